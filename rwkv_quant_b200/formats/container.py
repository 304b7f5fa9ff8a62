"""``.rwkvq`` container: reader, writer and the checkpoint dataclasses.

The container is a safetensors file (u64 little-endian header length, JSON
header, raw buffers) whose ``__metadata__["rwkvq"]`` entry is a JSON manifest;
buffers are named ``"<key>::<field>"``.  This mirrors the reference's
``formats/reader.py`` (load_raw, :42-93), ``formats/codec.py`` (open_rwkvq,
:462-511) and the manifest written by ``formats/writer.py`` (save_rwkvq,
:82-142): same field names, same manifest keys, same error behaviour
(``ValueError`` for a foreign / future container).

Only numpy is needed to parse the file; buffers are zero-copy views on an mmap
and are handed to the CUDA backend as CPU torch tensors.
"""
from __future__ import annotations

import json
import mmap
import re
import warnings
from dataclasses import dataclass, field

import numpy as np
import torch

FORMAT = "rwkvq"
FORMAT_VERSION = 2
MAGIC_ZIP = b"PK\x03\x04"

# buffers a QuantizedTensor may carry on disk (formats/writer.py:39-44)
TENSOR_FIELDS = ("codes", "codes_packed", "scale", "dense",
                 "outlier_indices", "outlier_values",
                 "gw_d", "gw_dm", "gw_qsqm", "gw_qh", "gw_qh2",
                 "gw_scale", "gw_min", "gw_qs")

_RAW_LORA_WORLD = re.compile(r"^blocks\.\d+\.att\.[wavg][12]$")

_NP_OF_ST = {"BOOL": np.bool_, "U8": np.uint8, "I8": np.int8, "I16": np.int16,
             "U16": np.uint16, "F16": np.float16, "BF16": np.uint16,
             "I32": np.int32, "U32": np.uint32, "F32": np.float32,
             "F64": np.float64, "I64": np.int64, "U64": np.uint64}
_ST_OF_TORCH = {torch.uint8: "U8", torch.int8: "I8", torch.int16: "I16",
                torch.float16: "F16", torch.bfloat16: "BF16",
                torch.int32: "I32", torch.float32: "F32", torch.int64: "I64",
                torch.bool: "BOOL"}


@dataclass
class QuantizedTensor:
    """One tensor of a ``.rwkvq`` file; field names follow the reference's
    ``formats/schema.py:45-81`` so that either loader's objects can be passed
    to the backend classes."""
    key: str
    group: str
    bits: int
    shape: tuple
    codes: torch.Tensor = None
    codes_packed: torch.Tensor = None
    scale: torch.Tensor = None
    dense: torch.Tensor = None
    outlier_indices: torch.Tensor = None
    outlier_values: torch.Tensor = None
    gw_mode: str = ""            # "" (per-row rtn / dense) | "sb6" | "sym" | "asym"
    gw_gs: int = 0
    gw_sb: int = 0
    gw_d: torch.Tensor = None
    gw_dm: torch.Tensor = None
    gw_qsqm: torch.Tensor = None
    gw_qh: torch.Tensor = None
    gw_qh2: torch.Tensor = None
    gw_scale: torch.Tensor = None
    gw_min: torch.Tensor = None
    gw_qs: torch.Tensor = None
    transposed: bool = False     # stored [in, out] (world-naming LoRA matrices)

    @property
    def kind(self) -> str:
        return "dense" if self.bits >= 16 else (self.gw_mode or "rtn")

    def nbytes(self) -> int:
        """Bytes this tensor occupies in the file format."""
        return sum(int(getattr(self, f).numel() * getattr(self, f).element_size())
                   for f in TENSOR_FIELDS if getattr(self, f) is not None)


@dataclass
class QuantizedCheckpoint:
    """Mirrors ``formats/schema.py:84-97``."""
    naming: str
    n_layer: int
    n_embd: int
    head_size: int
    vocab_size: int
    tensors: dict = field(default_factory=dict)
    config_repr: str = ""
    config: object = None
    tokenizer: str = None

    def weight_bytes(self, exclude=("emb.weight",)) -> int:
        """File-format bytes of everything a decode step streams: all tensors
        except the embedding table (one row is gathered per token)."""
        return sum(qt.nbytes() for k, qt in self.tensors.items() if k not in exclude)


def expected_field_elems(kind: str, bits: int, rows: int, cols: int, gs: int, sb: int,
                         int8_codes: bool) -> dict:
    """Element count every buffer of a tensor must have for its stored shape [rows, cols]
    (formats/writer.py:236-337, codec.py:81-105): what the kernels index without further
    checks.  ``int8_codes``: the tensor carries ``codes`` rather than ``codes_packed``."""
    n = rows * cols
    if kind == "dense":
        return {"dense": n}
    if kind == "sb6":
        if gs <= 0 or sb <= 0 or cols % (gs * sb):
            raise ValueError(f"sb6 tensor with {cols} columns, group {gs} x {sb}")
        nsb = cols // (gs * sb)
        out = {"codes_packed": n // 2, "gw_qsqm": rows * nsb * (sb * 12 // 8), "gw_d": rows * nsb,
               "gw_dm": rows * nsb}
        if bits >= 5:
            out["gw_qh"] = n // 8
        if bits >= 6:
            out["gw_qh2"] = n // 8
        return out
    if kind == "sym":
        if gs <= 0 or sb <= 0 or cols % (gs * sb):
            raise ValueError(f"sym tensor with {cols} columns, group {gs} x {sb}")
        out = {"gw_qs": rows * (cols // gs), "gw_d": rows * (cols // (gs * sb))}
        if int8_codes:
            out["codes"] = n
        else:
            out["codes_packed"] = n // 2
            if bits >= 5:
                out["gw_qh"] = n // 8
            if bits >= 6:
                out["gw_qh2"] = n // 8
        return out
    if kind == "asym":
        if gs <= 0:
            raise ValueError(f"asym tensor with group {gs}")
        nb = (cols + gs - 1) // gs
        return {"codes": n, "gw_scale": rows * nb, "gw_min": rows * nb}
    if kind == "rtn":
        return {("codes" if int8_codes else "codes_packed"): n if int8_codes else rows * ((cols + 1) // 2),
                "scale": rows}
    raise ValueError(f"unknown layout kind {kind!r}")


def check_tensor_sizes(qt) -> None:
    """Refuse (ValueError) a tensor whose buffers do not have the sizes its manifest shape, layout
    and bit width imply, or whose sparse overrides point outside it, before any kernel indexes
    them.  The reference fails on the host for such files too (numpy reshape in its codec).
    Works on this package's QuantizedTensor and on the reference's (same field names)."""
    shape = tuple(int(v) for v in qt.shape)
    bits = int(qt.bits)
    kind = "dense" if bits >= 16 else (getattr(qt, "gw_mode", "") or "rtn")
    key = getattr(qt, "key", "?")
    if not shape or min(shape) < 1:
        raise ValueError(f"{key}: unusable shape {shape}")
    cols = shape[-1]
    rows = 1
    for v in shape[:-1]:
        rows *= v
    have = lambda f: getattr(qt, f, None) is not None and getattr(qt, f).numel() > 0
    want = expected_field_elems(kind, bits, rows, cols, int(getattr(qt, "gw_gs", 0) or 0),
                                int(getattr(qt, "gw_sb", 0) or 0), have("codes"))
    if kind in ("sb6", "sym"):                  # a plane the bit width does not call for is still read when present
        for f in ("gw_qh", "gw_qh2"):
            if have(f):
                want.setdefault(f, rows * cols // 8)
    for f, n in want.items():
        got = getattr(qt, f).numel() if have(f) else 0
        if got != n:
            raise ValueError(f"{key}: buffer {f} has {got} elements, its {kind}@{bits} layout of shape "
                             f"{list(shape)} needs {n}")
    if have("outlier_indices"):
        oi = qt.outlier_indices.reshape(-1, 2)
        nv = qt.outlier_values.numel() if have("outlier_values") else 0
        if oi.shape[0] != nv:
            raise ValueError(f"{key}: {oi.shape[0]} outlier positions for {nv} values")
        if len(shape) != 2:
            raise ValueError(f"{key}: outlier overrides on a {len(shape)}-D tensor")
        r, c = oi[:, 0].long(), oi[:, 1].long()
        if bool(((r < 0) | (r >= rows) | (c < 0) | (c >= cols)).any()):
            raise ValueError(f"{key}: an outlier override points outside the [{rows}, {cols}] tensor")


def is_raw_lora_world(key: str) -> bool:
    """World checkpoints keep blocks.N.att.{w,a,v,g}{1,2} as [in, out]
    (formats/codec.py:529-535)."""
    return _RAW_LORA_WORLD.match(key) is not None


# --------------------------------------------------------------------------
# safetensors, torch-free parsing
# --------------------------------------------------------------------------

def read_safetensors(path: str):
    """(metadata dict, {name: read-only ndarray view on the mmap})."""
    with open(path, "rb") as f:
        head = f.read(8)
        if head[:4] == MAGIC_ZIP:
            raise ValueError(f"{path}: legacy pickle (torch.save) container; "
                             f"only the safetensors container is supported")
        if len(head) < 8:
            raise ValueError(f"{path}: truncated file")
        n = int.from_bytes(head, "little")
        try:
            header = json.loads(f.read(n))
        except Exception as e:  # noqa: BLE001
            raise ValueError(f"{path}: unreadable safetensors header ({e})") from None
        mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
    raw = np.frombuffer(mm, dtype=np.uint8)
    meta = header.pop("__metadata__", {}) or {}
    arrays = {}
    for name, info in header.items():
        b, e = info["data_offsets"]
        dt = _NP_OF_ST[info["dtype"]]
        shp = tuple(info["shape"])
        a = raw[8 + n + b: 8 + n + e]
        arrays[name] = (a.view(dt).reshape(shp) if a.size else np.empty(shp, dt),
                        info["dtype"])
    return meta, arrays


def open_rwkvq(path: str):
    """(manifest, {"<key>::<field>": ndarray}); bf16 buffers arrive as uint16."""
    meta, arrays = read_safetensors(path)
    if "rwkvq" not in meta:
        raise ValueError(f"{path}: not a .rwkvq file (no rwkvq manifest)")
    manifest = json.loads(meta["rwkvq"])
    if manifest.get("format") != FORMAT:
        raise ValueError(f"{path}: format {manifest.get('format')!r}, expected {FORMAT!r}")
    if manifest.get("format_version", 0) > FORMAT_VERSION:
        raise ValueError(f"{path}: format_version {manifest['format_version']} is newer "
                         f"than this reader understands ({FORMAT_VERSION})")
    return manifest, {k: v[0] for k, v in arrays.items()}, {k: v[1] for k, v in arrays.items()}


def _to_torch(a: np.ndarray, st_dtype: str) -> torch.Tensor:
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")          # read-only mmap view
        t = torch.from_numpy(a)
    if st_dtype == "BF16":
        t = t.view(torch.bfloat16)
    return t


def load_raw(path: str) -> QuantizedCheckpoint:
    """``.rwkvq`` -> QuantizedCheckpoint (buffers are CPU tensors viewing the mmap)."""
    manifest, arrays, dtypes = open_rwkvq(path)
    tensors = {}
    for key, t in manifest["tensors"].items():
        kind = t["kind"]
        qt = QuantizedTensor(
            key=key, group=t.get("group", "other"), bits=int(t["bits"]),
            shape=tuple(t["shape"]),
            gw_mode=kind if kind in ("sb6", "sym", "asym") else "",
            gw_gs=int(t.get("gw_gs", 0)), gw_sb=int(t.get("gw_sb", 0)),
            transposed=bool(t["transposed"]) if "transposed" in t else
            (manifest.get("naming") == "world" and is_raw_lora_world(key)))
        for f in t["fields"]:
            name = f"{key}::{f}"
            setattr(qt, f, _to_torch(arrays[name], dtypes[name]))
        check_tensor_sizes(qt)
        if kind == "dense" and qt.dense is not None:
            qt.dense = qt.dense.reshape(qt.shape)
        tensors[key] = qt
    return QuantizedCheckpoint(
        naming=manifest["naming"], n_layer=int(manifest["n_layer"]),
        n_embd=int(manifest["n_embd"]), head_size=int(manifest["head_size"]),
        vocab_size=int(manifest["vocab_size"]), tensors=tensors,
        config_repr=manifest.get("config_repr", ""), config=manifest.get("config"),
        tokenizer=manifest.get("tokenizer"))


# --------------------------------------------------------------------------
# writer (used for synthetic random-init builds and round-trip tests)
# --------------------------------------------------------------------------

def _n_blocks(qt: QuantizedTensor) -> int:
    if qt.gw_mode == "sb6":
        return int(qt.gw_qsqm.shape[-2]) * int(qt.gw_sb)
    if qt.gw_mode == "asym":
        return int(qt.gw_scale.shape[-1])
    if qt.gw_mode == "sym":
        return int(qt.gw_qs.shape[-1])
    return 0


def save_rwkvq(ckpt: QuantizedCheckpoint, path: str) -> None:
    """Write the safetensors container with the version-2 manifest layout."""
    entries, manifest_t = [], {}
    for key, qt in ckpt.tensors.items():
        fields = []
        for f in TENSOR_FIELDS:
            v = getattr(qt, f, None)
            if v is None or v.numel() == 0:
                continue
            entries.append((f"{key}::{f}", v.detach().cpu().contiguous()))
            fields.append(f)
        manifest_t[key] = {
            "kind": qt.kind, "shape": [int(x) for x in qt.shape],
            "bits": int(qt.bits), "group": qt.group or "other",
            "gw_gs": int(qt.gw_gs), "gw_sb": int(qt.gw_sb),
            "n_blocks": _n_blocks(qt),
            "transposed": ckpt.naming == "world" and is_raw_lora_world(key),
            "fields": fields}
    manifest = {"format": FORMAT, "format_version": FORMAT_VERSION,
                "naming": ckpt.naming, "n_layer": int(ckpt.n_layer),
                "n_embd": int(ckpt.n_embd), "head_size": int(ckpt.head_size),
                "vocab_size": int(ckpt.vocab_size),
                "config_repr": ckpt.config_repr,
                "config": ckpt.config if isinstance(ckpt.config, (dict, type(None))) else None,
                "tokenizer": ckpt.tokenizer, "tensors": manifest_t}
    header, off = {"__metadata__": {"rwkvq": json.dumps(manifest)}}, 0
    for name, t in entries:
        nb = t.numel() * t.element_size()
        header[name] = {"dtype": _ST_OF_TORCH[t.dtype], "shape": list(t.shape),
                        "data_offsets": [off, off + nb]}
        off += nb
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((-len(hj)) % 8)
    with open(path, "wb") as f:
        f.write(len(hj).to_bytes(8, "little"))
        f.write(hj)
        for _, t in entries:
            f.write(t.reshape(-1).view(torch.uint8).numpy().tobytes())
