"""numpy restatement of the ``.rwkvq`` bit layouts and dequantisers.

TEST INFRASTRUCTURE (parity oracle / CPU baseline) -- not a product code path.

Every function states the layout as index arithmetic on the packed bytes and
cites the reference function it restates (paths relative to the reference
project root).  The restatement is pinned against the reference's own numpy
codec and against vectors produced by the reference's packers (see
tests/test_oracle_codec.py and tests/golden/).

Layout glossary (weights are [OUT, IN], blocks run along IN):
  sb6   block gs=32, super-block sb=8 blocks.  4 low code bits as block-local
        split nibbles, optional bit-planes for code bits 4 and 5, 6-bit block
        scale/min codes (8+8 per super-block in 12 bytes, min stored +31)
        against fp16 super-scales d / dm.          w = q*half(qs*d) + half(qm*dm)
  sym   block gs=16, sb=16.  Signed codes: int8 bytes (8 bit) or (code+32)
        packed like sb6 (6 bit); int8 block scale code against fp16 d.
                                                   w = q*half(qs*d)
  asym  block gs (64 for LoRA), fp32 scale and min per block, uint8 codes,
        ceil(IN/gs) blocks (ragged tail has its own pair).   w = q*scale + min
  rtn   per-row fp16 scale, int8 codes or biased split nibbles (code+8),
        optional sparse outlier overrides.         w = code*scale[row]
"""
from __future__ import annotations

import json
import mmap

import numpy as np

F32 = np.float32


# --------------------------------------------------------------------------
# bit-level unpackers
# --------------------------------------------------------------------------

def nibbles_blocklocal(packed: np.ndarray, gs: int) -> np.ndarray:
    """uint8 [OUT, IN/2] -> codes 0..15 [OUT, IN].

    Column c of block p=c//gs sits in byte p*gs/2 + (c%gs)%(gs/2); the low
    nibble holds the first half of the block, the high nibble the second half.
    Restates codec.unpack_nib_block (formats/codec.py:149-157)."""
    out_rows, half_cols = packed.shape
    n_in = half_cols * 2
    c = np.arange(n_in)
    j = c % gs
    byte = (c // gs) * (gs // 2) + j % (gs // 2)
    shift = np.where(j >= gs // 2, 4, 0).astype(np.uint8)
    return (packed[:, byte] >> shift) & np.uint8(0xF)


def bitplane(plane: np.ndarray, n_in: int) -> np.ndarray:
    """uint8 [OUT, IN/8] -> {0,1} [OUT, IN]; column c is bit c%8 of byte c//8.
    Restates codec.unpack_bitplane (formats/codec.py:172-178)."""
    c = np.arange(n_in)
    return (plane[:, c >> 3] >> (c & 7).astype(np.uint8)) & np.uint8(1)


def sixbit_stream(b: np.ndarray, n: int) -> np.ndarray:
    """Little-endian 6-bit stream: value i occupies bits [6i, 6i+6) of the byte
    string along the last axis.  Restates codec.unpack6 (formats/codec.py:122-131)."""
    b = np.asarray(b, dtype=np.uint8)
    i = np.arange(n)
    bit0 = 6 * i
    lo = b[..., bit0 >> 3].astype(np.uint16)
    hi_idx = np.minimum((bit0 >> 3) + 1, b.shape[-1] - 1)
    hi = b[..., hi_idx].astype(np.uint16)
    word = lo | (hi << 8)
    return ((word >> (bit0 & 7).astype(np.uint16)) & 0x3F).astype(np.uint8)


def nibbles_split_biased(packed: np.ndarray, n_cols: int) -> np.ndarray:
    """per-row rtn at <=4 bits: uint8 [rows, ceil(cols/2)] -> int8 [rows, cols].
    Low nibble of byte i is column i, high nibble is column i+ceil(cols/2);
    the nibble stores code+8.  Restates codec.unpack_int4 (formats/codec.py:99-105)."""
    half = packed.shape[1]
    c = np.arange(n_cols)
    hi = c >= half
    byte = np.where(hi, c - half, c)
    v = (packed[:, byte] >> np.where(hi, 4, 0).astype(np.uint8)) & np.uint8(0xF)
    return (v.astype(np.int16) - 8).astype(np.int8)


def bf16_bits_to_f32(u16: np.ndarray) -> np.ndarray:
    """bf16 carried as uint16 -> float32 (exact).  codec.bf16_to_f32 (formats/codec.py:456-459)."""
    return (np.asarray(u16).astype(np.uint32) << np.uint32(16)).view(F32)


def f32_to_bf16_rne(x: np.ndarray) -> np.ndarray:
    """float32 -> float32 holding the nearest-even bf16 value (what
    ``tensor.to(torch.bfloat16)`` does; reader._dequantize_one rounds every
    dequantised tensor this way, formats/reader.py:114-127)."""
    x = np.ascontiguousarray(x, dtype=F32)
    out = np.empty_like(x)
    flat_in, flat_out = x.reshape(-1), out.reshape(-1)

    def part(a, b):
        u = flat_in[a:b].view(np.uint32)
        nan = np.isnan(flat_in[a:b])
        r = u + (np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1)))     # wraps only for NaN patterns
        r &= np.uint32(0xFFFF0000)
        o = r.view(F32)
        o[nan] = np.nan
        flat_out[a:b] = o
    n, step = flat_in.size, 1 << 22
    if n <= step:
        part(0, n)
    else:
        import os
        from concurrent.futures import ThreadPoolExecutor
        with ThreadPoolExecutor(max_workers=min(32, os.cpu_count() or 1)) as ex:
            list(ex.map(lambda a: part(a, min(a + step, n)), range(0, n, step)))
    return out


def _half_roundtrip(x: np.ndarray) -> np.ndarray:
    return x.astype(np.float16).astype(F32)


# --------------------------------------------------------------------------
# dequantisers (float32 out, exact superset of the bf16 the torch reader emits)
# --------------------------------------------------------------------------

def dequant_sb6(codes_packed, qsqm, d, dm, *, shape, gs=32, sb=8, qh=None, qh2=None):
    """Restates codec.dequant_sb6 (formats/codec.py:183-216)."""
    n_out, n_in = shape
    nb = n_in // gs
    nsb = nb // sb
    assert qsqm.shape == (n_out, nsb, 12), qsqm.shape
    q = nibbles_blocklocal(np.asarray(codes_packed), gs).astype(F32)
    if qh is not None:
        q += bitplane(np.asarray(qh), n_in).astype(F32) * F32(16)
    if qh2 is not None:
        q += bitplane(np.asarray(qh2), n_in).astype(F32) * F32(32)
    qs = sixbit_stream(qsqm[..., 0:6], sb).reshape(n_out, nb).astype(F32)
    qm = sixbit_stream(qsqm[..., 6:12], sb).reshape(n_out, nb).astype(F32) - F32(31)
    blk2sb = np.arange(nb) // sb
    s = np.maximum(_half_roundtrip(qs * np.asarray(d, F32)[:, blk2sb]), F32(1e-8))
    m = _half_roundtrip(qm * np.asarray(dm, F32)[:, blk2sb])
    col2blk = np.arange(n_in) // gs
    return q * s[:, col2blk] + m[:, col2blk]


def dequant_sym(qs, d, *, shape, gs=16, sb=16, codes=None, codes_packed=None,
                qh=None, qh2=None):
    """Restates codec.dequant_sym (formats/codec.py:219-257).  Which code buffer
    is present decides the bit width (int8 ``codes`` = 8 bit, ``codes_packed`` = 6)."""
    n_out, n_in = shape
    nb = n_in // gs
    assert np.asarray(qs).shape == (n_out, nb)
    assert np.asarray(d).shape[-1] * sb == nb
    if codes is not None:
        q = np.asarray(codes).astype(F32)
    else:
        u = nibbles_blocklocal(np.asarray(codes_packed), gs).astype(np.int16)
        if qh is not None:
            u += bitplane(np.asarray(qh), n_in).astype(np.int16) * 16
        if qh2 is not None:
            u += bitplane(np.asarray(qh2), n_in).astype(np.int16) * 32
        q = (u - 32).astype(F32)
    blk2sb = np.arange(nb) // sb
    s = _half_roundtrip(np.asarray(qs).astype(F32) * np.asarray(d, F32)[:, blk2sb])
    return q * s[:, np.arange(n_in) // gs]


def dequant_asym(codes, scale, mn, *, shape, gs):
    """Restates codec.dequant_asym (formats/codec.py:260-276); ceil(IN/gs) blocks."""
    n_out, n_in = shape
    nb = -(-n_in // gs)
    assert np.asarray(scale).shape == (n_out, nb), (np.asarray(scale).shape, nb)
    blk = np.arange(n_in) // gs
    return (np.asarray(codes).astype(F32) * np.asarray(scale, F32)[:, blk]
            + np.asarray(mn, F32)[:, blk])


def dequant_rtn(scale, *, shape, codes=None, codes_packed=None,
                outlier_indices=None, outlier_values=None):
    """Restates codec.dequant_rtn (formats/codec.py:279-292)."""
    if codes is None:
        codes = nibbles_split_biased(np.asarray(codes_packed), shape[1])
    w = np.asarray(codes).astype(F32) * np.asarray(scale, F32)
    if outlier_indices is not None and len(outlier_indices):
        oi = np.asarray(outlier_indices)
        w[oi[:, 0], oi[:, 1]] = np.asarray(outlier_values, F32)
    return w


# --------------------------------------------------------------------------
# container
# --------------------------------------------------------------------------

_ST_DTYPES = {"BOOL": np.bool_, "U8": np.uint8, "I8": np.int8, "I16": np.int16,
              "U16": np.uint16, "F16": np.float16, "BF16": np.uint16,
              "I32": np.int32, "U32": np.uint32, "F32": np.float32,
              "F64": np.float64, "I64": np.int64, "U64": np.uint64}


def open_rwkvq(path: str):
    """(manifest, {"<key>::<field>": ndarray view on the mmap}).
    Restates codec.read_safetensors + codec.open_rwkvq (formats/codec.py:462-511):
    u64 little-endian header length, JSON header, raw buffers; the manifest is
    the JSON string under ``__metadata__["rwkvq"]``."""
    with open(path, "rb") as f:
        head = f.read(8)
        if head[:4] == b"PK\x03\x04":
            raise ValueError(f"{path}: legacy pickle container, not safetensors")
        n = int.from_bytes(head, "little")
        header = json.loads(f.read(n))
        mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
    raw = np.frombuffer(mm, dtype=np.uint8)
    meta = header.pop("__metadata__", {})
    if "rwkvq" not in meta:
        raise ValueError(f"{path}: no rwkvq manifest in __metadata__")
    manifest = json.loads(meta["rwkvq"])
    if manifest.get("format") != "rwkvq":
        raise ValueError(f"{path}: format {manifest.get('format')!r}")
    if manifest.get("format_version", 0) > 2:
        raise ValueError(f"{path}: format_version {manifest['format_version']} is newer than 2")
    arrays = {}
    for name, info in header.items():
        b, e = info["data_offsets"]
        dt = _ST_DTYPES[info["dtype"]]
        shp = tuple(info["shape"])
        a = raw[8 + n + b: 8 + n + e]
        arrays[name] = a.view(dt).reshape(shp) if a.size else np.empty(shp, dt)
    return manifest, arrays


def dequant_key(manifest, arrays, key) -> np.ndarray:
    """One tensor -> float32 in the stored orientation.
    Restates codec.dequant_key (formats/codec.py:538-571).  Large 2-D block-quantized tensors
    are decoded in row chunks on a thread pool (rows are independent in every layout and numpy
    releases the interpreter lock inside its loops); the result is the same array."""
    m = manifest["tensors"][key]
    kind, shape = m["kind"], tuple(m["shape"])
    if kind in ("sb6", "sym") and len(shape) == 2 and shape[0] * shape[1] >= (1 << 22) and shape[0] >= 64:
        import os
        from concurrent.futures import ThreadPoolExecutor
        rows = shape[0]
        step = max(16, min(1024, rows // 8))
        out = np.empty(shape, F32)
        names = [f for f in m["fields"] if arrays[f"{key}::{f}"].shape[:1] == (rows,)]

        def chunk(a):
            b = min(a + step, rows)
            sub = {f"{key}::{f}": arrays[f"{key}::{f}"][a:b] for f in names}
            man = {"tensors": {key: dict(m, shape=[b - a, shape[1]])}}
            out[a:b] = _dequant_one(man, sub, key)
        with ThreadPoolExecutor(max_workers=min(32, os.cpu_count() or 1)) as ex:
            list(ex.map(chunk, range(0, rows, step)))
        return out
    return _dequant_one(manifest, arrays, key)


def _dequant_one(manifest, arrays, key) -> np.ndarray:
    m = manifest["tensors"][key]
    kind, shape = m["kind"], tuple(m["shape"])
    g = lambda f: arrays.get(f"{key}::{f}")
    if kind == "dense":
        return bf16_bits_to_f32(g("dense")).reshape(shape)
    if kind == "sb6":
        return dequant_sb6(g("codes_packed"), g("gw_qsqm"), g("gw_d"), g("gw_dm"),
                           shape=shape, gs=m["gw_gs"], sb=m["gw_sb"],
                           qh=g("gw_qh"), qh2=g("gw_qh2"))
    if kind == "sym":
        return dequant_sym(g("gw_qs"), g("gw_d"), shape=shape, gs=m["gw_gs"],
                           sb=m["gw_sb"], codes=g("codes"),
                           codes_packed=g("codes_packed"), qh=g("gw_qh"), qh2=g("gw_qh2"))
    if kind == "asym":
        return dequant_asym(g("codes"), g("gw_scale"), g("gw_min"), shape=shape,
                            gs=m["gw_gs"])
    if kind == "rtn":
        ov = g("outlier_values")
        return dequant_rtn(g("scale"), shape=shape, codes=g("codes"),
                           codes_packed=g("codes_packed"),
                           outlier_indices=g("outlier_indices"),
                           outlier_values=None if ov is None else bf16_bits_to_f32(ov))
    raise ValueError(f"{key}: unknown layout {kind!r}")


def is_transposed(manifest, key) -> bool:
    """True when the stored tensor is [in, out] (world-naming LoRA matrices).
    Restates codec.is_transposed (formats/codec.py:514-535)."""
    m = manifest["tensors"][key]
    if "transposed" in m:
        return bool(m["transposed"])
    import re
    return (manifest.get("naming") == "world"
            and re.match(r"^blocks\.\d+\.att\.[wavg][12]$", key) is not None)
