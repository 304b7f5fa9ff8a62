"""PyTorch custom ops (namespace ``rwkvq``) over the C ABI, and the device-side
view of a quantized tensor.

Every op takes the tensor's file buffers as a fixed-order list plus six
integers, builds the ``rwkvq_qtensor`` descriptor and calls the library on the
current CUDA stream.  Nothing here computes on the CPU.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import List, Optional, Sequence

import torch

from ... import _lib
from ..._lib import QTensorStruct

_BUF_ORDER = ("codes", "qh", "qh2", "qsqm", "qs", "d", "dm", "scale", "mn",
              "dev_meta", "dev_planes")


def _descr(bufs: Sequence[torch.Tensor], meta: Sequence[int]) -> QTensorStruct:
    s = QTensorStruct()
    s.kind, s.bits, s.rows, s.cols, s.gs, s.sb = (int(v) for v in meta[:6])
    for name, b in zip(_BUF_ORDER, bufs):
        setattr(s, name, b.data_ptr() if b.numel() else None)
    return s


def _require_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("rwkvq ops run on CUDA tensors only (there is no CPU path)")


class DeviceQT:
    """A QuantizedTensor uploaded to the GPU in the file layout (no repack).

    Accepts this package's ``QuantizedTensor`` or the reference's (same field
    names, formats/schema.py:45-81).  ``rows, cols`` is the stored 2-D shape."""

    def __init__(self, qt, device="cuda", relayout=True):
        shape = tuple(qt.shape)
        if len(shape) != 2:
            raise ValueError(f"{getattr(qt, 'key', '?')}: only 2-D tensors, got {shape}")
        # the descriptor carries no buffer sizes: a short buffer or an override outside the
        # tensor must be refused here, on the host, before a kernel indexes it
        from ...formats.container import check_tensor_sizes
        check_tensor_sizes(qt)
        self.outliers = None          # (rows, cols, values fp32, first index of each row run, run lengths)
        self.key = getattr(qt, "key", "")
        self.rows, self.cols = int(shape[0]), int(shape[1])
        self.bits = int(qt.bits)
        mode = getattr(qt, "gw_mode", "") or ""
        self.kind = "dense" if self.bits >= 16 else (mode or "rtn")
        self.gs, self.sb = int(getattr(qt, "gw_gs", 0) or 0), int(getattr(qt, "gw_sb", 0) or 0)
        dev = torch.device(device)

        def up(t, dtype=None):
            if t is None:
                return torch.empty(0, dtype=torch.uint8, device=dev)
            t = t.to(dev, non_blocking=True)
            if dtype is not None and t.dtype != dtype:
                t = t.to(dtype)
            return t.contiguous()

        g = lambda f: getattr(qt, f, None)
        none = up(None)
        b = dict.fromkeys(_BUF_ORDER, none)
        if self.kind == "dense":
            b["codes"] = up(qt.dense, torch.bfloat16)
        elif self.kind == "sb6":
            b.update(codes=up(qt.codes_packed), qh=up(g("gw_qh")), qh2=up(g("gw_qh2")),
                     qsqm=up(qt.gw_qsqm), d=up(qt.gw_d, torch.float16), dm=up(qt.gw_dm, torch.float16))
        elif self.kind == "sym":
            codes = qt.codes if g("codes") is not None else qt.codes_packed
            b.update(codes=up(codes), qh=up(g("gw_qh")), qh2=up(g("gw_qh2")),
                     qs=up(qt.gw_qs, torch.int8), d=up(qt.gw_d, torch.float16))
        elif self.kind == "asym":
            b.update(codes=up(qt.codes), scale=up(qt.gw_scale, torch.float32),
                     mn=up(qt.gw_min, torch.float32))
        elif self.kind == "rtn":
            codes = qt.codes if g("codes") is not None else qt.codes_packed
            b.update(codes=up(codes), scale=up(qt.scale.reshape(-1), torch.float16))
        else:
            raise NotImplementedError(f"{self.key}: layout {self.kind!r}")
        self.bufs: List[torch.Tensor] = [b[n] for n in _BUF_ORDER]
        self.meta: List[int] = [_lib.KIND[self.kind], self.bits, self.rows, self.cols, self.gs, self.sb]
        self.struct = _descr(self.bufs, self.meta)
        if relayout and dev.type == "cuda":
            self._relayout()
        oi = getattr(qt, "outlier_indices", None)
        if oi is not None and oi.numel() > 0:
            self._attach_outliers(oi, qt.outlier_values, dev)

    def _attach_outliers(self, oi, ov, dev):
        """Sparse overrides of per-row tensors (formats/codec.py:279-292): W[r, c] = value.  Kept
        sorted by (row, column); ``delta`` = value - quantized value is what a product over the
        packed codes is short of."""
        if self.kind != "rtn":
            raise NotImplementedError(f"{self.key}: outlier overrides on a {self.kind!r} tensor")
        oi = oi.to(dev).long().reshape(-1, 2)
        vals = ov.to(dev).to(torch.bfloat16).float().reshape(-1)
        order = torch.argsort(oi[:, 0] * self.cols + oi[:, 1], stable=True)
        # a position listed twice keeps its last value, as the codec's fancy assignment does
        key = (oi[:, 0] * self.cols + oi[:, 1])[order]
        last = torch.ones_like(key, dtype=torch.bool)
        last[:-1] = key[1:] != key[:-1]
        order = order[last]
        rows, cols, vals = oi[order, 0], oi[order, 1], vals[order]
        wq = dequant(self.bufs, self.meta, torch.float32, False)[rows, cols]
        # CSR over the rows for the tail kernel: row_ptr [rows + 1], columns and deltas in (row, column) order
        row_ptr = torch.zeros(self.rows + 1, dtype=torch.int32, device=dev)
        row_ptr[1:] = torch.cumsum(torch.bincount(rows, minlength=self.rows), 0).to(torch.int32)
        self.outliers = (rows, cols, vals, (vals - wq).contiguous(), row_ptr, cols.to(torch.int32).contiguous())

    def dequant(self, out_dtype: torch.dtype = torch.float32, round_bf16: bool = False) -> torch.Tensor:
        """Dense [rows, cols] with the outlier overrides applied (fp32: the codec's bits)."""
        w = dequant(self.bufs, self.meta, out_dtype, round_bf16)
        if self.outliers is not None:
            rows, cols, vals = self.outliers[:3]
            w[rows, cols] = vals.to(out_dtype)
        return w

    def gemv(self, x: torch.Tensor, epilogue: int = 0, resid: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x [N, cols] -> [N, rows]; tensors with outliers: the product over the packed codes, then the
        CSR tail kernel adds every row's override terms in column order (deterministic) and applies the
        epilogue (the reference's per-row kernels carry the same tail, quant_linear_v2.py:47-55)."""
        if self.outliers is None:
            return gemv(self.bufs, self.meta, x, epilogue, resid)
        delta, row_ptr, cols32 = self.outliers[3:6]
        y = gemv(self.bufs, self.meta, x, 0, None)
        _lib.check(_lib.load().rwkvq_outlier_tail(row_ptr.data_ptr(), cols32.data_ptr(), delta.data_ptr(), self.rows,
                                                  x.data_ptr(), _lib.DTYPE_CODE[x.dtype], x.shape[0], x.stride(0),
                                                  y.data_ptr(), y.stride(0), epilogue, _lib.ptr(resid), _lib.stream_ptr()),
                   "rwkvq_outlier_tail")
        return y

    def densified(self) -> "DeviceQT":
        """The tensor as a dense bf16 one with the overrides applied (what the kernels that read
        packed codes directly are given instead of a tensor with outliers)."""
        from ...formats.container import QuantizedTensor
        w = self.dequant(torch.float32, True).to(torch.bfloat16)
        qt = QuantizedTensor(key=self.key, group="", bits=16, shape=(self.rows, self.cols))
        qt.dense = w
        return DeviceQT(qt, device=w.device)

    def transposed_dense(self) -> "DeviceQT":
        """W^T as a dense bf16 tensor [cols, rows] (overrides applied): how a LoRA matrix stored
        as an nn.Linear weight [out, in] is handed to the kernels, which read LoRA matrices
        [in, out]."""
        from ...formats.container import QuantizedTensor
        w = self.dequant(torch.float32, True).t().contiguous().to(torch.bfloat16)
        qt = QuantizedTensor(key=self.key, group="", bits=16, shape=(self.cols, self.rows))
        qt.dense = w
        return DeviceQT(qt, device=w.device)

    def _relayout(self):
        """Regroup the scale records / bit-planes for the decode kernels (same bytes,
        done once at load on the device)."""
        lib = _lib.load()
        dev = self.bufs[0].device
        i_meta, i_planes = _BUF_ORDER.index("dev_meta"), _BUF_ORDER.index("dev_planes")
        with torch.cuda.device(dev):
            if self.kind == "sb6":
                m = torch.empty((self.rows, self.cols // 256, 16), dtype=torch.uint8, device=dev)
                _lib.check(lib.rwkvq_relayout_meta(C.byref(self.struct), m.data_ptr(), _lib.stream_ptr()),
                           "rwkvq_relayout_meta")
                self.bufs[i_meta] = m
            words = {("sb6", 5): self.cols // 32, ("sb6", 6): self.cols // 16,
                     ("sym", 6): self.cols // 16}.get((self.kind, self.bits))
            if words:
                p = torch.empty((self.rows, words), dtype=torch.int32, device=dev)
                _lib.check(lib.rwkvq_relayout_planes(C.byref(self.struct), p.data_ptr(), _lib.stream_ptr()),
                           "rwkvq_relayout_planes")
                self.bufs[i_planes] = p
        self.struct = _descr(self.bufs, self.meta)

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.bufs)

    def nbytes_file(self) -> int:
        """Bytes of the tensor in the file format (the relayout copies excluded)."""
        return sum(t.numel() * t.element_size() for t in self.bufs[:9])

    def slice_rows(self, a: int, b: int) -> "DeviceQT":
        """Rows [a, b) as a view: every layout stores rows first and blocks along
        the columns, so any row range is a valid tensor (formats/reader.py:130-152)."""
        out = object.__new__(DeviceQT)
        out.__dict__.update(self.__dict__)
        out.rows = b - a
        out.bufs = [t[a:b] if t.numel() else t for t in self.bufs]
        out.meta = list(self.meta)
        out.meta[2] = b - a
        out.struct = _descr(out.bufs, out.meta)
        return out


# ---------------------------------------------------------------------------
# custom ops
# ---------------------------------------------------------------------------

@torch.library.custom_op("rwkvq::dequant", mutates_args=())
def dequant(bufs: Sequence[torch.Tensor], meta: Sequence[int], out_dtype: torch.dtype,
            round_bf16: bool) -> torch.Tensor:
    _require_cuda(bufs[0])
    lib = _lib.load()
    d = _descr(bufs, meta)
    out = torch.empty((meta[2], meta[3]), dtype=out_dtype, device=bufs[0].device)
    _lib.check(lib.rwkvq_dequant(C.byref(d), out.data_ptr(), _lib.DTYPE_CODE[out_dtype],
                                 int(round_bf16), _lib.stream_ptr()), "rwkvq_dequant")
    return out


@dequant.register_fake
def _(bufs, meta, out_dtype, round_bf16):
    return torch.empty((meta[2], meta[3]), dtype=out_dtype, device=bufs[0].device)


@torch.library.custom_op("rwkvq::gemv", mutates_args=())
def gemv(bufs: Sequence[torch.Tensor], meta: Sequence[int], x: torch.Tensor, epilogue: int,
         resid: Optional[torch.Tensor]) -> torch.Tensor:
    """x [N, IN] (fp32 / fp16 / bf16, contiguous rows) -> y [N, OUT] fp32."""
    _require_cuda(bufs[0], x, resid)
    lib = _lib.load()
    d = _descr(bufs, meta)
    n = x.shape[0]
    y = torch.empty((n, meta[2]), dtype=torch.float32, device=x.device)
    _lib.check(lib.rwkvq_gemv(C.byref(d), x.data_ptr(), _lib.DTYPE_CODE[x.dtype], n, x.stride(0),
                              y.data_ptr(), y.stride(0), epilogue, _lib.ptr(resid),
                              _lib.stream_ptr()), "rwkvq_gemv")
    return y


@gemv.register_fake
def _(bufs, meta, x, epilogue, resid):
    return torch.empty((x.shape[0], meta[2]), dtype=torch.float32, device=x.device)


@torch.library.custom_op("rwkvq::gemv_t", mutates_args=())
def gemv_t(bufs: Sequence[torch.Tensor], meta: Sequence[int], x: torch.Tensor, act: int,
           round_w: bool) -> torch.Tensor:
    """x [N, rows] fp32 against a tensor stored [rows=in, cols=out] -> [N, cols]."""
    _require_cuda(bufs[0], x)
    lib = _lib.load()
    d = _descr(bufs, meta)
    n = x.shape[0]
    y = torch.empty((n, meta[3]), dtype=torch.float32, device=x.device)
    _lib.check(lib.rwkvq_gemv_t(C.byref(d), x.data_ptr(), n, x.stride(0), y.data_ptr(),
                                y.stride(0), act, int(round_w), _lib.stream_ptr()), "rwkvq_gemv_t")
    return y


@gemv_t.register_fake
def _(bufs, meta, x, act, round_w):
    return torch.empty((x.shape[0], meta[3]), dtype=torch.float32, device=x.device)


def batch_fast() -> bool:
    """RWKVQ_BATCH_FAST=1 in the environment: the small-batch linears use single fp16 operands
    (and the tcgen05 kernel above 32 rows) instead of the default two-term kernel.  The library
    reads the variable once, at its first small-batch call."""
    return os.environ.get("RWKVQ_BATCH_FAST", "")[:1] == "1"


def has_batch_layout(dq: "DeviceQT") -> bool:
    """Whether ``gemv_batch`` serves the tensor (the layouts of the tensor-core GEMV family)."""
    if dq.outliers is not None:
        return False
    if dq.kind == "sb6":
        return dq.cols % 256 == 0
    if dq.kind == "sym":
        return dq.cols % 256 == 0
    return dq.kind == "rtn" and dq.bits > 4 and dq.cols % 128 == 0


def gemv_batch(dq: "DeviceQT", x: torch.Tensor, epilogue: int = 0, resid: Optional[torch.Tensor] = None,
               check: bool = False) -> torch.Tensor:
    """x [N, IN] -> y [N, OUT] fp32 with the packed weights read once for all N rows (mma.sync
    tensor cores, tokens as the MMA columns, fp16 operands, fp32 accumulation)."""
    _require_cuda(x, resid)
    lib = _lib.load()
    x = x.float()
    if x.stride(-1) != 1 or x.stride(0) % 4 or x.data_ptr() % 16:
        x = x.contiguous()
    n = x.shape[0]
    y = torch.empty((n, dq.rows), dtype=torch.float32, device=x.device)
    nws = lib.rwkvq_gemv_batch_workspace_bytes(n)
    ws = torch.empty(nws, dtype=torch.uint8, device=x.device)
    _lib.check(lib.rwkvq_gemv_batch(C.byref(dq.struct), x.data_ptr(), n, x.stride(0), y.data_ptr(), y.stride(0),
                                    epilogue, _lib.ptr(resid), ws.data_ptr(), nws, _lib.stream_ptr()), "rwkvq_gemv_batch")
    if check:          # synchronises: the kernel's own report that a bounded pipeline wait ran out
        _lib.check(int(ws[:4].view(torch.int32).item()), "rwkvq_gemv_batch(kernel status)")
    return y


def lora_pair_ok(pairs, D: int) -> bool:
    """Whether ``lora_pair`` serves these (W1 [D, r], W2 [r, C]) tensor pairs (one C for all, a multiple of 32)."""
    C_out = pairs[0][1].cols
    return D % 128 == 0 and C_out % 32 == 0 and all(a.rows == D and b.cols == C_out and a.cols == b.rows and a.cols % 16 == 0
                                and 16 <= a.cols <= 512 and a.outliers is None and b.outliers is None for a, b in pairs)


def lora_pair(pairs, xs: Sequence[torch.Tensor], acts: Sequence[int]) -> List[torch.Tensor]:
    """y_i = act_i(x_i @ W1_i) @ W2_i for up to four (W1, W2) pairs of tensors stored [in, out], x_i
    [N, D] fp32 -> y_i [N, C]: two tensor-core launches for all branches (act: 0 none, 1 tanh, 2 sigmoid)."""
    lib = _lib.load()
    n_br = len(pairs)
    xs = [x.float().contiguous() for x in xs]
    _require_cuda(*xs)
    N, D = xs[0].shape
    ys = [torch.empty((N, pairs[0][1].cols), dtype=torch.float32, device=xs[0].device) for _ in range(n_br)]
    t1 = (QTensorStruct * n_br)(*[a.struct for a, _ in pairs])
    t2 = (QTensorStruct * n_br)(*[b.struct for _, b in pairs])
    nws = lib.rwkvq_lora_pair_workspace_bytes(N, max(a.cols for a, _ in pairs))
    ws = torch.empty(nws, dtype=torch.uint8, device=xs[0].device)
    _lib.check(lib.rwkvq_lora_pair(t1, t2, n_br, (C.c_void_p * n_br)(*[x.data_ptr() for x in xs]),
                                   (C.c_void_p * n_br)(*[y.data_ptr() for y in ys]), (C.c_int * n_br)(*acts), N, D,
                                   ws.data_ptr(), nws, _lib.stream_ptr()), "rwkvq_lora_pair")
    return ys


def gemm(dq: "DeviceQT", x: torch.Tensor, epilogue: int = 0, resid: Optional[torch.Tensor] = None,
         check: bool = False) -> torch.Tensor:
    """x [M, IN] fp32 -> y [M, OUT] fp32 on the tcgen05 tensor cores with the dequantisation
    fused into the operand producer (sb6 / sym tensors).  ``check`` synchronises and raises
    if the kernel reported that a bounded pipeline wait ran out."""
    _require_cuda(x, resid)
    lib = _lib.load()
    x = x.float().contiguous()
    m = x.shape[0]
    nws = lib.rwkvq_gemm_workspace_bytes_for(m, dq.cols)
    ws = torch.empty(nws, dtype=torch.uint8, device=x.device)
    y = torch.empty((m, dq.rows), dtype=torch.float32, device=x.device)
    _lib.check(lib.rwkvq_gemm(C.byref(dq.struct), x.data_ptr(), m, x.stride(0), y.data_ptr(), y.stride(0),
                              epilogue, _lib.ptr(resid), ws.data_ptr(), nws, _lib.stream_ptr()), "rwkvq_gemm")
    if check:
        st = int(ws[:4].view(torch.int32).item())
        _lib.check(st, "rwkvq_gemm(kernel status)")
    return y


class PreparedRows:
    """Activation rows in the forms their consumers read (made by ``seq_ln_shift_mix_prep``):
    ``x16``/``scale`` for ``gemm_x16``, ``split`` ([hi | lo] fp16) for the LoRA products, ``f32``."""
    __slots__ = ("x16", "scale", "split", "f32", "n", "cols")

    def __init__(self, n, cols):
        self.x16 = self.scale = self.split = self.f32 = None
        self.n, self.cols = n, cols


PREP_SCALED, PREP_SPLIT, PREP_F32 = 1, 2, 4


def gemm_x16(dq: "DeviceQT", rows: PreparedRows, epilogue: int = 0, resid: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``gemm`` on rows already scaled and rounded to fp16 (no pre-pass over the activations)."""
    _require_cuda(rows.x16, resid)
    lib = _lib.load()
    m = rows.n
    nws = lib.rwkvq_gemm_workspace_bytes_for(m, 0)
    ws = torch.empty(nws, dtype=torch.uint8, device=rows.x16.device)
    y = torch.empty((m, dq.rows), dtype=torch.float32, device=rows.x16.device)
    _lib.check(lib.rwkvq_gemm_x16(C.byref(dq.struct), rows.x16.data_ptr(), rows.scale.data_ptr(), m, y.data_ptr(),
                                  y.stride(0), epilogue, _lib.ptr(resid), ws.data_ptr(), nws, _lib.stream_ptr()),
               "rwkvq_gemm_x16")
    return y


def seq_ln_shift_mix_prep(x: torch.Tensor, ln_w, ln_b, shift_in: Optional[torch.Tensor], mix: torch.Tensor,
                          modes: Sequence[int]):
    """``seq_ln_shift_mix`` writing every mix row in the forms ``modes[m]`` selects (PREP_SCALED |
    PREP_SPLIT | PREP_F32) -> ([PreparedRows] * n_mix, new shift state [B, 1, D])."""
    _require_cuda(x, shift_in, mix)
    lib = _lib.load()
    B, T, D = x.shape
    N = B * T
    x = x.float().contiguous()
    mix2 = mix.reshape(-1, D).contiguous()
    n_mix = mix2.shape[0]
    assert len(modes) == n_mix
    pitch = lib.rwkvq_gemm_x16_pitch(D)
    dev = x.device
    rows, tabs = [], [[None] * n_mix for _ in range(4)]
    for m, mode in enumerate(modes):
        r = PreparedRows(N, D)
        if mode & PREP_SCALED:
            r.x16 = torch.empty((N, pitch), dtype=torch.float16, device=dev)
            r.scale = torch.empty(N, dtype=torch.float32, device=dev)
            tabs[0][m], tabs[1][m] = r.x16.data_ptr(), r.scale.data_ptr()
        if mode & PREP_SPLIT:
            r.split = torch.empty((N, 2 * D), dtype=torch.float16, device=dev)
            tabs[2][m] = r.split.data_ptr()
        if mode & PREP_F32:
            r.f32 = torch.empty((N, D), dtype=torch.float32, device=dev)
            tabs[3][m] = r.f32.data_ptr()
        rows.append(r)
    new_shift = torch.empty((B, 1, D), dtype=torch.float32, device=dev)
    sin = None if shift_in is None else shift_in.float().contiguous()
    ctab = [(C.c_void_p * n_mix)(*t) for t in tabs]
    _lib.check(lib.rwkvq_seq_ln_shift_mix_prep(x.data_ptr(), ln_w.data_ptr(), ln_b.data_ptr(), _lib.ptr(sin),
                                               mix2.data_ptr(), n_mix, (C.c_int * n_mix)(*modes), ctab[0], ctab[1],
                                               ctab[2], ctab[3], new_shift.data_ptr(), B, T, D, _lib.stream_ptr()),
               "rwkvq_seq_ln_shift_mix_prep")
    return rows, new_shift


def gemv_fused(dqts: Sequence[DeviceQT], xstack: torch.Tensor) -> torch.Tensor:
    """K same-shape matrices, K inputs [K, IN] -> [K, OUT], one launch."""
    _require_cuda(xstack)
    lib = _lib.load()
    k = len(dqts)
    arr = (QTensorStruct * k)(*[d.struct for d in dqts])
    y = torch.empty((k, dqts[0].rows), dtype=torch.float32, device=xstack.device)
    _lib.check(lib.rwkvq_gemv_fused(arr, k, xstack.data_ptr(), _lib.DTYPE_CODE[xstack.dtype],
                                    y.data_ptr(), _lib.stream_ptr()), "rwkvq_gemv_fused")
    return y


def seq_ln_shift_mix(x: torch.Tensor, ln_w, ln_b, shift_in: Optional[torch.Tensor], mix: torch.Tensor):
    """x [B, T, D] fp32 -> (out [n_mix, B, T, D], new shift state [B, 1, D]); mix [n_mix, D] or [D]."""
    _require_cuda(x, shift_in, mix)
    B, T, D = x.shape
    x = x.float().contiguous()
    mix2 = mix.reshape(-1, D).contiguous()
    out = torch.empty((mix2.shape[0], B, T, D), dtype=torch.float32, device=x.device)
    new_shift = torch.empty((B, 1, D), dtype=torch.float32, device=x.device)
    sin = None if shift_in is None else shift_in.float().contiguous()
    _lib.check(_lib.load().rwkvq_seq_ln_shift_mix(x.data_ptr(), ln_w.data_ptr(), ln_b.data_ptr(), _lib.ptr(sin),
                                                  mix2.data_ptr(), mix2.shape[0], out.data_ptr(), new_shift.data_ptr(),
                                                  B, T, D, _lib.stream_ptr()), "rwkvq_seq_ln_shift_mix")
    return out, new_shift


def seq_embed_ln0(emb: "DeviceQT", idx: torch.Tensor, ln_w: torch.Tensor, ln_b: torch.Tensor) -> torch.Tensor:
    """idx [...] int64 -> LayerNorm0(rows of the packed embedding table) [..., D] fp32, one kernel."""
    _require_cuda(idx, ln_w)
    flat = idx.reshape(-1).contiguous().long()
    out = torch.empty((flat.numel(), emb.cols), dtype=torch.float32, device=idx.device)
    _lib.check(_lib.load().rwkvq_seq_embed_ln0(C.byref(emb.struct), flat.data_ptr(), ln_w.data_ptr(), ln_b.data_ptr(),
                                               out.data_ptr(), flat.numel(), emb.cols, _lib.stream_ptr()), "rwkvq_seq_embed_ln0")
    return out.reshape(*idx.shape, emb.cols)


def seq_layer_norm(x: torch.Tensor, ln_w: torch.Tensor, ln_b: torch.Tensor) -> torch.Tensor:
    """LayerNorm over the last axis (eps 1e-5) of fp32 rows, one kernel."""
    _require_cuda(x, ln_w)
    x2 = x.float().contiguous()
    out = torch.empty_like(x2)
    D = x2.shape[-1]
    _lib.check(_lib.load().rwkvq_seq_layer_norm(x2.data_ptr(), ln_w.data_ptr(), ln_b.data_ptr(), out.data_ptr(),
                                                x2.numel() // D, D, _lib.stream_ptr()), "rwkvq_seq_layer_norm")
    return out


def split_fp16(x: torch.Tensor) -> torch.Tensor:
    """x fp32 [N, K] -> fp16 [N, 2K] = [hi | lo], hi + lo = x to ~2^-22 relative."""
    _require_cuda(x)
    x = x.float().contiguous()
    out = torch.empty((x.shape[0], 2 * x.shape[1]), dtype=torch.float16, device=x.device)
    _lib.check(_lib.load().rwkvq_split_fp16(x.data_ptr(), out.data_ptr(), x.shape[0], x.shape[1], _lib.stream_ptr()),
               "rwkvq_split_fp16")
    return out


def seq_tmix_pre(k, v, yw, ya, yv, v_first, w0, a0, v0, k_k, k_a, n_head: int):
    """[N, D] fp32 inputs -> (w, k2, v2, -kk, kk*a), each [N, D]; yv / v_first None on layer 0."""
    _require_cuda(k, v, yw, ya)
    k, v, yw, ya = (t.contiguous() for t in (k, v, yw, ya))
    if yv is not None:
        yv, v_first = yv.contiguous(), v_first.contiguous()
    outs = [torch.empty_like(k) for _ in range(5)]
    _lib.check(_lib.load().rwkvq_seq_tmix_pre(k.data_ptr(), v.data_ptr(), yw.data_ptr(), ya.data_ptr(), _lib.ptr(yv),
                                              _lib.ptr(v_first), w0.data_ptr(), a0.data_ptr(),
                                              _lib.ptr(v0) if yv is not None else None, k_k.data_ptr(), k_a.data_ptr(),
                                              *[o.data_ptr() for o in outs], k.shape[0], n_head, _lib.stream_ptr()),
               "rwkvq_seq_tmix_pre")
    return outs


def as_rows(x: torch.Tensor, n_in: int):
    """[..., IN] -> contiguous [N, IN] of a supported dtype plus the leading shape."""
    if x.shape[-1] != n_in:
        raise AssertionError(f"last dim {x.shape[-1]} != in_features {n_in}")
    lead = x.shape[:-1]
    x2 = x.reshape(-1, n_in)
    if x2.dtype not in _lib.DTYPE_CODE:
        x2 = x2.float()
    if x2.stride(-1) != 1 or (x2.stride(0) * x2.element_size()) % 16 or x2.data_ptr() % 16:
        x2 = x2.contiguous()
    return x2, lead
