"""Device-side quantizers for the `sb6` and `sym` layouts.

The counterpart of the reference's host-side packer for its block formats
(`formats/writer.py:236-269` `_make_qt_gw_sb6` over `calibration/groupwise.py:207-300`): the
scale search and code selection run in one CUDA kernel (`rwkvq_quantize_sb6`, a warp per
super-block of 256 weights), the bit packing into the file buffers with the package's packers.
The result is a `QuantizedTensor` a `.rwkvq` file can hold and the kernels can read.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _lib
from .formats import QuantizedTensor
from .synth import pack_6bit, pack_bitplane, pack_nibbles_blocklocal

MODES = {"asym_sb6": False, "asym_sb6_search": True, "asym_sb6_aw": True}
SYM_MODES = ("sym", "sym_aw", "sym_plain")


def sym_factors() -> torch.Tensor:
    """The scale factors the reference's symmetric search visits: the float32 nodes of
    torch.linspace(0.7, 1.15, 19) (calibration/groupwise.py:305)."""
    return torch.linspace(0.7, 1.15, 19)


def quantize_sb6_parts(w: torch.Tensor, bits: int, search: bool = True, ex2: Optional[torch.Tensor] = None):
    """(q u8 [OUT, IN], qs u8 [OUT, IN/32], qm i8 [OUT, IN/32], d f16 [OUT, IN/256], dm f16) on the device."""
    if not w.is_cuda or w.dim() != 2:
        raise ValueError("quantize_sb6: a 2-D CUDA tensor is required")
    o, n = w.shape
    if n % 256:
        raise ValueError(f"quantize_sb6: IN={n} is not a multiple of 256")
    w32 = w.float().contiguous()
    e = None
    if ex2 is not None:
        e = ex2.to(device=w.device, dtype=torch.float32).contiguous()
        if e.numel() != n:
            raise ValueError("quantize_sb6: ex2 needs one value per input channel")
    dev = w.device
    q = torch.empty((o, n), dtype=torch.uint8, device=dev)
    qs = torch.empty((o, n // 32), dtype=torch.uint8, device=dev)
    qm = torch.empty((o, n // 32), dtype=torch.int8, device=dev)
    d = torch.empty((o, n // 256), dtype=torch.float16, device=dev)
    dm = torch.empty((o, n // 256), dtype=torch.float16, device=dev)
    lib = _lib.load(check_device=True)
    with torch.cuda.device(dev):
        _lib.check(lib.rwkvq_quantize_sb6(w32.data_ptr(), n, o, n, bits, 1 if search else 0,
                                          e.data_ptr() if e is not None else None, q.data_ptr(), qs.data_ptr(),
                                          qm.data_ptr(), d.data_ptr(), dm.data_ptr(), _lib.stream_ptr()), "rwkvq_quantize_sb6")
    return q, qs, qm, d, dm


def quantize_sb6(key: str, group: str, w: torch.Tensor, bits: int, mode: str = "asym_sb6_search",
                 ex2: Optional[torch.Tensor] = None) -> QuantizedTensor:
    """`w` [OUT, IN] -> a packed sb6 `QuantizedTensor` (buffers stay on w's device).  mode: one of
    asym_sb6 (min / max scales), asym_sb6_search (scale search + least-squares refit), asym_sb6_aw
    (the search weighted by `ex2`, E[x^2] per input channel)."""
    if mode not in MODES:
        raise ValueError(f"quantize_sb6: mode {mode!r}")
    if (mode == "asym_sb6_aw") != (ex2 is not None):
        raise ValueError("quantize_sb6: ex2 goes with mode asym_sb6_aw, and only with it")
    q, qs, qm, d, dm = quantize_sb6_parts(w, bits, MODES[mode], ex2)
    o, n = w.shape
    qsqm = torch.cat([pack_6bit(qs.reshape(o, -1, 8)), pack_6bit((qm.to(torch.int16) + 31).to(torch.uint8).reshape(o, -1, 8))], dim=-1)
    return QuantizedTensor(
        key=key, group=group, bits=bits, shape=(o, n), gw_mode="sb6", gw_gs=32, gw_sb=8,
        codes_packed=pack_nibbles_blocklocal(q & 0xF, 32),
        gw_qh=pack_bitplane((q >> 4) & 1) if bits >= 5 else None,
        gw_qh2=pack_bitplane((q >> 5) & 1) if bits >= 6 else None,
        gw_qsqm=qsqm.contiguous(), gw_d=d, gw_dm=dm)


def quantize_sym_parts(w: torch.Tensor, bits: int, search: bool = True, ex2: Optional[torch.Tensor] = None):
    """(q i8 [OUT, IN], qs i8 [OUT, IN/16], d f16 [OUT, IN/256]) on the device."""
    if not w.is_cuda or w.dim() != 2:
        raise ValueError("quantize_sym: a 2-D CUDA tensor is required")
    o, n = w.shape
    if n % 256:
        raise ValueError(f"quantize_sym: IN={n} is not a multiple of 256")
    w32 = w.float().contiguous()
    dev = w.device
    e = None
    if ex2 is not None:
        e = ex2.to(device=dev, dtype=torch.float32).contiguous()
        if e.numel() != n:
            raise ValueError("quantize_sym: ex2 needs one value per input channel")
    f = (sym_factors() if search else torch.ones(1)).to(dev)
    q = torch.empty((o, n), dtype=torch.int8, device=dev)
    qs = torch.empty((o, n // 16), dtype=torch.int8, device=dev)
    d = torch.empty((o, n // 256), dtype=torch.float16, device=dev)
    lib = _lib.load(check_device=True)
    with torch.cuda.device(dev):
        _lib.check(lib.rwkvq_quantize_sym(w32.data_ptr(), n, o, n, bits, f.data_ptr(), f.numel(),
                                          e.data_ptr() if e is not None else None, q.data_ptr(), qs.data_ptr(), d.data_ptr(),
                                          _lib.stream_ptr()), "rwkvq_quantize_sym")
    return q, qs, d


def quantize_sym(key: str, group: str, w: torch.Tensor, bits: int, mode: str = "sym",
                 ex2: Optional[torch.Tensor] = None) -> QuantizedTensor:
    """`w` [OUT, IN] -> a packed sym `QuantizedTensor` (bits 6 or 8).  mode: sym (scale search), sym_aw (the
    search weighted by `ex2`), sym_plain (no search); the counterpart of `formats/writer.py::_make_qt_gw_sym`."""
    if mode not in SYM_MODES:
        raise ValueError(f"quantize_sym: mode {mode!r}")
    if (mode == "sym_aw") != (ex2 is not None):
        raise ValueError("quantize_sym: ex2 goes with mode sym_aw, and only with it")
    q, qs, d = quantize_sym_parts(w, bits, mode != "sym_plain", ex2)
    o, n = w.shape
    qt = QuantizedTensor(key=key, group=group, bits=bits, shape=(o, n), gw_mode="sym", gw_gs=16, gw_sb=16, gw_qs=qs, gw_d=d)
    if bits == 8:
        qt.codes = q
    else:
        u = (q.to(torch.int16) + 32).to(torch.uint8)
        qt.codes_packed = pack_nibbles_blocklocal(u & 0xF, 16)
        qt.gw_qh = pack_bitplane((u >> 4) & 1)
        qt.gw_qh2 = pack_bitplane((u >> 5) & 1)
    return qt
