"""Time-mix tail in one launch: group_norm + bonus + gate.

Same contract as the reference's ``fused_tail.wkv_tail`` / ``can_fuse_tail``
(backends/metal/fused_tail.py:88-110): all inputs fp32 with N*H*S elements, r_k /
ln_w / ln_b of H*S elements, returns ``[N, D]``.
"""
from __future__ import annotations

import torch

from ... import _lib


def can_fuse_tail(H, S):
    return S == 64


def wkv_tail(wkv, r, k, v, r_k, ln_w, ln_b, g, H, S, eps=64e-5):
    D = H * S
    n = wkv.numel() // D
    f = lambda t, shape: t.contiguous().float().reshape(shape)
    ins = [f(wkv, (n, D)), f(r, (n, D)), f(k, (n, D)), f(v, (n, D)), f(r_k, (D,)), f(ln_w, (D,)),
           f(ln_b, (D,)), f(g, (n, D))]
    if not all(t.is_cuda for t in ins):
        raise RuntimeError("wkv_tail: CUDA tensors are required")
    out = torch.empty((n, D), dtype=torch.float32, device=wkv.device)
    lib = _lib.load()
    _lib.check(lib.rwkvq_wkv_tail(*[t.data_ptr() for t in ins], out.data_ptr(), n, H, S, float(eps),
                                  _lib.stream_ptr()), "rwkvq_wkv_tail")
    return out
