"""WKV-7 recurrence with carried state (head size 64).

Same call contract as ``rwkv_metal.kernel.wkv7.wkv7_infer`` as the reference uses it
(backends/metal/quant_model.py:118-125): ``wkv7_infer(r, w, k, v, a, b, state) ->
(out, new_state)`` with r..b ``[B, T, H, 64]`` fp32 (``w`` is the decay itself),
state ``[B, H, 64, 64]`` fp32, any T >= 1.  The input state is not modified.
"""
from __future__ import annotations

import torch

from ... import _lib

CHUNK = 16      # kept for callers that import it; no padding or chunking is needed here


def wkv7_infer(r, w, k, v, a, b, state):
    B, T, H, S = r.shape
    ts = [t.contiguous().float() for t in (r, w, k, v, a, b)]
    for t in ts:
        if not t.is_cuda or t.shape != (B, T, H, S):
            raise RuntimeError("wkv7_infer: CUDA tensors of one shape [B, T, H, 64] are required")
    h_in = state.contiguous().float()
    out = torch.empty((B, T, H, S), dtype=torch.float32, device=r.device)
    h_out = torch.empty_like(h_in)
    lib = _lib.load()
    _lib.check(lib.rwkvq_wkv7(*[t.data_ptr() for t in ts], h_in.data_ptr(), out.data_ptr(),
                              h_out.data_ptr(), B, T, H, S, _lib.stream_ptr()), "rwkvq_wkv7")
    return out, h_out


def wkv7_train(r, w, k, v, a, b):
    """Zero initial state, no state out (quant_model.py:394)."""
    B, T, H, S = r.shape
    return wkv7_infer(r, w, k, v, a, b, torch.zeros((B, H, S, S), device=r.device))[0]
