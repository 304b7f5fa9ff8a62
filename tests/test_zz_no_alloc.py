"""rwkvq_gemv_static: the single-vector GEMV whose K-split scratch lives inside the
library (it allocates nothing) against the allocating entry point rwkvq_gemv.

Collected last (file name) so that it also runs after every other GPU test has used
the library; it must pass alone as well.

  * two calls in a row: the second reuses the scratch the first one left behind and
    must give the same bits as the first;
  * both against rwkvq_gemv on the same tensor and vector: the K split only changes
    the order of the fp32 partial sums, so |dy| <= 2e-5 * max|y| (written tolerance);
  * sizes beyond the built-in scratch and layouts without the relayouted records are
    refused with their documented error codes, before anything is launched.
"""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
TOL = 2e-5

E_DTYPE, E_LIMIT = -3, -8


def _linear(layout, bits, rows, cols, seed, relayout=True):
    from rwkv_quant_b200 import synth
    from rwkv_quant_b200.backends.cuda import ops
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(rows, cols, generator=g) * 0.02
    fn = {"sb6": synth.quant_sb6, "sym": synth.quant_sym, "rtn": synth.quant_rtn}[layout]
    return ops.DeviceQT(fn("w", "g", w, bits), relayout=relayout)


def _static(lib, dq, x, epilogue=0, resid=None):
    from rwkv_quant_b200 import _lib
    y = torch.full((dq.rows,), float("nan"), dtype=torch.float32, device=x.device)
    rc = lib.rwkvq_gemv_static(C.byref(dq.struct), x.data_ptr(), _lib.DTYPE_CODE[x.dtype], y.data_ptr(),
                               epilogue, _lib.ptr(resid), _lib.stream_ptr())
    return rc, y


@pytest.mark.parametrize("layout,bits,rows,cols", [
    ("sb6", 4, 2048, 2048),     # K split 2 ways
    ("sb6", 5, 512, 8192),      # K split 4 ways (ffn.value-like: few rows, long rows)
    ("sb6", 6, 272, 4096),      # rows not a multiple of the 16-row tile
    ("sym", 6, 1024, 2048),
    ("sym", 8, 4096, 1024),     # largest row count served; too short for a K split
    ("rtn", 8, 640, 4096),      # per-row int8
    ("sb6", 6, 1024, 17 * 256),   # 17 iterations: no even split, every column must still be multiplied
    ("sym", 8, 1024, 34 * 128),   # 34 iterations: 2 slices, not 4
    ("rtn", 8, 1024, 34 * 128),
    ("sb6", 4, 512, 33 * 256),    # odd count at the 4-way size
])
def test_static_matches_allocating_entry_point_twice(cuda_lib, layout, bits, rows, cols):
    from rwkv_quant_b200.backends.cuda import ops
    dq = _linear(layout, bits, rows, cols, seed=rows + cols + bits)
    g = torch.Generator().manual_seed(7)
    x = torch.randn(cols, generator=g).cuda()
    ref = ops.gemv(dq.bufs, dq.meta, x.view(1, -1), 0, None)[0]
    rc1, y1 = _static(cuda_lib, dq, x)
    rc2, y2 = _static(cuda_lib, dq, x)
    torch.cuda.synchronize()
    assert rc1 == 0 and rc2 == 0, cuda_lib.rwkvq_last_error_detail()
    assert torch.isfinite(y1).all() and torch.isfinite(y2).all()
    assert torch.equal(y1, y2), "second call (scratch reused) differs from the first"
    scale = ref.abs().max().item()
    assert (y1 - ref).abs().max().item() <= TOL * scale
    assert (y2 - ref).abs().max().item() <= TOL * scale


def test_static_epilogues_and_half_input(cuda_lib):
    from rwkv_quant_b200.backends.cuda import ops
    dq = _linear("sb6", 5, 768, 4096, seed=3)
    g = torch.Generator().manual_seed(11)
    x = torch.randn(4096, generator=g).cuda().half()
    resid = torch.randn(768, generator=g).cuda()
    for epi, r in ((1, None), (2, resid)):
        ref = ops.gemv(dq.bufs, dq.meta, x.view(1, -1), epi, None if r is None else r.view(1, -1))[0]
        for _ in range(2):
            rc, y = _static(cuda_lib, dq, x, epi, r)
            assert rc == 0, cuda_lib.rwkvq_last_error_detail()
            assert (y - ref).abs().max().item() <= TOL * max(ref.abs().max().item(), 1e-6)


def test_static_refuses_what_does_not_fit(cuda_lib):
    x = torch.zeros(32768, device="cuda")
    too_many_rows = _linear("sym", 8, 4096 + 16, 256, seed=1)
    rc, _ = _static(cuda_lib, too_many_rows, x[:256])
    assert rc == E_LIMIT and b"4096" in cuda_lib.rwkvq_last_error_detail()
    too_long = _linear("sym", 8, 16, 32768, seed=2)
    rc, _ = _static(cuda_lib, too_long, x)
    assert rc == E_LIMIT
    no_records = _linear("sb6", 5, 256, 512, seed=3, relayout=False)
    rc, _ = _static(cuda_lib, no_records, x[:512])
    assert rc == E_DTYPE
    rtn4 = _linear("rtn", 4, 256, 512, seed=4)          # packed nibbles: no tensor-core layout
    rc, _ = _static(cuda_lib, rtn4, x[:512])
    assert rc == E_DTYPE
    torch.cuda.synchronize()
