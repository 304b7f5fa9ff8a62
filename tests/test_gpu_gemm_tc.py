"""Dequant-fused tcgen05 GEMM (rwkvq_gemm) against the oracle.

Operands are fp16 (weights fp16(q*s+m), tokens scaled per row by a power of two) with
fp32 accumulation in tensor memory, so the bar is the reference's own GEMM-path gate:
relmax <= 2e-3 against x @ dequant(W).T (tests/test_gemm_prefill.py:45); measured
values are printed.  The kernel status word must stay 0 (no bounded wait expired).
"""
import numpy as np
import pytest
import torch

from helpers import relmax
from test_gpu_dequant_gemv import LAYOUTS, _oracle_w, _synth_linear

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("layout,bits", [lb for lb in LAYOUTS if lb[0] in ("sb6", "sym")])
@pytest.mark.parametrize("rows,cols,M", [(256, 256, 5), (128, 512, 16), (100, 768, 40), (384, 2048, 128),
                                         (2048, 2048, 300), (256, 8192, 64)])
def test_gemm_tc_matches_oracle(cuda_lib, layout, bits, rows, cols, M):
    from rwkv_quant_b200.backends.cuda import ops
    qt = _synth_linear(layout, bits, rows, cols, seed=rows + cols + M)
    dq = ops.DeviceQT(qt)
    w = _oracle_w(qt).astype(np.float64)
    rs = np.random.default_rng(M * 7 + cols)
    x = rs.standard_normal((M, cols)).astype(np.float32)
    x[0] *= 1e3                      # rows of very different magnitude: the per-row scale must cope
    if M > 2:
        x[2] *= 1e-4
    xt = torch.from_numpy(x).cuda()
    y = ops.gemm(dq, xt, 0, None, check=True).cpu().numpy()
    ref = x.astype(np.float64) @ w.T
    per_row = np.abs(y - ref).max(axis=1) / np.abs(ref).max(axis=1)
    assert per_row.max() <= 2e-3, per_row.max()
    print(f"{layout}{bits} [{rows},{cols}] M={M}: worst row relmax {per_row.max():.2e}")


def test_gemm_tc_epilogues_and_determinism(cuda_lib):
    from rwkv_quant_b200.backends.cuda import ops
    qt = _synth_linear("sb6", 5, 512, 1024, seed=3)
    dq = ops.DeviceQT(qt)
    x = torch.randn(70, 1024, device="cuda")
    y = ops.gemm(dq, x, 0, None, check=True)
    assert torch.equal(y, ops.gemm(dq, x, 0, None, check=True)), "two runs differ"
    assert torch.equal(ops.gemm(dq, x, 1, None, check=True), torch.relu(y) ** 2)
    resid = torch.randn(70, 512, device="cuda")
    assert torch.equal(ops.gemm(dq, x, 2, resid, check=True), y + resid)
    # the first 16 tokens alone give the same rows (token tiles are independent)
    y16 = ops.gemm(dq, x[:16].contiguous(), 0, None, check=True)
    assert relmax(y16.cpu().numpy(), y[:16].cpu().numpy()) <= 1e-6
    # against the exact single-vector kernel
    y1 = ops.gemv(dq.bufs, dq.meta, x[:4].contiguous(), 0, None)
    assert relmax(y[:4].cpu().numpy(), y1.cpu().numpy()) <= 2e-3


@pytest.fixture
def two_accumulators(cuda_lib):
    """256-row tiles (two accumulators per activation slab) wherever the shape allows: the
    launcher takes them by itself only once they fill the SMs (row tiles x token tiles >= 148)."""
    import ctypes as C
    f = cuda_lib.rwkvq_profiling_gemm_acc_mode          # rwkvq_profiling.h: not part of the C ABI
    f.restype, f.argtypes = None, [C.c_int]
    f(2)
    yield f
    f(0)


@pytest.mark.parametrize("layout,bits", [("sb6", 4), ("sb6", 5), ("sb6", 6), ("sym", 6), ("sym", 8)])
@pytest.mark.parametrize("rows,cols,M", [(256, 256, 129), (512, 1024, 300), (2048, 2048, 520), (256, 8192, 256)])
def test_gemm_tc_two_accumulator_tiles(cuda_lib, two_accumulators, layout, bits, rows, cols, M):
    """Same bar as the one-accumulator form, bit-equal to it (the same MMAs in the same order per
    output element), on shapes with one CTA, a K split (few tiles, long K) and a ragged token tile;
    the epilogues go through both accumulators."""
    from rwkv_quant_b200.backends.cuda import ops
    qt = _synth_linear(layout, bits, rows, cols, seed=rows + cols + M + 1)
    dq = ops.DeviceQT(qt)
    w = _oracle_w(qt).astype(np.float64)
    x = np.random.default_rng(M + cols).standard_normal((M, cols)).astype(np.float32)
    x[1] *= 1e3
    xt = torch.from_numpy(x).cuda()
    y2 = ops.gemm(dq, xt, 0, None, check=True)
    ref = x.astype(np.float64) @ w.T
    per_row = np.abs(y2.cpu().numpy() - ref).max(axis=1) / np.abs(ref).max(axis=1)
    assert per_row.max() <= 2e-3, per_row.max()
    resid = torch.randn(M, rows, device="cuda")
    r2 = ops.gemm(dq, xt, 2, resid, check=True)
    q2 = ops.gemm(dq, xt, 1, None, check=True)
    two_accumulators(1)                                  # the same call on 128-row tiles
    y1 = ops.gemm(dq, xt, 0, None, check=True)
    two_accumulators(2)
    assert torch.equal(r2, y2 + resid) and torch.equal(q2, torch.relu(y2) ** 2)
    assert relmax(y2.cpu().numpy(), y1.cpu().numpy()) <= 1e-6
    print(f"{layout}{bits} [{rows},{cols}] M={M} (256-row tiles): worst row relmax {per_row.max():.2e}")
