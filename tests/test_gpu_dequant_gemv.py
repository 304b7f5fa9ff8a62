"""CUDA kernels against the oracle, through the C ABI (via the rwkvq:: ops).

  dequant  fp32 output equal BIT FOR BIT to the reference codec (digests of
           tests/golden/codec_cases.npz, made by the reference's packers);
  GEMV     relmax(|y - x @ dequant(W).T|) / max|ref| <= 1e-3 (the reference's own
           kernel gates allow 3e-3: tests/test_gw_kernel.py:29), N in {1,2,3,8};
  claims restated from the reference's equality gates: batch invariance
  (tests/test_gw_nb_parity.py), fused == separate (tests/test_sym_fuse_parity.py),
  poison-filled outputs to catch rows the grid does not cover.
"""
import os
import zlib

import numpy as np
import pytest
import torch

from helpers import case_to_qt, digest_f32, oracle_dequant_case, relmax
from oracle import codec_np as oc

pytestmark = pytest.mark.gpu
TOL = 1e-3


def _x(n, k, seed, dtype=torch.float32):
    x = np.random.default_rng(seed).standard_normal((n, k)).astype(np.float32)
    return torch.from_numpy(x).to("cuda", dtype)


def test_dequant_bit_exact_all_golden_cases(cuda_lib, codec_cases):
    from rwkv_quant_b200.backends.cuda import ops
    n_outlier_cases = 0
    for name, (meta, bufs, _) in codec_cases.items():
        n_outlier_cases += "outlier_indices" in bufs        # sparse overrides: applied by DeviceQT.dequant
        dq = ops.DeviceQT(case_to_qt(name, meta, bufs))
        w = dq.dequant(torch.float32, False).cpu().numpy()
        assert digest_f32(w) == meta["digest"], f"{name}: device dequant differs from the codec"
        ref = oracle_dequant_case(meta, bufs)
        h = dq.dequant(torch.float16, False).cpu().numpy()
        np.testing.assert_array_equal(h, ref.astype(np.float16), err_msg=name)
        b = dq.dequant(torch.bfloat16, True).float().cpu().numpy()
        np.testing.assert_array_equal(b, oc.f32_to_bf16_rne(ref), err_msg=name)
    assert n_outlier_cases >= 1, "the golden set lost its outlier case"


@pytest.mark.parametrize("xdtype", [torch.float32, torch.float16, torch.bfloat16])
def test_gemv_golden_cases(cuda_lib, codec_cases, xdtype):
    from rwkv_quant_b200.backends.cuda import ops
    for name, (meta, bufs, _) in codec_cases.items():
        dq = ops.DeviceQT(case_to_qt(name, meta, bufs))
        w = oracle_dequant_case(meta, bufs).astype(np.float64)
        for n in (1, 2, 3, 8):
            x = _x(n, dq.cols, zlib.crc32(f"{name}-{n}".encode()), xdtype)
            y = dq.gemv(x, 0, None).cpu().numpy()
            ref = x.float().cpu().numpy().astype(np.float64) @ w.T
            assert relmax(y, ref) <= TOL, (name, n, relmax(y, ref))


def _synth_linear(layout, bits, rows, cols, seed=0):
    from rwkv_quant_b200 import synth
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(rows, cols, generator=g) * 0.02
    fn = {"sb6": synth.quant_sb6, "sym": synth.quant_sym, "rtn": synth.quant_rtn}[layout]
    return fn("w", "g", w, bits)


def _oracle_w(qt):
    n = lambda t: None if t is None else t.numpy()
    if qt.gw_mode == "sb6":
        return oc.dequant_sb6(n(qt.codes_packed), n(qt.gw_qsqm), n(qt.gw_d), n(qt.gw_dm), shape=qt.shape,
                              qh=n(qt.gw_qh), qh2=n(qt.gw_qh2))
    if qt.gw_mode == "sym":
        return oc.dequant_sym(n(qt.gw_qs), n(qt.gw_d), shape=qt.shape, codes=n(qt.codes),
                              codes_packed=n(qt.codes_packed), qh=n(qt.gw_qh), qh2=n(qt.gw_qh2))
    return oc.dequant_rtn(n(qt.scale), shape=qt.shape, codes=n(qt.codes), codes_packed=n(qt.codes_packed))


LAYOUTS = [("sb6", 4), ("sb6", 5), ("sb6", 6), ("sym", 6), ("sym", 8), ("rtn", 8), ("rtn", 4)]


@pytest.mark.parametrize("layout,bits", LAYOUTS)
@pytest.mark.parametrize("rows,cols", [(16, 256), (48, 512), (2048, 2048), (100, 2560), (2048, 8192), (1024, 4352)])
def test_gemv_shapes_and_uncovered_rows(cuda_lib, layout, bits, rows, cols):
    """Exhaustive small shapes plus model shapes; rows not a multiple of the CTA
    tile; the output is NaN-filled first so an unwritten row cannot pass."""
    from rwkv_quant_b200 import _lib
    from rwkv_quant_b200.backends.cuda import ops
    import ctypes as C
    qt = _synth_linear(layout, bits, rows, cols, seed=rows + cols)
    dq = ops.DeviceQT(qt)
    w = _oracle_w(qt)
    wd = ops.dequant(dq.bufs, dq.meta, torch.float32, False).cpu().numpy()
    assert np.array_equal(wd.view(np.uint32), w.view(np.uint32)), "device dequant != oracle, bit level"
    x = _x(1, cols, rows * 31 + cols)
    y = torch.full((1, rows), float("nan"), device="cuda")
    d = ops._descr(dq.bufs, dq.meta)
    _lib.check(cuda_lib.rwkvq_gemv(C.byref(d), x.data_ptr(), 0, 1, cols, y.data_ptr(), rows, 0, None,
                                   _lib.stream_ptr()), "rwkvq_gemv")
    y = y.cpu().numpy()
    assert np.isfinite(y).all(), "a row was not written"
    ref = x.cpu().numpy().astype(np.float64) @ w.astype(np.float64).T
    assert relmax(y, ref) <= TOL, relmax(y, ref)


@pytest.mark.parametrize("layout,bits", LAYOUTS[:6])
def test_batch_invariance_and_epilogues(cuda_lib, layout, bits):
    """Column n of an N-column call equals the single-vector call bit for bit;
    relu^2 and residual-add epilogues equal their unfused forms."""
    from rwkv_quant_b200.backends.cuda import ops
    qt = _synth_linear(layout, bits, 512, 1024, seed=bits)
    dq = ops.DeviceQT(qt)
    x = _x(7, 1024, 99)
    y = ops.gemv(dq.bufs, dq.meta, x, 0, None)
    for n in range(7):
        y1 = ops.gemv(dq.bufs, dq.meta, x[n:n + 1].contiguous(), 0, None)
        assert torch.equal(y1[0], y[n]), f"column {n} depends on the batch it was computed in"
    assert torch.equal(ops.gemv(dq.bufs, dq.meta, x, 1, None), torch.relu(y) ** 2)
    resid = _x(7, 512, 5)
    assert torch.equal(ops.gemv(dq.bufs, dq.meta, x, 2, resid), resid + y)


@pytest.mark.parametrize("layout,bits", [("sb6", 5), ("sym", 8), ("sb6", 4)])
def test_fused_projections_equal_separate(cuda_lib, layout, bits):
    from rwkv_quant_b200.backends import cuda as be
    cls, fused = ((be.GwQuantLinear, be.GwQuantLinearFused) if layout == "sb6"
                  else (be.SymQuantLinear, be.SymQuantLinearFused))
    lins = [cls(_synth_linear(layout, bits, 768, 768, seed=s)) for s in (1, 2, 3)]
    xs = _x(3, 768, 17)
    out = fused(lins)(xs)
    assert out.shape == (3, 768)
    for k in range(3):
        assert torch.equal(out[k], lins[k](xs[k])), f"matrix {k}"


def test_linear_classes_contract(cuda_lib):
    """Any leading shape, fp32 out, attributes, from_buffers, dispatch by layout."""
    from rwkv_quant_b200.backends import cuda as be
    qt = _synth_linear("sym", 6, 256, 512, seed=8)
    lin = be.linear_for(qt)
    assert isinstance(lin, be.SymQuantLinear) and (lin.in_features, lin.out_features) == (512, 256)
    x = _x(6, 512, 3).reshape(2, 3, 512)
    y = lin(x)
    assert y.shape == (2, 3, 256) and y.dtype == torch.float32
    n = lambda t: None if t is None else t.numpy()
    lin2 = be.SymQuantLinear.from_buffers(shape=qt.shape, bits=6, qs=n(qt.gw_qs), d=n(qt.gw_d),
                                          codes_packed=n(qt.codes_packed), qh=n(qt.gw_qh), qh2=n(qt.gw_qh2))
    assert torch.equal(lin2(x), y)
    w = lin._dequant_w(torch.float32).cpu().numpy()
    assert np.array_equal(w.view(np.uint32), _oracle_w(qt).view(np.uint32))
    assert not np.array_equal(lin._dequant_w(torch.float16).float().cpu().numpy(), w)   # control
    assert isinstance(be.linear_for(_synth_linear("sb6", 4, 64, 256)), be.GwQuantLinear)
    assert isinstance(be.linear_for(_synth_linear("rtn", 8, 64, 256)), be.QuantLinearV2)
    with pytest.raises(AssertionError):
        lin(_x(1, 256, 0))


def test_gemv_t_lora_orientation(cuda_lib, codec_cases):
    """Tensors stored [in, out]: y = act(x @ W) with the reference's load-time
    rounding fp16(bf16(w)) of LoRA weights (quant_model.py:128-154)."""
    from rwkv_quant_b200.backends.cuda import ops
    for name in ("asym/ragged", "asym/wide", "rtn/8", "rtn/8wide", "rtn/4odd"):
        meta, bufs, _ = codec_cases[name]
        dq = ops.DeviceQT(case_to_qt(name, meta, bufs))
        w = oracle_dequant_case(meta, bufs)
        wr = oc.f32_to_bf16_rne(w).astype(np.float16).astype(np.float64)
        for n in (1, 5, 11):
            x = _x(n, dq.rows, zlib.crc32(name.encode()) + n)
            xh = x.cpu().numpy().astype(np.float64)
            y = ops.gemv_t(dq.bufs, dq.meta, x, 0, True).cpu().numpy()
            assert relmax(y, xh @ wr) <= 2e-5, (name, n)
            y = ops.gemv_t(dq.bufs, dq.meta, x, 0, False).cpu().numpy()
            assert relmax(y, xh @ w.astype(np.float64)) <= 2e-5, (name, n)
            y = ops.gemv_t(dq.bufs, dq.meta, x, 1, True).cpu().numpy()
            assert relmax(y, np.tanh(xh @ wr)) <= 2e-5, (name, n)
            y = ops.gemv_t(dq.bufs, dq.meta, x, 2, True).cpu().numpy()
            assert relmax(y, 1 / (1 + np.exp(-(xh @ wr)))) <= 2e-5, (name, n)


def test_config1_single_gemv(cuda_lib, config1_case):
    """W [8192, 2048] ~N(0, 0.02) int4 sb6 packed by the reference's asym_sb6_search packer
    (9 437 184 packed bytes), x fp16 [1, 2048]: dequantised W equal to the reference codec bit
    for bit (its digest), y relmax <= 1e-3 against the reference's numpy dequant + matvec."""
    from rwkv_quant_b200.backends import cuda as be
    meta, bufs, x, y_ref = config1_case
    qt = case_to_qt("config1", meta, bufs)
    assert qt.nbytes() == 9437184
    lin = be.GwQuantLinear(qt)
    assert digest_f32(lin._dequant_w().cpu().numpy()) == meta["digest"]
    y = lin(torch.from_numpy(x).cuda()).cpu().numpy()
    assert relmax(y, y_ref) <= TOL, relmax(y, y_ref)
    print(f"config 1: y relmax vs the reference's dequant + matvec {relmax(y, y_ref):.2e}")


@pytest.mark.parametrize("layout,bits", LAYOUTS[:6])
@pytest.mark.parametrize("n", [1, 8])
def test_gemv_wide_dynamic_range_activations(cuda_lib, layout, bits, n):
    """One channel 1000 x larger than the rest: the single-vector kernel turns x into fixed point
    against max|x|, so the small channels keep only ~11 bits; the result must still meet the
    1e-3 bar against the fp64 product (the batched kernels round x to fp16 per row instead)."""
    from rwkv_quant_b200.backends.cuda import ops
    qt = _synth_linear(layout, bits, 1024, 2048, seed=40 + bits)
    dq = ops.DeviceQT(qt)
    w = _oracle_w(qt).astype(np.float64)
    x = _x(n, 2048, 77)
    x[:, 5] *= 1000.0
    ref = x.cpu().numpy().astype(np.float64) @ w.T
    y = dq.gemv(x, 0, None).cpu().numpy()
    assert relmax(y, ref) <= TOL, relmax(y, ref)
    # the same with the outlier column removed from both sides: the error of the small channels
    # measured against THEIR contribution, not against the outlier's
    ref_small = ref - np.outer(x[:, 5].cpu().numpy().astype(np.float64), w[:, 5])
    y_small = y - np.outer(x[:, 5].cpu().numpy().astype(np.float64), w[:, 5])
    print(f"{layout}@{bits} n={n}: relmax {relmax(y, ref):.2e}; small-channel part {relmax(y_small, ref_small):.2e}")
    assert relmax(y_small, ref_small) <= 5e-3


BATCH_SHAPES = [(16, 256), (48, 512), (2048, 2048), (100, 2560), (2048, 8192), (1024, 4352), (8192, 2048), (2560, 10240)]


@pytest.fixture(params=["two-term", "tcgen05-two-term", "mma.sync-fast", "tcgen05-fast"])
def batch_kernel(request, cuda_lib):
    """The four kernels behind rwkvq_gemv_batch: the two-term kernels (both operands as fp16 pairs:
    fp32-grade results) on mma.sync and on tcgen05, and, selected by RWKVQ_BATCH_FAST=1 in production
    and by the library's profiling switches (not part of the C ABI) here, the single-term mma.sync
    kernel and the single-term tcgen05 kernel (fp16 operands, the arithmetic of the prefill GEMM)."""
    import ctypes as C
    f = cuda_lib.rwkvq_profiling_tcb_force
    f.restype, f.argtypes = None, [C.c_int]
    fast = cuda_lib.rwkvq_profiling_batch_fast
    fast.restype, fast.argtypes = None, [C.c_int]
    fast(0 if request.param.endswith("two-term") else 1)
    f(1000 if request.param.startswith("tcgen05") else -1)   # 1000: tcgen05 at every batch size (no valid cluster size: launcher's choice)
    yield request.param
    f(0)
    fast(-1)


BATCH_TOL = {"two-term": 2e-5, "tcgen05-two-term": 2e-5, "mma.sync-fast": TOL, "tcgen05-fast": TOL}


@pytest.mark.parametrize("layout,bits", LAYOUTS[:6])
@pytest.mark.parametrize("rows,cols", BATCH_SHAPES)
def test_gemv_batch_matches_oracle(cuda_lib, batch_kernel, layout, bits, rows, cols):
    """The weights-once small-batch kernel against the fp64 product with the oracle's weights, for
    every batch-size class (1, 2, 4, 8 token tiles; a ragged last tile; more than one 64-token
    group) and every K split the launcher can choose (cluster of 1, 2, 4, 5, 8 CTAs; one or
    several staged chunks); NaN-filled output so that an unwritten element cannot pass."""
    import ctypes as C
    from rwkv_quant_b200 import _lib
    from rwkv_quant_b200.backends.cuda import ops
    qt = _synth_linear(layout, bits, rows, cols, seed=rows + cols + bits)
    dq = ops.DeviceQT(qt)
    assert ops.has_batch_layout(dq)
    if layout == "rtn" and batch_kernel.startswith("tcgen05"):
        pytest.skip("per-row int8 has no tcgen05 form")
    w = _oracle_w(qt).astype(np.float64)
    worst = 0.0
    for n in (3, 8, 13, 32, 64, 70):
        x = _x(n, cols, rows * 31 + cols + n)
        y = torch.full((n, rows), float("nan"), device="cuda")
        ws = torch.empty(cuda_lib.rwkvq_gemv_batch_workspace_bytes(n), dtype=torch.uint8, device="cuda")
        _lib.check(cuda_lib.rwkvq_gemv_batch(C.byref(dq.struct), x.data_ptr(), n, cols, y.data_ptr(), rows, 0, None,
                                             ws.data_ptr(), ws.numel(), _lib.stream_ptr()), "rwkvq_gemv_batch")
        torch.cuda.synchronize()
        assert int(ws[:4].view(torch.int32).item()) == 0, "the kernel reported a pipeline time-out"
        y = y.cpu().numpy()
        assert np.isfinite(y).all(), f"n={n}: an element was not written"
        ref = x.cpu().numpy().astype(np.float64) @ w.T
        worst = max(worst, relmax(y, ref))
        assert relmax(y, ref) <= BATCH_TOL[batch_kernel], (n, relmax(y, ref))
    print(f"gemv_batch ({batch_kernel}) {layout}@{bits} [{rows},{cols}]: worst relmax {worst:.2e}")


def test_gemv_batch_epilogues_scaling_and_refusals(cuda_lib, batch_kernel):
    import ctypes as C
    from rwkv_quant_b200 import _lib
    from rwkv_quant_b200.backends.cuda import ops
    qt = _synth_linear("sb6", 5, 768, 2048, seed=4)
    dq = ops.DeviceQT(qt)
    w = _oracle_w(qt).astype(np.float64)
    x = _x(9, 2048, 12)
    resid = _x(9, 768, 13)
    y0 = ops.gemv_batch(dq, x)
    assert torch.equal(ops.gemv_batch(dq, x, 1, None), torch.relu(y0) ** 2)
    assert torch.equal(ops.gemv_batch(dq, x, 2, resid), resid + y0)
    assert torch.equal(ops.gemv_batch(dq, x), y0), "two launches on the same input differ"
    # rows of very different magnitude in one batch, and a channel 1000 x larger than the rest:
    # every token is scaled on its own, per staged chunk
    xs = x.clone()
    xs[0] *= 1e-6
    xs[1] *= 3e4
    xs[2, 5] *= 1000.0
    xs[3] = 0.0
    ref = xs.cpu().numpy().astype(np.float64) @ w.T
    y = ops.gemv_batch(dq, xs).cpu().numpy()
    for n in range(9):
        assert np.abs(y[n] - ref[n]).max() <= BATCH_TOL[batch_kernel] * max(np.abs(ref[n]).max(), 1e-30), n
    assert (y[3] == 0).all()
    # non-finite input propagates to its own row only
    xs[4, 100] = float("inf")
    y = ops.gemv_batch(dq, xs)
    assert not torch.isfinite(y[4]).any() and torch.isfinite(y[[0, 1, 2, 3, 5, 6, 7, 8]]).all()
    # strided rows
    xp = torch.zeros(9, 2048 + 64, device="cuda")
    xp[:, :2048] = x
    assert torch.equal(ops.gemv_batch(dq, xp[:, :2048]), y0)
    # layouts without the tensor-core form are refused, not served by something else
    rtn4 = ops.DeviceQT(_synth_linear("rtn", 4, 64, 256))
    yb = torch.empty(3, 64, device="cuda")
    ws = torch.empty(512, dtype=torch.uint8, device="cuda")
    assert cuda_lib.rwkvq_gemv_batch(C.byref(rtn4.struct), x.data_ptr(), 3, 256, yb.data_ptr(), 64, 0, None,
                                     ws.data_ptr(), 512, _lib.stream_ptr()) == _lib.E_DTYPE
    assert cuda_lib.rwkvq_gemv_batch(C.byref(dq.struct), x.data_ptr() + 4, 3, 2048, y0.data_ptr(), 768, 0, None,
                                     ws.data_ptr(), 512, _lib.stream_ptr()) == _lib.E_ALIGN
    assert cuda_lib.rwkvq_gemv_batch(C.byref(dq.struct), x.data_ptr(), 3, 2048, y0.data_ptr(), 768, 0, None,
                                     ws.data_ptr(), 4, _lib.stream_ptr()) == _lib.E_LIMIT


def test_linear_classes_route_small_batches_through_the_batch_kernel(cuda_lib):
    """3 <= N < 128 through the operator class: one pass over the weights (the reference reads them
    once per chunk of 4 columns), result within fp32 rounding of the single-vector kernel."""
    from rwkv_quant_b200.backends import cuda as be
    from rwkv_quant_b200.backends.cuda import ops
    for layout, bits in (("sb6", 4), ("sym", 6), ("rtn", 8)):
        qt = _synth_linear(layout, bits, 512, 1024, seed=bits)
        lin = be.linear_for(qt)
        x = _x(40, 1024, 3)
        y = lin(x)
        assert torch.equal(y, ops.gemv_batch(lin.dq, x))
        exact = ops.gemv(lin.dq.bufs, lin.dq.meta, x, 0, None)
        assert (y - exact).abs().max().item() <= 2e-5 * exact.abs().max().item()
        assert torch.equal(lin(x[:2]), exact[:2])          # 1 and 2 rows: the exact kernel


def test_errors_surface_as_exceptions(cuda_lib):
    from rwkv_quant_b200 import _lib
    from rwkv_quant_b200.backends.cuda import ops
    qt = _synth_linear("sb6", 4, 64, 256)
    dq = ops.DeviceQT(qt)
    bad = list(dq.meta)
    bad[3] = 250
    with pytest.raises(_lib.RwkvqError):
        ops.gemv(dq.bufs, bad, _x(1, 256, 0), 0, None)
    with pytest.raises(RuntimeError):
        ops.gemv(dq.bufs, dq.meta, torch.zeros(1, 256), 0, None)      # CPU tensor: no fallback


def test_rtn_outlier_overrides(cuda_lib):
    """Sparse outlier overrides of per-row tensors (formats/codec.py:279-292): the dense result is
    the codec's bit for bit, a position listed twice keeps its last value, the GEMV adds the
    sparse correction before the epilogue (rel <= 1e-3) and is reproducible, and the dense bf16
    stand-in the model uses equals bf16(dequant)."""
    from rwkv_quant_b200 import synth
    from rwkv_quant_b200.backends.cuda import QuantLinearV2, ops
    g = torch.Generator().manual_seed(5)
    rows, cols = 96, 256
    qt = synth.quant_rtn("w", "g", torch.randn(rows, cols, generator=g) * 0.02, 8)
    idx = torch.tensor([[3, 7], [3, 200], [0, 0], [95, 255], [40, 13], [3, 7], [40, 12]], dtype=torch.int32)
    val = torch.tensor([0.5, -0.25, 1.0, -2.0, 0.125, 0.75, 3.0]).to(torch.bfloat16)
    qt.outlier_indices, qt.outlier_values = idx, val
    n = lambda t: None if t is None else t.numpy()
    ref = oc.dequant_rtn(n(qt.scale), shape=qt.shape, codes=n(qt.codes), codes_packed=n(qt.codes_packed),
                         outlier_indices=idx.numpy(), outlier_values=val.float().numpy())
    assert ref[3, 7] == 0.75
    lin = QuantLinearV2(qt)
    np.testing.assert_array_equal(lin._dequant_w(torch.float32).cpu().numpy(), ref)
    x = _x(3, cols, 17)
    resid = _x(3, rows, 18)
    for epi, r in ((0, None), (1, None), (2, resid)):
        y1 = lin(x, epilogue=epi, resid=r)
        y2 = lin(x, epilogue=epi, resid=r)
        assert torch.equal(y1, y2)
        want = x.cpu().numpy().astype(np.float64) @ ref.astype(np.float64).T
        if epi == 1:
            want = np.maximum(want, 0) ** 2
        elif epi == 2:
            want = want + resid.cpu().numpy()
        assert relmax(y1.cpu().numpy(), want) <= TOL, epi
    dense = lin.dq.densified()
    assert dense.kind == "dense" and dense.outliers is None
    np.testing.assert_array_equal(dense.dequant(torch.float32, False).cpu().numpy(), oc.f32_to_bf16_rne(ref))


@pytest.mark.parametrize("name", ["toy_compression", "toy_reduction", "toy_custom_int8"])
def test_c_reader_upload_feeds_the_kernels(cuda_lib, name):
    """rwkvq_file_open -> rwkvq_file_upload: the device descriptor made without Python or torch
    dequantises to the codec's bits (every tensor of a reference-written file), and a GEMV on it
    equals the GEMV on the Python loader's descriptor."""
    import ctypes as C
    from conftest import GOLDEN
    from oracle import codec_np as oc
    from rwkv_quant_b200 import _lib
    from rwkv_quant_b200.backends.cuda import ops
    from rwkv_quant_b200.formats import load_raw
    path = os.path.join(GOLDEN, name + ".rwkvq")
    man, arr = oc.open_rwkvq(path)
    ck = load_raw(path)
    h = C.c_void_p()
    _lib.check(cuda_lib.rwkvq_file_open(path.encode(), C.byref(h)), "rwkvq_file_open")
    slabs = []
    try:
        for key, t in man["tensors"].items():
            v, slab = _lib.QTensorStruct(), C.c_void_p()
            _lib.check(cuda_lib.rwkvq_file_upload(h, key.encode(), C.byref(v), C.byref(slab), _lib.stream_ptr()),
                       "rwkvq_file_upload")
            slabs.append(slab)
            out = torch.empty((v.rows, v.cols), dtype=torch.float32, device="cuda")
            _lib.check(cuda_lib.rwkvq_dequant(C.byref(v), out.data_ptr(), _lib.DTYPE_CODE[torch.float32], 0,
                                              _lib.stream_ptr()), "rwkvq_dequant")
            qt = ck.tensors[key]
            has_outliers = getattr(qt, "outlier_indices", None) is not None and qt.outlier_indices.numel() > 0
            want = oc.dequant_key(man, arr, key).reshape(v.rows, v.cols)
            if has_outliers:                           # the descriptor carries the packed codes only
                want = ops.DeviceQT(qt, "cuda", relayout=False)
                want = ops.dequant(want.bufs, want.meta, torch.float32, False).cpu().numpy()
            assert np.array_equal(out.cpu().numpy(), want), key
            if t["kind"] in ("sb6", "sym") and v.cols % 256 == 0:
                x = torch.randn(1, v.cols, device="cuda")
                y = torch.empty((1, v.rows), dtype=torch.float32, device="cuda")
                _lib.check(cuda_lib.rwkvq_gemv(C.byref(v), x.data_ptr(), 0, 1, v.cols, y.data_ptr(), v.rows, 0, None,
                                               _lib.stream_ptr()), "rwkvq_gemv")
                d = ops.DeviceQT(qt, "cuda", relayout=False)
                assert torch.equal(y, ops.gemv(d.bufs, d.meta, x, 0, None)), key
        torch.cuda.synchronize()
    finally:
        for s in slabs:
            cuda_lib.rwkvq_file_free_slab(s)
        cuda_lib.rwkvq_file_close(h)


@pytest.mark.parametrize("layout,bits", LAYOUTS[:6])
def test_gemv_skips_all_zero_activation_groups_exactly(cuda_lib, layout, bits):
    """relu(k)^2 leaves most channel-mix activations exactly zero; the single-vector kernel does not
    read the codes of a 32-column group whose activations are all zero.  Same bar as the dense
    case (and the rows of a 2-row call, which run one by one, agree bit for bit with single calls)."""
    import ctypes as C
    from rwkv_quant_b200.backends.cuda import ops
    sw = cuda_lib.rwkvq_profiling_zero_skip          # rwkvq_profiling.h: the skip is opt-in (RWKVQ_ZERO_SKIP=1)
    sw.restype, sw.argtypes = None, [C.c_int]
    try:
        sw(1)
        y_on = _zero_group_case(ops, layout, bits)
        sw(0)
        y_off = _zero_group_case(ops, layout, bits)
    finally:
        sw(-1)
    assert np.array_equal(y_on, y_off), "the skip changed a bit of the result"


def _zero_group_case(ops, layout, bits):
    rows, cols = 2048, 8192
    qt = _synth_linear(layout, bits, rows, cols, seed=17 + bits)
    dq = ops.DeviceQT(qt)
    w = _oracle_w(qt).astype(np.float64)
    rs = np.random.default_rng(5)
    x = np.maximum(rs.standard_normal((2, cols)), 0.0).astype(np.float32) ** 2       # ~50 % zeros
    groups = rs.random((2, cols // 32)) < 0.6                                         # + 60 % of the groups entirely zero
    x = (x.reshape(2, cols // 32, 32) * ~groups[..., None]).reshape(2, cols)
    x[1, :32 * 200] = 0.0                                                             # a long zero run, whole iterations
    xt = torch.from_numpy(x).cuda()
    y = ops.gemv(dq.bufs, dq.meta, xt, 0, None).cpu().numpy()
    ref = x.astype(np.float64) @ w.T
    assert relmax(y, ref) <= TOL and np.isfinite(y).all()
    print(f"{layout}@{bits} zero-group skip: relmax {relmax(y, ref):.2e}")
    for r in range(2):
        y1 = ops.gemv(dq.bufs, dq.meta, xt[r:r + 1].contiguous(), 0, None).cpu().numpy()
        assert np.array_equal(y1[0], y[r])
    # an all-zero vector gives exact zeros
    z = ops.gemv(dq.bufs, dq.meta, torch.zeros(1, cols, device="cuda"), 0, None)
    assert (z == 0).all()
    return y
