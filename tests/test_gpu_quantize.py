"""Device-side sb6 quantizer (rwkvq_quantize_sb6) against the numpy oracle of the reference's
search quantizer and against a tensor the reference itself packed.  Codes are compared as fractions
of equal entries (block sums run in different orders, see oracle/quant_np.py); the quantization
error must match the oracle's to 1e-4 relative, and the packed tensor must decode, through the
kernels, to exactly q * s + m of its own parts."""
import json
import os

import numpy as np
import pytest
import torch

from oracle import codec_np as oc
from oracle import quant_np as qn

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("bits,mode", [(4, "asym_sb6_search"), (5, "asym_sb6_search"), (6, "asym_sb6"), (4, "asym_sb6_aw"),
                                       (6, "asym_sb6_aw"), (5, "asym_sb6")])
def test_quantize_sb6_matches_oracle(cuda_lib, bits, mode):
    from rwkv_quant_b200 import quantize
    g = torch.Generator().manual_seed(bits * 11 + len(mode))
    w = torch.randn(300, 2048, generator=g) * 0.03
    w[7] = -0.125                               # constant row
    w[9, 100:130] *= 40.0                       # outliers across a block boundary
    w[11] = 0.0
    ex2 = (torch.rand(2048, generator=g) ** 2 * 3 + 1e-3) if mode.endswith("_aw") else None
    ref = qn.quant_sb6(w.numpy(), bits, mode != "asym_sb6", None if ex2 is None else ex2.numpy())
    q, qs, qm, d, dm = quantize.quantize_sb6_parts(w.cuda(), bits, mode != "asym_sb6", None if ex2 is None else ex2.cuda())
    q, qs, qm, d, dm = (t.cpu().numpy() for t in (q, qs, qm, d, dm))
    eq = {"q": (q == ref["q"]).mean(), "qs": (qs == ref["qs"]).mean(), "qm": (qm == ref["qm"]).mean(),
          "d": (d == ref["d"]).mean(), "dm": (dm == ref["dm"]).mean()}
    print(f"sb6@{bits} {mode}: equal fractions", {k: f"{v:.6f}" for k, v in eq.items()})
    assert eq["q"] >= 0.9995 and eq["qs"] >= 0.999 and eq["qm"] >= 0.999 and eq["d"] >= 0.995 and eq["dm"] >= 0.995
    # the packed tensor decodes (CUDA dequant kernel, bit-exact codec) to q * s + m of its own parts
    qt = quantize.quantize_sb6("blocks.0.ffn.key.weight", "cmix", w.cuda(), bits, mode, None if ex2 is None else ex2.cuda())
    from rwkv_quant_b200.backends.cuda import ops
    dq = ops.DeviceQT(qt)
    deq = dq.dequant().cpu().numpy()
    s = np.maximum((qs.astype(np.float32).reshape(300, -1, 8) * d.astype(np.float32)[..., None]).astype(np.float16).astype(np.float32), 1e-8)
    m = (qm.astype(np.float32).reshape(300, -1, 8) * dm.astype(np.float32)[..., None]).astype(np.float16).astype(np.float32)
    own = q.reshape(300, -1, 32).astype(np.float32) * s.reshape(300, -1, 1) + m.reshape(300, -1, 1)
    assert np.array_equal(deq, own.reshape(300, 2048))
    e_ref, e_our = float(((ref["deq"] - w.numpy()) ** 2).sum()), float(((deq - w.numpy()) ** 2).sum())
    assert abs(e_our - e_ref) <= 1e-4 * e_ref, (e_our, e_ref)
    # and runs through the GEMV
    x = torch.randn(1, 2048, device="cuda")
    y = ops.gemv(dq.bufs, dq.meta, x, 0, None).cpu().numpy()
    yr = x.cpu().numpy().astype(np.float64) @ deq.astype(np.float64).T
    assert np.abs(y - yr).max() <= 1e-3 * np.abs(yr).max()


def test_quantize_sb6_matches_reference_packed_tensor(cuda_lib):
    """W [8192, 2048] of the single-GEMV configuration, packed by the reference's
    quantize_tensor(... asym_sb6_search ...) (tests/golden/make_golden.py::make_config1)."""
    from rwkv_quant_b200 import quantize
    z = np.load(os.path.join(HERE, "golden", "config1_gemv.npz"))
    w = torch.randn(8192, 2048, generator=torch.Generator().manual_seed(0)) * 0.02
    qt = quantize.quantize_sb6("blocks.0.ffn.key.weight", "cmix", w.cuda(), 4, "asym_sb6_search")
    same = {"codes_packed": (qt.codes_packed.cpu().numpy() == z["config1::codes_packed"]).mean(),
            "gw_qsqm": (qt.gw_qsqm.cpu().numpy() == z["config1::gw_qsqm"]).mean(),
            "gw_d": (qt.gw_d.cpu().numpy() == z["config1::gw_d"]).mean(),
            "gw_dm": (qt.gw_dm.cpu().numpy() == z["config1::gw_dm"]).mean()}
    print("bytes equal to the reference-packed tensor:", {k: f"{v:.6f}" for k, v in same.items()})
    assert same["codes_packed"] >= 0.9999 and same["gw_qsqm"] >= 0.999 and same["gw_d"] >= 0.999 and same["gw_dm"] >= 0.999
    # the reference's y = x @ dequant(W).T of that configuration, through our tensor and kernel: rows whose
    # bytes all equal the reference's must reproduce its y; a row where one block chose another (equally good)
    # factor differs at the level of the quantization noise
    from rwkv_quant_b200.backends.cuda import ops
    dq = ops.DeviceQT(qt)
    x = torch.from_numpy(z["x"].astype(np.float32)).cuda()
    y = ops.gemv(dq.bufs, dq.meta, x, 0, None).cpu().numpy()[0]
    same_row = ((qt.codes_packed.cpu().numpy() == z["config1::codes_packed"]).all(axis=1) &
                (qt.gw_qsqm.cpu().numpy() == z["config1::gw_qsqm"]).all(axis=(1, 2)) &
                (qt.gw_d.cpu().numpy() == z["config1::gw_d"]).all(axis=1) & (qt.gw_dm.cpu().numpy() == z["config1::gw_dm"]).all(axis=1))
    print(f"rows identical to the reference's: {same_row.mean():.4f}")
    assert same_row.mean() >= 0.97
    ref_y = z["y"][0]
    assert np.abs(y - ref_y)[same_row].max() <= 1e-5 * np.abs(ref_y).max()
    assert np.abs(y - ref_y).max() <= 2e-2 * np.abs(ref_y).max()


def test_quantize_sb6_refusals(cuda_lib):
    from rwkv_quant_b200 import quantize
    with pytest.raises(ValueError):
        quantize.quantize_sb6_parts(torch.randn(4, 300, device="cuda"), 4)
    with pytest.raises(ValueError):
        quantize.quantize_sb6_parts(torch.randn(4, 512), 4)
    with pytest.raises(Exception):
        quantize.quantize_sb6_parts(torch.randn(4, 512, device="cuda"), 7)
    with pytest.raises(ValueError):
        quantize.quantize_sb6("k", "cmix", torch.randn(4, 512, device="cuda"), 4, "asym_sb6_aw")


@pytest.mark.parametrize("bits,mode", [(6, "sym"), (8, "sym"), (6, "sym_plain"), (8, "sym_aw"), (6, "sym_aw")])
def test_quantize_sym_matches_oracle(cuda_lib, bits, mode):
    from rwkv_quant_b200 import quantize
    from rwkv_quant_b200.backends.cuda import ops
    g = torch.Generator().manual_seed(bits * 5 + len(mode))
    w = torch.randn(200, 2048, generator=g) * 0.03
    w[3] = 0.0                                  # all-zero row: scale codes and codes 0
    w[5, 10:14] *= 60.0
    ex2 = (torch.rand(2048, generator=g) ** 2 * 3 + 1e-3) if mode == "sym_aw" else None
    factors = quantize.sym_factors().tolist() if mode != "sym_plain" else (1.0,)
    ref = qn.quant_sym(w.numpy(), bits, factors, None if ex2 is None else ex2.numpy())
    q, qs, d = (t.cpu().numpy() for t in quantize.quantize_sym_parts(w.cuda(), bits, mode != "sym_plain", None if ex2 is None else ex2.cuda()))
    eq = {"q": (q == ref["q"]).mean(), "qs": (qs == ref["qs"]).mean(), "d": (d == ref["d"]).mean()}
    print(f"sym@{bits} {mode}: equal fractions", {k: f"{v:.6f}" for k, v in eq.items()})
    assert eq["q"] >= 0.9995 and eq["qs"] >= 0.999 and eq["d"] >= 0.995
    qt = quantize.quantize_sym("blocks.0.att.key.weight", "proj", w.cuda(), bits, mode, None if ex2 is None else ex2.cuda())
    dq = ops.DeviceQT(qt)
    deq = dq.dequant().cpu().numpy()
    s = (qs.astype(np.float32).reshape(200, -1, 16) * d.astype(np.float32)[..., None]).astype(np.float16).astype(np.float32)
    own = q.reshape(200, -1, 16).astype(np.float32) * s.reshape(200, -1, 1)
    assert np.array_equal(deq, own.reshape(200, 2048))
    assert (deq[3] == 0).all()
    e_ref, e_our = float(((ref["deq"] - w.numpy()) ** 2).sum()), float(((deq - w.numpy()) ** 2).sum())
    assert abs(e_our - e_ref) <= 1e-4 * e_ref
    x = torch.randn(1, 2048, device="cuda")
    y = ops.gemv(dq.bufs, dq.meta, x, 0, None).cpu().numpy()
    yr = x.cpu().numpy().astype(np.float64) @ deq.astype(np.float64).T
    assert np.abs(y - yr).max() <= 1e-3 * np.abs(yr).max()
