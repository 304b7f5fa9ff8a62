"""The numpy restatement of the reference's sb6 search quantizer (oracle/quant_np.py) against
tensors the reference itself packed, and against the reference run live where it is present.

Sums over a block run in a different order in numpy and in torch, so the two agree to the last
bits of each block's (s, m) and not bit for bit; the bars below are fractions of equal codes."""
import json
import os
import sys

import numpy as np
import pytest
import torch

from oracle import quant_np as qn

HERE = os.path.dirname(os.path.abspath(__file__))
# the reference checkout: RWKVQ_REFERENCE_DIR, else a directory "reference" beside the repository
REF = os.environ.get("RWKVQ_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def config1_weights(rows):
    """The seeded W of the single-GEMV configuration (tests/golden/make_golden.py::make_config1)."""
    w = torch.randn(8192, 2048, generator=torch.Generator().manual_seed(0)) * 0.02
    return w[:rows].numpy()


def test_quantizer_oracle_matches_reference_packed_tensor():
    rows = 768
    z = np.load(os.path.join(HERE, "golden", "config1_gemv.npz"))
    meta = json.loads(bytes(z["__meta__"]).decode())["config1"]
    assert (meta["kind"], meta["bits"]) == ("sb6", 4)
    r = qn.quant_sb6(config1_weights(rows), 4, search=True)
    q, qs, qm = qn.unpack_sb6(z["config1::codes_packed"][:rows], z["config1::gw_qsqm"][:rows], None, None, shape=(rows, 2048))
    eq = {"q": (q == r["q"]).mean(), "qs": (qs == r["qs"]).mean(), "qm": (qm == r["qm"]).mean(),
          "d": (z["config1::gw_d"][:rows] == r["d"]).mean(), "dm": (z["config1::gw_dm"][:rows] == r["dm"]).mean()}
    print("equal fractions against the reference-packed tensor:", {k: f"{v:.6f}" for k, v in eq.items()})
    assert eq["q"] >= 0.9999 and eq["qs"] >= 0.9995 and eq["qm"] >= 0.9995 and eq["d"] >= 0.999 and eq["dm"] >= 0.999


@pytest.mark.skipif(not os.path.isdir(REF), reason="reference tree not present")
@pytest.mark.parametrize("bits,search,aw", [(4, True, False), (5, True, False), (6, False, False), (4, True, True), (6, True, True)])
def test_quantizer_oracle_matches_reference_live(bits, search, aw):
    sys.path.insert(0, REF)
    try:
        from rwkv_quant.calibration.groupwise import _gw_one
    finally:
        sys.path.remove(REF)
    g = torch.Generator().manual_seed(bits * 7 + search + 2 * aw)
    w = torch.randn(96, 1024, generator=g) * 0.05
    w[3] = 0.25                                  # a constant row: degenerate blocks
    w[5, :40] *= 30.0                            # outliers inside a block
    ex2 = (torch.rand(1024, generator=g) ** 2 * 4 + 1e-3) if aw else None
    ref = _gw_one(w, bits, 32, sb=8, sb_bits=(-6 if search else 6), ex2=ex2, return_parts=True)
    r = qn.quant_sb6(w.numpy(), bits, search, None if ex2 is None else ex2.numpy())
    assert (r["q"] == ref["q"].numpy()).mean() >= 0.9995
    assert (r["qs"] == ref["qs"].numpy()).mean() >= 0.999 and (r["qm"] == ref["qm"].numpy()).mean() >= 0.999
    assert (r["d"] == ref["d"].numpy()).mean() >= 0.995 and (r["dm"] == ref["dm"].numpy()).mean() >= 0.995
    e_ref = float(((ref["deq"].numpy() - w.numpy()) ** 2).sum()), 
    e_our = float(((r["deq"] - w.numpy()) ** 2).sum())
    assert abs(e_our - e_ref[0]) <= 1e-3 * e_ref[0]


@pytest.mark.skipif(not os.path.isdir(REF), reason="reference tree not present")
@pytest.mark.parametrize("bits,search,aw", [(6, True, False), (8, True, False), (6, False, False), (8, True, True)])
def test_sym_quantizer_oracle_matches_reference_live(bits, search, aw):
    sys.path.insert(0, REF)
    try:
        from rwkv_quant.calibration.groupwise import _SYM_FACTORS, _sym_one
    finally:
        sys.path.remove(REF)
    assert list(_SYM_FACTORS) == torch.linspace(0.7, 1.15, 19).tolist()
    g = torch.Generator().manual_seed(bits + 3 * search + aw)
    w = torch.randn(64, 1024, generator=g) * 0.05
    w[2] = 0.0                                   # an all-zero row: degenerate super-blocks
    w[4, 16:20] *= 50.0
    ex2 = (torch.rand(1024, generator=g) ** 2 * 4 + 1e-3) if aw else None
    ref = _sym_one(w, bits, 16, 16, ex2, search, 0.0, True)
    r = qn.quant_sym(w.numpy(), bits, _SYM_FACTORS if search else (1.0,), None if ex2 is None else ex2.numpy())
    assert (r["q"] == ref["q"].numpy()).mean() >= 0.9995
    assert (r["qs"] == ref["qs"].numpy()).mean() >= 0.999 and (r["d"] == ref["d"].numpy()).mean() >= 0.995
    e_ref, e_our = float(((ref["deq"].numpy() - w.numpy()) ** 2).sum()), float(((r["deq"] - w.numpy()) ** 2).sum())
    assert abs(e_our - e_ref) <= 1e-3 * e_ref
