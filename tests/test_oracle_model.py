"""The stateful CPU forward against the reference's own PyTorch forward.

Golden: ``RWKV7Ref(cpu, fp32)`` logits on the dequantised state dict of a toy
model quantized by ``rwkv_quant.quantize()`` (tests/golden/make_golden.py).
With linears rounded to bf16 (what RWKV7Ref sees) the restatement agrees to
float noise; with exact linears (what the kernels compute) the distance is the
bf16 rounding of the weights, which is recorded, not gated tightly.
"""
import os

import numpy as np
import pytest

from conftest import GOLDEN
from helpers import relmax
from oracle import codec_np as oc
from oracle.model_np import OracleRWKV7, wkv7_np


@pytest.mark.parametrize("preset", ["reduction", "compression"])
def test_matches_reference_forward(preset):
    man, arr = oc.open_rwkvq(os.path.join(GOLDEN, f"toy_{preset}.rwkvq"))
    z = np.load(os.path.join(GOLDEN, f"toy_{preset}_ref.npz"))
    m = OracleRWKV7(man, arr, linear_weights="bf16")
    trace = []
    hidden, _ = m.forward_hidden(z["idx"], m.init_state(z["idx"].shape[0]), trace=trace)
    logits = hidden @ m.head.T
    assert relmax(logits, z["logits"]) < 5e-6
    for i, t in enumerate(trace):
        assert relmax(t, z["trace"][i]) < 5e-6, f"residual stream after block {i}"
    exact = OracleRWKV7(man, arr, linear_weights="exact")(z["idx"])
    d = relmax(exact, z["logits"])
    assert d < 1e-2          # the reference's own model-level gate (tests/test_quant_parity.py:138)
    print(f"{preset}: exact-linears vs all-bf16 reference forward relmax {d:.3e}")


@pytest.mark.parametrize("cfg", ["int8", "compression", "d128_int8"])
def test_custom_naming_matches_reference_forward(cfg):
    """Custom-naming checkpoints written by the reference's writer.save() (tmix./cmix. keys, LoRA
    pairs as [out, in] linears with biases; tests/test_quant_parity.py:97-118)."""
    man, arr = oc.open_rwkvq(os.path.join(GOLDEN, f"toy_custom_{cfg}.rwkvq"))
    assert man["naming"] == "custom"
    z = np.load(os.path.join(GOLDEN, f"toy_custom_{cfg}_ref.npz"))
    m = OracleRWKV7(man, arr, linear_weights="bf16")
    hidden, _ = m.forward_hidden(z["idx"], m.init_state(z["idx"].shape[0]))
    assert relmax(hidden @ m.head.T, z["logits"]) < 5e-6
    assert relmax(OracleRWKV7(man, arr)(z["idx"]), z["logits"]) < 1e-2


@pytest.mark.parametrize("preset", ["reduction", "compression"])
def test_streaming_equals_whole(preset):
    """Whole prompt == chunks == token by token (tests/test_streaming_inference.py)."""
    man, arr = oc.open_rwkvq(os.path.join(GOLDEN, f"toy_{preset}.rwkvq"))
    idx = np.load(os.path.join(GOLDEN, f"toy_{preset}_ref.npz"))["idx"]
    m = OracleRWKV7(man, arr)
    whole, st_whole = m.forward_stateful(idx, m.init_state(idx.shape[0]))
    for step in (1, 7):
        st, outs = m.init_state(idx.shape[0]), []
        for t0 in range(0, idx.shape[1], step):
            lo, st = m.forward_stateful(idx[:, t0:t0 + step], st)
            outs.append(lo)
        assert relmax(np.concatenate(outs, 1), whole) < 1e-5
        for (a, b, c), (a2, b2, c2) in zip(st, st_whole):
            assert np.abs(a - a2).max() < 1e-5
            np.testing.assert_allclose(b, b2, atol=1e-6)
            np.testing.assert_allclose(c, c2, atol=1e-6)
    lo, _ = m.forward_stateful(idx, m.init_state(idx.shape[0]), last_only=True)
    np.testing.assert_allclose(lo, whole[:, -1:], atol=3e-6)   # BLAS blocking differs with M
    lo, _ = m.forward_stateful(idx, m.init_state(idx.shape[0]), tail_only=3)
    np.testing.assert_allclose(lo, whole[:, -3:], atol=3e-6)


def test_wkv7_matches_reference_loop(reference):
    """wkv7_np with a zero state == RWKV7Ref._wkv7 (models/rwkv7_ref.py:236-255)."""
    import torch
    from rwkv_quant.models.rwkv7_ref import RWKV7Ref
    rs = np.random.RandomState(5)
    B, T, H, S = 2, 9, 3, 64
    r, k, v = (rs.randn(B, T, H, S).astype(np.float32) for _ in range(3))
    a, b = (0.1 * rs.randn(B, T, H, S).astype(np.float32) for _ in range(2))
    wlog = (rs.randn(B, T, H, S) * 0.5 - 0.5).astype(np.float32)     # w_ of the reference
    decay = np.exp(-np.exp(wlog)).astype(np.float32)
    out, _ = wkv7_np(r, decay, k, v, a, b, np.zeros((B, H, S, S), np.float32))
    t = lambda x: torch.from_numpy(x.reshape(B, T, H * S))
    ref = RWKV7Ref._wkv7(t(r), t(wlog), t(k), t(v), t(a), t(b), H, S).numpy().reshape(B, T, H, S)
    assert relmax(out, ref) < 1e-5


def test_wkv7_state_carry():
    """Running T steps at once == running them in two calls carrying the state."""
    rs = np.random.RandomState(7)
    B, T, H, S = 1, 12, 2, 64
    r, k, v = (rs.randn(B, T, H, S).astype(np.float32) for _ in range(3))
    a, b = (0.1 * rs.randn(B, T, H, S).astype(np.float32) for _ in range(2))
    w = (0.85 + 0.14 * rs.rand(B, T, H, S)).astype(np.float32)
    h0 = (0.05 * rs.randn(B, H, S, S)).astype(np.float32)
    o, h = wkv7_np(r, w, k, v, a, b, h0)
    o1, h1 = wkv7_np(r[:, :5], w[:, :5], k[:, :5], v[:, :5], a[:, :5], b[:, :5], h0)
    o2, h2 = wkv7_np(r[:, 5:], w[:, 5:], k[:, 5:], v[:, 5:], a[:, 5:], b[:, 5:], h1)
    np.testing.assert_array_equal(np.concatenate([o1, o2], 1), o)
    np.testing.assert_array_equal(h2, h)
