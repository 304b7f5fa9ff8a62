"""The chunked restatement of WKV-7 (oracle/wkv7_chunked_np.py) against the sequential oracle
(oracle/model_np.py::wkv7_np, pinned to the reference and to the C restatement elsewhere): inputs shaped
like the model's (decay exp(-0.606531 sigmoid(.)), a = -kk, b = kk * gate with kk normalised per head),
several chunk lengths, a ragged last chunk, a non-zero initial state.  Tolerances written here:
fp32 chunked vs fp32 sequential 1e-5 of max|y| and of max(1, max|S|); fp64 chunked vs an fp64
sequential loop 1e-12."""
import numpy as np
import pytest

from oracle.model_np import wkv7_np
from oracle.wkv7_chunked_np import wkv7_chunked_np


def _inputs(B, T, H, S, seed):
    g = np.random.default_rng(seed)
    r, k, v = (g.standard_normal((B, T, H, S)).astype(np.float32) for _ in range(3))
    w = np.exp(-0.606531 / (1.0 + np.exp(-g.standard_normal((B, T, H, S))))).astype(np.float32)
    kk = k * g.uniform(0.5, 1.5, (1, 1, H, S)).astype(np.float32)
    kk = kk / np.sqrt((kk * kk).sum(-1, keepdims=True) + 1e-12)
    gate = (1.0 / (1.0 + np.exp(-g.standard_normal((B, T, H, S))))).astype(np.float32)
    st = (0.5 * g.standard_normal((B, H, S, S))).astype(np.float32)
    return r, w, k, v, (-kk).astype(np.float32), (kk * gate).astype(np.float32), st


def _seq64(r, w, k, v, a, b, st):
    r, w, k, v, a, b = (x.astype(np.float64) for x in (r, w, k, v, a, b))
    st = st.astype(np.float64).copy()
    out = np.empty(r.shape, dtype=np.float64)
    for t in range(r.shape[1]):
        sa = np.einsum("bhvk,bhk->bhv", st, a[:, t])
        st = st * w[:, t][:, :, None, :] + sa[..., None] * b[:, t][:, :, None, :] + v[:, t][..., None] * k[:, t][:, :, None, :]
        out[:, t] = np.einsum("bhvk,bhk->bhv", st, r[:, t])
    return out, st


@pytest.mark.parametrize("T,chunk", [(1, 16), (16, 16), (37, 16), (64, 32), (50, 8), (96, 64)])
def test_chunked_matches_sequential_fp32(T, chunk):
    x = _inputs(2, T, 3, 64, seed=T * 100 + chunk)
    y0, s0 = wkv7_np(*x)
    y1, s1 = wkv7_chunked_np(*x, chunk=chunk)
    ey = np.abs(y1 - y0).max() / max(np.abs(y0).max(), 1e-30)
    es = np.abs(s1 - s0).max() / max(1.0, np.abs(s0).max())
    print(f"T={T} chunk={chunk}: y relmax {ey:.2e}, state {es:.2e}")
    assert ey <= 1e-5 and es <= 1e-5, (ey, es)


def test_chunked_matches_sequential_fp64():
    x = _inputs(1, 70, 2, 64, seed=7)
    y0, s0 = _seq64(*x)
    y1, s1 = wkv7_chunked_np(*x, chunk=16, dtype=np.float64)
    assert np.abs(y1 - y0).max() <= 1e-12 * max(1.0, np.abs(y0).max())
    assert np.abs(s1 - s0).max() <= 1e-12 * max(1.0, np.abs(s0).max())


def test_chunks_compose():
    """Two calls over halves of a sequence, state handed over, equal one call over the whole."""
    x = _inputs(1, 48, 2, 64, seed=11)
    r, w, k, v, a, b, st = x
    y, s = wkv7_chunked_np(*x, chunk=16)
    ya, sa = wkv7_chunked_np(r[:, :32], w[:, :32], k[:, :32], v[:, :32], a[:, :32], b[:, :32], st, chunk=16)
    yb, sb = wkv7_chunked_np(r[:, 32:], w[:, 32:], k[:, 32:], v[:, 32:], a[:, 32:], b[:, 32:], sa, chunk=16)
    assert np.array_equal(np.concatenate([ya, yb], 1), y) and np.array_equal(sb, s)
