"""Chunked form of the WKV-7 recurrence on the CPU (test infrastructure: only tests import this).

The sequential scan (`oracle/model_np.py::wkv7_np`, which restates the reference's
`rwkv_quant/models/rwkv7_ref.py:236-255`) applies, per head and per token,

    S_t = S_{t-1} diag(w_t) + (S_{t-1} a_t) b_t^T + v_t k_t^T ,      y_t = S_t r_t

with S [value row, key column].  Every row of S obeys the same linear recurrence, and with
u_t = S_{t-1} a_t the update is a diagonal decay plus two rank-one terms, so a chunk of C tokens
can be advanced with small matrix products instead of C dependent steps.  With the running decay
P_t = w_1 * ... * w_t (per key column, P_0 = 1) and the scaled vectors

    a~_t = a_t * P_{t-1},   r~_t = r_t * P_t,   b^_j = b_j / P_j,   k^_j = k_j / P_j

the chunk is

    u_t  = S_0 a~_t + sum_{j<t}  ( u_j (b^_j . a~_t) + v_j (k^_j . a~_t) )        forward substitution over t
    y_t  = S_0 r~_t + sum_{j<=t} ( u_j (b^_j . r~_t) + v_j (k^_j . r~_t) )
    S_C  = ( S_0 + sum_j ( u_j b^_j^T + v_j k^_j^T ) ) diag(P_C)

i.e. four C x C Gram matrices (contractions over the 64 key columns), two products of the state
with C columns, one triangular solve of size C, and one rank-2C update of the state.  RWKV-7's decay
is w = exp(-0.606531 sigmoid(.)) > 0.545, so 1 / P_j stays below 0.545^-C (1.6e4 for C = 16, 2.7e8
for C = 32) and fp32 carries the scaled vectors without trouble; the tests hold the chunked form
to 1e-5 of the sequential one in fp32.  This is the arithmetic a chunked GPU scan would run (Gram
matrices and state products on the tensor cores, the substitution on a warp); the library's
`rwkvq_wkv7` is the sequential scan.
"""
from __future__ import annotations

import numpy as np


def wkv7_chunked_np(r, w, k, v, a, b, state, chunk: int = 16, dtype=np.float32):
    """Same contract as `wkv7_np`: r, w, k, v, a, b [B, T, H, S] (w is the decay itself),
    state [B, H, S, S] indexed [value row, key column] -> (y [B, T, H, S], final state)."""
    f = dtype
    r, w, k, v, a, b = (np.asarray(x, dtype=f) for x in (r, w, k, v, a, b))
    B, T, H, S = r.shape
    st = np.array(state, dtype=f, copy=True)
    out = np.empty((B, T, H, S), dtype=f)
    for t0 in range(0, T, chunk):
        C = min(chunk, T - t0)
        sl = slice(t0, t0 + C)
        # [B, H, C, S] views of the chunk
        rc, wc, kc, vc, ac, bc = (np.moveaxis(x[:, sl], 1, 2) for x in (r, w, k, v, a, b))
        P = np.cumprod(wc, axis=2, dtype=f)                                   # P_t, t = 1..C
        P_prev = np.concatenate([np.ones_like(P[:, :, :1]), P[:, :, :-1]], axis=2)
        a_s, r_s = ac * P_prev, rc * P
        b_h, k_h = bc / P, kc / P
        # Gram matrices [B, H, j, t]
        g_ba = np.einsum("bhjs,bhts->bhjt", b_h, a_s)
        g_ka = np.einsum("bhjs,bhts->bhjt", k_h, a_s)
        g_br = np.einsum("bhjs,bhts->bhjt", b_h, r_s)
        g_kr = np.einsum("bhjs,bhts->bhjt", k_h, r_s)
        strict = np.triu(np.ones((C, C), dtype=f), 1)                         # j < t
        upper = np.triu(np.ones((C, C), dtype=f), 0)                          # j <= t
        # u [B, H, value row, t]: right-hand side, then forward substitution over t
        rhs = np.einsum("bhvs,bhts->bhvt", st, a_s) + np.einsum("bhjv,bhjt->bhvt", vc, g_ka * strict)
        u = np.zeros_like(rhs)
        gs = g_ba * strict
        for t in range(C):
            u[..., t] = rhs[..., t] + np.einsum("bhvj,bhj->bhv", u[..., :t], gs[..., :t, t])
        y = np.einsum("bhvs,bhts->bhvt", st, r_s) + np.einsum("bhvj,bhjt->bhvt", u, g_br * upper) \
            + np.einsum("bhjv,bhjt->bhvt", vc, g_kr * upper)
        out[:, sl] = np.transpose(y, (0, 3, 1, 2))                            # [B, C, H, S]
        st = (st + np.einsum("bhvj,bhjs->bhvs", u, b_h) + np.einsum("bhjv,bhjs->bhvs", vc, k_h)) * P[:, :, -1][:, :, None, :]
    return out, st
