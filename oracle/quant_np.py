"""CPU oracle of the sb6 and sym block quantizers (test infrastructure: only tests import this).

A numpy restatement of the reference's search quantizer for the `sb6` layout,
`rwkv_quant/calibration/groupwise.py:207-300` (`_gw_one` with sb = 8 and sb_bits = -6 for the
search modes `asym_sb6_search` / `asym_sb6_aw`, sb_bits = 6 for plain `asym_sb6`):

  per block of 32 weights   min / max scale; with search, for each of 8 factors of that scale:
                            codes -> closed-form least-squares (s, m) for those codes (optionally
                            weighted by E[x^2] of the input channel) -> codes again -> squared
                            error; the (s, m) of the smallest error wins (first factor on ties)
  per super-block of 8      d = fp16(max s / 63), qs = clamp(round(s / d), 1, 63);
                            dm = fp16(max|m| / 31), qm = clamp(round(m / dm), -31, 31);
                            s' = max(fp16(qs d), 1e-8), m' = fp16(qm dm)
  per weight                q = clamp(round((w - m') / s'), 0, 2^bits - 1)

All arithmetic is float32 like the reference's torch code.  Sums over the 32 weights of a block are
taken in numpy's order, the reference takes them in torch's, the CUDA kernel as a shuffle tree: the
three agree to the last bits of (s, m), not bit for bit, so codes may differ where a quotient falls
within an ulp of a rounding boundary or two factors tie.  Pinned against tensors packed by the
reference itself (tests/golden/config1_gemv.npz: the codes, scale codes and super-scales the
reference's `quantize_tensor(... asym_sb6_search ...)` chose for a seeded W [8192, 2048]).
"""
from __future__ import annotations

import numpy as np

FACTORS = (0.7, 0.75, 0.8, 0.85, 0.9, 0.95, 1.0, 1.05)      # groupwise.py:241


def _h(x):
    return x.astype(np.float16).astype(np.float32)


def quant_sb6(w: np.ndarray, bits: int, search: bool = True, ex2: np.ndarray | None = None):
    """w [OUT, IN] float32, IN a multiple of 256 -> dict(q u8 [OUT, IN], qs u8 [OUT, IN/32],
    qm i8 [OUT, IN/32], d f16 [OUT, IN/256], dm f16 [OUT, IN/256], deq f32 [OUT, IN])."""
    f32 = np.float32
    w = np.ascontiguousarray(w, dtype=f32)
    OUT, IN = w.shape
    assert IN % 256 == 0
    gs, sb = 32, 8
    wg = w.reshape(OUT, IN // gs, gs)
    mn = wg.min(axis=2, keepdims=True)
    mx = wg.max(axis=2, keepdims=True)
    qmax = f32(2 ** bits - 1)
    scale = np.maximum((mx - mn) / qmax, f32(1e-8))
    evg = None
    if ex2 is not None:
        evg = np.maximum(np.asarray(ex2, dtype=f32), f32(1e-12)).reshape(1, IN // gs, gs)
    if search:
        best_s = best_m = best_e = None
        for f in FACTORS:
            sc = scale * f32(f)
            qq = np.clip(np.rint((wg - mn) / sc), 0, qmax)
            if evg is None:
                qm_ = qq.mean(axis=2, keepdims=True, dtype=f32)
                wm_ = wg.mean(axis=2, keepdims=True, dtype=f32)
                cov = ((qq - qm_) * (wg - wm_)).sum(axis=2, keepdims=True, dtype=f32)
                var = np.maximum(((qq - qm_) ** 2).sum(axis=2, keepdims=True, dtype=f32), f32(1e-12))
            else:
                wsum = evg.sum(axis=2, keepdims=True, dtype=f32)
                qm_ = (evg * qq).sum(axis=2, keepdims=True, dtype=f32) / wsum
                wm_ = (evg * wg).sum(axis=2, keepdims=True, dtype=f32) / wsum
                cov = (evg * (qq - qm_) * (wg - wm_)).sum(axis=2, keepdims=True, dtype=f32)
                var = np.maximum((evg * (qq - qm_) ** 2).sum(axis=2, keepdims=True, dtype=f32), f32(1e-12))
            s_ls = cov / var
            m_ls = wm_ - s_ls * qm_
            s_ls = np.where(s_ls > f32(1e-8), s_ls, sc)
            q2 = np.clip(np.rint((wg - m_ls) / s_ls), 0, qmax)
            e2 = (q2 * s_ls + m_ls - wg) ** 2
            err = (e2 if evg is None else evg * e2).sum(axis=2, keepdims=True, dtype=f32)
            if best_e is None:
                best_s, best_m, best_e = s_ls, m_ls, err
            else:
                b = err < best_e
                best_s = np.where(b, s_ls, best_s)
                best_m = np.where(b, m_ls, best_m)
                best_e = np.minimum(best_e, err)
        scale, mn = np.maximum(best_s, f32(1e-8)), best_m
    nb = IN // gs
    with np.errstate(divide="ignore", invalid="ignore"):      # fp16(1e-12) is 0: a constant-zero super-block divides by it, as in torch
        return _superblocks(wg, scale, mn, OUT, IN, nb, sb, qmax)


def _superblocks(wg, scale, mn, OUT, IN, nb, sb, qmax):
    f32 = np.float32
    ssb = scale.reshape(OUT, nb // sb, sb, 1)
    msb = mn.reshape(OUT, nb // sb, sb, 1)
    d = _h(np.maximum(ssb.max(axis=2, keepdims=True) / f32(63), f32(1e-12)))
    qs = np.clip(np.rint(ssb / d), 1, 63)
    dm = _h(np.maximum(np.abs(msb).max(axis=2, keepdims=True) / f32(31), f32(1e-12)))
    # an all-zero super-block has dm = fp16(1e-12) = 0 and the reference's 0 / 0 leaves NaN min codes
    # (and a NaN dequantised block); here, as in the CUDA kernel, such a block gets min code 0
    qm = np.clip(np.nan_to_num(np.rint(msb / dm), nan=0.0), -31, 31)
    s2 = np.maximum(_h((qs * d).reshape(OUT, nb, 1)), f32(1e-8))
    m2 = _h((qm * dm).reshape(OUT, nb, 1))
    qv = np.clip(np.rint((wg - m2) / s2), 0, qmax)
    deq = (qv * s2 + m2).reshape(OUT, IN)
    return {"q": qv.reshape(OUT, IN).astype(np.uint8), "qs": qs.reshape(OUT, nb).astype(np.uint8),
            "qm": qm.reshape(OUT, nb).astype(np.int8), "d": d.reshape(OUT, -1).astype(np.float16),
            "dm": dm.reshape(OUT, -1).astype(np.float16), "deq": deq.astype(np.float32)}


def unpack_sb6(codes_packed, qsqm, d, dm, *, shape, qh=None, qh2=None):
    """The (q, qs, qm) a packed sb6 tensor holds (inverse of the reference's packers,
    formats/writer.py:236-269), through the codec restatement of this package."""
    from . import codec_np as oc
    OUT, IN = shape
    q = oc.nibbles_blocklocal(np.asarray(codes_packed), 32).astype(np.uint8)
    if qh is not None:
        q = q | (oc.bitplane(np.asarray(qh), IN).astype(np.uint8) << 4)
    if qh2 is not None:
        q = q | (oc.bitplane(np.asarray(qh2), IN).astype(np.uint8) << 5)
    rec = np.asarray(qsqm).reshape(OUT, IN // 256, 12)
    qs = oc.sixbit_stream(rec[..., :6], 8).reshape(OUT, IN // 32).astype(np.uint8)
    qm = (oc.sixbit_stream(rec[..., 6:], 8).reshape(OUT, IN // 32).astype(np.int16) - 31).astype(np.int8)
    return q.reshape(OUT, IN), qs, qm


def quant_sym(w: np.ndarray, bits: int, factors, ex2: np.ndarray | None = None):
    """The symmetric layout (blocks of 16, super-blocks of 16 blocks): restates
    `calibration/groupwise.py:358-473` `_sym_one` without outliers.  `factors`: the float32 nodes the
    reference searches over (torch.linspace(0.7, 1.15, 19)) or (1.0,) for the plain mode.
    -> dict(q i8 [OUT, IN], qs i8 [OUT, IN/16], d f16 [OUT, IN/256], deq f32)."""
    f32 = np.float32
    w = np.ascontiguousarray(w, dtype=f32)
    OUT, IN = w.shape
    assert IN % 256 == 0
    gs, sb = 16, 16
    nb = IN // gs
    wg = w.reshape(OUT, nb, gs)
    evg = None if ex2 is None else np.maximum(np.asarray(ex2, dtype=f32), f32(1e-12)).reshape(1, nb, gs)
    qmax = f32(2 ** (bits - 1) - 1)
    qmin = -qmax - f32(1)
    base = np.maximum(np.abs(wg).max(axis=2, keepdims=True), f32(1e-12)) / qmax
    best_s, best_e = base.copy(), None
    for f in factors:
        s = base * f32(f)
        qv = np.clip(np.rint(wg / s), qmin, qmax)
        e = (wg - qv * s) ** 2
        err = (e if evg is None else evg * e).sum(axis=2, keepdims=True, dtype=f32)
        if best_e is None:
            best_s, best_e = s, err
        else:
            b = err < best_e
            best_s = np.where(b, s, best_s)
            best_e = np.minimum(best_e, err)
    with np.errstate(divide="ignore", invalid="ignore"):
        ssb = best_s.reshape(OUT, nb // sb, sb, 1)
        d = _h(np.maximum(ssb.max(axis=2, keepdims=True) / f32(127), f32(1e-12)))
        qs = np.clip(np.rint(ssb / d), -128, 127)
        scale_q = _h((qs * d).reshape(OUT, nb, 1))
        nz = np.abs(scale_q) > 0
        qv = np.clip(np.rint(wg / np.where(nz, scale_q, f32(1))), qmin, qmax)
        qv = np.where(nz, qv, f32(0))
    deq = (qv * scale_q).reshape(OUT, IN)
    return {"q": qv.reshape(OUT, IN).astype(np.int8), "qs": np.nan_to_num(qs, nan=0.0).reshape(OUT, nb).astype(np.int8),
            "d": d.reshape(OUT, -1).astype(np.float16), "deq": deq.astype(np.float32)}
