"""Shared helpers of the test-suite."""
import hashlib

import numpy as np
import torch

from oracle import codec_np as oc


def digest_f32(a) -> str:
    """sha256 over shape, dtype tag and raw bytes of a float32 array: the digest
    format of the reference's known-answer file (tests/make_gw_golden.py:55-62)."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    h = hashlib.sha256()
    h.update(str(tuple(a.shape)).encode())
    h.update(b"torch.float32")
    h.update(a.tobytes())
    return h.hexdigest()


def oracle_dequant_case(meta, bufs):
    kind, shape = meta["kind"], tuple(meta["shape"])
    g = bufs.get
    if kind == "sb6":
        return oc.dequant_sb6(g("codes_packed"), g("gw_qsqm"), g("gw_d"), g("gw_dm"), shape=shape,
                              gs=meta["gs"], sb=meta["sb"], qh=g("gw_qh"), qh2=g("gw_qh2"))
    if kind == "sym":
        return oc.dequant_sym(g("gw_qs"), g("gw_d"), shape=shape, gs=meta["gs"], sb=meta["sb"],
                              codes=g("codes"), codes_packed=g("codes_packed"),
                              qh=g("gw_qh"), qh2=g("gw_qh2"))
    if kind == "asym":
        return oc.dequant_asym(g("codes"), g("gw_scale"), g("gw_min"), shape=shape, gs=meta["gs"])
    ov = g("outlier_values")
    return oc.dequant_rtn(g("scale"), shape=shape, codes=g("codes"), codes_packed=g("codes_packed"),
                          outlier_indices=g("outlier_indices"),
                          outlier_values=None if ov is None else oc.bf16_bits_to_f32(ov))


def case_to_qt(name, meta, bufs):
    """A golden codec case as this package's QuantizedTensor (CPU tensors)."""
    from rwkv_quant_b200.formats.container import QuantizedTensor
    kind = meta["kind"]
    qt = QuantizedTensor(key=name, group="", bits=meta["bits"], shape=tuple(meta["shape"]),
                         gw_mode=kind if kind != "rtn" else "", gw_gs=meta["gs"], gw_sb=meta["sb"])
    for f, a in bufs.items():
        t = torch.from_numpy(np.array(a))
        if f == "outlier_values":
            t = t.view(torch.bfloat16)
        setattr(qt, f, t)
    return qt


def relmax(y, ref) -> float:
    """max|y - ref| / max|ref|: the error measure of the reference's kernel gates
    (tests/test_gw_kernel.py:21-29)."""
    y = np.asarray(y, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.abs(y - ref).max() / max(np.abs(ref).max(), 1e-30))
