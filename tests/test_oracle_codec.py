"""The numpy oracle of the codec against the reference's vectors.

(1) packed buffers made by the reference's packers -> oracle dequant must hit the
    sha256 of the reference codec's output (tests/golden/codec_cases.npz);
(2) for the `known/` cases that digest is the reference's OWN known answer
    (tests/fixtures/gw_golden.json, synthetic gauss entries);
(3) where the reference is present, the oracle is compared live against
    formats/codec.py on fresh random tensors of every layout.
"""
import json
import os

import numpy as np
import pytest

from conftest import GOLDEN
from helpers import digest_f32, oracle_dequant_case
from oracle import codec_np as oc


def test_golden_codec_cases_bit_exact(codec_cases):
    assert len(codec_cases) >= 19
    for name, (meta, bufs, sample) in codec_cases.items():
        w = oracle_dequant_case(meta, bufs)
        assert w.dtype == np.float32 and w.shape == tuple(meta["shape"])
        step = max(1, w.size // 257)
        np.testing.assert_array_equal(w.reshape(-1)[::step][:257], sample, err_msg=name)
        assert digest_f32(w) == meta["digest"], name


def test_config1_reference_packed(config1_case):
    """The single-GEMV configuration (W [8192, 2048] int4 g32, packed by the reference's
    asym_sb6_search packer): 9 437 184 packed bytes, oracle dequant hits the reference codec's
    digest, and the oracle's matvec reproduces the reference's y."""
    meta, bufs, x, y = config1_case
    assert (meta["kind"], meta["bits"], meta["shape"]) == ("sb6", 4, [8192, 2048])
    assert sum(a.nbytes for a in bufs.values()) == 9437184
    w = oracle_dequant_case(meta, bufs)
    assert digest_f32(w) == meta["digest"]
    np.testing.assert_allclose(x.astype(np.float32) @ w.T, y, rtol=0, atol=1e-5 * np.abs(y).max())


def test_reference_known_answers(codec_cases):
    """digest(oracle(packed)) == the hash the reference froze for its quantiser."""
    known = json.load(open(os.path.join(GOLDEN, "gw_known_answers.json")))["hashes"]
    assert len(known) >= 6
    for key, want in known.items():
        _, mode, bits = key.split("|")
        meta, bufs, _ = codec_cases[f"known/{mode}/{bits}"]
        assert digest_f32(oracle_dequant_case(meta, bufs)) == want, key


def test_layout_sizes(codec_cases):
    """bits per weight of the file layouts: sb6 bits+0.5, sym bits+0.5625."""
    for name, (meta, bufs, _) in codec_cases.items():
        n = meta["shape"][0] * meta["shape"][1]
        nbytes = sum(a.nbytes for a in bufs.values())
        if meta["kind"] == "sb6":
            assert nbytes * 8 / n == meta["bits"] + 0.5, name
        if meta["kind"] == "sym":
            assert nbytes * 8 / n == meta["bits"] + 0.5625, name


def test_bit_unpackers_roundtrip():
    rng = np.random.default_rng(1)
    from rwkv_quant_b200 import synth
    import torch
    q = rng.integers(0, 16, (5, 128), dtype=np.uint8)
    for gs in (16, 32):
        p = synth.pack_nibbles_blocklocal(torch.from_numpy(q), gs).numpy()
        np.testing.assert_array_equal(oc.nibbles_blocklocal(p, gs), q)
    b = rng.integers(0, 2, (5, 128), dtype=np.uint8)
    np.testing.assert_array_equal(oc.bitplane(synth.pack_bitplane(torch.from_numpy(b)).numpy(), 128), b)
    v = rng.integers(0, 64, (5, 3, 8), dtype=np.uint8)
    np.testing.assert_array_equal(oc.sixbit_stream(synth.pack_6bit(torch.from_numpy(v)).numpy(), 8), v)
    c = rng.integers(-8, 8, (5, 65), dtype=np.int8)
    np.testing.assert_array_equal(
        oc.nibbles_split_biased(synth.pack_nibbles_split_biased(torch.from_numpy(c)).numpy(), 65), c)


def test_bf16_rounding_matches_torch():
    import torch
    x = np.random.default_rng(0).standard_normal(4096).astype(np.float32) * 0.02
    np.testing.assert_array_equal(oc.f32_to_bf16_rne(x),
                                  torch.from_numpy(x).bfloat16().float().numpy())


def test_oracle_matches_reference_codec_live(reference):
    import torch
    from rwkv_quant.calibration.group_config import QuantConfig
    from rwkv_quant.formats import codec as rc
    from rwkv_quant.formats.writer import quantize_tensor
    torch.manual_seed(123)
    n = lambda t: None if t is None else t.numpy()
    cases = [("blocks.0.ffn.key.weight", (32, 512), QuantConfig(cmix=b, group_scale={"cmix": 32},
              group_scale_mode={"cmix": m})) for b in (4, 5, 6) for m in ("asym_sb6", "asym_sb6_search")]
    cases += [("blocks.0.ffn.key.weight", (32, 512), QuantConfig(cmix=b, group_scale={"cmix": 16},
               group_scale_mode={"cmix": "sym"})) for b in (6, 8)]
    cases += [("blocks.0.att.w1", (300, 96), QuantConfig(w_lora=6, group_scale={"w_lora": 64})),
              ("blocks.0.att.g1", (64, 33), QuantConfig(g_lora=4)),
              ("blocks.0.att.g1", (64, 33), QuantConfig(g_lora=8))]
    for key, shape, cfg in cases:
        qt = quantize_tensor(key, torch.randn(*shape) * 0.02, cfg, real_gw=True)
        kind = qt.gw_mode or "rtn"
        if kind == "sb6":
            a = rc.dequant_sb6(n(qt.codes_packed), n(qt.gw_qsqm), n(qt.gw_d), n(qt.gw_dm), shape=qt.shape,
                               gs=32, sb=8, qh=n(qt.gw_qh), qh2=n(qt.gw_qh2))
            b = oc.dequant_sb6(n(qt.codes_packed), n(qt.gw_qsqm), n(qt.gw_d), n(qt.gw_dm), shape=qt.shape,
                               qh=n(qt.gw_qh), qh2=n(qt.gw_qh2))
        elif kind == "sym":
            kw = dict(shape=qt.shape, gs=16, sb=16, codes=n(qt.codes), codes_packed=n(qt.codes_packed),
                      qh=n(qt.gw_qh), qh2=n(qt.gw_qh2))
            a = rc.dequant_sym(n(qt.gw_qs), n(qt.gw_d), **kw)
            b = oc.dequant_sym(n(qt.gw_qs), n(qt.gw_d), **kw)
        elif kind == "asym":
            a = rc.dequant_asym(n(qt.codes), n(qt.gw_scale), n(qt.gw_min), shape=qt.shape, gs=64)
            b = oc.dequant_asym(n(qt.codes), n(qt.gw_scale), n(qt.gw_min), shape=qt.shape, gs=64)
        else:
            a = rc.dequant_rtn(n(qt.scale), shape=qt.shape, codes=n(qt.codes), codes_packed=n(qt.codes_packed))
            b = oc.dequant_rtn(n(qt.scale), shape=qt.shape, codes=n(qt.codes), codes_packed=n(qt.codes_packed))
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32)), (key, kind, qt.bits)
