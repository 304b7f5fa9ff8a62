"""Sharding of a checkpoint for the head-sharded tensor-parallel model (rwkv_quant_b200/tp_model.py):
row and column ranges of every layout decode (CPU oracle codec) to the same values as the range of
the whole tensor, and the shards of all ranks together cover every tensor exactly once."""
import numpy as np
import pytest
import torch

from oracle import codec_np as oc
from rwkv_quant_b200 import synth, tp_model


def _deq(qt):
    f = lambda t: None if t is None else t.cpu().numpy()
    if qt.kind == "dense":
        return qt.dense.float().cpu().numpy()
    if qt.kind == "sb6":
        return oc.dequant_sb6(f(qt.codes_packed), f(qt.gw_qsqm).reshape(qt.shape[0], -1, 12), f(qt.gw_d), f(qt.gw_dm),
                              shape=tuple(qt.shape), qh=f(qt.gw_qh), qh2=f(qt.gw_qh2))
    if qt.kind == "sym":
        return oc.dequant_sym(f(qt.gw_qs), f(qt.gw_d), shape=tuple(qt.shape), codes=f(qt.codes), codes_packed=f(qt.codes_packed),
                              qh=f(qt.gw_qh), qh2=f(qt.gw_qh2))
    if qt.kind == "asym":
        return oc.dequant_asym(f(qt.codes), f(qt.gw_scale), f(qt.gw_min), shape=tuple(qt.shape), gs=qt.gw_gs)
    return oc.dequant_rtn(f(qt.scale), shape=tuple(qt.shape), codes=f(qt.codes), codes_packed=f(qt.codes_packed))


@pytest.mark.parametrize("maker,bits", [(synth.quant_sb6, 4), (synth.quant_sb6, 5), (synth.quant_sb6, 6), (synth.quant_sym, 6),
                                        (synth.quant_sym, 8), (synth.quant_rtn, 8)])
def test_row_and_column_ranges_decode_like_the_whole_tensor(maker, bits):
    w = torch.randn(96, 1024, generator=torch.Generator().manual_seed(bits)) * 0.05
    qt = maker("blocks.0.att.output.weight", "proj", w, bits)
    full = _deq(qt)
    assert np.array_equal(_deq(tp_model.slice_rows(qt, 32, 80)), full[32:80])
    assert np.array_equal(_deq(tp_model.slice_cols(qt, 256, 768)), full[:, 256:768])
    if qt.kind in ("sb6", "sym"):
        with pytest.raises(ValueError):
            tp_model.slice_cols(qt, 128, 512)


def test_asym_column_ranges():
    w = torch.randn(96, 640, generator=torch.Generator().manual_seed(1)) * 0.05
    qt = synth.quant_asym("blocks.1.att.w2", "lora", w, 8)
    full = _deq(qt)
    assert np.array_equal(_deq(tp_model.slice_cols(qt, 320, 640)), full[:, 320:640])
    assert np.array_equal(_deq(tp_model.slice_rows(qt, 10, 50)), full[10:50])


@pytest.mark.parametrize("recipe", ["compression", "reduction"])
def test_shards_cover_the_checkpoint(recipe):
    ck = synth.build_checkpoint("1.5b", recipe, seed=3, n_layer=2, n_embd=512, ffn=2048, vocab=1024)
    world = 2
    shards = [tp_model.shard_checkpoint(ck, r, world) for r in range(world)]
    D, H = 512, 8
    for key, qt in ck.tensors.items():
        full = _deq(qt)
        parts = [_deq(s.tensors[key]) for s in shards]
        rows_split = (".att." in key and key.endswith(("receptance.weight", "key.weight", "value.weight"))) or \
            key.endswith("ffn.key.weight") or key == "head.weight"
        if rows_split:
            assert np.array_equal(np.concatenate(parts, 0), full), key
        elif key.endswith(("output.weight", "ffn.value.weight", ".w2", ".a2", ".g2", ".v2")):
            assert np.array_equal(np.concatenate(parts, 1), full), key
        elif ".att." in key and key.split(".")[-1] in ("w0", "a0", "v0", "k_k", "k_a") or "ln_x" in key:
            assert np.array_equal(np.concatenate([p.reshape(-1) for p in parts]), full.reshape(-1)), key
        elif key.endswith("r_k"):
            assert np.array_equal(np.concatenate(parts, 0), full.reshape(H, -1)), key
        else:
            for p in parts:
                assert np.array_equal(p, full), key
    with pytest.raises(ValueError):
        tp_model.shard_checkpoint(ck, 0, 3)
