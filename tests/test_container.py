"""``.rwkvq`` container: files written by the reference load here, files written
here load in the reference, manifests carry the documented fields, and foreign or
future containers are refused with ValueError (formats/reader.py:64-73)."""
import json
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN
from oracle import codec_np as oc
from rwkv_quant_b200 import synth
from rwkv_quant_b200.formats import container


@pytest.mark.parametrize("preset", ["reduction", "compression"])
def test_reads_reference_written_file(preset):
    path = os.path.join(GOLDEN, f"toy_{preset}.rwkvq")
    ck = container.load_raw(path)
    assert (ck.naming, ck.n_layer, ck.n_embd, ck.head_size, ck.vocab_size) == ("world", 2, 256, 64, 512)
    man, arr = oc.open_rwkvq(path)
    assert set(ck.tensors) == set(man["tensors"])
    kinds = {qt.kind for qt in ck.tensors.values()}
    assert kinds == ({"sym", "asym", "rtn", "dense"} if preset == "reduction"
                     else {"sb6", "asym", "rtn", "dense"})
    for key, qt in ck.tensors.items():
        m = man["tensors"][key]
        assert tuple(m["shape"]) == qt.shape and m["bits"] == qt.bits
        assert qt.transposed == oc.is_transposed(man, key)
        for f in m["fields"]:
            a = getattr(qt, f)
            b = arr[f"{key}::{f}"]
            a = a.view(torch.uint16).numpy() if a.dtype == torch.bfloat16 else a.numpy()
            np.testing.assert_array_equal(a.reshape(b.shape), b)
    w1 = ck.tensors["blocks.1.att.w1"]
    assert w1.transposed and w1.gw_scale.shape[-1] == -(-w1.shape[1] // w1.gw_gs)
    # bits per weight from real buffer sizes
    k = ck.tensors["blocks.0.ffn.key.weight"]
    bpw = k.nbytes() * 8 / (k.shape[0] * k.shape[1])
    assert bpw == (6.5625 if preset == "reduction" else 4.5)


@pytest.mark.parametrize("recipe", sorted(synth.RECIPES))
def test_roundtrip_own_writer(tmp_path, recipe):
    ck = synth.build_checkpoint("toy", recipe, seed=3)
    p = str(tmp_path / "m.rwkvq")
    container.save_rwkvq(ck, p)
    ck2 = container.load_raw(p)
    assert set(ck2.tensors) == set(ck.tensors)
    for key, qt in ck.tensors.items():
        qt2 = ck2.tensors[key]
        assert (qt2.kind, qt2.bits, qt2.shape, qt2.gw_gs, qt2.gw_sb) == \
               (qt.kind, qt.bits, qt.shape, qt.gw_gs, qt.gw_sb)
        for f in container.TENSOR_FIELDS:
            a, b = getattr(qt, f), getattr(qt2, f)
            assert (a is None) == (b is None), (key, f)
            if a is not None:
                assert torch.equal(a.reshape(b.shape), b), (key, f)
    man, arr = oc.open_rwkvq(p)
    w = oc.dequant_key(man, arr, "blocks.1.ffn.key.weight")
    assert w.shape == (1024, 256) and np.isfinite(w).all() and 0.01 < w.std() < 0.03


def test_reference_reads_our_file(reference, tmp_path):
    from rwkv_quant.formats import codec as rc, reader as rr
    for recipe in ("reduction", "compression"):
        ck = synth.build_checkpoint("toy", recipe, seed=4)
        p = str(tmp_path / f"{recipe}.rwkvq")
        container.save_rwkvq(ck, p)
        man, arr = rc.open_rwkvq(p)
        man2, arr2 = oc.open_rwkvq(p)
        rck = rr.load_raw(p)
        assert rck.n_layer == 2 and rck.naming == "world"
        for key in man["tensors"]:
            a = rc.dequant_key(man, arr, key)
            b = oc.dequant_key(man2, arr2, key)
            assert np.array_equal(a.reshape(-1).view(np.uint32), b.reshape(-1).view(np.uint32)), key
            c = rr._dequantize_one(rck.tensors[key]).float().numpy()
            np.testing.assert_array_equal(oc.f32_to_bf16_rne(a).reshape(c.shape), c)


def _rewrite_manifest(src, dst, edit, drop=False):
    raw = open(src, "rb").read()
    n = int.from_bytes(raw[:8], "little")
    header = json.loads(raw[8:8 + n])
    man = json.loads(header["__metadata__"]["rwkvq"])
    edit(man, header)
    header["__metadata__"]["rwkvq"] = json.dumps(man)
    if drop:
        del header["__metadata__"]["rwkvq"]
    hj = json.dumps(header).encode()
    open(dst, "wb").write(len(hj).to_bytes(8, "little") + hj + raw[8 + n:])


def test_rejects_foreign_and_future(tmp_path):
    src = os.path.join(GOLDEN, "toy_compression.rwkvq")
    p = str(tmp_path / "x.rwkvq")
    _rewrite_manifest(src, p, lambda m, h: m.__setitem__("format_version", 3))
    with pytest.raises(ValueError):
        container.load_raw(p)
    _rewrite_manifest(src, p, lambda m, h: m.__setitem__("format", "gguf"))
    with pytest.raises(ValueError):
        container.load_raw(p)
    _rewrite_manifest(src, p, lambda m, h: None, drop=True)
    with pytest.raises(ValueError):
        container.load_raw(p)
    open(p, "wb").write(b"PK\x03\x04" + b"\0" * 64)
    with pytest.raises(ValueError):
        container.load_raw(p)
    # version-1 manifests (no n_blocks / transposed) stay readable
    def v1(m, h):
        m["format_version"] = 1
        for t in m["tensors"].values():
            t.pop("transposed", None)
            t.pop("n_blocks", None)
    _rewrite_manifest(src, p, v1)
    ck = container.load_raw(p)
    assert ck.tensors["blocks.0.att.w1"].transposed and not ck.tensors["head.weight"].transposed


def test_rejects_buffers_that_do_not_fit_the_manifest_shape(tmp_path):
    """A manifest whose shape is larger than its buffers, a short side buffer, or a sparse
    override outside the tensor is refused on the host (ValueError), by the reader and by the
    device-side tensor view alike: the kernels' descriptors carry no buffer sizes."""
    src = os.path.join(GOLDEN, "toy_compression.rwkvq")
    p = str(tmp_path / "x.rwkvq")
    def grow_rows(m, h):
        m["tensors"]["blocks.0.ffn.key.weight"]["shape"][0] += 16
    _rewrite_manifest(src, p, grow_rows)
    with pytest.raises(ValueError, match="codes_packed"):
        container.load_raw(p)
    def wrong_bits(m, h):                      # 5-bit layout whose plane buffer is not listed
        t = m["tensors"]["blocks.0.att.key.weight"]
        t["fields"] = [f for f in t["fields"] if f != "gw_qh"]
    _rewrite_manifest(src, p, wrong_bits)
    with pytest.raises(ValueError, match="gw_qh"):
        container.load_raw(p)
    def grow_lora(m, h):
        m["tensors"]["blocks.1.att.w1"]["shape"][1] += 64      # one more block than gw_scale holds
    _rewrite_manifest(src, p, grow_lora)
    with pytest.raises(ValueError):
        container.load_raw(p)
    # the in-memory objects are checked too (no file involved)
    qt = synth.quant_sb6("w", "g", torch.randn(32, 512) * 0.02, 5)
    container.check_tensor_sizes(qt)
    qt.gw_d = qt.gw_d[:-1]
    with pytest.raises(ValueError, match="gw_d"):
        container.check_tensor_sizes(qt)
    qt = synth.quant_rtn("w", "g", torch.randn(32, 64) * 0.02, 8)
    qt.outlier_indices = torch.tensor([[3, 5], [32, 0]], dtype=torch.int32)
    qt.outlier_values = torch.zeros(2, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="outside"):
        container.check_tensor_sizes(qt)
    qt.outlier_indices = torch.tensor([[3, 5], [31, 63]], dtype=torch.int32)
    container.check_tensor_sizes(qt)
    from rwkv_quant_b200.backends.cuda import ops
    qt.outlier_indices = torch.tensor([[3, 64]], dtype=torch.int32)
    qt.outlier_values = torch.zeros(1, dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        ops.DeviceQT(qt, device="cpu", relayout=False)


def test_weight_bytes_of_full_size_recipes():
    """Per-token streamed bytes of the 1.5B builds from the layout arithmetic:
    about 876 MB (compression) and 1289 MB (reduction) without the embedding."""
    D, F, V, L = 2048, 8192, 65536, 24
    r = synth.lora_ranks(D)
    assert r == {"w": 96, "a": 96, "v": 64, "g": 256}
    lora = 2 * D * (r["w"] + r["a"] + r["v"]) * 9 / 8 + 2 * D * r["g"] + 2 * (D + r["g"])
    comp = L * (4 * D * D * 5.5 / 8 + 2 * D * F * 4.5 / 8 + lora) + V * D * 5.5 / 8
    red = L * (4 * D * D * 8.5625 / 8 + 2 * D * F * 6.5625 / 8 + lora) + V * D * 8.5625 / 8
    assert 870e6 < comp < 885e6 and 1280e6 < red < 1300e6
