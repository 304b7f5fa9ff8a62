"""Generate the golden fixtures of this directory from the UNMODIFIED reference.

    python tests/golden/make_golden.py [/path/to/reference] [all|codec|toy|custom|config1]

Needs the reference project importable (default: a `reference` directory beside this
repository, or $RWKVQ_REFERENCE); the fixtures
it writes are committed so that the tests run where the reference is absent.

  codec_cases.npz      packed buffers made by the reference's packers
                       (formats/writer.py quantize_tensor) for every layout,
                       with the sha256 digest of the reference numpy codec's
                       dequantised fp32 output (formats/codec.py)
  gw_known_answers.json  the subset of the reference's own known-answer file
                       tests/fixtures/gw_golden.json that a packed layout exists
                       for: digest(fake-dequant) which packer -> dequant must
                       reproduce (the claim of tests/test_groupwise_parity.py:82-115)
  config1_gemv.npz     W [8192, 2048] = randn(seed 0) * 0.02 packed by quantize_tensor with
                       cmix = 4, group 32, asym_sb6_search (the single-GEMV benchmark
                       configuration), the codec digest of its dequantised form, x fp16
                       [1, 2048] = default_rng(0).standard_normal and y = x.f32 @ Wdq.T
  toy_<preset>.rwkvq   2-layer D=256 world-naming random-init model quantized by
                       rwkv_quant.quantize() with both presets
  toy_<preset>_ref.npz token ids, RWKV7Ref (cpu, fp32) logits on the dequantised
                       state dict, residual-stream trace
  toy_custom_<cfg>.rwkvq / _ref.npz  the same model under custom naming, written by the
                       reference's writer.save(); RWKV7Ref logits
"""
import hashlib
import json
import os
import sys
import zlib

import numpy as np
import torch

HERE_ = os.path.dirname(os.path.abspath(__file__))
REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get(
    "RWKVQ_REFERENCE", os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(HERE_))), "reference"))
sys.path.insert(0, REF)
HERE = os.path.dirname(os.path.abspath(__file__))

from rwkv_quant import quantize  # noqa: E402
from rwkv_quant.calibration.group_config import QuantConfig  # noqa: E402
from rwkv_quant.formats import codec, reader  # noqa: E402
from rwkv_quant.formats.writer import (_make_qt_gw_sb6, _make_qt_gw_sym,  # noqa: E402
                                       quantize_tensor)
from rwkv_quant.models.rwkv7_ref import RWKV7Ref  # noqa: E402
from rwkv_quant.presets import PRESETS  # noqa: E402

FIELDS = ("codes", "codes_packed", "scale", "gw_d", "gw_dm", "gw_qsqm", "gw_qh", "gw_qh2",
          "gw_scale", "gw_min", "gw_qs", "outlier_indices", "outlier_values")


def digest_f32(a: np.ndarray) -> str:
    """Same digest as tests/make_gw_golden.py:55-62 for a float32 torch tensor."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    h = hashlib.sha256()
    h.update(str(tuple(a.shape)).encode())
    h.update(b"torch.float32")
    h.update(a.tobytes())
    return h.hexdigest()


def to_np(t):
    if t is None:
        return None
    if t.dtype == torch.bfloat16:
        return t.view(torch.uint16).numpy()
    return t.numpy()


def ref_dequant(qt):
    kind = qt.gw_mode or "rtn"
    n = to_np
    if kind == "sb6":
        return codec.dequant_sb6(n(qt.codes_packed), n(qt.gw_qsqm), n(qt.gw_d), n(qt.gw_dm),
                                 shape=qt.shape, gs=qt.gw_gs, sb=qt.gw_sb, qh=n(qt.gw_qh), qh2=n(qt.gw_qh2))
    if kind == "sym":
        return codec.dequant_sym(n(qt.gw_qs), n(qt.gw_d), shape=qt.shape, gs=qt.gw_gs, sb=qt.gw_sb,
                                 codes=n(qt.codes), codes_packed=n(qt.codes_packed),
                                 qh=n(qt.gw_qh), qh2=n(qt.gw_qh2))
    if kind == "asym":
        return codec.dequant_asym(n(qt.codes), n(qt.gw_scale), n(qt.gw_min), shape=qt.shape, gs=qt.gw_gs)
    ov = qt.outlier_values
    return codec.dequant_rtn(n(qt.scale), shape=qt.shape, codes=n(qt.codes), codes_packed=n(qt.codes_packed),
                             outlier_indices=n(qt.outlier_indices),
                             outlier_values=None if ov is None else codec.bf16_to_f32(n(ov)))


def add_case(store, meta, name, qt, expect_digest=None):
    deq = ref_dequant(qt)
    dg = digest_f32(deq)
    if expect_digest is not None:
        assert dg == expect_digest, f"{name}: reference packer -> codec does not hit the known answer"
    meta[name] = {"kind": qt.gw_mode or "rtn", "bits": int(qt.bits), "shape": list(qt.shape),
                  "gs": int(qt.gw_gs), "sb": int(qt.gw_sb), "digest": dg,
                  "fields": [f for f in FIELDS if getattr(qt, f, None) is not None
                             and getattr(qt, f).numel() > 0]}
    for f in meta[name]["fields"]:
        store[f"{name}::{f}"] = to_np(getattr(qt, f))
    # a few raw values so that a failing digest can be localised
    store[f"{name}::sample"] = deq.reshape(-1)[:: max(1, deq.size // 257)][:257].copy()


def make_codec_cases():
    store, meta = {}, {}
    known = json.load(open(os.path.join(REF, "tests/fixtures/gw_golden.json")))["hashes"]
    kept = {}
    # -- the reference's own known answers (synthetic gauss, seed 20260810)
    g = torch.Generator().manual_seed(20260810)
    w = torch.randn(128, 512, generator=g)
    for bits in (4, 5, 6):
        for mode, search in (("asym_sb6", False), ("asym_sb6_search", True)):
            key = f"synth::gauss|{mode}|{bits}"
            qt = _make_qt_gw_sb6("k", "cmix", bits, w, 32, None, search=search)
            try:
                add_case(store, meta, f"known/{mode}/{bits}", qt, known[key])
                kept[key] = known[key]
            except AssertionError as e:      # platform float differences: see the reference's own notes
                print("skip", e)
    # The sym known answers hash the quantiser's fake-dequant tensor, which holds
    # negative zeros (round(-0.3) * s); a packed int8 code 0 dequantises to +0.0,
    # so packer -> codec is value-equal but not digest-equal and these are skipped.
    for mode, search in (("sym", True), ("sym_plain", False)):
        key = f"synth::gauss|{mode}|6"
        qt = _make_qt_gw_sym("k", "cmix", 6, w, 16, 16, None, search=search)
        try:
            add_case(store, meta, f"known/{mode}/6", qt, known[key])
            kept[key] = known[key]
        except AssertionError as e:
            print("skip", e)
    json.dump({"source": "tests/fixtures/gw_golden.json of the reference", "hashes": kept},
              open(os.path.join(HERE, "gw_known_answers.json"), "w"), indent=1, sort_keys=True)

    # -- every layout through quantize_tensor, N(0, 0.02) weights, crc32 seeds
    def W(name, *shape, std=0.02):
        gg = torch.Generator().manual_seed(zlib.crc32(name.encode()) & 0x7FFFFFFF)
        return torch.randn(*shape, generator=gg) * std

    for bits in (4, 5, 6):
        cfg = QuantConfig(cmix=bits, group_scale={"cmix": 32}, group_scale_mode={"cmix": "asym_sb6_search"})
        add_case(store, meta, f"sb6/{bits}", quantize_tensor("blocks.0.ffn.key.weight", W(f"sb6{bits}", 48, 768), cfg, real_gw=True))
    for bits in (6, 8):
        cfg = QuantConfig(cmix=bits, group_scale={"cmix": 16}, group_scale_mode={"cmix": "sym"})
        add_case(store, meta, f"sym/{bits}", quantize_tensor("blocks.0.ffn.key.weight", W(f"sym{bits}", 48, 768), cfg, real_gw=True))
    # degenerate rows: all-zero row (sym scale 0), constant row (sb6 scale clamp)
    wz = W("degenerate", 16, 512)
    wz[3] = 0.0
    wz[5] = 1e-9
    wz[7] = 0.25
    cfg = QuantConfig(cmix=4, group_scale={"cmix": 32}, group_scale_mode={"cmix": "asym_sb6"})
    add_case(store, meta, "sb6/degenerate", quantize_tensor("blocks.0.ffn.key.weight", wz, cfg, real_gw=True))
    cfg = QuantConfig(cmix=8, group_scale={"cmix": 16}, group_scale_mode={"cmix": "sym"})
    add_case(store, meta, "sym/degenerate", quantize_tensor("blocks.0.ffn.key.weight", wz, cfg, real_gw=True))
    # LoRA: asym@6 gs64, ragged [2048-like, 96] and its partner; stored [in, out]
    cfg = QuantConfig(w_lora=6, group_scale={"w_lora": 64})
    add_case(store, meta, "asym/ragged", quantize_tensor("blocks.1.att.w1", W("w1", 512, 96), cfg, real_gw=True))
    add_case(store, meta, "asym/wide", quantize_tensor("blocks.1.att.w2", W("w2", 96, 512), cfg, real_gw=True))
    # per-row: int8, packed nibbles with odd column count
    add_case(store, meta, "rtn/8", quantize_tensor("blocks.1.att.g1", W("g1", 512, 64), QuantConfig(g_lora=8), real_gw=True))
    add_case(store, meta, "rtn/8wide", quantize_tensor("blocks.1.att.g2", W("g2", 64, 512), QuantConfig(g_lora=8), real_gw=True))
    add_case(store, meta, "rtn/4odd", quantize_tensor("blocks.1.att.g1", W("g1o", 40, 65), QuantConfig(g_lora=4), real_gw=True))
    add_case(store, meta, "rtn/8lin", quantize_tensor("blocks.0.att.key.weight", W("rl", 48, 256), QuantConfig(proj=8), real_gw=True))
    # per-row int8 with sparse outlier overrides (2 % of the columns of every row)
    add_case(store, meta, "rtn/8outliers", quantize_tensor("blocks.1.att.g1", W("g1x", 96, 256),
                                                            QuantConfig(g_lora=8, outlier_fracs={"g_lora": 0.02}), real_gw=True))
    store["__meta__"] = np.frombuffer(json.dumps(meta).encode(), dtype=np.uint8)
    np.savez_compressed(os.path.join(HERE, "codec_cases.npz"), **store)
    print("codec cases:", len(meta))


def make_config1():
    """The single-GEMV configuration, packed by the reference's search packer."""
    w = torch.randn(8192, 2048, generator=torch.Generator().manual_seed(0)) * 0.02
    cfg = QuantConfig(cmix=4, group_scale={"cmix": 32}, group_scale_mode={"cmix": "asym_sb6_search"},
                      act_stats_path=None)
    qt = quantize_tensor("blocks.0.ffn.key.weight", w, cfg, real_gw=True)
    store, meta = {}, {}
    add_case(store, meta, "config1", qt)
    deq = ref_dequant(qt)
    x = np.random.default_rng(0).standard_normal((1, 2048)).astype(np.float16)
    store["x"] = x
    store["y"] = (x.astype(np.float32) @ deq.T).astype(np.float32)
    store["__meta__"] = np.frombuffer(json.dumps(meta).encode(), dtype=np.uint8)
    path = os.path.join(HERE, "config1_gemv.npz")
    np.savez_compressed(path, **store)
    nbytes = sum(store[f"config1::{f}"].nbytes for f in meta["config1"]["fields"])
    print("config 1:", meta["config1"]["kind"], meta["config1"]["bits"], nbytes, "packed bytes;",
          os.path.getsize(path), "bytes on disk")


# ---------------------------------------------------------------- toy model
def lora_ranks(d):
    f = lambda c, p: max(32, int(round((c * (d ** p)) / 32) * 32))
    return {"w": f(1.8, 0.5), "a": f(1.8, 0.5), "v": f(1.3, 0.5), "g": f(0.6, 0.8)}


def toy_world_state_dict(L=2, D=256, V=512, S=64, seed=0):
    """World-naming shapes (tests_local/build_world_ckpt_v2.py:42-74) with the
    value distributions of tests/test_quant_parity.py:44-94."""
    g = torch.Generator().manual_seed(seed)
    H, r = D // S, lora_ranks(D)
    rn = lambda *s, std=0.02: torch.randn(*s, generator=g) * std
    ru = lambda *s, lo=0.0, hi=1.0: torch.rand(*s, generator=g) * (hi - lo) + lo
    sd = {"emb.weight": rn(V, D), "blocks.0.ln0.weight": torch.ones(D), "blocks.0.ln0.bias": torch.zeros(D)}
    for i in range(L):
        p = f"blocks.{i}."
        for ln in ("ln1", "ln2"):
            sd[p + ln + ".weight"] = 1 + rn(D, std=0.1)
            sd[p + ln + ".bias"] = rn(D, std=0.1)
        a = p + "att."
        for nm in ("x_r", "x_w", "x_k", "x_v", "x_a", "x_g"):
            sd[a + nm] = ru(1, 1, D, lo=0.2, hi=0.8)
        for br in ("w", "a", "v"):
            sd[a + br + "0"] = rn(1, 1, D, std=0.1)
            sd[a + br + "1"] = rn(D, r[br])
            sd[a + br + "2"] = rn(r[br], D)
        sd[a + "g1"] = rn(D, r["g"])
        sd[a + "g2"] = rn(r["g"], D)
        sd[a + "k_k"] = ru(1, 1, D, lo=0.5, hi=1.0)
        sd[a + "k_a"] = ru(1, 1, D, lo=0.0, hi=0.5)
        sd[a + "r_k"] = rn(H, S, std=0.1)
        for nm in ("receptance", "key", "value", "output"):
            sd[a + nm + ".weight"] = rn(D, D)
        sd[a + "ln_x.weight"] = 1 + rn(D, std=0.1)
        sd[a + "ln_x.bias"] = rn(D, std=0.1)
        f = p + "ffn."
        sd[f + "x_k"] = ru(1, 1, D, lo=0.2, hi=0.8)
        sd[f + "key.weight"] = rn(4 * D, D)
        sd[f + "value.weight"] = rn(D, 4 * D)
    sd["ln_out.weight"] = 1 + rn(D, std=0.1)
    sd["ln_out.bias"] = rn(D, std=0.1)
    sd["head.weight"] = rn(V, D)
    return sd


def make_toy_models():
    sd = toy_world_state_dict()
    pth = "/tmp/rwkvq_toy_world.pth"
    torch.save(sd, pth)
    idx = torch.from_numpy(np.random.default_rng(0).integers(1, 500, (2, 24)))
    for preset in ("reduction", "compression"):
        cfg = PRESETS[preset]
        cfg.act_stats_path = None      # deterministic: no activation statistics file
        out = os.path.join(HERE, f"toy_{preset}.rwkvq")
        quantize(pth, out, config=cfg)
        deq = reader.load_dequantized(out)
        dq_pth = f"/tmp/rwkvq_toy_{preset}_deq.pth"
        torch.save(deq, dq_pth)
        model = RWKV7Ref(dq_pth, device="cpu", dtype=torch.float32)
        trace = []
        with torch.no_grad():
            logits = model.forward(idx, trace=trace)
        np.savez_compressed(os.path.join(HERE, f"toy_{preset}_ref.npz"), idx=idx.numpy(),
                            logits=logits.numpy().astype(np.float32),
                            trace=np.stack([t.numpy() for t in trace]).astype(np.float32))
        print(preset, os.path.getsize(out), "bytes; logits", tuple(logits.shape),
              "absmax", float(logits.abs().max()))


WORLD_TO_CUSTOM = {"receptance": "r_proj", "key": "k_proj", "value": "v_proj", "output": "o_proj"}


def toy_custom_state_dict(**kw):
    """The same random model under "custom" naming (tests/test_quant_model_smoke.py:31-73):
    blocks.N.tmix.* / cmix.*, top-level ln0, LoRA pairs as nn.Linear weights [out, in] with the
    world w0/a0/v0 vectors as the B biases."""
    sd, out = toy_world_state_dict(**kw), {}
    for k, v in sd.items():
        parts = k.split(".")
        if k.startswith("blocks.0.ln0."):
            out["ln0." + parts[-1]] = v
        elif len(parts) >= 4 and parts[2] == "att":
            tp, nm = ".".join(parts[:2]) + ".tmix.", parts[3]
            if nm in WORLD_TO_CUSTOM:
                out[tp + WORLD_TO_CUSTOM[nm] + ".weight"] = v
            elif len(nm) == 2 and nm[0] in "wavg" and nm[1] in "012":
                if nm[1] == "0":
                    out[tp + nm[0] + "_lora_B.bias"] = v.reshape(-1)
                else:
                    out[tp + nm[0] + "_lora_" + ("A" if nm[1] == "1" else "B") + ".weight"] = v.t().contiguous()
            else:
                out[tp + ".".join(parts[3:])] = v
        elif len(parts) >= 4 and parts[2] == "ffn":
            out[".".join(parts[:2]) + ".cmix." + ".".join(parts[3:])] = v
        else:
            out[k] = v
    # layer 0 has no value-residual branch under custom naming
    for k in [k for k in out if k.startswith("blocks.0.tmix.v_lora_")]:
        del out[k]
    return out


def make_toy_custom():
    """toy_custom_<cfg>.rwkvq: custom-naming checkpoints written by the reference's save() (the
    int8 + SpQR configuration of tests/test_quant_parity.py:97 and the compression preset), with
    RWKV7Ref logits on the dequantised weights."""
    from safetensors.torch import save_file
    from rwkv_quant.formats.writer import save
    cfg_c = PRESETS["compression"]
    cfg_c.act_stats_path = None
    int8 = QuantConfig(proj=8, cmix=8, outlier_fracs={"proj": 0.02, "cmix": 0.01})
    # d128: the dimensions of the reference's own model-level tests (D=128, H=2, V=256)
    for name, cfg, (L, D, S, V) in (("int8", int8, (2, 256, 64, 512)), ("compression", cfg_c, (2, 256, 64, 512)),
                                    ("d128_int8", int8, (2, 128, 64, 256))):
        sd = toy_custom_state_dict(L=L, D=D, V=V, S=S)
        idx = torch.from_numpy(np.random.default_rng(1).integers(1, V - 12, (2, 24)))
        out = os.path.join(HERE, f"toy_custom_{name}.rwkvq")
        save(sd, cfg, out, naming="custom", n_layer=L, n_embd=D, head_size=S, vocab_size=V)
        deq = reader.load_dequantized(out)
        d = f"/tmp/rwkvq_toy_custom_{name}"
        os.makedirs(d, exist_ok=True)
        save_file({k: v.contiguous() for k, v in deq.items()}, f"{d}/model.safetensors")
        with open(f"{d}/config.json", "w") as f:
            json.dump({"n_layer": L, "n_embd": D, "head_size": S, "vocab_size": V}, f)
        model = RWKV7Ref(d, device="cpu", dtype=torch.float32)
        with torch.no_grad():
            logits = model.forward(idx)
        np.savez_compressed(os.path.join(HERE, f"toy_custom_{name}_ref.npz"), idx=idx.numpy(),
                            logits=logits.numpy().astype(np.float32))
        print("custom", name, os.path.getsize(out), "bytes; logits", tuple(logits.shape),
              "absmax", float(logits.abs().max()))


if __name__ == "__main__":
    which = sys.argv[2] if len(sys.argv) > 2 else "all"
    if which in ("all", "codec"):
        make_codec_cases()
    if which in ("all", "toy"):
        make_toy_models()
    if which in ("all", "custom"):
        make_toy_custom()
    if which in ("all", "config1"):
        make_config1()
