"""Random-init quantized RWKV-7 builds in the ``.rwkvq`` layouts.

There is no real checkpoint to load on a benchmark box, so throughput runs and
full-size parity tests use seeded random-init weights packed straight into the
file format.  The packers here are plain min/max block quantisers (no grid
search, no activation statistics): they produce valid sb6 / sym / asym / rtn
buffers that any ``.rwkvq`` reader dequantises, which is all the inference path
needs.  The reference's calibrated quantiser (calibration/groupwise.py) is
offline tooling and is not reproduced.

Shapes follow a "world"-naming state dict (tests_local/build_world_ckpt_v2.py:42-74)
with the LoRA rank rule of tests/test_quant_model_smoke.py:25-27, and the value
distributions of tests/test_quant_parity.py:44-94.

All packers take and return torch tensors on the input's device, so a 1.5B build
is produced on the GPU in seconds.
"""
from __future__ import annotations

import zlib

import torch

from .formats.container import QuantizedCheckpoint, QuantizedTensor

# ---------------------------------------------------------------------------
# recipes: group -> (layout, bits).  Mirrors rwkv_quant/presets.py:97-133.
# ---------------------------------------------------------------------------
RECIPES = {
    # Q6_K-style sym: proj/emb/head at 8 bits, cmix at 6; LoRA w/a/v asym@6 gs64,
    # g per-row 8 bit; k_k/k_a/r_k, lerp vectors, biases and norms dense bf16.
    "reduction": {"proj": ("sym", 8), "cmix": ("sym", 6), "emb": ("sym", 8),
                  "head": ("sym", 8), "wav_lora": ("asym", 6), "g_lora": ("rtn", 8)},
    # sb6: proj/emb/head int5, cmix int4.
    "compression": {"proj": ("sb6", 5), "cmix": ("sb6", 4), "emb": ("sb6", 5),
                    "head": ("sb6", 5), "wav_lora": ("asym", 6), "g_lora": ("rtn", 8)},
    # the variant of the compression recipe with 8-bit embedding / head
    "compression_eh8": {"proj": ("sb6", 5), "cmix": ("sb6", 4), "emb": ("sym", 8),
                        "head": ("sym", 8), "wav_lora": ("asym", 6), "g_lora": ("rtn", 8)},
    # sb6 at 6 bits everywhere (exercises both bit-planes)
    "sb6_int6": {"proj": ("sb6", 6), "cmix": ("sb6", 6), "emb": ("sb6", 6),
                 "head": ("sb6", 6), "wav_lora": ("asym", 6), "g_lora": ("rtn", 8)},
    # per-row configurations (legacy files): int8 codes / packed biased nibbles
    "rtn8": {"proj": ("rtn", 8), "cmix": ("rtn", 8), "emb": ("rtn", 8),
             "head": ("rtn", 8), "wav_lora": ("rtn", 8), "g_lora": ("rtn", 8)},
}

MODEL_DIMS = {
    "1.5b": dict(n_layer=24, n_embd=2048, ffn=8192, vocab=65536),
    "2.9b": dict(n_layer=32, n_embd=2560, ffn=10240, vocab=65536),
    "toy": dict(n_layer=2, n_embd=256, ffn=1024, vocab=512),
}


def lora_ranks(d: int) -> dict:
    f = lambda c, p: max(32, int(round(c * d ** p / 32)) * 32)
    return {"w": f(1.8, 0.5), "a": f(1.8, 0.5), "v": f(1.3, 0.5), "g": f(0.6, 0.8)}


# ---------------------------------------------------------------------------
# bit packers
# ---------------------------------------------------------------------------

def pack_nibbles_blocklocal(q: torch.Tensor, gs: int) -> torch.Tensor:
    """codes 0..15 [OUT, IN] -> uint8 [OUT, IN/2]; inside each block of ``gs``
    columns byte j carries column j (low nibble) and column j+gs/2 (high)."""
    o, n = q.shape
    b = q.reshape(o, n // gs, 2, gs // 2).to(torch.uint8)
    return (b[:, :, 0] | (b[:, :, 1] << 4)).reshape(o, n // 2).contiguous()


def pack_bitplane(bit: torch.Tensor) -> torch.Tensor:
    """{0,1} [OUT, IN] -> uint8 [OUT, IN/8]; column c is bit c%8 of byte c//8."""
    o, n = bit.shape
    w = (1 << torch.arange(8, device=bit.device, dtype=torch.int32))
    return (bit.reshape(o, n // 8, 8).to(torch.int32) * w).sum(-1).to(torch.uint8)


def pack_6bit(v: torch.Tensor) -> torch.Tensor:
    """values 0..63 [..., 4k] -> bytes [..., 3k], little-endian bit stream."""
    x = v.to(torch.int32).reshape(*v.shape[:-1], -1, 4)
    word = x[..., 0] | (x[..., 1] << 6) | (x[..., 2] << 12) | (x[..., 3] << 18)
    out = torch.stack([word & 0xFF, (word >> 8) & 0xFF, (word >> 16) & 0xFF], dim=-1)
    return out.reshape(*v.shape[:-1], -1).to(torch.uint8)


def pack_nibbles_split_biased(codes: torch.Tensor) -> torch.Tensor:
    """per-row rtn <=4 bit: int8 [-8,7] [rows, cols] -> uint8 [rows, ceil(cols/2)];
    nibble = code+8, low nibble column i, high nibble column i+ceil(cols/2)."""
    r, c = codes.shape
    half = (c + 1) // 2
    u = (codes.to(torch.int16) + 8).to(torch.uint8)
    hi = torch.zeros(r, half, dtype=torch.uint8, device=codes.device) + 8
    hi[:, : c - half] = u[:, half:]
    return (u[:, :half] | (hi << 4)).contiguous()


def _h(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.float16).to(torch.float32)


# ---------------------------------------------------------------------------
# block quantisers (min/max, no search)
# ---------------------------------------------------------------------------

def quant_sb6(key, group, w: torch.Tensor, bits: int) -> QuantizedTensor:
    """asymmetric block-32 codes, 6-bit block scale/min against fp16 super-scales."""
    gs, sb = 32, 8
    o, n = w.shape
    assert n % (gs * sb) == 0, f"{key}: IN={n} is not a multiple of {gs * sb}"
    qmax = (1 << bits) - 1
    wb = w.float().reshape(o, n // gs, gs)
    lo, hi = wb.amin(-1), wb.amax(-1)
    step = ((hi - lo) / qmax).clamp_min(1e-8).reshape(o, -1, sb)
    lo = lo.reshape(o, -1, sb)
    d = _h((step.amax(-1, keepdim=True) / 63).clamp_min(1e-12))
    qs = torch.round(step / d).clamp(1, 63)
    dm = _h((lo.abs().amax(-1, keepdim=True) / 31).clamp_min(1e-12))
    qm = torch.round(lo / dm).clamp(-31, 31)
    s = _h(qs * d).clamp_min(1e-8).reshape(o, -1, 1)
    m = _h(qm * dm).reshape(o, -1, 1)
    q = torch.round((wb - m) / s).clamp(0, qmax).to(torch.uint8).reshape(o, n)
    qsqm = torch.cat([pack_6bit(qs.to(torch.uint8)),
                      pack_6bit((qm + 31).to(torch.uint8))], dim=-1)
    return QuantizedTensor(
        key=key, group=group, bits=bits, shape=(o, n), gw_mode="sb6", gw_gs=gs, gw_sb=sb,
        codes_packed=pack_nibbles_blocklocal(q & 0xF, gs),
        gw_qh=pack_bitplane((q >> 4) & 1) if bits >= 5 else None,
        gw_qh2=pack_bitplane((q >> 5) & 1) if bits >= 6 else None,
        gw_qsqm=qsqm.contiguous(), gw_d=d.squeeze(-1).half(), gw_dm=dm.squeeze(-1).half())


def quant_sym(key, group, w: torch.Tensor, bits: int) -> QuantizedTensor:
    """symmetric block-16 codes, int8 block-scale code against one fp16 per 256."""
    gs, sb = 16, 16
    o, n = w.shape
    assert n % (gs * sb) == 0, f"{key}: IN={n} is not a multiple of {gs * sb}"
    qmax = (1 << (bits - 1)) - 1
    wb = w.float().reshape(o, n // gs, gs)
    step = (wb.abs().amax(-1) / qmax).reshape(o, -1, sb)
    d = _h((step.amax(-1, keepdim=True) / 127).clamp_min(1e-12))
    qs = torch.nan_to_num(torch.round(step / d), 0.0).clamp(-128, 127)
    qs = torch.where(d > 0, qs, torch.zeros_like(qs))
    s = _h(qs * d).reshape(o, -1, 1)
    safe = torch.where(s != 0, s, torch.ones_like(s))
    q = torch.where(s != 0, torch.round(wb / safe).clamp(-qmax - 1, qmax),
                    torch.zeros_like(wb)).to(torch.int8).reshape(o, n)
    qt = QuantizedTensor(key=key, group=group, bits=bits, shape=(o, n), gw_mode="sym",
                         gw_gs=gs, gw_sb=sb, gw_qs=qs.reshape(o, -1).to(torch.int8),
                         gw_d=d.squeeze(-1).half())
    if bits == 8:
        qt.codes = q.contiguous()
    else:
        u = (q.to(torch.int16) + 32).to(torch.uint8)
        qt.codes_packed = pack_nibbles_blocklocal(u & 0xF, gs)
        qt.gw_qh = pack_bitplane((u >> 4) & 1)
        qt.gw_qh2 = pack_bitplane((u >> 5) & 1)
    return qt


def quant_asym(key, group, w: torch.Tensor, bits: int, gs: int = 64) -> QuantizedTensor:
    """uint8 codes with fp32 scale/min per block of ``gs`` stored columns;
    ceil(cols/gs) blocks, the ragged tail block has its own pair."""
    o, n = w.shape
    nb = -(-n // gs)
    qmax = (1 << bits) - 1
    pad = nb * gs - n
    wf = w.float()
    big = torch.finfo(torch.float32).max
    lo = torch.nn.functional.pad(wf, (0, pad), value=big).reshape(o, nb, gs).amin(-1)
    hi = torch.nn.functional.pad(wf, (0, pad), value=-big).reshape(o, nb, gs).amax(-1)
    step = ((hi - lo) / qmax).clamp_min(1e-8)
    blk = torch.arange(n, device=w.device) // gs
    q = torch.round((wf - lo[:, blk]) / step[:, blk]).clamp(0, qmax).to(torch.uint8)
    return QuantizedTensor(key=key, group=group, bits=bits, shape=(o, n), gw_mode="asym",
                           gw_gs=gs, codes=q.contiguous(), gw_scale=step.contiguous(),
                           gw_min=lo.contiguous())


def quant_rtn(key, group, w: torch.Tensor, bits: int) -> QuantizedTensor:
    """per-row symmetric round-to-nearest with an fp16 scale per stored row."""
    qmax = (1 << (bits - 1)) - 1
    wf = w.float()
    scale = (wf.abs().amax(dim=tuple(range(1, wf.dim())), keepdim=True).clamp_min(1e-8)
             / qmax)
    codes = torch.round(wf / scale).clamp(-qmax - 1, qmax).to(torch.int8)
    qt = QuantizedTensor(key=key, group=group, bits=bits, shape=tuple(w.shape),
                         scale=scale.half())
    if bits <= 4:
        qt.codes_packed = pack_nibbles_split_biased(codes)
    else:
        qt.codes = codes.contiguous()
    return qt


def dense(key, w: torch.Tensor, group="other") -> QuantizedTensor:
    return QuantizedTensor(key=key, group=group, bits=16, shape=tuple(w.shape),
                           dense=w.to(torch.bfloat16).contiguous())


_QUANT = {"sb6": quant_sb6, "sym": quant_sym, "asym": quant_asym, "rtn": quant_rtn}


def quantize(key: str, group: str, w: torch.Tensor, recipe: dict) -> QuantizedTensor:
    layout, bits = recipe[group]
    grp = {"wav_lora": key.rsplit(".", 1)[-1][0] + "_lora"}.get(group, group)
    return _QUANT[layout](key, grp, w, bits)


# ---------------------------------------------------------------------------
# random-init world-naming checkpoint
# ---------------------------------------------------------------------------

def _gen(key: str, seed: int, device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed((zlib.crc32(key.encode()) ^ (seed * 0x9E3779B1)) & 0x7FFFFFFF)
    return g


def build_checkpoint(model="1.5b", recipe="compression", seed=0, device="cpu",
                     n_layer=None, n_embd=None, ffn=None, vocab=None,
                     head_size=64, keep_on_device=True) -> QuantizedCheckpoint:
    """Seeded random-init RWKV-7 build packed in ``recipe``'s layouts.

    Matrices ~N(0, 0.02); lerp vectors U(0.2, 0.8); w0/a0/v0 0.1*N(0,1);
    k_k U(0.5,1); k_a U(0,0.5); r_k 0.1*N(0,1); norm weights 1, biases 0."""
    dims = dict(MODEL_DIMS[model]) if isinstance(model, str) else dict(model)
    L = n_layer or dims["n_layer"]
    D = n_embd or dims["n_embd"]
    F = ffn or dims["ffn"]
    V = vocab or dims["vocab"]
    H = D // head_size
    rec = RECIPES[recipe] if isinstance(recipe, str) else recipe
    rk = lora_ranks(D)
    dev = torch.device(device)
    tensors = {}

    def randn(key, *shape, std=0.02):
        return torch.randn(*shape, generator=_gen(key, seed, dev), device=dev) * std

    def rand(key, *shape, lo=0.0, hi=1.0):
        return torch.rand(*shape, generator=_gen(key, seed, dev), device=dev) * (hi - lo) + lo

    def put(qt):
        if not keep_on_device:
            for f in ("codes", "codes_packed", "scale", "dense", "gw_d", "gw_dm", "gw_qsqm",
                      "gw_qh", "gw_qh2", "gw_scale", "gw_min", "gw_qs"):
                v = getattr(qt, f)
                if v is not None:
                    setattr(qt, f, v.cpu())
        tensors[qt.key] = qt

    def mat(key, group, *shape):
        put(quantize(key, group, randn(key, *shape), rec))

    mat("emb.weight", "emb", V, D)
    for nm in ("blocks.0.ln0", "ln_out"):
        put(dense(nm + ".weight", torch.ones(D, device=dev)))
        put(dense(nm + ".bias", torch.zeros(D, device=dev)))
    for i in range(L):
        p = f"blocks.{i}."
        for ln in ("ln1", "ln2"):
            put(dense(p + ln + ".weight", torch.ones(D, device=dev)))
            put(dense(p + ln + ".bias", torch.zeros(D, device=dev)))
        a = p + "att."
        for nm in ("x_r", "x_w", "x_k", "x_v", "x_a", "x_g"):
            put(dense(a + nm, rand(a + nm, 1, 1, D, lo=0.2, hi=0.8)))
        for br in ("w", "a", "v"):
            if br == "v" and i == 0:
                continue      # layer 0 has no value-residual branch
            put(dense(a + br + "0", randn(a + br + "0", 1, 1, D, std=0.1), group=br + "_lora"))
            mat(a + br + "1", "wav_lora", D, rk[br])
            mat(a + br + "2", "wav_lora", rk[br], D)
        mat(a + "g1", "g_lora", D, rk["g"])
        mat(a + "g2", "g_lora", rk["g"], D)
        put(dense(a + "k_k", rand(a + "k_k", 1, 1, D, lo=0.5, hi=1.0), group="small"))
        put(dense(a + "k_a", rand(a + "k_a", 1, 1, D, lo=0.0, hi=0.5), group="small"))
        put(dense(a + "r_k", randn(a + "r_k", H, head_size, std=0.1), group="small"))
        for nm in ("receptance", "key", "value", "output"):
            mat(a + nm + ".weight", "proj", D, D)
        put(dense(a + "ln_x.weight", torch.ones(D, device=dev)))
        put(dense(a + "ln_x.bias", torch.zeros(D, device=dev)))
        f = p + "ffn."
        put(dense(f + "x_k", rand(f + "x_k", 1, 1, D, lo=0.2, hi=0.8)))
        mat(f + "key.weight", "cmix", F, D)
        mat(f + "value.weight", "cmix", D, F)
    mat("head.weight", "head", V, D)
    for k, qt in tensors.items():
        qt.transposed = k.split(".")[-1] in ("w1", "w2", "a1", "a2", "v1", "v2", "g1", "g2")
    return QuantizedCheckpoint(naming="world", n_layer=L, n_embd=D, head_size=head_size,
                               vocab_size=V, tensors=tensors,
                               config_repr=f"synth({recipe if isinstance(recipe, str) else 'custom'}, seed={seed})",
                               config=None, tokenizer=None)
