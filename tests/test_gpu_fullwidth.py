"""Model-level parity at the FULL width of the benchmark configurations.

The reference-written toy files pin the model at D = 256; here the same comparisons run on
2-layer builds with the real width, heads, LoRA ranks, channel-mix width and vocabulary of
RWKV-7 1.5B (D 2048, 32 heads, FFN 8192, ranks 96/96/64/256) and 2.9B (D 2560, 40 heads,
FFN 10240, ranks 96/96/64/320), vocabulary 65536, in both recipes, so that every launch
geometry of the benchmark (K-split GEMVs, the persistent 296-CTA head launch, the 65536-row
argmax, 32/40-head time-mix core, 256-token GEMM tiles, 8192-token glue) runs inside a model
and is compared with the CPU oracle (the reference's model gate is tests/test_quant_parity.py:129-138).

  decode   8 teacher-forced tokens at batch 1 and batch 64, eager launches and CUDA-graph
           replay; at batch 64 the oracle follows streams 0, 31 and 63 (streams are independent)
  prefill  pp512: batch 1 all positions + final states; batch 16 last position + states
           (oracle on sequences 0 and 15)
  hand-over  prefill of 37 tokens, then 4 decoded tokens from the returned state

Tolerances (written here): logits relmax <= 1e-3; WKV state max|delta| <= 1e-3 * max(1, max|state|)
(printed); shift states relmax <= 1e-3.
"""
import os

import numpy as np
import pytest
import torch

from helpers import relmax
from oracle import codec_np as oc
from oracle.model_np import OracleRWKV7

pytestmark = pytest.mark.gpu
TOL = 1e-3

BUILDS = [("1.5b", "compression"), ("1.5b", "reduction"), ("2.9b", "compression"), ("2.9b", "reduction")]


@pytest.fixture(scope="module", params=BUILDS, ids=lambda p: f"{p[0]}-{p[1]}")
def build(request, tmp_path_factory, cuda_lib):
    """(QuantRWKV7 on the GPU, OracleRWKV7 on the CPU) over the same seeded 2-layer build."""
    from rwkv_quant_b200 import synth
    from rwkv_quant_b200.backends.cuda import QuantRWKV7
    from rwkv_quant_b200.formats import load_raw, save_rwkvq
    name, recipe = request.param
    ck = synth.build_checkpoint(name, recipe, seed=5, device="cuda", n_layer=2, keep_on_device=False)
    path = str(tmp_path_factory.mktemp("fw") / f"{name}_{recipe}.rwkvq")
    save_rwkvq(ck, path)
    del ck
    model = QuantRWKV7(load_raw(path))
    man, arr = oc.open_rwkvq(path)
    oracle = OracleRWKV7(man, arr)
    dims = synth.MODEL_DIMS[name]
    assert (model.n_embd, model.ffn_dim, model.vocab_size) == (dims["n_embd"], dims["ffn"], 65536)
    yield model, oracle, f"{name} {recipe}"
    del model, oracle
    torch.cuda.empty_cache()
    os.remove(path)


def _check_states(tag, got, ref, rows=None):
    """got: model states (torch), ref: oracle states; rows: batch rows of `got` the oracle followed."""
    worst = 0.0
    for (w, ts, cs), (rw, rts, rcs) in zip(got, ref):
        sel = (lambda t: t) if rows is None else (lambda t: t[rows])
        w = sel(w).cpu().numpy()
        d = float(np.abs(w - rw).max())
        worst = max(worst, d)
        assert d <= TOL * max(1.0, float(np.abs(rw).max())), (tag, "wkv state", d)
        B = w.shape[0]
        assert relmax(sel(ts).reshape(B, -1).cpu().numpy(), rts.reshape(B, -1)) <= TOL, (tag, "tmix shift")
        assert relmax(sel(cs).reshape(B, -1).cpu().numpy(), rcs.reshape(B, -1)) <= TOL, (tag, "cmix shift")
    print(f"{tag}: wkv state max|delta| {worst:.2e}")


@pytest.mark.parametrize("B,rows", [(1, [0]), (64, [0, 31, 63])])
def test_decode_full_width(build, B, rows):
    model, oracle, name = build
    n = 8
    toks = np.random.default_rng(100 + B).integers(1, 65000, (B, n))
    ref_st = oracle.init_state(len(rows))
    ref = []
    for t in range(n):
        lo, ref_st = oracle.forward_stateful(toks[rows, t:t + 1], ref_st)
        ref.append(lo[:, 0])
    ref = np.stack(ref, 1)                                         # [rows, n, V]
    tk = torch.from_numpy(toks).cuda()
    for graph in (False, True):
        dec = model.decoder(B, use_graph=graph)
        got, arg = [], []
        for t in range(n):
            nxt = dec.step(tk[:, t])
            got.append(dec.logits[rows].cpu().numpy())
            arg.append(nxt[rows].cpu().numpy())
        got = np.stack(got, 1)
        err = relmax(got, ref)
        print(f"{name} decode B={B} {'graph' if graph else 'eager'}: logits relmax {err:.2e}")
        assert np.isfinite(got).all() and err <= TOL, err
        # the 65536-row argmax against the oracle wherever its top-2 margin is clear
        arg = np.stack(arg, 1)
        top2 = np.sort(ref, axis=-1)[..., -2:]
        clear = (top2[..., 1] - top2[..., 0]) > 2 * TOL * np.abs(ref).max()
        assert (arg[clear] == ref.argmax(-1)[clear]).all()
        assert (arg == got.argmax(-1)).all(), "device argmax differs from its own logits"
        _check_states(f"{name} decode B={B}", dec.states, ref_st, rows)


def test_prefill_pp512_full_width(build):
    model, oracle, name = build
    idx = np.random.default_rng(7).integers(1, 60000, (16, 512))
    # batch 1: every position and the final state
    ref, ref_st = oracle.forward_stateful(idx[:1], oracle.init_state(1))
    lo, st = model.forward_stateful(idx[:1], model.init_state(1))
    err = relmax(lo.cpu().numpy(), ref)
    print(f"{name} pp512 B=1: logits relmax (all positions) {err:.2e}")
    assert err <= TOL, err
    _check_states(f"{name} pp512 B=1", st, ref_st)
    del lo
    # batch 16: last position and the states; the oracle follows sequences 0 and 15
    rows = [0, 15]
    ref, ref_st = oracle.forward_stateful(idx[rows], oracle.init_state(2), last_only=True)
    lo, st = model.forward_stateful(idx, model.init_state(16), last_only=True)
    assert lo.shape == (16, 1, model.vocab_size)
    err = relmax(lo[rows].cpu().numpy(), ref)
    print(f"{name} pp512 B=16: logits relmax (last position, sequences 0 and 15) {err:.2e}")
    assert err <= TOL, err
    _check_states(f"{name} pp512 B=16", st, ref_st, rows)


def test_prefill_then_decode_full_width(build):
    model, oracle, name = build
    idx = np.random.default_rng(9).integers(1, 60000, (2, 41))
    ref, _ = oracle.forward_stateful(idx, oracle.init_state(2))
    lo, st = model.forward_stateful(idx[:, :37], model.init_state(2), last_only=True)
    assert relmax(lo.cpu().numpy(), ref[:, 36:37]) <= TOL
    for t in range(37, 41):
        lo, st = model.forward_stateful(idx[:, t:t + 1], st)
        err = relmax(lo.cpu().numpy(), ref[:, t:t + 1])
        assert err <= TOL, (t, err)
    print(f"{name} prefill(37) -> decode(4): last-step logits relmax {err:.2e}")


@pytest.mark.parametrize("B", [40, 64])
def test_decode_two_term_tcgen05_linears(build, cuda_lib, B):
    """Batched decode above 32 streams runs some linears on the two-term tcgen05 kernel, fed with fp16
    pairs and block sums by the LayerNorm kernels: r / k / v, the ffn key and the head up to 48 streams,
    the head alone up to 64 (RWKVQ_TCB_EXACT=1 / 0 force all three / none; here through the library's
    profiling switch, not part of the C ABI).  With all three forced: the tolerance of the default path
    against the oracle (streams 0 and B - 1) and fp32-grade agreement with the all-mma.sync step; at 40
    streams the launcher's own choice must be exactly the forced one."""
    import ctypes as C
    model, oracle, name = build
    hook = cuda_lib.rwkvq_profiling_tcb_exact
    hook.restype, hook.argtypes = None, [C.c_int]
    n, rows = 4, [0, B - 1]
    toks = np.random.default_rng(300 + B).integers(1, 65000, (B, n))
    ref_st = oracle.init_state(len(rows))
    ref = []
    for t in range(n):
        lo, ref_st = oracle.forward_stateful(toks[rows, t:t + 1], ref_st)
        ref.append(lo[:, 0])
    ref = np.stack(ref, 1)
    tk = torch.from_numpy(toks).cuda()
    got = {}
    try:
        for on in (1, 0, -1):
            hook(on)
            dec = model.decoder(B, use_graph=False)
            out = []
            for t in range(n):
                dec.step(tk[:, t])
                out.append(dec.logits.cpu().numpy())
            dec.check()
            got[on] = np.stack(out, 1)
            del dec
    finally:
        hook(-1)
    err = relmax(got[1][rows], ref)
    both = relmax(got[1], got[0])
    own = relmax(got[-1][rows], ref)
    print(f"{name} decode B={B}, two-term tcgen05 linears: logits relmax {err:.2e} vs oracle, {both:.2e} vs the mma.sync form; "
          f"launcher's choice {own:.2e} vs oracle")
    assert np.isfinite(got[1]).all() and err <= TOL, err
    assert both <= 2e-4, both
    assert np.isfinite(got[-1]).all() and own <= TOL, own
    if B == 40:
        assert np.array_equal(got[-1], got[1])


def test_full_depth_decode_and_prefill(tmp_path, cuda_lib):
    """All 24 layers of the 1.5B compression build (the benchmark's model): rounding that stays
    under the tolerance on 2 layers must not grow past it over the real depth.  Batched decode
    (8 streams: one token tile; 64 streams: two stream groups of 32) runs on the two-term
    small-batch linears and stays at fp32 grade, 2e-4 asserted.  The pp512 prefill runs its linears
    on fp16 operands, which is the reference's own prefill arithmetic (fp16 dequantise + fp16 matmul
    from 128 rows on, gated there at 2e-3 per linear): its last-position logits are held to 2e-3
    and the top-1 token must agree."""
    from rwkv_quant_b200 import synth
    from rwkv_quant_b200.backends.cuda import QuantRWKV7
    from rwkv_quant_b200.formats import load_raw, save_rwkvq
    ck = synth.build_checkpoint("1.5b", "compression", seed=5, device="cuda", keep_on_device=False)
    path = str(tmp_path / "full.rwkvq")
    save_rwkvq(ck, path)
    del ck
    model = QuantRWKV7(load_raw(path))
    man, arr = oc.open_rwkvq(path)
    oracle = OracleRWKV7(man, arr)
    assert model.n_layer == 24
    for B in (1, 8, 64):
        toks = np.random.default_rng(B).integers(1, 60000, (B, 3))
        rows = list(range(min(B, 3)))
        rs = oracle.init_state(len(rows))
        dec = model.decoder(B, use_graph=True)
        tk = torch.from_numpy(toks).cuda()
        worst = 0.0
        for t in range(3):
            ref, rs = oracle.forward_stateful(toks[rows, t:t + 1], rs)
            dec.step(tk[:, t])
            worst = max(worst, relmax(dec.logits[rows].cpu().numpy(), ref[:, 0]))
        print(f"1.5b compression, 24 layers, decode B={B} ({dec.groups} group(s)): logits relmax {worst:.2e}")
        assert worst <= 2e-4, (B, worst)
        del dec
    idx = np.random.default_rng(7).integers(1, 60000, (1, 512))
    ref, _ = oracle.forward_stateful(idx, oracle.init_state(1), last_only=True)
    lo, _ = model.forward_stateful(idx, model.init_state(1), last_only=True)
    err = relmax(lo.cpu().numpy(), ref)
    print(f"1.5b compression, 24 layers, pp512 B=1: last-position logits relmax {err:.2e}")
    assert err <= 2e-3, err
    assert int(lo[0, -1].argmax()) == int(ref[0, -1].argmax())
    del model, oracle
    torch.cuda.empty_cache()
