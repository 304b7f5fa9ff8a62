"""WKV-7, time-mix tail and the whole model on the GPU against the CPU oracle.

Tolerances: logits relmax <= 1e-3 against the fp32 oracle with the same weight
precision policy; WKV state max|delta| is asserted and printed; greedy tokens must
agree wherever the oracle's top-2 margin exceeds the logit tolerance.
"""
import os
import zlib

import numpy as np
import pytest
import torch

from conftest import GOLDEN
from helpers import relmax
from oracle import codec_np as oc
from oracle.build_c import wkv7_seq
from oracle.model_np import OracleRWKV7, wkv7_np

pytestmark = pytest.mark.gpu

# (B, T, H) of the reference's WKV gate (tests/test_wkv_infer_parity.py:34-36)
WKV_CASES = [(1, 1, 32), (1, 3, 32), (1, 16, 32), (1, 512, 32), (1, 1, 40), (1, 512, 40), (1, 512, 16),
             (2, 128, 32), (1, 7, 32), (1, 8, 32), (1, 9, 32), (2, 24, 16), (1, 25, 32), (3, 41, 4)]    # chunk edges (8 steps)


def wkv_inputs(B, T, H, S=64):
    """Input recipe of tests/test_wkv_infer_parity.py:38-53."""
    rs = np.random.RandomState(zlib.crc32(f"wkv7-infer-{B}-{T}-{H}".encode()) & 0x7FFFFFFF)
    g = lambda sc=1.0: (rs.randn(B, T, H, S) * sc).astype(np.float32)
    r, k, v, a, b = g(), g(), g(), g(0.1), g(0.1)
    w = (0.85 + 0.14 * rs.rand(B, T, H, S)).astype(np.float32)
    h = (rs.randn(B, H, S, S) * 0.05).astype(np.float32)
    return r, w, k, v, a, b, h


@pytest.mark.parametrize("case", WKV_CASES)
def test_wkv7_infer(cuda_lib, case):
    from rwkv_quant_b200.backends.cuda import wkv7_infer
    ins = wkv_inputs(*case)
    ref_out, ref_h = wkv7_seq(*ins)          # sequential order of the reference's kernel
    dev = [torch.from_numpy(x).cuda() for x in ins]
    h_before = dev[6].clone()
    out, h = wkv7_infer(*dev)
    assert torch.equal(dev[6], h_before), "the input state must not be modified"
    out, h = out.cpu().numpy(), h.cpu().numpy()
    d_state = float(np.abs(h - ref_h).max())
    print(f"wkv7 {case}: out relmax {relmax(out, ref_out):.2e}, state max|delta| {d_state:.2e}")
    assert relmax(out, ref_out) <= 1e-4 and d_state <= 1e-3 * max(1.0, np.abs(ref_h).max())
    # state carry: two calls == one call
    if case[1] >= 2:
        c = case[1] // 2
        o1, h1 = wkv7_infer(*[t[:, :c].contiguous() for t in dev[:6]], dev[6])
        o2, h2 = wkv7_infer(*[t[:, c:].contiguous() for t in dev[:6]], h1)
        assert torch.equal(torch.cat([o1, o2], 1).cpu(), torch.from_numpy(out))
        assert torch.equal(h2.cpu(), torch.from_numpy(h))


def test_wkv_tail(cuda_lib):
    from rwkv_quant_b200.backends.cuda import can_fuse_tail, wkv_tail
    assert can_fuse_tail(32, 64)
    rs = np.random.RandomState(3)
    N, H, S = 5, 32, 64
    D = H * S
    wkv, r, k, v, g = (rs.randn(N, D).astype(np.float32) for _ in range(5))
    r_k, lw, lb = (rs.randn(D).astype(np.float32) for _ in range(3))
    x = wkv.reshape(N, H, S).astype(np.float64)
    mu = x.mean(-1, keepdims=True)
    var = ((x - mu) ** 2).mean(-1, keepdims=True)
    nrm = ((x - mu) / np.sqrt(var + 64e-5)).reshape(N, D) * lw + lb
    dp = (r * k * r_k).reshape(N, H, S).astype(np.float64).sum(-1, keepdims=True)
    ref = (nrm + (dp * v.reshape(N, H, S)).reshape(N, D)) * g
    t = lambda a: torch.from_numpy(a).cuda()
    out = wkv_tail(t(wkv), t(r), t(k), t(v), t(r_k), t(lw), t(lb), t(g), H, S).cpu().numpy()
    assert relmax(out, ref) <= 1e-5


def _load(preset):
    from rwkv_quant_b200.backends.cuda import QuantRWKV7
    from rwkv_quant_b200.formats import load_raw
    path = os.path.join(GOLDEN, f"toy_{preset}.rwkvq")
    man, arr = oc.open_rwkvq(path)
    return QuantRWKV7(load_raw(path)), OracleRWKV7(man, arr), np.load(os.path.join(GOLDEN, f"toy_{preset}_ref.npz"))


@pytest.mark.parametrize("preset", ["reduction", "compression"])
def test_model_matches_oracle(cuda_lib, preset):
    """Reference-written toy checkpoint: sequence path, token-by-token path and the
    mixed use of both against the oracle (logits and every state tensor)."""
    model, oracle, z = _load(preset)
    idx = z["idx"]
    B, T = idx.shape
    ref, ref_st = oracle.forward_stateful(idx, oracle.init_state(B))
    # distance to the reference's own all-bf16 forward, for the record
    print(f"{preset}: oracle vs RWKV7Ref relmax {relmax(ref, z['logits']):.2e}")
    # whole sequence
    lo, st = model.forward_stateful(idx, model.init_state(B))
    assert lo.shape == (B, T, model.vocab_size) and lo.dtype == torch.float32
    assert relmax(lo.cpu().numpy(), ref) <= 1e-3, relmax(lo.cpu().numpy(), ref)
    assert relmax(model(idx).cpu().numpy(), ref) <= 1e-3
    # token by token (the decode kernels), states updated in place
    st1 = model.init_state(B)
    outs = []
    for t in range(T):
        lo1, st1 = model.forward_stateful(idx[:, t:t + 1], st1)
        outs.append(lo1.cpu().numpy())
    tb = np.concatenate(outs, 1)
    print(f"{preset}: decode path vs oracle relmax {relmax(tb, ref):.2e}")
    assert relmax(tb, ref) <= 1e-3
    for (w, ts, cs), (w2, ts2, cs2), (rw, rts, rcs) in zip(st, st1, ref_st):
        for got in (w, w2):
            d = float(np.abs(got.cpu().numpy() - rw).max())
            assert d <= 1e-3 * max(1.0, np.abs(rw).max()), d
        for got in (ts, ts2):
            assert relmax(got.reshape(B, -1).cpu().numpy(), rts) <= 1e-3
        for got in (cs, cs2):
            assert relmax(got.reshape(B, -1).cpu().numpy(), rcs) <= 1e-3
    # prefill then decode; last_only / tail_only
    lo_p, st_p = model.forward_stateful(idx[:, :10], model.init_state(B), last_only=True)
    assert lo_p.shape == (B, 1, model.vocab_size)
    assert relmax(lo_p.cpu().numpy(), ref[:, 9:10]) <= 1e-3
    lo_n, st_p = model.forward_stateful(idx[:, 10:11], st_p)
    assert relmax(lo_n.cpu().numpy(), ref[:, 10:11]) <= 1e-3
    lo_t, _ = model.forward_stateful(idx, model.init_state(B), tail_only=3)
    assert relmax(lo_t.cpu().numpy(), ref[:, -3:]) <= 1e-3
    hid, _ = model.forward_hidden(idx, model.init_state(B))
    rh, _ = oracle.forward_hidden(idx, oracle.init_state(B))
    assert relmax(hid.cpu().numpy(), rh) <= 1e-3


@pytest.mark.parametrize("cfg", ["int8", "compression", "d128_int8"])
def test_custom_naming_model(cuda_lib, cfg):
    """Custom-naming checkpoints written by the reference (tmix./cmix. keys, LoRA pairs stored
    [out, in] with biases; int8 + sparse overrides as in tests/test_quant_parity.py:97, and the
    compression preset): sequence path, decode path and the graph decoder against the oracle and
    against the reference's own RWKV7Ref logits (its model-level gate is 1e-2)."""
    from rwkv_quant_b200.backends.cuda import QuantRWKV7
    from rwkv_quant_b200.formats import load_raw
    path = os.path.join(GOLDEN, f"toy_custom_{cfg}.rwkvq")
    man, arr = oc.open_rwkvq(path)
    z = np.load(os.path.join(GOLDEN, f"toy_custom_{cfg}_ref.npz"))
    ck = load_raw(path)
    assert ck.naming == "custom"
    model = QuantRWKV7(ck)
    # tensors with overrides reach the kernels as dense bf16: compare those with the oracle's bf16 linears
    has_overrides = any(getattr(q, "outlier_indices", None) is not None and q.outlier_indices.numel() > 0
                        for q in ck.tensors.values())
    oracle = OracleRWKV7(man, arr, linear_weights="bf16" if has_overrides else "exact")
    idx = z["idx"]
    B, T = idx.shape
    ref, _ = oracle.forward_stateful(idx, oracle.init_state(B))
    lo, _ = model.forward_stateful(idx, model.init_state(B))
    d_seq = relmax(lo.cpu().numpy(), ref)
    st, outs = model.init_state(B), []
    for t in range(T):
        lo1, st = model.forward_stateful(idx[:, t:t + 1], st)
        outs.append(lo1.cpu().numpy())
    d_dec = relmax(np.concatenate(outs, 1), ref)
    print(f"custom {cfg}: sequence {d_seq:.2e}, decode {d_dec:.2e}, vs RWKV7Ref {relmax(lo.cpu().numpy(), z['logits']):.2e}")
    assert d_seq <= 1e-3 and d_dec <= 1e-3
    assert relmax(lo.cpu().numpy(), z["logits"]) <= 1e-2
    toks, _ = model.generate(idx[:, :6], 8)           # the graph decoder runs on it too
    assert toks.shape == (B, 8)


@pytest.mark.parametrize("recipe", ["compression", "reduction", "sb6_int6", "compression_eh8"])
def test_greedy_decode_graph_and_eager(cuda_lib, recipe):
    """Synthetic toy build: greedy tokens of the CUDA-graph decoder == eager decoder,
    and == the oracle wherever its top-2 margin is clear of the tolerance."""
    from rwkv_quant_b200 import synth
    from rwkv_quant_b200.backends.cuda import QuantRWKV7
    from rwkv_quant_b200.formats import save_rwkvq
    import tempfile
    ck = synth.build_checkpoint("toy", recipe, seed=11)
    with tempfile.TemporaryDirectory() as d:
        p = os.path.join(d, "m.rwkvq")
        save_rwkvq(ck, p)
        man, arr = oc.open_rwkvq(p)
        oracle = OracleRWKV7(man, arr)
        prompt = np.random.default_rng(5).integers(1, 500, (3, 9))
        model = QuantRWKV7(ck)
        toks, _ = model.generate(prompt, 12)
        # graph replay from the same prefilled state
        lo, st = model.forward_stateful(prompt, model.init_state(3), last_only=True)
        dec = model.decoder(3, states=st, use_graph=True)
        tok, got = lo[:, -1].argmax(-1), []
        for _ in range(12):
            got.append(tok.clone())
            tok = dec.step(tok).clone()
        assert torch.equal(torch.stack(got, 1), toks), "graph replay and eager decode disagree"
        # oracle, teacher-forced on our tokens
        ours = toks.cpu().numpy()
        logits, ost = oracle.forward_stateful(prompt, oracle.init_state(3), last_only=True)
        for t in range(12):
            top2 = np.sort(logits[:, -1], axis=-1)[:, -2:]
            clear = (top2[:, 1] - top2[:, 0]) > 2e-3 * np.abs(logits).max()
            assert (logits[:, -1].argmax(-1)[clear] == ours[clear, t]).all(), f"step {t}"
            logits, ost = oracle.forward_stateful(ours[:, t:t + 1], ost)


def test_sequence_glue_kernels_against_fp32_torch(cuda_lib):
    """rwkvq_seq_ln_shift_mix / rwkvq_seq_tmix_pre against the same formulas in plain torch fp32
    (tolerance 2e-6 of the output scale: different reduction orders only), including the carried
    shift state, a fresh stream (no state) and the layer-0 form without the v branch."""
    import torch.nn.functional as F
    from rwkv_quant_b200.backends.cuda import ops
    g = torch.Generator().manual_seed(21)
    B, T, D, H = 3, 5, 512, 8
    rnd = lambda *s: torch.randn(*s, generator=g).cuda()
    x, lw, lb, mix6, prev = rnd(B, T, D), rnd(D), rnd(D), torch.rand(6, D, generator=g).cuda(), rnd(B, 1, D)
    for shift_in in (prev, None):
        for mix in (mix6, mix6[2]):
            out, new_shift = ops.seq_ln_shift_mix(x, lw, lb, shift_in, mix)
            xn = F.layer_norm(x, (D,), lw, lb)
            p0 = shift_in if shift_in is not None else torch.zeros(B, 1, D, device="cuda")
            shifted = torch.cat([p0, xn[:, :-1]], dim=1)
            ref = torch.stack([xn + (shifted - xn) * m for m in mix.reshape(-1, D)])
            assert out.shape == ref.shape
            assert (out - ref).abs().max().item() <= 2e-6 * ref.abs().max().item() + 1e-6
            assert (new_shift - xn[:, -1:]).abs().max().item() <= 2e-6 * xn.abs().max().item() + 1e-6
    N = B * T
    k, v, yw, ya, yv, vf = (rnd(N, D) for _ in range(6))
    w0, a0, v0, k_k, k_a = (rnd(D) for _ in range(5))
    for layer0 in (False, True):
        w, k2, v2, na, nb = ops.seq_tmix_pre(k, v, yw, ya, None if layer0 else yv, None if layer0 else vf,
                                             w0, a0, v0, k_k, k_a, H)
        rw = torch.exp(-0.606531 * torch.sigmoid(yw + w0))
        ra = torch.sigmoid(ya + a0)
        kk = (k * k_k).reshape(N, H, 64)
        kk = (kk / torch.sqrt((kk * kk).sum(-1, keepdim=True) + 1e-12)).reshape(N, D)
        rk = k * (1.0 + (ra - 1.0) * k_a)
        rv = v if layer0 else v + (vf - v) * torch.sigmoid(yv + v0)
        for got, ref, nm in ((w, rw, "w"), (k2, rk, "k"), (v2, rv, "v"), (na, -kk, "-kk"), (nb, kk * ra, "kk*a")):
            assert (got - ref).abs().max().item() <= 3e-6 * ref.abs().max().item() + 1e-6, (layer0, nm)


def test_split_fp16_and_stacked_lora_product(cuda_lib):
    """rwkvq_split_fp16: [hi | lo] with hi = fp16(x) and hi + lo = x to 2^-21 of |x|; the product with
    a twice-stacked fp16 matrix equals the fp64 product to 1e-5 of its scale (fp32 accumulation on the
    tensor cores over K = 512 terms; a plain fp16 product of x.half() would be off by ~5e-4)."""
    from rwkv_quant_b200.backends.cuda import ops
    g = torch.Generator().manual_seed(31)
    x = (torch.randn(37, 256, generator=g) * 3).cuda()
    s = ops.split_fp16(x)
    assert s.shape == (37, 512) and s.dtype == torch.float16
    hi, lo = s[:, :256], s[:, 256:]
    assert torch.equal(hi, x.half())
    assert ((hi.double() + lo.double()) - x.double()).abs().max().item() <= 2.0 ** -21 * x.abs().max().item()
    w = (torch.randn(256, 96, generator=g) * 0.05).cuda().half()
    y = torch.mm(s, torch.cat([w, w], 0), out_dtype=torch.float32)
    ref = x.double() @ w.double()
    err = (y.double() - ref).abs().max().item() / ref.abs().max().item()
    assert err <= 1e-5, err
    plain = (torch.mm(x.half(), w, out_dtype=torch.float32).double() - ref).abs().max().item() / ref.abs().max().item()
    assert err < 0.1 * plain, (err, plain)


def test_prepared_rows_match_unfused_glue(cuda_lib):
    """rwkvq_seq_ln_shift_mix_prep: every form of a mix row equals what the separate passes make
    of the fp32 row (pre-pass scaling of rwkvq_gemm, rwkvq_split_fp16), and rwkvq_gemm_x16 on
    the prepared rows equals rwkvq_gemm on the fp32 rows bit for bit."""
    from rwkv_quant_b200 import synth
    from rwkv_quant_b200.backends.cuda import ops
    g = torch.Generator().manual_seed(17)
    B, T, D = 2, 37, 512
    x = torch.randn(B, T, D, generator=g).cuda() * 2
    lw, lb = (1 + 0.1 * torch.randn(D, generator=g)).cuda(), (0.1 * torch.randn(D, generator=g)).cuda()
    mix = torch.rand(6, D, generator=g).cuda()
    shift = torch.randn(B, 1, D, generator=g).cuda()
    for sh in (None, shift):
        ref, ref_shift = ops.seq_ln_shift_mix(x, lw, lb, sh, mix)
        rows, new_shift = ops.seq_ln_shift_mix_prep(x, lw, lb, sh, mix, [7, 2, 1, 3, 4, 6])
        assert (new_shift - ref_shift).abs().max().item() <= 2e-6
        for m, r in enumerate(rows):
            want = ref[m].reshape(B * T, D)
            if r.f32 is not None:
                assert (r.f32 - want).abs().max().item() <= 3e-6 * want.abs().max().item()
        full = rows[0]                                    # mode 7: all three forms of one row
        assert torch.equal(full.split, ops.split_fp16(full.f32))
        amax = full.f32.abs().amax(dim=1)
        sc = torch.ldexp(torch.ones_like(amax), 14 - torch.frexp(amax)[1])
        assert torch.equal(full.scale, sc)
        assert torch.equal(full.x16[:, :D], (full.f32 * sc[:, None]).half())
        assert rows[1].x16 is None and rows[2].split is None and rows[4].split is None
    qt = synth.quantize("blocks.0.att.key.weight", "proj", torch.randn(256, D, generator=g) * 0.02,
                        {"proj": ("sb6", 5)})
    dq = ops.DeviceQT(qt, "cuda")
    resid = torch.randn(B * T, 256, generator=g).cuda()
    for epi, rs in ((0, None), (1, None), (2, resid)):
        assert torch.equal(ops.gemm_x16(dq, full, epi, rs), ops.gemm(dq, full.f32, epi, rs))


def test_sequence_path_prepared_rows_vs_separate_passes(cuda_lib):
    """The sequence path with rows prepared in the LN kernel against the one with separate passes.
    The two LayerNorms add in different orders (1e-7), which moves a few fp16 roundings of the GEMM
    operands: the same 1e-3 gate as against the oracle."""
    model, oracle, z = _load("compression")
    idx = np.tile(z["idx"], (1, 3))
    B = idx.shape[0]
    assert model.fused_prep
    lo1, st1 = model.forward_stateful(idx, model.init_state(B))
    model.fused_prep = False
    lo0, st0 = model.forward_stateful(idx, model.init_state(B))
    d = relmax(lo1.cpu().numpy(), lo0.cpu().numpy())
    print(f"prepared rows vs separate passes: logits relmax {d:.2e}")
    assert d <= 1e-3
    ref, _ = oracle.forward_stateful(idx, oracle.init_state(B))
    assert relmax(lo1.cpu().numpy(), ref) <= 1e-3 and relmax(lo0.cpu().numpy(), ref) <= 1e-3
    for a, b in zip(st1, st0):
        for u, w in zip(a, b):
            assert (u - w).abs().max().item() <= 1e-3 * max(1.0, w.abs().max().item())


def test_speculative_decoding_matches_greedy(cuda_lib):
    """History n-gram drafts verified through forward_stateful(tail_only=...) on the small-T path
    (semantics of tests/spec_decode_champ.py:89-137): same tokens as plain greedy decoding."""
    from rwkv_quant_b200.spec_decode import generate_speculative
    model, oracle, z = _load("compression")
    prompt = [int(t) for t in z["idx"][0, :10]] * 3
    want, _ = model.generate(np.asarray([prompt]), 40)
    to_idx = lambda rows: torch.as_tensor(rows, device=model.device)
    st = generate_speculative(model, prompt, 40, k=4, flush=6, to_idx=to_idx)
    print(f"speculative: {st.rounds} rounds, {st.accepted}/{st.drafted} accepted, {st.flushes} flushes, "
          f"{st.tokens_per_call:.2f} tokens per model call")
    assert st.tokens == want[0].tolist()
    assert st.drafted > 0


def test_two_decoders_on_two_streams_match_serial_runs(cuda_lib):
    """Two decoders of one model stepping on two streams of one device, issued alternately and
    from two host threads: the fork/join events of the LoRA side branch belong to the caller's
    stream, so the tokens equal those of the same decoders run one after the other."""
    import threading
    from rwkv_quant_b200 import synth
    from rwkv_quant_b200.backends.cuda import QuantRWKV7
    model = QuantRWKV7(synth.build_checkpoint("toy", "compression", seed=21))
    starts = [torch.tensor([3], device="cuda"), torch.tensor([7, 11], device="cuda")]

    def run_serial(B, t0, n=12):
        dec = model.decoder(B, use_graph=False)
        out, tok = [], t0
        for _ in range(n):
            tok = dec.step(tok).clone()
            out.append(tok.cpu())
        return torch.stack(out)

    want = [run_serial(1, starts[0]), run_serial(2, starts[1])]
    torch.cuda.synchronize()
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    # (a) one host thread, steps issued alternately on the two streams
    decs = [model.decoder(1, use_graph=False), model.decoder(2, use_graph=False)]
    toks, outs = [t.clone() for t in starts], [[], []]
    for _ in range(12):
        for i in (0, 1):
            with torch.cuda.stream(streams[i]):
                toks[i] = decs[i].step(toks[i]).clone()
                outs[i].append(toks[i])
    torch.cuda.synchronize()
    for i in (0, 1):
        assert torch.equal(torch.stack(outs[i]).cpu(), want[i]), f"decoder {i} (alternating streams)"
    # (b) two host threads, one stream each
    decs = [model.decoder(1, use_graph=False), model.decoder(2, use_graph=False)]
    res, errs = [None, None], []

    def worker(i):
        try:
            with torch.cuda.stream(streams[i]):
                tok, out = starts[i].clone(), []
                for _ in range(12):
                    tok = decs[i].step(tok).clone()
                    out.append(tok)
                streams[i].synchronize()
                res[i] = torch.stack(out).cpu()
        except Exception as e:      # noqa: BLE001
            errs.append(e)

    th = [threading.Thread(target=worker, args=(i,)) for i in (0, 1)]
    [t.start() for t in th]
    [t.join() for t in th]
    assert not errs, errs
    for i in (0, 1):
        assert torch.equal(res[i], want[i]), f"decoder {i} (two threads)"


@pytest.mark.parametrize("preset", ["reduction", "compression"])
@pytest.mark.parametrize("B", [3, 9, 20, 40, 70])
def test_decode_batches_match_oracle(cuda_lib, preset, B):
    """Batched decode on the reference-written toy files: 3..8 streams (small-batch linears, per-
    stream LoRA kernels), 9..64 (tensor-core LoRA pair: one, two and four 16-stream tiles) and
    more than 64 (two stream groups), 4 teacher-forced tokens, logits and states against the oracle."""
    model, oracle, _ = _load(preset)
    toks = np.random.default_rng(B).integers(1, 500, (B, 4))
    ref_st = oracle.init_state(B)
    dec = model.decoder(B, use_graph=False)
    tk = torch.from_numpy(toks).cuda()
    for t in range(4):
        ref, ref_st = oracle.forward_stateful(toks[:, t:t + 1], ref_st)
        dec.step(tk[:, t])
        err = relmax(dec.logits.cpu().numpy(), ref[:, 0])
        assert err <= 1e-3, (t, err)
    for (w, ts, cs), (rw, rts, rcs) in zip(dec.states, ref_st):
        assert float(np.abs(w.cpu().numpy() - rw).max()) <= 1e-3 * max(1.0, np.abs(rw).max())
        assert relmax(ts.reshape(B, -1).cpu().numpy(), rts) <= 1e-3
        assert relmax(cs.reshape(B, -1).cpu().numpy(), rcs) <= 1e-3


@pytest.mark.parametrize("D,n", [(256, 3), (256, 17), (2048, 64), (2048, 130), (2560, 700)])
def test_lora_pair_matches_numpy(cuda_lib, D, n):
    """rwkvq_lora_pair through the C ABI: four branches (asym@6 w / a / v, per-row int8 g; tanh / none /
    sigmoid / none) in two launches against y = act(x @ W1) @ W2 in float64 with the loader's weight
    precision fp16(bf16(.)) (quant_model.py:128-154, 462-526), for one, two and four 16-row tiles, several
    64-row groups and a ragged last group.  rel <= 2e-5: fp16-pair operands, fp32 accumulation."""
    from rwkv_quant_b200 import synth
    from rwkv_quant_b200.backends.cuda import ops
    ranks = synth.lora_ranks(D)
    g = torch.Generator().manual_seed(D + n)
    pairs, acts, refs = [], [1, 0, 2, 0], []
    for br, fn, bits in (("w", synth.quant_asym, 6), ("a", synth.quant_asym, 6), ("g", synth.quant_rtn, 8), ("v", synth.quant_asym, 6)):
        r = ranks[br]
        q1 = fn(br + "1", "l", torch.randn(D, r, generator=g) * 0.05, bits)
        q2 = fn(br + "2", "l", torch.randn(r, D, generator=g) * 0.05, bits)
        d1, d2 = ops.DeviceQT(q1), ops.DeviceQT(q2)
        pairs.append((d1, d2))
        refs.append(tuple(d.dequant(torch.float32, True).half().double().cpu().numpy() for d in (d1, d2)))
    assert ops.lora_pair_ok(pairs, D)
    xs = [torch.randn(n, D, generator=g).cuda() for _ in range(4)]
    ys = ops.lora_pair(pairs, xs, acts)
    for i, (w1, w2) in enumerate(refs):
        h = xs[i].double().cpu().numpy() @ w1
        h = np.tanh(h) if acts[i] == 1 else 1 / (1 + np.exp(-h)) if acts[i] == 2 else h
        want = h @ w2
        assert ys[i].shape == (n, D) and relmax(ys[i].cpu().numpy(), want) <= 2e-5, (i, relmax(ys[i].cpu().numpy(), want))
    assert all(torch.equal(a, b) for a, b in zip(ys, ops.lora_pair(pairs, xs, acts))), "two calls differ"
    # three branches (layer 0 has no value-residual branch)
    ys3 = ops.lora_pair(pairs[:3], xs[:3], acts[:3])
    assert all(torch.equal(a, b) for a, b in zip(ys3, ys[:3]))


def test_seq_embed_and_layer_norm_kernels(cuda_lib):
    """Embedding gather + LayerNorm 0 and the final LayerNorm of the sequence path against torch on
    the loader-precision table."""
    import torch.nn.functional as F
    model, _, _ = _load("compression")
    idx = torch.from_numpy(np.random.default_rng(2).integers(0, model.vocab_size, (3, 19))).cuda()
    from rwkv_quant_b200.backends.cuda import ops
    got = ops.seq_embed_ln0(model.emb, idx, *model.ln0)
    want = F.layer_norm(model._embed(idx), (model.n_embd,), *model.ln0)
    assert got.shape == want.shape and (got - want).abs().max().item() <= 2e-6 * want.abs().max().item() + 1e-6
    x = torch.randn(7, 5, model.n_embd, device="cuda") * 3 + 1
    assert (ops.seq_layer_norm(x, *model.ln_out) - F.layer_norm(x, (model.n_embd,), *model.ln_out)).abs().max().item() <= 1e-5
