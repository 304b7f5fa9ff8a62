#!/usr/bin/env python
"""Decode-throughput benchmark of the quantized RWKV-7 forward path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--impl reference]

Workload: greedy decode (tg128 of tests/bench_decode_vs_gguf.py:84-96) of a seeded
random-init RWKV-7 1.5B build in the `compression` recipe (sb6 int5 projections / head,
int4 channel-mix, LoRA asym@6 / rtn@8), B independent streams per GPU.  One "step" is
one decoded token for every stream.  With N GPUs every rank holds a full replica and
its own B streams (no collective on the data path; weak scaling).

One JSON line is printed by rank 0:
  value      tokens/s, whole job, token fed back on the device, one CUDA-graph replay
             per token, timed with CUDA events, max over ranks
  e2e        tokens/s through QuantRWKV7.decoder().step() with the token ids coming
             from pinned host memory and the argmax read back to the host every step
  roofline   the quantized-linear GEMV launches of one token (6 per layer + head):
             file-format weight bytes / CUDA-event time, against the measured HBM peak
  cpu_baseline  the CPU oracle (numpy port of the reference forward) on the host cores
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

PUBLISHED_M4_TG128_COMPRESSION = 75.3       # tok/s, Apple M4 (reference README.md:22, 40)
FALLBACK_HBM_GBS = 6650.0


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=1, help="streams per GPU")
    ap.add_argument("--model", default="1.5b")
    ap.add_argument("--recipe", default="compression")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the b=64 decode and pp512 measurements")
    ap.add_argument("--decoder", default="chain", choices=["persistent", "chain"],
                    help="batch-1 decoder: one persistent kernel per token, or the launch chain")
    return ap.parse_args()


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:  # noqa: BLE001
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, text=True)
            self.t = threading.Thread(target=lambda: self.rows.extend(self.proc.stdout), daemon=True)
            self.t.start()
        except Exception:  # noqa: BLE001
            self.proc = None
        return self

    def __exit__(self, *a):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
            self.t.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            c = [x.strip() for x in r.split(",")]
            if len(c) < 6 or not c[0].isdigit():
                continue
            sm.append(int(c[0]))
            mx = max(mx, int(c[1]))
            reasons |= {n for n, v in zip(names, c[2:6]) if v.lower().startswith("active")}
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------ CPU arm (oracle port)
def cpu_decode_tok_s(model_name, recipe, seconds=20.0, seed=0):
    """tokens/s of the CPU oracle for the full-depth model, measured on a 2-layer build
    with the full width, vocabulary and head: t_token = (t_2layer_model - t_head) * L/2 + t_head."""
    import numpy as np
    import torch
    from oracle import codec_np as oc
    from oracle.model_np import OracleRWKV7
    from rwkv_quant_b200 import synth
    from rwkv_quant_b200.formats import save_rwkvq
    dims = synth.MODEL_DIMS[model_name]
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    ck = synth.build_checkpoint(model_name, recipe, seed=seed, device=dev, n_layer=2, keep_on_device=False)
    path = f"/tmp/rwkvq_bench_cpu_{os.getpid()}.rwkvq"
    save_rwkvq(ck, path)
    del ck
    man, arr = oc.open_rwkvq(path)
    m = OracleRWKV7(man, arr)
    st = m.init_state(1)
    tok = np.array([[17]])
    m.forward_stateful(tok, st)                       # warm
    t0, n = time.perf_counter(), 0
    while n < 3 or (time.perf_counter() - t0 < seconds / 2 and n < 64):
        logits, st = m.forward_stateful(tok, st)
        tok = logits[:, -1].argmax(-1)[:, None]
        n += 1
    t_tok = (time.perf_counter() - t0) / n
    x = np.random.default_rng(0).standard_normal((1, m.D)).astype(np.float32)
    t0 = time.perf_counter()
    for _ in range(5):
        _ = x @ m.head.T
    t_head = (time.perf_counter() - t0) / 5
    os.remove(path)
    L = dims["n_layer"]
    full = max(t_tok - t_head, 1e-9) * (L / 2.0) + t_head
    return 1.0 / full, {"tokens_timed": n, "s_per_token_2layer": t_tok, "s_head": t_head,
                        "threads": os.cpu_count()}


def run_reference(a, rank):
    if rank != 0:
        return
    t0 = time.perf_counter()
    vals = []
    for _ in range(max(1, min(a.steps, 3))):
        v, info = cpu_decode_tok_s(a.model, a.recipe, seconds=20.0)
        vals.append(v)
        if time.perf_counter() - t0 > 150:
            break
    v = sorted(vals)[len(vals) // 2]
    line = {"impl": "reference", "metric": "decode_tokens_per_s", "value": v, "unit": "tok/s",
            "n_gpus": a.gpus, "steps": a.steps, "warmup": a.warmup, "ms_per_step": 1e3 / v,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": f"rwkv7-{a.model} {a.recipe} greedy decode, batch 1, CPU oracle port "
                                   f"(numpy fp32, weights dequantised once)"},
            "cpu_baseline": {"value": v, "unit": "tok/s", "cores": os.cpu_count(), "kind": "port",
                             "sample": "2-layer build at full width/vocab, per-token time scaled to "
                                       f"{info['tokens_timed']} tokens x L/2 layers + head"},
            "e2e": {"value": v, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------ own arm
def gemv_phase(model, steps, warmup):
    """All quantized-linear GEMVs of one token (6 per layer + head) replayed as one CUDA
    graph: (file-format bytes, launches, seconds per replay)."""
    import torch
    from rwkv_quant_b200 import _lib
    lib = _lib.load()
    dev = model.device
    D, F_ = model.n_embd, model.ffn_dim
    xd = torch.randn(1, D, device=dev)
    xf = torch.randn(1, F_, device=dev).abs()
    yd = torch.empty(1, D, device=dev)
    yf = torch.empty(1, F_, device=dev)
    yv = torch.empty(1, model.vocab_size, device=dev)
    mats = []
    for L in model.blocks:
        mats += [(L.Wr, xd, yd), (L.Wk, xd, yd), (L.Wv, xd, yd), (L.Wo, xd, yd), (L.Wfk, xd, yf), (L.Wfv, xf, yd)]
    mats.append((model.head, xd, yv))
    nbytes = sum(m[0].nbytes_file() for m in mats)

    def run():
        s = _lib.stream_ptr()
        for dq, x, y in mats:
            _lib.check(lib.rwkvq_gemv(C.byref(dq.struct), x.data_ptr(), 0, 1, x.shape[1], y.data_ptr(),
                                      y.shape[1], 0, None, s), "rwkvq_gemv")
    st = torch.cuda.Stream(device=dev)
    st.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(st):
        run()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=st):
            run()
    torch.cuda.current_stream().wait_stream(st)
    for _ in range(warmup):
        g.replay()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(steps):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return nbytes, len(mats), e0.elapsed_time(e1) * 1e-3 / steps


# dram__bytes_read.sum + dram__bytes_write.sum of the quantized-linear GEMV launches of one decoded
# token (1.5B compression, b = 1), from the ncu capture summarised under profiles/
NCU_GEMV_PHASE_DRAM_BYTES = 828225280 + 342272


def other_configs(model, a, dev, w_bytes, peak):
    """The other configurations the metric names, measured in the same process on the same
    build: 64 concurrent decode streams and prefill pp512 (one stateful call over 512 random
    token ids, logits of the last position) at batch 1 and 16."""
    import torch
    out = {"build": f"{a.model} {a.recipe}"}
    dec = model.decoder(64, use_graph=True, self_feed=True)
    dec.tokens.copy_(torch.randint(1, 60000, (64,), device=dev))
    for _ in range(3):
        dec.step()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    n = 16
    e0.record()
    for _ in range(n):
        dec.step()
    e1.record()
    torch.cuda.synchronize()
    sec = e0.elapsed_time(e1) * 1e-3 / n
    state = 2 * model.n_layer * model.n_head * 64 * 64 * 4 * 64
    out["decode_b64"] = {"tok_s": 64 / sec, "ms_per_step": sec * 1e3, "hbm_gbs": (w_bytes + state) / sec / 1e9,
                         "frac_of_peak": (w_bytes + state) / sec / 1e9 / peak}
    del dec
    for b in (1, 16):
        idx = torch.randint(1, 60000, (b, 512), device=dev)
        model.forward_stateful(idx, model.init_state(b), last_only=True)          # warm-up
        torch.cuda.synchronize()
        best = float("inf")
        for _ in range(3):
            st = model.init_state(b)
            e0.record()
            model.forward_stateful(idx, st, last_only=True)
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1) * 1e-3)
        out[f"pp512_b{b}"] = {"tok_s": b * 512 / best, "ms": best * 1e3}
    return out


def run_ours(a, rank, world, local_rank):
    import torch
    import torch.distributed as dist
    from rwkv_quant_b200 import dp, synth
    from rwkv_quant_b200.backends.cuda import QuantRWKV7

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dp.init("nccl", dev)
    ck = synth.build_checkpoint(a.model, a.recipe, seed=0, device=dev)
    model = QuantRWKV7(ck, device=dev)
    del ck
    torch.cuda.empty_cache()
    B = a.batch
    w_bytes = model.weight_nbytes()
    state_bytes = 2 * model.n_layer * model.n_head * 64 * 64 * 4 * B

    def sync_all():
        torch.cuda.synchronize()
        dp.barrier()
        torch.cuda.synchronize()

    max_over_ranks = lambda sec: dp.max_over_ranks(sec, dev)

    prompt = torch.from_numpy(__import__("numpy").random.default_rng(rank).integers(1, 60000, (B,))).to(dev)
    # ---- device-resident loop: one graph replay per token, argmax fed back on the device
    persistent = a.decoder == "persistent"
    dec = model.decoder(B, use_graph=True, self_feed=True, persistent=persistent)
    dec_kind = type(dec).__name__
    dec.tokens.copy_(prompt)
    for _ in range(a.warmup):
        dec.step()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    with ClockSampler(local_rank) as clk:
        e0.record()
        for _ in range(a.steps):
            dec.step()
        e1.record()
        torch.cuda.synchronize()
    sync_all()
    t_dev = max_over_ranks(e0.elapsed_time(e1) * 1e-3)
    clocks = clk.summary()

    # ---- end to end: token ids from pinned host memory, argmax read back every step
    dec2 = model.decoder(B, use_graph=True, self_feed=False, persistent=persistent)
    host_tok = torch.empty(B, dtype=torch.long).pin_memory()
    host_tok.copy_(prompt.cpu())
    host_out = torch.empty(B, dtype=torch.long).pin_memory()
    for _ in range(a.warmup):
        host_out.copy_(dec2.step(host_tok), non_blocking=False)
        host_tok.copy_(host_out)
    sync_all()
    t0 = time.perf_counter()
    e0.record()
    for _ in range(a.steps):
        nxt = dec2.step(host_tok)                     # H2D of the token ids + graph replay
        host_out.copy_(nxt, non_blocking=True)        # D2H of the result
        torch.cuda.current_stream().synchronize()
        host_tok.copy_(host_out)
    e1.record()
    torch.cuda.synchronize()
    sync_all()
    t_e2e = max_over_ranks(max(e0.elapsed_time(e1) * 1e-3, 0.0))
    _ = t0

    # ---- roofline of the GEMV launches of one token
    g_bytes, g_launches, g_sec = gemv_phase(model, a.steps, a.warmup)
    peak, peak_kind = measured_peak()
    extras = None
    if world == 1 and B == 1 and not a.no_extras:
        extras = other_configs(model, a, dev, w_bytes, peak)
    if rank != 0:
        dp.finalize()
        return
    total_tokens = world * B * a.steps
    value = total_tokens / t_dev
    line = {
        "metric": "decode_tokens_per_s", "value": value, "unit": "tok/s", "n_gpus": world,
        "steps": a.steps, "warmup": a.warmup, "ms_per_step": t_dev / a.steps * 1e3,
        "higher_is_better": True, "scaling": "weak",
        "vs_baseline": (value / PUBLISHED_M4_TG128_COMPRESSION
                        if (a.model, a.recipe, B, world) == ("1.5b", "compression", 1, 1) else None),
        "dtype": "u8 codes x s8 activation digits -> s32, block scales and accumulation f32",
        "data": "synthetic",
        "config": {"workload": f"rwkv7-{a.model} {a.recipe} random-init, greedy decode tg{a.steps}, "
                               f"{B} stream(s) per GPU, full replica per GPU",
                   "streams_per_gpu": B, "weight_bytes_per_token": w_bytes,
                   "decoder": ("one persistent cooperative kernel per token" if dec_kind == "PersistentDecoder"
                               else "CUDA-graph replay of the launch chain"),
                   "state_bytes_per_step": state_bytes,
                   "l2": "weights per token (>= 800 MB) exceed the 126 MB L2; no flush needed",
                   "vs_baseline_ref": "75.3 tok/s tg128 on Apple M4 (reference README), other hardware"},
        "e2e": {"value": total_tokens / t_e2e, "unit": "tok/s", "h2d_bytes_per_step": 8 * B,
                "d2h_bytes_per_step": 8 * B},
        "gpu_launches": (dec.launches_per_step or (model.launches_per_token + 1)) * a.steps,
        "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": g_bytes / g_sec / 1e9, "peak": peak, "unit": "GB/s",
                     "frac": g_bytes / g_sec / 1e9 / peak,
                     "traffic": NCU_GEMV_PHASE_DRAM_BYTES if (a.model, a.recipe, B) == ("1.5b", "compression", 1) else None,
                     "traffic_source": "profiles/decode_gemv_phase_dram_traffic_1p5b_compression.md (ncu, one token)",
                     "peak_kind": peak_kind,
                     "kernel": f"gemv_mma_kernel, the {g_launches} quantized-linear launches of one token",
                     "bytes_per_replay": g_bytes, "us_per_replay": g_sec * 1e6},
        "whole_step": {"hbm_gbs": (w_bytes + state_bytes) / (t_dev / a.steps) / 1e9,
                       "frac_of_peak": (w_bytes + state_bytes) / (t_dev / a.steps) / 1e9 / peak},
    }
    if extras is not None:
        line["extras"] = extras
    if not a.no_cpu_baseline:
        v, info = cpu_decode_tok_s(a.model, a.recipe, seconds=16.0)
        line["cpu_baseline"] = {"value": v, "unit": "tok/s", "cores": os.cpu_count(), "kind": "port",
                                "sample": f"{info['tokens_timed']} tokens on a 2-layer build at full width / "
                                          f"vocabulary, scaled to {model.n_layer} layers + head"}
    print(json.dumps(line), flush=True)
    dp.finalize()


def main():
    a = parse()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if a.impl == "reference":
        run_reference(a, rank)
        return
    if world == 1 and a.gpus > 1:
        # launched without torchrun: re-launch one process per GPU
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={a.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", "29533", os.path.abspath(__file__)] + sys.argv[1:]
        sys.exit(subprocess.call(cmd))
    run_ours(a, rank, world, local_rank)


if __name__ == "__main__":
    main()
