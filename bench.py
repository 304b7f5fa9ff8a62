#!/usr/bin/env python
"""Throughput benchmark of the quantized RWKV-7 forward path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--streams S] [--impl reference]

Workload (the line's `value`): greedy decode (tg128 of tests/bench_decode_vs_gguf.py:84-96) of a
seeded random-init RWKV-7 1.5B build in the `compression` recipe (sb6 int5 projections / head, int4
channel-mix, LoRA asym@6 / rtn@8) for S = 64 concurrent streams, split data-parallel over the N GPUs
(64/N streams per GPU, a full replica per GPU, no collective on the data path: strong scaling).  One
"step" is one decoded token for every stream.

One JSON line is printed by rank 0:
  value      tokens/s, whole job, token fed back on the device, one CUDA-graph replay per step,
             timed with CUDA events, max over ranks
  e2e        tokens/s through QuantRWKV7.decoder().step() with the token ids coming from pinned host
             memory and the argmax read back to the host every step
  roofline   the dominant kernel: the quantized-linear launches of one step (6 per layer + head) replayed
             as a graph; algorithmic bytes = their file-format bytes + activation rows, against the
             measured HBM copy bandwidth; `traffic` = the DRAM bytes of the same launches under ncu
  step_roofline  the whole step of one GPU: (file-format weight bytes + WKV state read and written for
             its streams) / step time
  fast_mode  (N = 1) the same step with RWKVQ_BATCH_FAST=1 arithmetic (single fp16 operands), for comparison
  b1         (N = 1) the single-stream configuration with its own device time, e2e and rooflines
  prefill    (N = 1) pp512 at batch 1 and 16 on a `reduction` build: tokens/s, e2e, FLOP rate against
             the measured bf16 tensor peak
  big        (N = 8) RWKV-7 2.9B, 256 streams, 32 per GPU
  cpu_baseline  the CPU oracle (numpy port of the reference forward) on the host cores, same workload
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

PUBLISHED_M4_TG128_COMPRESSION = 75.3       # tok/s, batch 1, Apple M4 (reference README.md:22, 40)
FALLBACK = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--streams", type=int, default=64, help="concurrent streams of the whole job")
    ap.add_argument("--model", default="1.5b")
    ap.add_argument("--recipe", default="compression")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the b1 / prefill / big blocks")
    ap.add_argument("--with-big", action="store_true", help="run the 2.9B 256-stream block at this N too (default: N = 8 only)")
    return ap.parse_args()


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            j = json.load(f)
        return {k: float(j[k]) for k in FALLBACK}, "measured"
    except Exception:  # noqa: BLE001
        return dict(FALLBACK), "fallback"


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
def cpu_threads():
    """All host cores for the BLAS behind numpy, whatever the launcher exported (torchrun sets
    OMP_NUM_THREADS=1); returns the thread count in use."""
    n = os.cpu_count() or 1
    try:
        import numpy  # noqa: F401  (the BLAS must be loaded before it can be configured)
        from threadpoolctl import threadpool_info, threadpool_limits
        threadpool_limits(limits=n)
        got = [p.get("num_threads") for p in threadpool_info() if p.get("user_api") == "blas"]
        return max(got) if got else n
    except Exception:  # noqa: BLE001
        return n


def cpu_decode_tok_s(model_name, recipe, streams, budget_s=20.0, seed=0):
    """tokens/s of the CPU oracle decoding `streams` concurrent streams on the full-depth build."""
    import numpy as np
    import torch
    from oracle import codec_np as oc
    from oracle.model_np import OracleRWKV7
    from rwkv_quant_b200 import synth
    from rwkv_quant_b200.formats import save_rwkvq
    threads = cpu_threads()
    dev = "cuda" if torch.cuda.is_available() else "cpu"       # the build is not part of the measurement
    ck = synth.build_checkpoint(model_name, recipe, seed=seed, device=dev, keep_on_device=False)
    path = f"/tmp/rwkvq_bench_cpu_{os.getpid()}.rwkvq"
    save_rwkvq(ck, path)
    n_layer = ck.n_layer
    del ck
    man, arr = oc.open_rwkvq(path)
    m = OracleRWKV7(man, arr)
    st = m.init_state(streams)
    tok = np.random.default_rng(0).integers(1, 60000, (streams, 1))
    logits, st = m.forward_stateful(tok, st)                      # warm
    tok = logits[:, -1].argmax(-1)[:, None]
    t0, n = time.perf_counter(), 0
    while n < 2 or (time.perf_counter() - t0 < budget_s and n < 128):
        logits, st = m.forward_stateful(tok, st)
        tok = logits[:, -1].argmax(-1)[:, None]
        n += 1
    sec = (time.perf_counter() - t0) / n
    os.remove(path)
    return streams / sec, {"steps_timed": n, "s_per_step": sec, "threads": threads, "n_layer": n_layer}


def run_reference(a, rank):
    if rank != 0:
        return
    v, info = cpu_decode_tok_s(a.model, a.recipe, a.streams, budget_s=25.0)
    sample = (f"{info['steps_timed']} decode steps of {a.streams} streams on the full {info['n_layer']}-layer build, "
              f"numpy fp32, weights dequantised once at load")
    line = {"impl": "reference", "metric": "decode_tokens_per_s", "value": v, "unit": "tok/s",
            "n_gpus": a.gpus, "steps": a.steps, "warmup": a.warmup, "ms_per_step": 1e3 * info["s_per_step"],
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": f"rwkv7-{a.model} {a.recipe} random-init, greedy decode, {a.streams} concurrent "
                                   f"streams, CPU oracle port (the Metal/MLX reference cannot run here)",
                       "threads": info["threads"]},
            "cpu_baseline": {"value": v, "unit": "tok/s", "cores": info["threads"], "kind": "port", "sample": sample},
            "e2e": {"value": v, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------ own arm
def state_bytes(model, B):
    """WKV state read and written per step for B streams."""
    return 2 * model.n_layer * model.n_head * 64 * 64 * 4 * B


def linear_phase(model, B, steps, warmup):
    """All quantized-linear launches of one step at batch B (6 per layer + head, the entry points the
    decode step itself uses) replayed as one CUDA graph: (bytes, launches, seconds per replay)."""
    import torch
    from rwkv_quant_b200 import _lib
    lib = _lib.load()
    dev = model.device
    D, F_ = model.n_embd, model.ffn_dim
    xd = torch.randn(B, D, device=dev)
    xf = torch.randn(B, F_, device=dev).abs()
    yd = torch.empty(B, D, device=dev)
    yf = torch.empty(B, F_, device=dev)
    yv = torch.empty(B, model.vocab_size, device=dev)
    mats = []
    for L in model.blocks:
        mats += [(L.Wr, xd, yd), (L.Wk, xd, yd), (L.Wv, xd, yd), (L.Wo, xd, yd), (L.Wfk, xd, yf), (L.Wfv, xf, yd)]
    mats.append((model.head, xd, yv))
    nbytes = sum(m[0].nbytes_file() + (m[1].numel() + m[2].numel()) * 4 for m in mats)
    ws = torch.empty(max(256, lib.rwkvq_gemv_batch_workspace_bytes(B)), dtype=torch.uint8, device=dev)

    def run():
        s = _lib.stream_ptr()
        for dq, x, y in mats:
            if B <= 2:
                _lib.check(lib.rwkvq_gemv(C.byref(dq.struct), x.data_ptr(), 0, B, x.shape[1], y.data_ptr(),
                                          y.shape[1], 0, None, s), "rwkvq_gemv")
            else:
                _lib.check(lib.rwkvq_gemv_batch(C.byref(dq.struct), x.data_ptr(), B, x.shape[1], y.data_ptr(),
                                                y.shape[1], 0, None, ws.data_ptr(), ws.numel(), s), "rwkvq_gemv_batch")
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
    return nbytes, len(mats) * (B if B <= 2 else 2), e0.elapsed_time(e1) * 1e-3 / steps


# dram__bytes_read.sum + dram__bytes_write.sum of the quantized-linear launches of one decoded token
# (1.5B compression, one stream), from the ncu capture summarised under profiles/
NCU_GEMV_PHASE_DRAM_BYTES_B1 = 828225280 + 342272
# the same for one step of 64 streams on the default (two-term) small-batch kernels: 24 x 45.60 MB per layer
# (r/k/v 12.63, output projection 6.11, ffn key 13.19, ffn value 13.68) + 101.84 MB for the head, from a 2-layer
# capture (profiles/decode_step_b64_b8_launch_list_1p5b_compression.md); traffic grows with the layer count
NCU_BATCH_PHASE_DRAM_BYTES_B64 = 24 * 45602560 + 101837824


def time_decode(model, B, prompt, steps, warmup, sync_all, clock_index=None, groups=None):
    """Device-resident loop (one graph replay per step, argmax fed back on the device) and the
    end-to-end loop (pinned host token ids in, argmax out, every step): (sec, sec_e2e, clocks, launches)."""
    import torch
    dec = model.decoder(B, use_graph=True, self_feed=True, groups=groups)
    dec.tokens.copy_(prompt)
    for _ in range(warmup):
        dec.step()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    with ClockSampler(clock_index if clock_index is not None else 0) as clk:
        e0.record()
        for _ in range(steps):
            dec.step()
        e1.record()
        torch.cuda.synchronize()
    sync_all()
    t_dev = e0.elapsed_time(e1) * 1e-3
    del dec
    dec2 = model.decoder(B, use_graph=True, self_feed=False, groups=groups)
    host_tok = torch.empty(B, dtype=torch.long).pin_memory()
    host_tok.copy_(prompt.cpu())
    host_out = torch.empty(B, dtype=torch.long).pin_memory()
    for _ in range(warmup):
        host_out.copy_(dec2.step(host_tok), non_blocking=False)
        host_tok.copy_(host_out)
    sync_all()
    e0.record()
    for _ in range(steps):
        nxt = dec2.step(host_tok)                     # H2D of the token ids + graph replay
        host_out.copy_(nxt, non_blocking=True)        # D2H of the result
        torch.cuda.current_stream().synchronize()
        host_tok.copy_(host_out)
    e1.record()
    torch.cuda.synchronize()
    sync_all()
    t_e2e = e0.elapsed_time(e1) * 1e-3
    del dec2
    return t_dev, t_e2e, clk.summary(), (model.launches_per_token + 1) * steps


def prefill_block(dev, model_name, peaks, peak_kind):
    """pp512 (one stateful call over 512 random token ids per sequence, logits of the last position)
    at batch 1 and 16 on a `reduction` build; e2e includes the token ids from pinned host memory and
    the argmax of the last position back on the host."""
    import torch
    from rwkv_quant_b200 import synth
    from rwkv_quant_b200.backends.cuda import QuantRWKV7
    ck = synth.build_checkpoint(model_name, "reduction", seed=0, device=dev)
    model = QuantRWKV7(ck, device=dev)
    del ck
    torch.cuda.empty_cache()
    mat_params = sum(getattr(L, nm).rows * getattr(L, nm).cols for L in model.blocks
                     for nm in ("Wr", "Wk", "Wv", "Wo", "Wfk", "Wfv"))
    lora_params = sum(getattr(L, nm).rows * getattr(L, nm).cols for L in model.blocks
                      for nm in ("w1", "w2", "a1", "a2", "g1", "g2", "v1", "v2") if getattr(L, nm) is not None)
    head_params = model.head.rows * model.head.cols
    out = {"build": f"{model_name} reduction", "peak_tflops": peaks["bf16_tflops_sustained"],
           "peak_kind": f"{peak_kind} bf16 cuBLAS, sustained (the pass is tens of milliseconds long)"}
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for b in (1, 16):
        host_idx = torch.randint(1, 60000, (b, 512)).pin_memory()
        host_out = torch.empty(b, dtype=torch.long).pin_memory()
        idx = host_idx.to(dev)
        for _ in range(3):                                                       # warm-up
            model.forward_stateful(idx, model.init_state(b), last_only=True)
        torch.cuda.synchronize()
        best, best_e2e = float("inf"), float("inf")
        for _ in range(3):
            st = model.init_state(b)
            e0.record()
            model.forward_stateful(idx, st, last_only=True)
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1) * 1e-3)
        for _ in range(3):
            st = model.init_state(b)
            e0.record()
            lo, _ = model.forward_stateful(host_idx.to(dev, non_blocking=True), st, last_only=True)
            host_out.copy_(lo[:, -1].argmax(-1), non_blocking=True)
            e1.record()
            torch.cuda.synchronize()
            best_e2e = min(best_e2e, e0.elapsed_time(e1) * 1e-3)
        flop = 2.0 * (mat_params + lora_params) * b * 512 + 2.0 * head_params * b
        out[f"pp512_b{b}"] = {"tok_s": b * 512 / best, "ms": best * 1e3, "e2e_tok_s": b * 512 / best_e2e,
                              "h2d_bytes": b * 512 * 8, "d2h_bytes": b * 8, "tflops": flop / best / 1e12,
                              "frac_of_peak": flop / best / 1e12 / peaks["bf16_tflops_sustained"]}
    del model
    torch.cuda.empty_cache()
    return out


def run_ours(a, rank, world, local_rank):
    import numpy as np
    import torch
    from rwkv_quant_b200 import _lib, dp, synth
    from rwkv_quant_b200.backends.cuda import QuantRWKV7, ops

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dp.init("nccl", dev)
    peaks, peak_kind = measured_peaks()
    peak = peaks["hbm_gbs"]
    ck = synth.build_checkpoint(a.model, a.recipe, seed=0, device=dev)
    model = QuantRWKV7(ck, device=dev)
    del ck
    torch.cuda.empty_cache()
    lo, hi = dp.shard_streams(a.streams, world, rank)
    B = hi - lo                                            # this GPU's streams
    if B < 1:
        raise SystemExit(f"{a.streams} streams cannot be split over {world} GPUs")
    w_bytes = model.weight_nbytes()

    def sync_all():
        torch.cuda.synchronize()
        dp.barrier()
        torch.cuda.synchronize()

    max_over_ranks = lambda sec: dp.max_over_ranks(sec, dev)
    prompts = torch.from_numpy(np.random.default_rng(0).integers(1, 60000, (a.streams,))).to(dev)
    model_groups = model.decode_groups(B)
    t_dev, t_e2e, clocks, launches = time_decode(model, B, prompts[lo:hi], a.steps, a.warmup, sync_all, local_rank)
    t_dev, t_e2e = max_over_ranks(t_dev), max_over_ranks(t_e2e)
    g_bytes, g_launches, g_sec = linear_phase(model, B, min(a.steps, 32), a.warmup)
    step_bytes = w_bytes + state_bytes(model, B)

    extras = {}
    fast_env = ops.batch_fast()
    if not a.no_extras and world == 1 and B > 2 and not fast_env:
        # the same step on single fp16 operands (what RWKVQ_BATCH_FAST=1 selects): faster, but its logits
        # drift to 2-3e-3 of the fp32 oracle over 24 layers, so it is not the default and not `value`
        lib = _lib.load()
        sw = lib.rwkvq_profiling_batch_fast            # rwkvq_profiling.h: not part of the C ABI
        sw.restype, sw.argtypes = None, [C.c_int]
        sw(1)
        try:
            tf, tf_e2e, _, lf = time_decode(model, B, prompts[lo:hi], a.steps, a.warmup, sync_all, local_rank, groups=1)
        finally:
            sw(-1)
        extras["fast_mode"] = {"value": a.streams * a.steps / tf, "unit": "tok/s", "ms_per_step": tf / a.steps * 1e3,
                               "e2e": {"value": a.streams * a.steps / tf_e2e, "unit": "tok/s"}, "gpu_launches": lf,
                               "what": "RWKVQ_BATCH_FAST=1: small-batch linears on single fp16 operands (tcgen05 kernel "
                                       "above 32 streams); logits within 1e-3 of the oracle on 2 layers, 2-3e-3 on 24"}
    if not a.no_extras and world == 1:
        # the single-stream configuration (the one the reference's tg128 number is quoted on)
        tb, tb_e2e, clk1, l1 = time_decode(model, 1, prompts[:1], a.steps, a.warmup, sync_all, local_rank)
        b_bytes, b_launches, b_sec = linear_phase(model, 1, min(a.steps, 64), a.warmup)
        sb = state_bytes(model, 1)
        extras["b1"] = {
            "value": a.steps / tb, "unit": "tok/s", "ms_per_step": tb / a.steps * 1e3,
            "e2e": {"value": a.steps / tb_e2e, "unit": "tok/s", "h2d_bytes_per_step": 8, "d2h_bytes_per_step": 8},
            "vs_baseline": (a.steps / tb) / PUBLISHED_M4_TG128_COMPRESSION if (a.model, a.recipe) == ("1.5b", "compression") else None,
            "vs_baseline_ref": "75.3 tok/s tg128, batch 1, Apple M4 (reference README): other hardware",
            "gpu_launches": l1, "clocks": clk1,
            "roofline": {"bound": "hbm", "achieved": (w_bytes + sb) / (tb / a.steps) / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": (w_bytes + sb) / (tb / a.steps) / 1e9 / peak, "traffic": None,
                         "what": "whole step: weight bytes + WKV state of one stream / step time"},
            "linear_phase": {"bound": "hbm", "achieved": b_bytes / b_sec / 1e9, "peak": peak, "unit": "GB/s",
                             "frac": b_bytes / b_sec / 1e9 / peak,
                             "traffic": NCU_GEMV_PHASE_DRAM_BYTES_B1 if (a.model, a.recipe) == ("1.5b", "compression") else None,
                             "kernel": f"gemv_mma_kernel, the {b_launches} quantized-linear launches of one token",
                             "bytes_per_replay": b_bytes, "us_per_replay": b_sec * 1e6}}
        del model
        torch.cuda.empty_cache()
        extras["prefill"] = prefill_block(dev, a.model, peaks, peak_kind)
        model = None
    if (not a.no_extras and world == 8) or a.with_big:
        # RWKV-7 2.9B, 256 concurrent streams, 32 per GPU
        del model
        torch.cuda.empty_cache()
        big = QuantRWKV7(synth.build_checkpoint("2.9b", a.recipe, seed=0, device=dev), device=dev)
        bb = 256 // world
        pr = torch.from_numpy(np.random.default_rng(1).integers(1, 60000, (256,))).to(dev)[rank * bb:(rank + 1) * bb]
        tg, tg_e2e, clk8, _ = time_decode(big, bb, pr, a.steps, a.warmup, sync_all, local_rank)
        tg, tg_e2e = max_over_ranks(tg), max_over_ranks(tg_e2e)
        bytes_gpu = big.weight_nbytes() + state_bytes(big, bb)
        extras["big"] = {"workload": f"rwkv7-2.9b {a.recipe} random-init, 256 streams, {bb} per GPU",
                         "value": 256 * a.steps / tg, "unit": "tok/s", "ms_per_step": tg / a.steps * 1e3,
                         "e2e": {"value": 256 * a.steps / tg_e2e, "unit": "tok/s", "h2d_bytes_per_step": 8 * bb,
                                 "d2h_bytes_per_step": 8 * bb},
                         "roofline": {"bound": "hbm", "achieved": bytes_gpu / (tg / a.steps) / 1e9, "peak": peak,
                                      "unit": "GB/s", "frac": bytes_gpu / (tg / a.steps) / 1e9 / peak, "traffic": None},
                         "clocks": clk8}
        del big
        model = None
    if rank != 0:
        dp.finalize()
        return
    total_tokens = a.streams * a.steps
    value = total_tokens / t_dev
    sec_step = t_dev / a.steps
    line = {
        "metric": "decode_tokens_per_s", "value": value, "unit": "tok/s", "n_gpus": world,
        "steps": a.steps, "warmup": a.warmup, "ms_per_step": sec_step * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": ("f16 operands (weights fp16(q*s+m), activations scaled per token) -> f32 accumulate" if fast_env else
                  "f16 operand pairs (weights q*s as product + rounding error, mins on block sums; activations hi + lo, "
                  "scaled per token) -> f32 accumulate") if B > 2
                 else "u8 codes x s8 activation digits -> s32, block scales and accumulation f32",
        "data": "synthetic",
        "config": {"workload": f"rwkv7-{a.model} {a.recipe} random-init, greedy decode tg{a.steps}, {a.streams} concurrent "
                               f"streams split over {world} GPU(s) ({B} per GPU), full replica per GPU",
                   "streams": a.streams, "streams_per_gpu": B, "weight_bytes_per_step": w_bytes,
                   "state_bytes_per_step": step_bytes - w_bytes,
                   "decoder": "CUDA-graph replay of the launch chain" +
                              (f", {model_groups} stream groups side by side" if model_groups > 1 else ""),
                   "precision": "RWKVQ_BATCH_FAST=1 (single fp16 operands)" if fast_env else "default (two-term operands)",
                   "l2": "weights per step (>= 800 MB) exceed the 126 MB L2; no flush needed",
                   "vs_baseline_ref": "no published number for the 64-stream metric; b1.vs_baseline divides by the "
                                      "reference's 75.3 tok/s at batch 1 on an Apple M4"},
        "e2e": {"value": total_tokens / t_e2e, "unit": "tok/s", "h2d_bytes_per_step": 8 * B, "d2h_bytes_per_step": 8 * B},
        "gpu_launches": launches,
        "clocks": clocks,
        "step_roofline": {"bound": "hbm", "achieved": step_bytes / sec_step / 1e9, "peak": peak, "unit": "GB/s",
                          "frac": step_bytes / sec_step / 1e9 / peak, "traffic": None, "peak_kind": peak_kind,
                          "what": "whole decode step of one GPU: file-format weight bytes + WKV state read and written "
                                  "for its streams, per step time",
                          "bytes_per_step": step_bytes, "us_per_step": sec_step * 1e6},
        "roofline": {"bound": "hbm", "achieved": g_bytes / g_sec / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": g_bytes / g_sec / 1e9 / peak, "peak_kind": peak_kind,
                         "traffic": NCU_BATCH_PHASE_DRAM_BYTES_B64 if (a.model, a.recipe, B, fast_env) == ("1.5b", "compression", 64, False) else None,
                         "what": "the dominant kernel (the mma.sync small-batch linear: 72 % of a 64-stream step in the ncu launch list "
                                 "when every linear runs on it, as timed here; the step itself runs r / k / v and the head on the "
                                 "tcgen05 form above 48 streams): file-format bytes of the quantized linears + their activation "
                                 "rows / time of those launches, all through rwkvq_gemv_batch, replayed as one graph",
                         "kernel": (f"row_amax_kernel + {'gemm_tcb_kernel' if (fast_env and B > 32) else 'gemv_batch_kernel'}, "
                                    f"the {g_launches} launches of the quantized linears of one step at "
                                    f"{B} streams" if B > 2 else f"gemv_mma_kernel, {g_launches} launches"),
                         "bytes_per_replay": g_bytes, "us_per_replay": g_sec * 1e6},
    }
    line.update(extras)
    if not a.no_cpu_baseline and world == 1:
        v, info = cpu_decode_tok_s(a.model, a.recipe, a.streams, budget_s=16.0)
        line["cpu_baseline"] = {"value": v, "unit": "tok/s", "cores": info["threads"], "kind": "port",
                                "sample": f"{info['steps_timed']} decode steps of {a.streams} streams on the full "
                                          f"{info['n_layer']}-layer build (numpy fp32, weights dequantised once)"}
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
