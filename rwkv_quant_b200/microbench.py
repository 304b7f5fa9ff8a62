"""Small single-purpose runs for profiling and A/B timing.

    python -m rwkv_quant_b200.microbench gemv LAYOUT BITS ROWS COLS [--n N] [--launches K]
    python -m rwkv_quant_b200.microbench decode [--layers L] [--recipe R] [--steps S] [--batch B]
    python -m rwkv_quant_b200.microbench sweep          # GEMV shapes of the 1.5B model, GB/s each
    python -m rwkv_quant_b200.microbench prefill [--T 512] [--batch B] [--recipe R]
    python -m rwkv_quant_b200.microbench wkv [--batch B] [--T 512] [--H 32]   # the WKV-7 scan alone
    python -m rwkv_quant_b200.microbench spec [--k 4] [--flush 8]            # speculative vs plain greedy decode

`gemv` and `decode` do a handful of launches and exit (suitable under a profiler);
`sweep` replays a ring of distinct weight buffers (working set >> L2) as a CUDA graph and
prints microseconds per launch and GB/s of file-format bytes.
"""
from __future__ import annotations

import argparse
import contextlib
import ctypes as C

import numpy as np
import torch

from . import _lib, synth
from .backends.cuda import QuantRWKV7, ops

_Q = {"sb6": synth.quant_sb6, "sym": synth.quant_sym, "rtn": synth.quant_rtn}


def _tensor(layout, bits, rows, cols, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    w = torch.randn(rows, cols, device="cuda", generator=g) * 0.02
    return ops.DeviceQT(_Q[layout]("w", "g", w, bits))


def gemv(layout, bits, rows, cols, n=1, launches=4, zero_groups=0.0):
    """A few plain rwkvq_gemv launches on different tensors (the target of ncu captures);
    zero_groups: share of the 32-column groups of x that are exactly zero."""
    lib = _lib.load(check_device=True)
    dqs = [_tensor(layout, bits, rows, cols, s) for s in range(launches)]
    x = torch.randn(n, cols, device="cuda")
    if zero_groups > 0:
        keep = torch.rand(n, cols // 32, device="cuda") >= zero_groups
        x = (x.view(n, cols // 32, 32) * keep[..., None]).reshape(n, cols).contiguous()
    y = torch.empty(n, rows, device="cuda")
    for d in dqs:
        _lib.check(lib.rwkvq_gemv(C.byref(d.struct), x.data_ptr(), 0, n, cols, y.data_ptr(), rows, 0, None,
                                  _lib.stream_ptr()), "rwkvq_gemv")
    torch.cuda.synchronize()
    print("ok", float(y.abs().sum()))


def decode(layers=4, recipe="compression", steps=3, batch=1, model="1.5b"):
    ck = synth.build_checkpoint(model, recipe, seed=0, device="cuda", n_layer=layers)
    m = QuantRWKV7(ck)
    del ck
    dec = m.decoder(batch, use_graph=False)
    for _ in range(steps):
        dec.step()
        dec.feed_back()
    torch.cuda.synchronize()
    print("ok", dec.next_tokens.tolist())


def tp_model_time(model="2.9b", recipe="compression", exchange="p2p", layers=32, steps=8):
    """Whole-model head-sharded decode (tp_model.TPQuantRWKV7, launches issued from Python) for the
    ranks of a torchrun launch: milliseconds per single-token step at 1 and 64 streams and per
    pp512 pass, max over ranks, beside the same calls on one GPU through the same Python path
    and through the one-call decode step."""
    import os

    import torch.distributed as dist

    from . import tp, tp_model
    rank, local = int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    ck = synth.build_checkpoint(model, recipe, seed=0, device=dev, n_layer=layers)
    g = tp.TPGroup(device=dev, exchange=exchange)
    m = tp_model.TPQuantRWKV7(ck, g, device=dev)
    ref = QuantRWKV7(ck, device=dev)

    def timed(fn, n):
        fn()
        torch.cuda.synchronize(); dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record(); torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / n], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())
    for B in (1, 64):
        tok = torch.randint(1, 60000, (B, 1), device=dev)
        st_t, st_r, st_c = m.init_state(B), ref.init_state(B), ref._materialize(ref.init_state(B), B)
        t_tp = timed(lambda: m.forward_stateful(tok, st_t), steps)
        x1, _ = ref.forward_hidden(tok, st_r)          # same Python path on one GPU
        t_py = timed(lambda: ref.forward_hidden(tok, st_r), steps)
        t_c = timed(lambda: ref._decode(tok.reshape(B), st_c), steps)
        dec_t = m.decoder(B, use_graph=True)
        t_tpg = timed(lambda: dec_t.step(), 4 * steps)
        dec_1 = ref.decoder(B, use_graph=True, self_feed=True)
        t_1g = timed(lambda: dec_1.step(), 4 * steps)
        del dec_t, dec_1
        if rank == 0:
            print(f"tp-model {model} {recipe} {layers} layers x{g.world} ({exchange}), {B} stream(s): plain calls {t_tp:.2f} ms per step, "
                  f"graph replay {t_tpg:.2f} ms; one GPU: same Python path {t_py:.2f} ms, one-call decode step {t_c:.2f} ms, "
                  f"its graph replay {t_1g:.2f} ms", flush=True)
    idx = torch.randint(1, 60000, (1, 512), device=dev)
    t_tp = timed(lambda: m.forward_stateful(idx, m.init_state(1), last_only=True), 2)
    t_1 = timed(lambda: ref.forward_stateful(idx, ref.init_state(1), last_only=True), 2)
    if rank == 0:
        print(f"tp-model pp512 batch 1: {t_tp:.1f} ms on {g.world} GPUs, {t_1:.1f} ms on one", flush=True)
    g.close()
    dist.destroy_process_group()


def tp_chain(model="2.9b", recipe="compression", exchange="p2p", iters=200):
    """Row-split tensor-parallel GEMV chain of one layer (output projection, ffn key, ffn
    value: three exchanges) plus the head, for the ranks of a torchrun launch (one process
    per GPU).  Prints microseconds per layer chain and per head, max over ranks, as a CUDA
    graph when the exchange allows it (peer stores) and as plain launches otherwise."""
    import os

    import torch.distributed as dist

    from . import tp
    rank, local = int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
    world = dist.get_world_size()
    dims = synth.MODEL_DIMS[model]
    D, F, V = dims["n_embd"], dims["ffn"], dims["vocab"]
    bits = {"compression": ("sb6", 5, "sb6", 4), "reduction": ("sym", 8, "sym", 6)}[recipe]

    def lin(layout, b, rows, cols, seed):
        g = torch.Generator().manual_seed(seed)
        w = torch.randn(rows, cols, generator=g) * 0.02
        fn = {"sb6": synth.quant_sb6, "sym": synth.quant_sym}[layout]
        return ops.DeviceQT(fn("w", "g", w, b), device=dev)

    out, key = lin(bits[0], bits[1], D, D, 1), lin(bits[2], bits[3], F, D, 2)
    val, head = lin(bits[2], bits[3], D, F, 3), lin(bits[0], bits[1], V, D, 4)
    x = torch.randn(D, device=dev)
    if exchange == "none":                     # every rank computes the whole matrices (no split)
        class _Whole:
            def __init__(self, dq): self.dq = dq
            def __call__(self, v, epi=0, resid=None):
                return ops.gemv(self.dq.bufs, self.dq.meta, v.reshape(1, -1), epi,
                                None if resid is None else resid.reshape(1, -1))[0]
        g = None
        lo, lk, lv, lh = _Whole(out), _Whole(key), _Whole(val), _Whole(head)
        split = 1
    else:
        g = tp.TPGroup(device=dev, exchange=exchange)
        lo, lk = tp.TPRowLinear(g, out, "out", 64), tp.TPRowLinear(g, key, "key", 64)
        lv, lh = tp.TPRowLinear(g, val, "value", 64), tp.TPRowLinear(g, head, "head", 64)
        split = world

    def layer(x):
        a = lo(x, 2, x)
        return lv(lk(a, 1), 2, a)

    def timed(fn, n):
        """fn replayed n times as one CUDA graph (plain launches if capture is refused)."""
        for _ in range(4):                     # an even count keeps the sites' buffer parity
            fn()
        torch.cuda.synchronize(); dist.barrier()
        graph = None
        try:
            st = torch.cuda.Stream(device=dev)
            st.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(st):
                graph = torch.cuda.CUDAGraph()
                with (g.graph_capture() if g is not None else contextlib.nullcontext()):
                    with torch.cuda.graph(graph, stream=st):
                        fn(); fn()
            torch.cuda.current_stream().wait_stream(st)
        except Exception as e:                 # noqa: BLE001 - report and fall back
            if rank == 0:
                print("graph capture refused:", str(e)[:120])
            graph = None
        run = (lambda: graph.replay()) if graph is not None else (lambda: (fn(), fn()))
        run(); torch.cuda.synchronize(); dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n // 2):
            run()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) * 1e3 / (2 * (n // 2))], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    t_layer = timed(lambda: layer(x), iters)
    t_head = timed(lambda: lh(x), iters)
    if g is not None:
        g.check()
    wbytes = (out.nbytes_file() + key.nbytes_file() + val.nbytes_file())
    if rank == 0:
        print(f"tp chain {model} {recipe} world {world} exchange {exchange}: layer (o, key, value) {t_layer:.1f} us "
              f"({wbytes / split / t_layer / 1e3:.0f} GB/s per GPU), head {t_head:.1f} us "
              f"({head.nbytes_file() / split / t_head / 1e3:.0f} GB/s per GPU)", flush=True)
    if g is not None:
        g.close()
    dist.barrier()
    dist.destroy_process_group()


def gemm_sweep(recipe="compression", Ms=(64, 512, 8192), reps=20, acc_mode=0):
    """rwkvq_gemm (pre-pass + tensor-core kernel) on the four linear shapes of a 1.5B layer
    and the head: microseconds per call (CUDA-graph replay, so that host time does not
    count) and TFLOP/s = 2 * M * OUT * IN / time.  acc_mode: 0 the launcher's tile choice,
    1 128-row tiles only, 2 256-row tiles wherever legal."""
    f = _lib.load().rwkvq_profiling_gemm_acc_mode      # rwkvq_profiling.h: not part of the C ABI
    f.restype, f.argtypes = None, [C.c_int]
    f(acc_mode)
    lay = {"compression": [("sb6", 5, 2048, 2048), ("sb6", 4, 8192, 2048), ("sb6", 4, 2048, 8192), ("sb6", 5, 65536, 2048)],
           "reduction": [("sym", 8, 2048, 2048), ("sym", 6, 8192, 2048), ("sym", 6, 2048, 8192), ("sym", 8, 65536, 2048)]}[recipe]
    for layout, bits, rows, cols in lay:
        dq = _tensor(layout, bits, rows, cols)
        for M in Ms:
            if rows == 65536 and M > 512:
                continue                                   # the head sees the last token of each sequence only
            x = torch.randn(M, cols, device="cuda")
            ops.gemm(dq, x, check=True)
            st = torch.cuda.Stream()
            st.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(st):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=st):
                    y = ops.gemm(dq, x)
            torch.cuda.current_stream().wait_stream(st)
            g.replay(); torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                g.replay()
            e1.record(); torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / reps
            print(f"gemm {layout}@{bits} [{rows},{cols}] M={M}: {us:8.1f} us  {2.0 * M * rows * cols / us / 1e6:7.1f} TFLOP/s", flush=True)


def batch_sweep(recipe="compression", Ns=(8, 64), reps=40, ring=24):
    """rwkvq_gemv_batch on the linear shapes of a 1.5B layer and the head: microseconds per launch in
    a CUDA graph over a ring of distinct weight copies (working set beyond the L2), GB/s of file
    bytes, and the in-kernel marks of CTA (0,0,0) for one launch."""
    lib = _lib.load()
    tr = lib.rwkvq_profiling_batch_trace            # rwkvq_profiling.h: not part of the C ABI
    tr.restype, tr.argtypes = None, [C.c_void_p, C.c_int]
    lay = {"compression": [("sb6", 5, 2048, 2048), ("sb6", 4, 8192, 2048), ("sb6", 4, 2048, 8192), ("sb6", 5, 65536, 2048)],
           "reduction": [("sym", 8, 2048, 2048), ("sym", 6, 8192, 2048), ("sym", 6, 2048, 8192), ("sym", 8, 65536, 2048)]}[recipe]
    for layout, bits, rows, cols in lay:
        n_ring = 2 if rows == 65536 else ring
        dqs = [_tensor(layout, bits, rows, cols, seed=i) for i in range(n_ring)]
        for N in Ns:
            x = torch.randn(N, cols, device="cuda")
            y = torch.empty(N, rows, device="cuda")
            ws = torch.empty(max(256, lib.rwkvq_gemv_batch_workspace_bytes(N)), dtype=torch.uint8, device="cuda")
            tf = lib.rwkvq_profiling_tcb_force
            tf.restype, tf.argtypes = None, [C.c_int]
            for ks in (0, 4, 8, 16):                          # forced cluster size of the tcgen05 kernel
                tr(None, 0)
                tf(ks)

                def run():
                    for dq in dqs:
                        _lib.check(lib.rwkvq_gemv_batch(C.byref(dq.struct), x.data_ptr(), N, cols, y.data_ptr(), rows, 0,
                                                        None, ws.data_ptr(), ws.numel(), _lib.stream_ptr()), "rwkvq_gemv_batch")
                run()
                st = torch.cuda.Stream()
                st.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(st):
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=st):
                        run()
                torch.cuda.current_stream().wait_stream(st)
                g.replay(); torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(reps):
                    g.replay()
                e1.record(); torch.cuda.synchronize()
                us = e0.elapsed_time(e1) * 1e3 / reps / n_ring
                buf = torch.zeros(16, dtype=torch.int64, device="cuda")
                tr(buf.data_ptr(), 0)
                _lib.check(lib.rwkvq_gemv_batch(C.byref(dqs[0].struct), x.data_ptr(), N, cols, y.data_ptr(), rows, 0, None,
                                                ws.data_ptr(), ws.numel(), _lib.stream_ptr()), "rwkvq_gemv_batch")
                torch.cuda.synchronize()
                tr(None, 0)
                tf(0)
                m = buf.cpu().numpy().astype(np.float64)
                marks = " ".join(f"{(m[i] - m[0]) * 1e-3:.1f}" for i in range(1, 9))
                print(f"batch {layout}@{bits} [{rows},{cols}] N={N} ks={ks or 'auto'}: {us:7.1f} us/launch "
                      f"{dqs[0].nbytes_file() / us / 1e3:7.0f} GB/s   marks(us) {marks}", flush=True)
        del dqs
        torch.cuda.empty_cache()


def batch_once(layout="sb6", bits=4, rows=8192, cols=2048, n=64, launches=3, tcgen05=False):
    """A few plain rwkvq_gemv_batch launches, each on its own tensor (cold weights): the target of
    ncu captures of the small-batch kernels.  tcgen05: the tensor-memory form of the kernel (two-term
    in the default precision) instead of the mma.sync form."""
    lib = _lib.load(check_device=True)
    if tcgen05:
        tf = lib.rwkvq_profiling_tcb_force           # rwkvq_profiling.h: not part of the C ABI
        tf.restype, tf.argtypes = None, [C.c_int]
        tf(1000)
    dqs = [_tensor(layout, bits, rows, cols, s) for s in range(launches)]
    x = torch.randn(n, cols, device="cuda")
    for d in dqs:
        y = ops.gemv_batch(d, x, check=True)
    torch.cuda.synchronize()
    print("ok", float(y.abs().sum()))


def batch_tune(layers=4, batch=64, recipe="compression", model="1.5b", reps=20):
    """Step time of a `layers`-layer decode graph at `batch` streams with the small-batch linear's
    launch geometry forced, one tensor shape at a time (cluster size x rows per group): what the
    launcher's cost model is calibrated against."""
    lib = _lib.load()
    force = lib.rwkvq_profiling_batch_force          # rwkvq_profiling.h: not part of the C ABI
    force.restype, force.argtypes = None, [C.c_int, C.c_int, C.c_int]
    ck = synth.build_checkpoint(model, recipe, seed=0, device="cuda", n_layer=layers)
    m = QuantRWKV7(ck)
    del ck
    D, F_, V = m.n_embd, m.ffn_dim, m.vocab_size

    def step_us():
        dec = m.decoder(batch, use_graph=True, self_feed=True)
        for _ in range(3):
            dec.step()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(reps):
            dec.step()
        e1.record(); torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / reps
    force(0, 0, 0)
    base = step_us()
    print(f"batch-tune {model} {recipe} {layers} layers, {batch} streams: launcher's choice {base:.1f} us/step", flush=True)
    for rows, cols, name in ((D, D, "r/k/v, o"), (F_, D, "ffn.key"), (D, F_, "ffn.value"), (V, D, "head")):
        out = []
        for tp in (32, 16):
            for ks in (1, 2, 4, 5, 8):
                force(ks | tp, rows, cols)
                try:
                    out.append((step_us() - base, ks, 128 if tp == 32 else 256))
                except Exception as e:      # noqa: BLE001
                    out.append((float("nan"), ks, 128 if tp == 32 else 256))
        force(0, 0, 0)
        print(f"  [{rows},{cols}] {name}: " + "  ".join(f"ks{k}/{r}:{d:+.0f}" for d, k, r in out), flush=True)


def decode_groups(layers=24, batch=64, recipe="compression", model="1.5b", reps=20):
    """Step time of batched decode with the streams split into 1, 2, 4, 8 groups whose launch
    chains run as parallel branches of the graph."""
    ck = synth.build_checkpoint(model, recipe, seed=0, device="cuda", n_layer=layers)
    m = QuantRWKV7(ck)
    del ck
    for g in (1, 2, 4, 8):
        if g > batch:
            break
        dec = m.decoder(batch, use_graph=True, self_feed=True, groups=g)
        for _ in range(3):
            dec.step()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(reps):
            dec.step()
        e1.record(); torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / reps
        print(f"decode {model} {recipe} {layers} layers, {batch} streams in {g} group(s): {us:.0f} us/step, {batch / us * 1e6:.0f} tok/s", flush=True)
        del dec


def gemm_once(layout="sb6", bits=5, rows=2048, cols=2048, M=8192, launches=3):
    """A few plain rwkvq_gemm launches of one shape (the target of ncu captures)."""
    dq = _tensor(layout, bits, rows, cols)
    x = torch.randn(M, cols, device="cuda")
    for _ in range(launches):
        y = ops.gemm(dq, x, check=True)
    torch.cuda.synchronize()
    print("ok", float(y.abs().sum()))


def gemm_timeline(layout="sb6", bits=5, rows=2048, cols=2048, M=8192, acc_mode=0):
    """Pipeline timeline of CTA (0,0,0) of one rwkvq_gemm launch: per macro-iteration
    when its weight stage was free, converted, seen full by the issuer and issued."""
    import numpy as np
    f = _lib.load().rwkvq_profiling_gemm_acc_mode      # rwkvq_profiling.h: not part of the C ABI
    f.restype, f.argtypes = None, [C.c_int]
    f(acc_mode)
    dq = _tensor(layout, bits, rows, cols)
    x = torch.randn(M, cols, device="cuda")
    ops.gemm(dq, x, check=True)
    buf = torch.zeros(512, dtype=torch.int64, device="cuda")
    lib = _lib.load()
    _trace = lib.rwkvq_profiling_gemm_trace          # rwkvq_profiling.h: not part of the C ABI
    _trace.restype, _trace.argtypes = None, [C.c_void_p]
    _trace(buf.data_ptr())
    ops.gemm(dq, x)
    torch.cuda.synchronize()
    _trace(None)
    t = buf.cpu().numpy().astype(np.float64)
    t0 = t[0]
    n = sum(1 for i in range(120) if t[8 + 4 * i] > 0)
    us = lambda v: (v - t0) / 1e3
    print(f"gemm timeline {layout}@{bits} [{rows},{cols}] M={M}: accumulator complete {us(t[1]):.2f} us, CTA end {us(t[2]):.2f} us, {n} macro-iterations")
    print("  i  stage free  converted  issuer full  issued")
    for i in range(n):
        r = t[8 + 4 * i: 12 + 4 * i]
        print(f"{i:3d} {us(r[1]) if r[1] else 0:10.2f} {us(r[0]):10.2f} {us(r[2]):12.2f} {us(r[3]):7.2f}")


def prefill(layers=24, recipe="reduction", T=512, batch=1, model="1.5b", reps=3):
    """pp{T}: one stateful call over a prompt of T tokens, logits for the last position."""
    ck = synth.build_checkpoint(model, recipe, seed=0, device="cuda", n_layer=layers)
    m = QuantRWKV7(ck)
    del ck
    g = torch.Generator().manual_seed(0)
    idx = torch.randint(1, 60000, (batch, T), generator=g).cuda()
    m.forward_stateful(idx, m.init_state(batch), last_only=True)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    best = 1e9
    for _ in range(reps):
        st = m.init_state(batch)
        e0.record()
        m.forward_stateful(idx, st, last_only=True)
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1))
    print(f"pp{T} batch {batch} {recipe} {layers} layers: {best:.2f} ms  {batch * T / best * 1e3:.0f} tok/s", flush=True)


def time_ring(layout, bits, rows, cols, n=1, ring_bytes=1.5e9, iters=5, zero_groups=0.0):
    lib = _lib.load(check_device=True)
    base = _tensor(layout, bits, rows, cols)
    nb = base.nbytes_file()
    k = max(2, min(64, int(ring_bytes // nb)))
    ring = [base]
    for _ in range(k - 1):
        d = object.__new__(ops.DeviceQT)
        d.__dict__.update(base.__dict__)
        d.bufs = [b.clone() if b.numel() else b for b in base.bufs]
        d.struct = ops._descr(d.bufs, d.meta)
        ring.append(d)
    x = torch.randn(n, cols, device="cuda")
    if zero_groups > 0:          # whole groups of 32 activations exactly zero (relu(k)^2 in the channel mix)
        keep = torch.rand(n, cols // 32, device="cuda") >= zero_groups
        x = (x.view(n, cols // 32, 32) * keep[..., None]).reshape(n, cols).contiguous()
    y = torch.empty(n, rows, device="cuda")

    def run():
        s = _lib.stream_ptr()
        for d in ring:
            lib.rwkvq_gemv(C.byref(d.struct), x.data_ptr(), 0, n, cols, y.data_ptr(), rows, 0, None, s)
    st = torch.cuda.Stream()
    st.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(st):
        run()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=st):
            run()
    torch.cuda.current_stream().wait_stream(st)
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    best = 1e9
    for _ in range(iters):
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1))
    us = best * 1e3 / k
    print(f"{layout}{bits} [{rows},{cols}] N={n}" + (f" {zero_groups:.0%} zero groups" if zero_groups else "") +
          f": {us:8.2f} us/launch {nb / us / 1e3:8.1f} GB/s ({nb / 1e6:.2f} MB, ring {k})", flush=True)
    return us


def quantize_time(rows=10240, cols=2560, reps=5):
    """rwkvq_quantize_sb6 (scale search + least-squares refit) on one channel-mix matrix of RWKV-7 2.9B:
    milliseconds per call and weights per second, kernel only and with the bit packing."""
    from . import quantize
    w = torch.randn(rows, cols, device="cuda") * 0.02
    for bits in (4, 5, 6):
        quantize.quantize_sb6_parts(w, bits)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize(); e0.record()
        for _ in range(reps):
            quantize.quantize_sb6_parts(w, bits)
        e1.record(); torch.cuda.synchronize()
        ms_k = e0.elapsed_time(e1) / reps
        e0.record()
        for _ in range(reps):
            quantize.quantize_sb6("k", "cmix", w, bits)
        e1.record(); torch.cuda.synchronize()
        ms_p = e0.elapsed_time(e1) / reps
        print(f"quantize sb6@{bits} [{rows},{cols}] search: kernel {ms_k:.2f} ms ({rows * cols / ms_k / 1e6:.1f} G weights/s), "
              f"with packing {ms_p:.2f} ms", flush=True)


def sparse_sweep():
    """The exact zero-group skip of the single-vector GEMV: launch time against the share of
    32-column groups whose activations are all zero (file bytes / time, so the rate rises)."""
    sw = _lib.load().rwkvq_profiling_zero_skip      # rwkvq_profiling.h: the skip is opt-in (RWKVQ_ZERO_SKIP=1)
    sw.restype, sw.argtypes = None, [C.c_int]
    sw(1)
    for args in [("sb6", 4, 2048, 8192), ("sb6", 5, 65536, 2048), ("sym", 6, 2048, 8192)]:
        for z in (0.0, 0.35, 0.7):
            time_ring(*args, zero_groups=z)
    sw(-1)


def sweep():
    for args in [("sb6", 4, 8192, 2048), ("sb6", 4, 2048, 8192), ("sb6", 5, 2048, 2048), ("sb6", 5, 65536, 2048),
                 ("sb6", 6, 8192, 2048), ("sym", 8, 2048, 2048), ("sym", 6, 8192, 2048), ("sym", 6, 2048, 8192),
                 ("sym", 8, 65536, 2048), ("rtn", 8, 8192, 2048)]:
        time_ring(*args)
    time_ring("sb6", 4, 8192, 2048, n=8)


def wkv(B, T, H, launches=6):
    """rwkvq_wkv7 alone on random rows: microseconds per launch (inputs rotate over sets that
    together exceed L2 when one set does not)."""
    from .backends.cuda.wkv7 import wkv7_infer
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(5)
    set_bytes = 7 * B * T * H * 64 * 4
    n_sets = max(2, min(8, int(300e6 // set_bytes) + 1))
    rnd = lambda: torch.randn(B, T, H, 64, device=dev, generator=g) * 0.5
    sets = []
    for _ in range(n_sets):
        r, k, v = rnd(), rnd(), rnd()
        w = torch.exp(-0.606531 * torch.sigmoid(rnd()))
        kk = torch.nn.functional.normalize(rnd(), dim=-1)
        sets.append((r, w, k, v, -kk, kk * torch.sigmoid(rnd())))
    st = torch.zeros(B, H, 64, 64, device=dev)
    for i in range(3):
        wkv7_infer(*sets[i % n_sets], st)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(launches + 1)]
    torch.cuda.synchronize()
    ev[0].record()
    for i in range(launches):
        wkv7_infer(*sets[i % n_sets], st)
        ev[i + 1].record()
    torch.cuda.synchronize()
    us = sorted(ev[i].elapsed_time(ev[i + 1]) * 1e3 for i in range(launches))
    nb = set_bytes
    print(f"wkv7 B={B} T={T} H={H}: median {us[len(us) // 2]:.1f} us  min {us[0]:.1f} us  "
          f"({nb / 1e6:.1f} MB of rows, {nb / us[len(us) // 2] / 1e3:.0f} GB/s)", flush=True)


def spec(recipe="compression", n_tokens=128, k=4, flush=8, period=16):
    """Speculative greedy decoding (n-gram drafts from the stream's own history, verified on the
    small-T path) against the plain CUDA-graph decoder, one stream, on a prompt of period
    ``period`` (random-init weights do not continue text, so the acceptance rate here is that of
    whatever cycle the model falls into, not of natural language)."""
    import time
    from .spec_decode import generate_speculative
    ck = synth.build_checkpoint("1.5b", recipe, seed=0, device="cuda")
    m = QuantRWKV7(ck)
    del ck
    rng = np.random.default_rng(0)
    prompt = [int(t) for t in rng.integers(1, 60000, period)] * (256 // period)
    to_idx = lambda rows: torch.as_tensor(rows, device=m.device)
    for _ in range(2):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        want, _ = m.generate(np.asarray([prompt]), n_tokens)
        torch.cuda.synchronize()
        t_plain = time.perf_counter() - t0
        t0 = time.perf_counter()
        st = generate_speculative(m, prompt, n_tokens, k=k, flush=flush, to_idx=to_idx)
        torch.cuda.synchronize()
        t_spec = time.perf_counter() - t0
    same = st.tokens == want[0].tolist()
    print(f"spec decode {recipe}: plain {n_tokens / t_plain:.0f} tok/s (eager decoder incl. prefill), speculative "
          f"{n_tokens / t_spec:.0f} tok/s; accepted {st.accepted}/{st.drafted}, {st.tokens_per_call:.2f} tokens per model "
          f"call, {st.flushes} flushes; tokens equal: {same}", flush=True)


def main():
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("gemv")
    g.add_argument("layout"); g.add_argument("bits", type=int); g.add_argument("rows", type=int)
    g.add_argument("cols", type=int); g.add_argument("--n", type=int, default=1)
    g.add_argument("--launches", type=int, default=4); g.add_argument("--zero-groups", type=float, default=0.0)
    d = sub.add_parser("decode")
    d.add_argument("--layers", type=int, default=4); d.add_argument("--recipe", default="compression")
    d.add_argument("--steps", type=int, default=3); d.add_argument("--batch", type=int, default=1)
    sub.add_parser("sweep")
    sub.add_parser("sparse-sweep")
    sub.add_parser("quantize")
    pf = sub.add_parser("prefill")
    pf.add_argument("--layers", type=int, default=24); pf.add_argument("--recipe", default="reduction")
    pf.add_argument("--T", type=int, default=512); pf.add_argument("--batch", type=int, default=1)
    tpp = sub.add_parser("tp")
    tpp.add_argument("--model", default="2.9b"); tpp.add_argument("--recipe", default="compression")
    tpp.add_argument("--exchange", default="p2p", choices=["p2p", "nccl", "none"])
    tm = sub.add_parser("tp-model")
    tm.add_argument("--model", default="2.9b"); tm.add_argument("--recipe", default="compression")
    tm.add_argument("--exchange", default="p2p", choices=["p2p", "nccl"]); tm.add_argument("--layers", type=int, default=32)
    go = sub.add_parser("gemm")
    go.add_argument("layout"); go.add_argument("bits", type=int); go.add_argument("rows", type=int)
    go.add_argument("cols", type=int); go.add_argument("--M", type=int, default=8192)
    go.add_argument("--launches", type=int, default=3)
    dg = sub.add_parser("decode-groups")
    dg.add_argument("--layers", type=int, default=24); dg.add_argument("--batch", type=int, default=64)
    dg.add_argument("--recipe", default="compression"); dg.add_argument("--model", default="1.5b")
    bo = sub.add_parser("batch-once")
    bo.add_argument("layout"); bo.add_argument("bits", type=int); bo.add_argument("rows", type=int)
    bo.add_argument("cols", type=int); bo.add_argument("--n", type=int, default=64); bo.add_argument("--launches", type=int, default=3)
    bo.add_argument("--tcgen05", action="store_true")
    bt = sub.add_parser("batch-tune")
    bt.add_argument("--layers", type=int, default=4); bt.add_argument("--batch", type=int, default=64)
    bt.add_argument("--recipe", default="compression"); bt.add_argument("--model", default="1.5b")
    bs = sub.add_parser("batch-sweep")
    bs.add_argument("--recipe", default="compression")
    gt = sub.add_parser("gemm-timeline")
    gt.add_argument("--M", type=int, default=8192); gt.add_argument("--rows", type=int, default=2048)
    gt.add_argument("--cols", type=int, default=2048); gt.add_argument("--acc-mode", type=int, default=0); gt.add_argument("--bits", type=int, default=5)
    gs = sub.add_parser("gemm-sweep"); gs.add_argument("--acc-mode", type=int, default=0)
    gs.add_argument("--recipe", default="compression")
    wk = sub.add_parser("wkv")
    wk.add_argument("--batch", type=int, default=1); wk.add_argument("--T", type=int, default=512)
    wk.add_argument("--H", type=int, default=32)
    sp = sub.add_parser("spec")
    sp.add_argument("--recipe", default="compression"); sp.add_argument("--n", type=int, default=128)
    sp.add_argument("--k", type=int, default=4); sp.add_argument("--flush", type=int, default=8)
    a = ap.parse_args()
    if a.cmd == "spec":
        spec(a.recipe, a.n, a.k, a.flush)
        return
    if a.cmd == "wkv":
        wkv(a.batch, a.T, a.H)
        return
    if a.cmd == "gemm":
        gemm_once(a.layout, a.bits, a.rows, a.cols, a.M, a.launches)
        return
    if a.cmd == "decode-groups":
        decode_groups(a.layers, a.batch, a.recipe, a.model)
        return
    if a.cmd == "batch-once":
        batch_once(a.layout, a.bits, a.rows, a.cols, a.n, a.launches, a.tcgen05)
        return
    if a.cmd == "batch-tune":
        batch_tune(a.layers, a.batch, a.recipe, a.model)
        return
    if a.cmd == "batch-sweep":
        batch_sweep(a.recipe)
        return
    if a.cmd == "gemm-timeline":
        gemm_timeline("sb6", a.bits, a.rows, a.cols, a.M, a.acc_mode)
        return
    if a.cmd == "quantize":
        quantize_time()
        return
    if a.cmd == "sparse-sweep":
        sparse_sweep()
        return
    if a.cmd == "gemm-sweep":
        gemm_sweep(a.recipe, acc_mode=a.acc_mode)
        return
    if a.cmd == "tp-model":
        tp_model_time(a.model, a.recipe, a.exchange, a.layers)
        return
    if a.cmd == "tp":
        tp_chain(a.model, a.recipe, a.exchange)
        return
    if a.cmd == "gemv":
        gemv(a.layout, a.bits, a.rows, a.cols, a.n, a.launches, a.zero_groups)
    elif a.cmd == "decode":
        decode(a.layers, a.recipe, a.steps, a.batch)
    elif a.cmd == "prefill":
        prefill(a.layers, a.recipe, a.T, a.batch)
    else:
        sweep()


if __name__ == "__main__":
    main()
