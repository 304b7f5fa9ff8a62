"""Row-split tensor-parallel GEMV on 2 GPUs: peer-store all-gather (and the NCCL baseline)
against the single-GPU GEMV of the whole matrix.  Needs two visible GPUs; one process per
GPU, rendezvous on 127.0.0.1.  Tolerance: the row slices may pick another work split than
the whole matrix, i.e. another fp32 summation order: |dy| <= 2e-5 * max|y|."""
import os
import socket
import subprocess
import sys

import pytest
import torch

from conftest import ROOT

pytestmark = pytest.mark.gpu

WORKER = r'''
import os, sys, numpy as np, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from rwkv_quant_b200 import synth, tp
from rwkv_quant_b200.backends.cuda import ops
rank = int(os.environ["RANK"]); local = int(os.environ["LOCAL_RANK"])
torch.cuda.set_device(local)
dev = torch.device("cuda", local)
dist.init_process_group("nccl", device_id=dev)
world = dist.get_world_size()

def linear(layout, bits, rows, cols, seed):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(rows, cols, generator=g) * 0.02
    fn = {"sb6": synth.quant_sb6, "sym": synth.quant_sym, "rtn": synth.quant_rtn}[layout]
    return ops.DeviceQT(fn("w", "g", w, bits), device=dev)

D, F = 2560, 10240                                   # the 2.9B build's widths
key = linear("sb6", 4, F, D, 1)
val = linear("sb6", 4, D, F, 2)
out = linear("sb6", 5, D, D, 3)
head = linear("sym", 8, 4096, D, 4)
gx = torch.Generator().manual_seed(9)
x0 = torch.randn(D, generator=gx).to(dev)
for exchange in ("p2p", "nccl"):
    g = tp.TPGroup(device=dev, exchange=exchange)
    lk = tp.TPRowLinear(g, key, "key", 64); lv = tp.TPRowLinear(g, val, "value", 64)
    lo = tp.TPRowLinear(g, out, "out", 64); lh = tp.TPRowLinear(g, head, "head", 64)
    x = x0.clone()
    for step in range(6):
        a = lo(x, 2, x)                              # projection + residual
        h = lk(a, 1)                                 # relu^2
        y = lv(h, 2, a)
        z = lh(y)
        ra = ops.gemv(out.bufs, out.meta, x.view(1, -1), 2, x.view(1, -1))[0]
        rh = ops.gemv(key.bufs, key.meta, ra.view(1, -1), 1, None)[0]
        ry = ops.gemv(val.bufs, val.meta, rh.view(1, -1), 2, ra.view(1, -1))[0]
        rz = ops.gemv(head.bufs, head.meta, ry.view(1, -1), 0, None)[0]
        torch.cuda.synchronize()
        g.check()
        for got, ref, nm in ((a, ra, "out"), (h, rh, "key"), (y, ry, "value"), (z, rz, "head")):
            err = (got - ref).abs().max().item() / max(ref.abs().max().item(), 1e-9)
            assert err <= 2e-5, (exchange, step, nm, err)
        x = (ry / (1.0 + ry.abs().max())).clone()
    g.close()
dist.barrier()
if rank == 0: print("RANK0_OK")
dist.destroy_process_group()
'''


def test_row_split_gemv_two_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", str(port), str(script), ROOT]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert "RANK0_OK" in r.stdout


MODEL_WORKER = r'''
import os, sys, numpy as np, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from rwkv_quant_b200 import synth, tp, tp_model
from rwkv_quant_b200.backends.cuda import QuantRWKV7
rank = int(os.environ["RANK"]); local = int(os.environ["LOCAL_RANK"])
torch.cuda.set_device(local)
dev = torch.device("cuda", local)
dist.init_process_group("nccl", device_id=dev)
rel = lambda a, b: float((a - b).abs().max() / b.abs().max())
for recipe in ("compression", "reduction"):
    # RWKV-7 2.9B widths (D 2560 = 40 heads, FFN 10240), 2 layers, a 4096-row vocabulary
    ck = synth.build_checkpoint("2.9b", recipe, seed=11, device="cpu", n_layer=2, vocab=4096, keep_on_device=False)
    ref = QuantRWKV7(ck, device=dev)
    for exchange in ("p2p", "nccl"):
        g = tp.TPGroup(device=dev, exchange=exchange)
        m = tp_model.TPQuantRWKV7(ck, g, device=dev)
        assert m.n_head_local == 20 and m.blocks[0].Wr.rows == 1280 and m.blocks[0].Wo.cols == 1280
        idx = torch.from_numpy(np.random.default_rng(5).integers(1, 4000, (2, 9))).to(dev)
        # prefill of 6 tokens, then 3 single-token steps from the returned (head-sharded) state
        lo_r, st_r = ref.forward_stateful(idx[:, :6], ref.init_state(2))
        lo_t, st_t = m.forward_stateful(idx[:, :6], m.init_state(2))
        errs = [rel(lo_t, lo_r)]
        for t in range(6, 9):
            lo_r, st_r = ref.forward_stateful(idx[:, t:t + 1], st_r)
            lo_t, st_t = m.forward_stateful(idx[:, t:t + 1], st_t)
            errs.append(rel(lo_t, lo_r))
        torch.cuda.synchronize(); g.check()
        assert max(errs) <= 2e-4, (recipe, exchange, errs)
        # this rank's heads of the WKV state, the replicated shift states
        for (w_t, ts_t, cs_t), (w_r, ts_r, cs_r) in zip(st_t, st_r):
            h0 = rank * 20
            assert (w_t - w_r[:, h0:h0 + 20]).abs().max().item() <= 1e-4 * max(1.0, w_r.abs().max().item())
            assert rel(ts_t.reshape(2, -1), ts_r.reshape(2, -1)) <= 1e-4 and rel(cs_t.reshape(2, -1), cs_r.reshape(2, -1)) <= 1e-4
        # every rank holds the same logits bit for bit
        both = [torch.empty_like(lo_t) for _ in range(2)]
        dist.all_gather(both, lo_t.contiguous())
        assert torch.equal(both[0], both[1])
        if rank == 0: print(f"{recipe} {exchange}: logits relmax vs one GPU {max(errs):.2e}")
        # the graph-replayed decoder against plain calls: same tokens, same logits, five steps
        tok = idx[:, 0]
        dec = m.decoder(2, use_graph=True)
        st_e = m.init_state(2)
        nxt_g = dec.step(tok).clone()
        for t in range(5):
            lo_e, st_e = m.forward_stateful((tok if t == 0 else nxt_e).reshape(2, 1), st_e)
            nxt_e = lo_e[:, 0].argmax(-1)
            assert torch.equal(nxt_g, nxt_e) and rel(dec.logits, lo_e[:, 0]) <= 1e-6, (recipe, exchange, t)
            if t < 4: nxt_g = dec.step().clone()
        torch.cuda.synchronize(); g.check()
        del dec
        del m
        g.close()
    del ref
dist.barrier()
if rank == 0: print("RANK0_OK")
dist.destroy_process_group()
'''


def test_head_sharded_model_two_gpus(tmp_path):
    """The whole model split over two GPUs (heads, WKV state, column-split output / ffn.value
    projections, row-split head) against the single-GPU model: logits over a prefill and three
    decode steps, final states, and bit-equality of the logits across ranks."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "model_worker.py"
    script.write_text(MODEL_WORKER)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", str(port), str(script), ROOT]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-5000:]
    assert "RANK0_OK" in r.stdout
    print(r.stdout[-600:])
