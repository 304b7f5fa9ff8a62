"""Row-split tensor parallelism: host logic on 2 CPU ranks (gloo).  Partitioning, the
per-site double buffers and the gather order; the local products are numpy matvecs over
``slice_rows`` of a stand-in tensor, so no GPU is involved."""
import os
import socket
import subprocess
import sys

import pytest

from conftest import ROOT
from rwkv_quant_b200 import tp


def test_row_partition_covers_every_row_once():
    for rows in (16, 64, 2048, 2560, 10240, 65536, 100):
        for world in (1, 2, 4, 8):
            for mult in (16, 64):
                b = tp.row_partition(rows, world, mult)
                assert b[0] == 0 and b[-1] == rows and len(b) == world + 1
                assert all(b[i] <= b[i + 1] for i in range(world))
                assert all((b[i + 1] - b[i]) % mult == 0 for i in range(world - 1) if b[i + 1] < rows)
    # the shapes of the 2.9B build split evenly at 2 / 4 / 8 ranks in head units
    for rows in (2560, 10240, 65536):
        for world in (2, 4, 8):
            b = tp.row_partition(rows, world, 64)
            assert len({b[i + 1] - b[i] for i in range(world)}) == 1
    with pytest.raises(ValueError):
        tp.row_partition(0, 2)


WORKER = r'''
import sys, numpy as np, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from rwkv_quant_b200 import tp
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()

class FakeQT:                      # rows first, like every .rwkvq layout
    def __init__(self, w): self.w, self.rows, self.cols = w, w.shape[0], w.shape[1]
    def slice_rows(self, a, b): return FakeQT(self.w[a:b])

def compute(local, x, epilogue, resid):
    y = torch.from_numpy(local.w @ x.numpy())
    if epilogue == 1: y = torch.relu(y) ** 2
    if epilogue == 2: y = y + resid
    return y

rng = np.random.default_rng(3)
W1 = rng.standard_normal((256, 128)).astype(np.float32)      # "ffn key"
W2 = rng.standard_normal((128, 256)).astype(np.float32)      # "ffn value"
g = tp.TPGroup(device=None, exchange="dist")
l1 = tp.TPRowLinear(g, FakeQT(W1), "key", multiple=64, compute=compute)
l2 = tp.TPRowLinear(g, FakeQT(W2), "value", multiple=64, compute=compute)
assert (l1.lo, l1.hi) == (128 * rank, 128 * rank + 128) and (l2.lo, l2.hi) == (64 * rank, 64 * rank + 64)
x = torch.from_numpy(rng.standard_normal(128).astype(np.float32))
outs = []
for step in range(5):              # the chain of a channel mix, several tokens: buffers alternate
    h = l1(x, 1)
    y = l2(h, 2, x)
    ref_h = np.maximum(W1 @ x.numpy(), 0) ** 2
    ref_y = W2 @ ref_h + x.numpy()
    np.testing.assert_allclose(h.numpy(), ref_h, rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(y.numpy(), ref_y, rtol=1e-4, atol=1e-3)
    outs.append(y)
    x = y.clone() / (1.0 + y.abs().max())
# a returned buffer stays valid for one more exchange at its site, not two
assert outs[-1].data_ptr() != outs[-2].data_ptr() and outs[-1].data_ptr() == outs[-3].data_ptr()
# graph-capture bookkeeping: a captured sequence must use every site an even number of times
with g.graph_capture():
    for _ in range(2):
        l2(l1(x, 1), 2, x)
try:
    with g.graph_capture():
        l2(l1(x, 1), 2, x)                 # once: the frozen buffer choice would repeat on every replay
    raise SystemExit("an odd number of uses of a site inside a capture was accepted")
except RuntimeError as e:
    assert "odd number" in str(e), e
l2(l1(x, 1), 2, x)                         # restores the parity of both sites on every rank
# interleaved graphs (two sites alternating) may use their sites an odd number of times ...
with g.graph_capture(interleaved=True):
    l2(l1(x, 1), 2, x)
l2(l1(x, 1), 2, x)
# ... a graph with a single site may not
try:
    with g.graph_capture(interleaved=True):
        l1(x, 1)
    raise SystemExit("one site used once inside an interleaved capture was accepted")
except RuntimeError as e:
    assert "odd number" in str(e), e
l1(x, 1)
dist.barrier()
if rank == 0: print("RANK0_OK")
dist.destroy_process_group()
'''


def test_two_rank_row_split_gloo(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", str(port), str(script), ROOT]
    env = dict(os.environ, OMP_NUM_THREADS="1")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=240, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert "RANK0_OK" in r.stdout
