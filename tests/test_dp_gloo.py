"""Data-parallel host logic on 2 CPU ranks (gloo): stream sharding, max-over-ranks
timing, result gather.  No GPU, no collective on a data path."""
import os
import socket
import subprocess
import sys

import pytest

from conftest import ROOT
from rwkv_quant_b200 import dp


def test_shard_streams_partitions_exactly():
    for total in (0, 1, 7, 64, 256):
        for world in (1, 2, 3, 8):
            seen = []
            for r in range(world):
                lo, hi = dp.shard_streams(total, world, r)
                assert 0 <= lo <= hi <= total
                seen += list(range(lo, hi))
            assert seen == list(range(total))
            sizes = [dp.shard_streams(total, world, r)[1] - dp.shard_streams(total, world, r)[0] for r in range(world)]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        dp.shard_streams(4, 2, 2)


WORKER = r'''
import sys, torch
sys.path.insert(0, sys.argv[1])
from rwkv_quant_b200 import dp
rank, world = dp.init("gloo")
assert world == 2
lo, hi = dp.shard_streams(5, world, rank)
# each rank "decodes" its streams: token t of stream s is 100*s + t
toks = torch.tensor([[100 * s + t for t in range(3)] for s in range(lo, hi)], dtype=torch.long).reshape(hi - lo, 3)
dp.barrier()
t = dp.max_over_ranks(0.25 + rank)            # rank 1 is the slow one
assert abs(t - 1.25) < 1e-12, t
allt = dp.gather_tokens(toks, 5)
if rank == 0:
    assert allt.tolist() == [[100 * s + t for t in range(3)] for s in range(5)], allt
    print("RANK0_OK")
else:
    assert allt is None
dp.finalize()
'''


def test_two_rank_gloo(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", str(port), str(script), ROOT]
    env = dict(os.environ, OMP_NUM_THREADS="1")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=240, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "RANK0_OK" in r.stdout
