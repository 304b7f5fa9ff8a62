"""Data-parallel decode across the GPUs of one box: host-side helpers.

Streams are independent (they share only read-only weights), so every rank holds a
full replica and its own slice of the streams; there is no collective on the data
path.  The only communication is a barrier around timed regions, a max-reduction of
per-rank timings and a gather of per-rank results.  Works with ``nccl`` (GPU) and
``gloo`` (CPU, used by the tests).
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist


def env_rank():
    """(rank, world_size, local_rank) from the torchrun environment (1 process: 0, 1, 0)."""
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")),
            int(os.environ.get("LOCAL_RANK", "0")))


def shard_streams(total_streams: int, world: int, rank: int):
    """Contiguous slice [lo, hi) of the global stream ids owned by ``rank``; sizes
    differ by at most one and every stream has exactly one owner."""
    if total_streams < 0 or world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad sharding request: {total_streams} streams, world {world}, rank {rank}")
    base, extra = divmod(total_streams, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def init(backend: str, device=None):
    """Initialise the default process group when WORLD_SIZE > 1; returns (rank, world)."""
    rank, world, _ = env_rank()
    if world > 1 and not dist.is_initialized():
        kw = {"device_id": device} if (backend == "nccl" and device is not None) else {}
        dist.init_process_group(backend, **kw)
    return rank, world


def barrier():
    if dist.is_initialized():
        dist.barrier()


def max_over_ranks(value: float, device="cpu") -> float:
    """Largest ``value`` over all ranks (the time a barrier-bracketed region took)."""
    if not dist.is_initialized():
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def gather_tokens(local_tokens: torch.Tensor, total_streams: int, device="cpu"):
    """Rank 0 receives the generated tokens of all streams in global stream order
    ([total_streams, n_tokens]); other ranks get None.  Host-side gather only."""
    if not dist.is_initialized():
        return local_tokens
    world, rank = dist.get_world_size(), dist.get_rank()
    n_tok = local_tokens.shape[1]
    most = -(-total_streams // world)
    pad = torch.zeros((most, n_tok), dtype=torch.long, device=device)
    pad[: local_tokens.shape[0]] = local_tokens.to(device)
    out = [torch.zeros_like(pad) for _ in range(world)] if rank == 0 else None
    dist.gather(pad, out, dst=0)
    if rank != 0:
        return None
    rows = []
    for r in range(world):
        lo, hi = shard_streams(total_streams, world, r)
        rows.append(out[r][: hi - lo])
    return torch.cat(rows, 0)


def finalize():
    if dist.is_initialized():
        dist.destroy_process_group()
