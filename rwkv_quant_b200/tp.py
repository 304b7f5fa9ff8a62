"""Row-split tensor parallelism for the decode GEMVs across the GPUs of one box.

Every rank keeps the output rows it owns of each big matrix (rows are independent in
every ``.rwkvq`` layout, so a row range of the file buffers is itself a valid tensor) and
computes its slice of ``y = W x`` with the ordinary weight-streaming GEMV; the slices are
then exchanged so that every rank holds the whole vector for the next stage:

``exchange="p2p"``   each rank stores its slice into every peer's buffer over NVLink and
                     raises a flag there (``rwkvq_tp_allgather_store``; buffers shared
                     through CUDA IPC, bounded waits, two buffers alternating per site);
``exchange="nccl"``  ``torch.distributed.all_gather_into_tensor`` - the baseline.

The host-side logic (partitioning, buffer bookkeeping, epochs) is independent of CUDA and
is exercised with the ``gloo`` backend in the CPU tests (``exchange="dist"``).
"""
from __future__ import annotations

import contextlib
import ctypes as C
from typing import List, Optional, Sequence

import torch
import torch.distributed as dist


def row_partition(rows: int, world: int, multiple: int = 16) -> List[int]:
    """Boundaries b[0..world] of a split of ``rows`` into ``world`` contiguous ranges whose
    sizes are multiples of ``multiple`` (16 = one GEMV tile, 64 = one head) except possibly
    the last; every row has exactly one owner; equal slices whenever rows % (world *
    multiple) == 0 (required by the p2p / nccl exchanges, which move equal segments)."""
    if rows <= 0 or world < 1 or multiple < 1:
        raise ValueError(f"bad partition request: rows={rows} world={world} multiple={multiple}")
    units = -(-rows // multiple)
    base, extra = divmod(units, world)
    b = [0]
    for r in range(world):
        b.append(min(rows, b[-1] + (base + (1 if r < extra else 0)) * multiple))
    b[-1] = rows
    return b


class _DevArray:
    """CUDA array interface over a raw device pointer (lets torch view memory that came
    from the library's own cudaMalloc / a peer's IPC mapping)."""

    def __init__(self, ptr: int, nbytes: int, typestr: str, shape):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (ptr, False),
                                         "version": 2, "strides": None}
        self.nbytes = nbytes


class TPGroup:
    """The ranks of one tensor-parallel group and their shared (IPC-mapped) buffers."""

    MAX_SPINS = 1 << 24          # about two seconds of polling before a rank gives up

    def __init__(self, device: Optional[torch.device] = None, exchange: str = "p2p"):
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed must be initialised (torchrun) before building a TPGroup")
        self.rank, self.world = dist.get_rank(), dist.get_world_size()
        self.exchange = exchange
        self.device = device
        self._epoch = 0
        self._owned, self._mapped = [], []
        self._sites, self._uses = {}, {}
        self._cap = None                 # site -> uses inside the capture in progress (graph_capture)
        if exchange == "p2p":
            from . import _lib
            self._lib = _lib.load(check_device=True)
            self._check = _lib.check
            self.status = torch.zeros(1, dtype=torch.int32, device=device)
            self._ctr = torch.zeros(8, dtype=torch.int32, device=device)      # exchange counters (device side)
            self._flags_ptrs = self._shared(4 * 8)          # [world] u32 arrival words, zero at start

    # ---- shared buffers ---------------------------------------------------------------
    def _shared(self, nbytes: int):
        """cudaMalloc here, exchange IPC handles, map every peer's buffer; returns the
        list of device pointers indexed by rank (own entry = own allocation)."""
        nbytes = (nbytes + 255) // 256 * 256
        p = C.c_void_p()
        self._check(self._lib.rwkvq_tp_alloc(nbytes, C.byref(p)), "rwkvq_tp_alloc")
        self._owned.append(p.value)
        h = (C.c_ubyte * 64)()
        self._check(self._lib.rwkvq_ipc_export(p, h), "rwkvq_ipc_export")
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(h))
        ptrs = []
        for r, hb in enumerate(handles):
            if r == self.rank:
                ptrs.append(p.value)
                continue
            q = C.c_void_p()
            buf = (C.c_ubyte * 64).from_buffer_copy(hb)
            self._check(self._lib.rwkvq_ipc_open(buf, C.byref(q)), "rwkvq_ipc_open")
            self._mapped.append(q.value)
            ptrs.append(q.value)
        return ptrs

    def site(self, name: str, n: int):
        """Destination buffers of one exchange site (a vector of ``n`` floats gathered from
        all ranks): two alternating buffers; returns (tensors[2], pointer tables[2])."""
        if name in self._sites:
            return self._sites[name]
        if self.exchange == "p2p":
            tens, tabs = [], []
            for _ in range(2):
                ptrs = self._shared(4 * n)
                tens.append(torch.as_tensor(_DevArray(ptrs[self.rank], 4 * n, "<f4", (n,)), device=self.device))
                tabs.append((C.c_void_p * self.world)(*ptrs))
            self._sites[name] = (tens, tabs)
        else:
            tens = [torch.empty(n, dtype=torch.float32, device=self.device) for _ in range(2)]
            self._sites[name] = (tens, [None, None])
        return self._sites[name]

    # ---- the exchange -----------------------------------------------------------------
    @contextlib.contextmanager
    def graph_capture(self, interleaved: bool = False):
        """Wrap the capture of a CUDA graph that contains exchanges.  Which of a site's two
        destination buffers an exchange writes is chosen by a host counter and therefore frozen into
        the graph: if a graph used a site an odd number of times, every replay would write the same
        buffer first and last, and a peer one exchange ahead could overwrite it before this rank's
        consumer has read it (the flags order arrival, not consumption).  On exit this raises unless
        every site was used an even number of times inside the capture; ``all_gather`` refuses to run
        under stream capture outside this context.

        ``interleaved=True`` lifts the even-count rule for graphs in which two consecutive uses of any
        one site, within a replay and from one replay to the next, are always separated by an exchange
        of ANOTHER site (the caller's promise; the graph must use at least two sites): a rank can only
        pass that other exchange once its peer has issued it, which the peer does, in stream order,
        after consuming the earlier buffer."""
        self._cap = {}
        try:
            yield self
        finally:
            cap, self._cap = self._cap, None
        odd = sorted(k for k, v in cap.items() if v % 2)
        if odd and not (interleaved and len(cap) >= 2):
            raise RuntimeError(f"captured graph uses exchange site(s) {odd} an odd number of times: replays would "
                               f"reuse one destination buffer; issue every site an even number of times per graph")

    def all_gather(self, name: str, local: torch.Tensor, n_total: int) -> torch.Tensor:
        """``local`` = this rank's slice (equal sizes on all ranks); returns the gathered
        vector [n_total] (a buffer owned by the group, valid until the site's next-but-one
        exchange).  Under CUDA-graph capture see ``graph_capture``."""
        if self._cap is not None:
            self._cap[name] = self._cap.get(name, 0) + 1
        elif local.is_cuda and torch.cuda.is_current_stream_capturing():
            raise RuntimeError("TPGroup.all_gather under stream capture: wrap the capture in TPGroup.graph_capture()")
        tens, tabs = self.site(name, n_total)
        self._epoch += 1
        k = self._uses.get(name, 0) & 1          # the site's two buffers alternate
        self._uses[name] = self._uses.get(name, 0) + 1
        out = tens[k]
        if self.exchange == "p2p":
            from . import _lib
            flags = (C.c_void_p * self.world)(*self._flags_ptrs)
            self._check(self._lib.rwkvq_tp_allgather_store(local.data_ptr(), local.numel(), tabs[k], flags, self.rank,
                                                           self.world, self._ctr.data_ptr(), self.status.data_ptr(),
                                                           self.MAX_SPINS, _lib.stream_ptr()),
                        "rwkvq_tp_allgather_store")
        elif self.exchange == "nccl":
            dist.all_gather_into_tensor(out, local.contiguous())
        else:                                   # any torch.distributed backend (gloo in the CPU tests)
            dist.all_gather(list(out.chunk(self.world)), local.contiguous())
        return out

    def check(self):
        """Synchronise and raise if a bounded wait of a p2p exchange ran out."""
        if self.exchange == "p2p":
            st = int(self.status.item())
            if st != 0:
                raise RuntimeError(f"tensor-parallel exchange gave up waiting for a peer (status {st})")

    def close(self):
        if self.exchange == "p2p":
            torch.cuda.synchronize(self.device)
            dist.barrier()
            for q in self._mapped:
                self._lib.rwkvq_ipc_close(C.c_void_p(q))
            dist.barrier()
            for p in self._owned:
                self._lib.rwkvq_tp_free(C.c_void_p(p))
            self._mapped, self._owned, self._sites = [], [], {}


class TPRowLinear:
    """One quantized linear split by output rows over the group: ``__call__(x[IN]) -> y[OUT]``
    (fp32, the whole vector on every rank).  ``epilogue`` / ``resid`` as in ``ops.gemv``,
    applied to the local rows before the exchange."""

    def __init__(self, group: TPGroup, dq, name: str, multiple: int = 16, compute=None):
        """``compute(local_slice, x, epilogue, resid_slice) -> y_slice`` replaces the CUDA
        GEMV (the CPU tests pass a numpy product over ``dq.slice_rows``)."""
        self.g, self.name, self._compute = group, name, compute
        self.rows, self.cols = dq.rows, dq.cols
        b = row_partition(dq.rows, group.world, multiple)
        sizes = {b[i + 1] - b[i] for i in range(group.world)}
        if len(sizes) != 1:
            raise ValueError(f"{name}: {dq.rows} rows do not split evenly over {group.world} ranks in units of {multiple}")
        self.lo, self.hi = b[group.rank], b[group.rank + 1]
        self.local = dq.slice_rows(self.lo, self.hi)

    def __call__(self, x: torch.Tensor, epilogue: int = 0, resid: Optional[torch.Tensor] = None) -> torch.Tensor:
        if self._compute is not None:
            y_loc = self._compute(self.local, x, epilogue, None if resid is None else resid[self.lo:self.hi])
        else:
            from .backends.cuda import ops
            r = None if resid is None else resid[self.lo:self.hi].reshape(1, -1)
            y_loc = ops.gemv(self.local.bufs, self.local.meta, x.reshape(1, -1), epilogue, r)[0]
        return self.g.all_gather(self.name, y_loc, self.rows)
