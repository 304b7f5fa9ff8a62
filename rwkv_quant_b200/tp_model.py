"""Head-sharded tensor-parallel RWKV-7 over the GPUs of one box (whole model, any B and T).

The reference runs on one device; what makes the split possible is that every ``.rwkvq`` layout
stores rows first and blocks along the columns (``formats/reader.py:130-152``), so a row range and
a block-aligned column range of the file buffers are themselves valid tensors.  Rank r of W owns
heads [r H/W, (r+1) H/W), i.e. channels [r D/W, (r+1) D/W):

    replicated (every rank, full width D)  embedding + LN0, LN1 / LN2 + token shift + lerps, the LoRA
                                           down projections (rank-wide), the residual stream, LN_out
    row-split (this rank's heads)          W_r, W_k, W_v, the LoRA up projections, the per-channel
                                           vectors, the WKV-7 state and scan, group norm + gate
    column-split (this rank's inputs)      W_o over its heads' channels, ffn.value over its slice of
                                           the hidden vector (ffn.key is row-split): partial sums of
                                           the full-width output
    row-split                              the head: vocabulary rows, logits gathered

Two exchanges per layer (the partial sums after W_o and after ffn.value, summed in rank order on
every rank so that the replicated residual stream stays bit-identical across ranks) and one for
the logits.  The exchange object is a ``tp.TPGroup`` (peer stores over NVLink or NCCL all-gather).
All compute runs through the same kernels as the single-GPU sequence path.

This is the functional whole-model split; it is not a fast path: per-layer launches are issued
from Python, nothing is captured in a graph, and at small batch the two exchanges cost more than
the halved weight stream saves (see the row-split GEMV measurements).
"""
from __future__ import annotations

import copy
from typing import Optional

import torch

from . import _lib
from .backends.cuda import ops
from .backends.cuda.fused_tail import wkv_tail
from .backends.cuda.quant_model import QuantRWKV7
from .backends.cuda.wkv7 import wkv7_infer
from .formats import QuantizedCheckpoint, QuantizedTensor

_ROW_FIELDS = ("codes", "codes_packed", "scale", "dense", "gw_d", "gw_dm", "gw_qsqm", "gw_qh", "gw_qh2", "gw_scale",
               "gw_min", "gw_qs")


def slice_rows(qt: QuantizedTensor, a: int, b: int) -> QuantizedTensor:
    """Stored rows [a, b) of a tensor (every buffer is row-major over the stored rows)."""
    if qt.outlier_indices is not None and qt.outlier_indices.numel():
        raise NotImplementedError(f"{qt.key}: sparse overrides are not sharded")
    rows = qt.shape[0]
    if not (0 <= a < b <= rows):
        raise ValueError(f"{qt.key}: rows [{a}, {b}) of {rows}")
    out = copy.copy(qt)
    for f in _ROW_FIELDS:
        v = getattr(qt, f)
        if v is not None:
            setattr(out, f, v.reshape(rows, -1)[a:b].reshape(b - a, *v.shape[1:]).contiguous())
    out.shape = (b - a,) + tuple(qt.shape[1:])
    return out


def slice_cols(qt: QuantizedTensor, a: int, b: int) -> QuantizedTensor:
    """Stored columns [a, b) of a 2-D tensor; a and b must fall on the layout's block structure
    (sb6 / sym: super-blocks of 256 columns; asym: its group size; per-row int8 and dense: any)."""
    if qt.outlier_indices is not None and qt.outlier_indices.numel():
        raise NotImplementedError(f"{qt.key}: sparse overrides are not sharded")
    rows, cols = qt.shape
    if not (0 <= a < b <= cols):
        raise ValueError(f"{qt.key}: columns [{a}, {b}) of {cols}")
    kind = qt.kind
    out = copy.copy(qt)
    out.shape = (rows, b - a)
    def take(v, num, den=1):
        """columns [a, b) of a per-row buffer holding num/den elements per stored column"""
        if v is None:
            return None
        lo, hi = a * num // den, b * num // den
        return v.reshape(rows, -1)[:, lo:hi].contiguous()
    if kind == "dense":
        out.dense = take(qt.dense, 1)
        return out
    if kind in ("sb6", "sym"):
        sbw = qt.gw_gs * qt.gw_sb
        if a % sbw or b % sbw:
            raise ValueError(f"{qt.key}: a column range of a {kind} tensor must fall on super-blocks of {sbw}")
        out.codes = take(qt.codes, 1)
        out.codes_packed = take(qt.codes_packed, 1, 2)
        out.gw_qh, out.gw_qh2 = take(qt.gw_qh, 1, 8), take(qt.gw_qh2, 1, 8)
        out.gw_d, out.gw_dm = take(qt.gw_d, 1, sbw), take(qt.gw_dm, 1, sbw)
        out.gw_qs = take(qt.gw_qs, 1, qt.gw_gs)
        if qt.gw_qsqm is not None:
            out.gw_qsqm = take(qt.gw_qsqm, 12, sbw).reshape(rows, (b - a) // sbw, 12)
        return out
    if kind == "asym":
        if a % qt.gw_gs or (b % qt.gw_gs and b != cols):
            raise ValueError(f"{qt.key}: a column range of an asym tensor must fall on groups of {qt.gw_gs}")
        out.codes = take(qt.codes, 1)
        nb = (cols + qt.gw_gs - 1) // qt.gw_gs
        lo, hi = a // qt.gw_gs, (b + qt.gw_gs - 1) // qt.gw_gs
        out.gw_scale = qt.gw_scale.reshape(rows, nb)[:, lo:hi].contiguous()
        out.gw_min = qt.gw_min.reshape(rows, nb)[:, lo:hi].contiguous()
        return out
    if kind == "rtn" and qt.codes is not None:
        out.codes = take(qt.codes, 1)
        return out
    raise NotImplementedError(f"{qt.key}: column ranges of layout {kind!r} at {qt.bits} bits")


def shard_checkpoint(ck: QuantizedCheckpoint, rank: int, world: int) -> QuantizedCheckpoint:
    """This rank's tensors of a world-naming checkpoint (see the module text for what is split how)."""
    if ck.naming != "world":
        raise NotImplementedError("tensor-parallel sharding is built for world-naming checkpoints")
    D, S = ck.n_embd, ck.head_size
    H = D // S
    if H % world:
        raise ValueError(f"{H} heads do not split over {world} ranks")
    c0, c1 = rank * (H // world) * S, (rank + 1) * (H // world) * S
    T = {}
    for key, qt in ck.tensors.items():
        leaf = ".".join(key.split(".")[-2:]) if key.endswith((".weight", ".bias")) else key.split(".")[-1]
        if ".att." in key:
            if leaf in ("receptance.weight", "key.weight", "value.weight"):
                qt = slice_rows(qt, c0, c1)
            elif leaf == "output.weight":
                qt = slice_cols(qt, c0, c1)
            elif leaf in ("w2", "a2", "g2", "v2"):                      # stored [rank, D]: the output channels are columns
                qt = slice_cols(qt, c0, c1)
            elif leaf in ("w0", "a0", "v0", "k_k", "k_a", "ln_x.weight", "ln_x.bias", "r_k") and qt.dense is None:
                raise NotImplementedError(f"{key}: a quantized per-channel vector is not sharded")
            elif leaf in ("w0", "a0", "v0", "k_k", "k_a", "ln_x.weight", "ln_x.bias"):
                flat = copy.copy(qt)
                flat.dense = qt.dense.reshape(-1)[c0:c1].contiguous()
                flat.shape = (c1 - c0,)
                qt = flat
            elif leaf == "r_k":                                          # [H, S]
                flat = copy.copy(qt)
                flat.dense = qt.dense.reshape(H, S)[c0 // S:c1 // S].contiguous()
                flat.shape = (c1 // S - c0 // S, S)
                qt = flat
        elif ".ffn." in key:
            F = qt.shape[0] if leaf == "key.weight" else qt.shape[1] if leaf == "value.weight" else 0
            if F and F % world:
                raise ValueError(f"{key}: hidden width {F} does not split over {world} ranks")
            if leaf == "key.weight":
                qt = slice_rows(qt, rank * (F // world), (rank + 1) * (F // world))
            elif leaf == "value.weight":
                qt = slice_cols(qt, rank * (F // world), (rank + 1) * (F // world))
        elif key == "head.weight":
            V = qt.shape[0]
            if V % world:
                raise ValueError(f"vocabulary {V} does not split over {world} ranks")
            qt = slice_rows(qt, rank * (V // world), (rank + 1) * (V // world))
        T[key] = qt
    return QuantizedCheckpoint(naming=ck.naming, n_layer=ck.n_layer, n_embd=ck.n_embd, head_size=ck.head_size,
                               vocab_size=ck.vocab_size, tensors=T)


class TPQuantRWKV7(QuantRWKV7):
    """``QuantRWKV7`` with the weights of one rank; ``forward_stateful`` / ``forward_hidden`` /
    ``init_state`` keep their contracts (logits and residual stream are full-size and identical on
    every rank; the WKV state holds this rank's heads only).  ``group``: a ``tp.TPGroup``."""

    def __init__(self, ckpt: QuantizedCheckpoint, group, device="cuda"):
        self.group = group
        self.rank, self.world = group.rank, group.world
        self.full_vocab = ckpt.vocab_size
        super().__init__(shard_checkpoint(ckpt, self.rank, self.world), device=device)
        self.n_head_local = self.n_head // self.world
        self.d_local = self.n_head_local * self.head_size
        self.fused_prep = False

    def _build_struct(self):           # the one-call decode step is a single-GPU path
        self._model_c = None

    def init_state(self, batch_size: int = 1):
        H, S = self.n_head_local, self.head_size
        return [(torch.zeros((batch_size, H, S, S), device=self.device), None, None) for _ in range(self.n_layer)]

    def decoder(self, batch_size: int = 1, use_graph: bool = True):
        """A ``TPDecoder``: one token of ``batch_size`` streams per call, replayed as a CUDA graph."""
        return TPDecoder(self, batch_size, use_graph)

    # ---- exchanges
    def _all_reduce(self, name: str, part: torch.Tensor) -> torch.Tensor:
        """Sum of every rank's [N, D] partial, added in rank order on every rank (bit-identical everywhere)."""
        n = part.numel()
        g = self.group.all_gather(name + f"/{n}", part.reshape(-1), n * self.world).view(self.world, *part.shape)
        out = g[0].clone()
        for r in range(1, self.world):
            out += g[r]
        return out

    def _gather_cols(self, name: str, loc: torch.Tensor) -> torch.Tensor:
        """[N, C_local] of every rank -> [N, world * C_local] in rank order."""
        n = loc.numel()
        g = self.group.all_gather(name + f"/{n}", loc.reshape(-1), n * self.world).view(self.world, *loc.shape)
        return g.permute(1, 0, 2).reshape(loc.shape[0], -1).contiguous()

    # ---- one layer over all B*T positions
    def _block_seq(self, i, L, x, v_first, state):
        B, T, D = x.shape
        Hl, S, Dl = self.n_head_local, self.head_size, self.d_local
        wkv, ts, cs = state
        N = B * T
        xs, ts = ops.seq_ln_shift_mix(x, L.ln1[0], L.ln1[1], ts, L.x_mix)              # replicated
        xr, xw, xk, xv, xa, xg = (xs[j].reshape(N, D) for j in range(6))
        r, k, v = self._linear(L.Wr, xr), self._linear(L.Wk, xk), self._linear(L.Wv, xv)   # [N, Dl]: this rank's heads
        pairs = [(L.w1, L.w2), (L.a1, L.a2), (L.g1, L.g2)] + ([(L.v1, L.v2)] if i > 0 else [])
        if N <= self.lora_pair_max and ops.lora_pair_ok(pairs, D):
            # down projections full width, up projections onto this rank's channels: two launches for all branches
            ys = ops.lora_pair(pairs, [xw, xa, xg] + ([xv] if i > 0 else []), [1, 0, 2, 0][:len(pairs)])
            y_w, y_a, g = ys[:3]
            y_v = ys[3] if i > 0 else None
        else:
            up = lambda dq, t: self._lora_seq(dq, t, 0)
            y_w = up(L.w2, self._lora_seq(L.w1, xw, 1))
            y_a = up(L.a2, self._lora_seq(L.a1, xa, 0))
            g = up(L.g2, self._lora_seq(L.g1, xg, 2))
            y_v = None if i == 0 else up(L.v2, self._lora_seq(L.v1, xv, 0))
        if i == 0:
            v_first = v
        w, k, v2, na, nb = ops.seq_tmix_pre(k, v, y_w, y_a, y_v, None if i == 0 else v_first, L.w0, L.a0, L.v0,
                                            L.k_k, L.k_a, Hl)
        r4 = lambda t: t.reshape(B, T, Hl, S)
        out, wkv = wkv7_infer(r4(r), r4(w), r4(k), r4(v2), r4(na), r4(nb), wkv)
        og = wkv_tail(out, r, k, v2, L.r_k, L.lnx[0], L.lnx[1], g, Hl, S)              # [N, Dl]
        part = self._linear(L.Wo, og.reshape(N, Dl))                                    # [N, D] partial sums
        x2 = x.reshape(N, D) + self._all_reduce("o", part)
        xk2, cs = ops.seq_ln_shift_mix(x2.reshape(B, T, D), L.ln2[0], L.ln2[1], cs, L.ffn_x_k)
        h = self._linear(L.Wfk, xk2.reshape(N, D), epilogue=_lib.EPI_RELU2)             # [N, F / world]
        part = self._linear(L.Wfv, h)
        x3 = x2 + self._all_reduce("v", part)
        return x3.reshape(B, T, D), v_first, (wkv, ts, cs)

    def forward_stateful(self, idx, states, last_only: bool = False, tail_only: int = 0):
        idx = torch.as_tensor(idx, device=self.device).long()
        B, T = idx.shape
        x, new_states = self.forward_hidden(idx, states)
        if last_only:
            x = x[:, -1:]
        elif tail_only and T > tail_only:
            x = x[:, -tail_only:]
        n = x.shape[1]
        loc = self._linear(self.head, x.reshape(B * n, self.n_embd).contiguous())       # [B n, V / world]
        logits = self._gather_cols("head", loc)
        return logits.reshape(B, n, self.full_vocab), new_states


class TPDecoder:
    """Greedy single-token steps of ``batch_size`` streams on a ``TPQuantRWKV7``: the whole step of this
    rank (its launches and its exchanges) captured once and replayed as one CUDA graph, state kept in
    place.  Every rank of the group must build and step its decoder in lockstep.

    ``step(tokens=None)``: feed ``tokens`` [B] (or the previous step's argmax) and return the next
    token ids [B] (a tensor of the decoder, overwritten by the next step); ``logits`` [B, V]."""

    def __init__(self, model: TPQuantRWKV7, batch_size: int, use_graph: bool = True):
        self.m, self.B = model, int(batch_size)
        dev = model.device
        self.tokens = torch.ones((self.B, 1), dtype=torch.long, device=dev)
        self.states = model._materialize(model.init_state(self.B), self.B)
        self.logits = torch.zeros((self.B, model.full_vocab), dtype=torch.float32, device=dev)
        self.next_tokens = torch.ones(self.B, dtype=torch.long, device=dev)
        self.graph = None
        if use_graph:
            self._body()                                   # sites, workspaces and library handles exist before the capture
            torch.cuda.synchronize(dev)
            for st in self.states:
                for t in st:
                    t.zero_()
            st = torch.cuda.Stream(device=dev)
            st.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(st):
                self.graph = torch.cuda.CUDAGraph()
                # o / v alternate layer by layer and the head exchange closes the step: consecutive uses of one
                # site always have another site's exchange between them
                with model.group.graph_capture(interleaved=True), torch.cuda.graph(self.graph, stream=st):
                    self._body()
            torch.cuda.current_stream(dev).wait_stream(st)

    def _body(self):
        logits, new = self.m.forward_stateful(self.tokens, self.states)
        for old, cur in zip(self.states, new):
            for o, c in zip(old, cur):
                if o.data_ptr() != c.data_ptr():
                    o.copy_(c.reshape(o.shape))
        self.logits.copy_(logits[:, 0])
        self.next_tokens.copy_(self.logits.argmax(dim=-1))

    def step(self, tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
        self.tokens.copy_((self.next_tokens if tokens is None else tokens).reshape(self.B, 1))
        if self.graph is not None:
            self.graph.replay()
        else:
            self._body()
        return self.next_tokens
