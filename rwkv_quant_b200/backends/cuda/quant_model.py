"""RWKV-7 (x070) inference model over a ``.rwkvq`` checkpoint on the CUDA kernels.

Same surface as the reference's ``QuantRWKV7`` (backends/metal/quant_model.py:839-990):
``QuantRWKV7(load_raw(path))``, ``init_state(B)``, ``step`` / ``forward_stateful(idx,
states, last_only, tail_only)``, ``forward_hidden``, ``__call__(idx)``; plus
``generate`` (the greedy loop of tests/bench_decode_vs_gguf.py:84-96) and
``decoder(B)`` which replays one whole token as a CUDA graph.

Two execution paths share the same weights (kept packed on the device):
  T == 1   one call of ``rwkvq_decode_step`` (all kernels of a token launched from C)
  T  > 1   per-layer ops over all B*T positions: quantized linears, LoRA products,
           ``wkv7_infer`` and ``wkv_tail`` are library kernels; layer norms, lerps and
           gates are elementwise torch ops on the device.
Weight precision follows the reference's loader (quant_model.py:128-154, 245-262):
quantized linears are used exactly as coded; every other tensor is rounded to bf16,
then to fp16 when it is 2-D with min(shape) >= 32 (LoRA, embedding, r_k).
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.nn.functional as F

from . import ops
from .fused_tail import wkv_tail
from .quant_linear_gw import GEMM_MIN_BATCH_NB
from .wkv7 import wkv7_infer
from ... import _lib
from ..._lib import LayerStruct, ModelStruct

_DECAY = -0.606531     # -exp(-0.5), quant_model.py:701


def _dense_param(qt, device):
    """A non-linear tensor as fp32 on the device in the reference's load-time precision."""
    if qt.bits >= 16:
        t = qt.dense.float()
    else:
        t = ops.DeviceQT(qt, device, relayout=False).dequant(torch.float32, True).cpu()
    if t.ndim == 2 and min(t.shape) >= 32:
        t = t.half().float()
    return t.to(device).contiguous()


class _Layer:
    pass


class QuantRWKV7:
    def __init__(self, ckpt, device="cuda", gemm_min_batch=GEMM_MIN_BATCH_NB, gemv_max_batch=2):
        if ckpt.naming not in ("world", "custom"):
            raise NotImplementedError(f"checkpoint naming {ckpt.naming!r} (world or custom)")
        _lib.load(check_device=True)
        self.device = torch.device(device)
        self.naming = ckpt.naming
        self.n_layer, self.n_embd = ckpt.n_layer, ckpt.n_embd
        self.head_size = ckpt.head_size
        self.n_head = ckpt.n_embd // ckpt.head_size
        self.vocab_size = ckpt.vocab_size
        self.gemm_min_batch = int(gemm_min_batch)
        self.gemv_max_batch = int(gemv_max_batch)
        self.batch_max = 64              # rows up to which the weights-once small-batch kernel serves a linear
        self.lora_pair_max = 1024        # rows up to which the sequence path uses rwkvq_lora_pair (measured: 512 rows equal, 8192 rows slower)
        T = ckpt.tensors
        dev = self.device
        def dq(key):
            d = ops.DeviceQT(T[key], dev)
            # the kernels of the model read packed codes directly: a tensor with sparse outlier
            # overrides is handed to them as a dense bf16 one (its load-time precision anyway)
            return d.densified() if d.outliers is not None else d
        vec = lambda key: _dense_param(T[key], dev).reshape(-1)

        self.emb, self.head = dq("emb.weight"), dq("head.weight")
        custom = self.naming == "custom"                     # key schemes: quant_model.py:317-364, 791, 856-859
        ln0 = "ln0." if custom else "blocks.0.ln0."
        self.ln0 = (vec(ln0 + "weight"), vec(ln0 + "bias"))
        self.ln_out = (vec("ln_out.weight"), vec("ln_out.bias"))
        proj = {"Wr": "r_proj", "Wk": "k_proj", "Wv": "v_proj", "Wo": "o_proj"} if custom else \
               {"Wr": "receptance", "Wk": "key", "Wv": "value", "Wo": "output"}
        self.blocks = []
        for i in range(self.n_layer):
            p = f"blocks.{i}."
            a, f = (p + "tmix.", p + "cmix.") if custom else (p + "att.", p + "ffn.")
            L = _Layer()
            L.ln1 = (vec(p + "ln1.weight"), vec(p + "ln1.bias"))
            L.ln2 = (vec(p + "ln2.weight"), vec(p + "ln2.bias"))
            L.x_mix = torch.stack([vec(a + n) for n in ("x_r", "x_w", "x_k", "x_v", "x_a", "x_g")]).contiguous()
            branches = ("w", "a", "g") + (("v",) if i > 0 else ())
            L.v0 = L.v1 = L.v2 = None
            for br in branches:
                if custom:
                    # nn.Linear weights [out, in] -> the [in, out] orientation the kernels read
                    setattr(L, br + "1", dq(a + br + "_lora_A.weight").transposed_dense())
                    setattr(L, br + "2", dq(a + br + "_lora_B.weight").transposed_dense())
                    if br != "g":
                        setattr(L, br + "0", vec(a + br + "_lora_B.bias"))
                else:
                    setattr(L, br + "1", dq(a + br + "1"))
                    setattr(L, br + "2", dq(a + br + "2"))
                    if br != "g":
                        setattr(L, br + "0", vec(a + br + "0"))
            L.k_k, L.k_a, L.r_k = vec(a + "k_k"), vec(a + "k_a"), vec(a + "r_k")
            L.lnx = (vec(a + "ln_x.weight"), vec(a + "ln_x.bias"))
            L.ffn_x_k = vec(f + "x_k")
            for nm, key in proj.items():
                setattr(L, nm, dq(a + key + ".weight"))
            L.Wfk, L.Wfv = dq(f + "key.weight"), dq(f + "value.weight")
            self.blocks.append(L)
        self.ffn_dim = self.blocks[0].Wfk.rows
        self.max_rank = max(max(L.w1.cols, L.a1.cols, L.g1.cols, L.v1.cols if L.v1 else 0)
                            for L in self.blocks)
        self._build_struct()
        self._ws = {}
        self._lora_dense = {}
        self.fused_prep = True       # sequence path: LN/shift/lerp rows written in their consumers' forms
        torch.cuda.synchronize(dev)

    # ------------------------------------------------------------------ C descriptors
    def _build_struct(self):
        n = self.n_layer
        self._layers_c = (LayerStruct * n)()
        p = lambda t: t.data_ptr() if t is not None else None
        for i, L in enumerate(self.blocks):
            s = self._layers_c[i]
            s.ln1_w, s.ln1_b, s.ln2_w, s.ln2_b = p(L.ln1[0]), p(L.ln1[1]), p(L.ln2[0]), p(L.ln2[1])
            s.x_mix, s.w0, s.a0, s.v0 = p(L.x_mix), p(L.w0), p(L.a0), p(L.v0)
            s.k_k, s.k_a, s.r_k = p(L.k_k), p(L.k_a), p(L.r_k)
            s.lnx_w, s.lnx_b, s.ffn_x_k = p(L.lnx[0]), p(L.lnx[1]), p(L.ffn_x_k)
            for nm in ("w1", "w2", "a1", "a2", "v1", "v2", "g1", "g2", "Wr", "Wk", "Wv", "Wo", "Wfk", "Wfv"):
                d = getattr(L, nm)
                if d is not None:
                    setattr(s, nm, d.struct)
        m = ModelStruct()
        m.n_layer, m.n_embd, m.head_size = self.n_layer, self.n_embd, self.head_size
        m.vocab_size, m.ffn_dim, m.max_rank = self.vocab_size, self.ffn_dim, self.max_rank
        m.emb, m.head = self.emb.struct, self.head.struct
        m.ln0_w, m.ln0_b = p(self.ln0[0]), p(self.ln0[1])
        m.lnout_w, m.lnout_b = p(self.ln_out[0]), p(self.ln_out[1])
        m.layers = C.cast(self._layers_c, C.POINTER(LayerStruct))
        self._model_c = m

    def weight_nbytes(self, with_emb=False) -> int:
        """File-format bytes a decode step streams (embedding excluded by default)."""
        n = self.head.nbytes_file()
        for L in self.blocks:
            for nm in ("w1", "w2", "a1", "a2", "v1", "v2", "g1", "g2", "Wr", "Wk", "Wv", "Wo", "Wfk", "Wfv"):
                d = getattr(L, nm)
                if d is not None:
                    n += d.nbytes_file()
        return n + (self.emb.nbytes_file() if with_emb else 0)

    # ------------------------------------------------------------------ state
    def init_state(self, batch_size: int = 1):
        """[(wkv [B,H,S,S], tmix_shift, cmix_shift)] * n_layer; shifts start as None
        (= zeros), as in the reference (quant_model.py:902-908)."""
        H, S = self.n_head, self.head_size
        return [(torch.zeros((batch_size, H, S, S), device=self.device), None, None)
                for _ in range(self.n_layer)]

    @staticmethod
    def clone_state(states):
        """Deep copy; T == 1 steps update a state in place, so keep a clone to roll back."""
        return [tuple(None if t is None else t.clone() for t in st) for st in states]

    def _materialize(self, states, B):
        out = []
        for wkv, ts, cs in states:
            z = lambda t: (torch.zeros((B, 1, self.n_embd), device=self.device) if t is None
                           else t.reshape(B, 1, self.n_embd).contiguous().float())
            out.append((wkv.contiguous().float(), z(ts), z(cs)))
        return out

    # ------------------------------------------------------------------ T == 1
    def _new_workspace(self, B):
        n = _lib.load().rwkvq_decode_workspace_bytes(C.byref(self._model_c), B)
        return torch.zeros(n, dtype=torch.uint8, device=self.device)               # counters start at zero

    def _workspace(self, B):
        if B not in self._ws:
            self._ws[B] = self._new_workspace(B)
        return self._ws[B]

    def _decode(self, tokens, states, logits=None, next_tokens=None, ws=None):
        """tokens [B] int64 on the device; states materialised; updates them in place.
        ``ws``: a workspace of the caller's own (steps that may overlap on the device must not
        share one); default: the model's workspace for this batch size."""
        B = tokens.shape[0]
        if ws is None:
            ws = self._workspace(B)
        arr = lambda k: (C.c_void_p * self.n_layer)(*[st[k].data_ptr() for st in states])
        if logits is None:
            logits = torch.empty((B, self.vocab_size), dtype=torch.float32, device=self.device)
        lib = _lib.load()
        _lib.check(lib.rwkvq_decode_step(C.byref(self._model_c), B, tokens.data_ptr(), arr(0), arr(1), arr(2),
                                         ws.data_ptr(), ws.numel(), logits.data_ptr(),
                                         None if next_tokens is None else next_tokens.data_ptr(),
                                         _lib.stream_ptr()), "rwkvq_decode_step")
        return logits

    # ------------------------------------------------------------------ T > 1
    def _linear(self, dq, x, epilogue=_lib.EPI_NONE, resid=None):
        """x [N, IN] fp32 -> [N, OUT].  Up to ``gemv_max_batch`` rows: the exact
        weight-streaming GEMV per row; more rows: the dequant-fused tensor-core GEMM
        (sb6 / sym); other layouts at large N: dequantise once + dense fp32 GEMM."""
        if x.shape[0] <= self.gemv_max_batch:
            return ops.gemv(dq.bufs, dq.meta, x, epilogue, resid)
        if x.shape[0] <= self.batch_max and ops.has_batch_layout(dq):
            return ops.gemv_batch(dq, x, epilogue, resid)
        if dq.kind in ("sb6", "sym"):
            return ops.gemm(dq, x, epilogue, resid)
        if x.shape[0] < self.gemm_min_batch:
            return ops.gemv(dq.bufs, dq.meta, x, epilogue, resid)
        y = x @ ops.dequant(dq.bufs, dq.meta, torch.float32, False).t()
        if epilogue == _lib.EPI_RELU2:
            y = torch.relu(y) ** 2
        elif epilogue == _lib.EPI_ADD:
            y = y + resid
        return y

    def _lora_seq(self, dq, x, act):
        """x [N, in] @ W [in, out] for a LoRA tensor stored [in, out].  Few rows: the packed
        kernel; many rows: a tensor-core GEMM on the weights dequantised once (kept in the
        loader's precision fp16(bf16(.)), stacked twice: 4 bytes per LoRA weight)."""
        if x.shape[0] <= 8:
            return ops.gemv_t(dq.bufs, dq.meta, x.contiguous(), act, True)
        w = self._lora_stacked(dq)
        # x = hi + lo with both halves fp16: [hi | lo] @ [W; W] on the tensor cores with fp32
        # accumulation gives x @ W to ~2^-22 relative (a plain fp32 GEMM runs on the SIMT pipes)
        if x.shape[1] % 2:
            y = x @ w[: x.shape[1]].float()
        else:
            y = torch.mm(ops.split_fp16(x), w, out_dtype=torch.float32)
        return torch.tanh(y) if act == 1 else torch.sigmoid(y) if act == 2 else y

    def _linear_rows(self, dq, rows, epilogue=_lib.EPI_NONE, resid=None):
        """``_linear`` on rows prepared by ``seq_ln_shift_mix_prep`` (sb6 / sym tensors read the
        scaled fp16 copy directly; other layouts take the fp32 rows)."""
        if rows.x16 is not None and dq.kind in ("sb6", "sym"):
            return ops.gemm_x16(dq, rows, epilogue, resid)
        return self._linear(dq, rows.f32, epilogue, resid)

    def _lora_rows(self, dq, rows, act):
        """``_lora_seq`` on prepared rows: the [hi | lo] fp16 split times the twice-stacked matrix."""
        if rows.split is None:
            return self._lora_seq(dq, rows.f32, act)
        y = torch.mm(rows.split, self._lora_stacked(dq), out_dtype=torch.float32)
        return torch.tanh(y) if act == 1 else torch.sigmoid(y) if act == 2 else y

    def _lora_stacked(self, dq):
        w = self._lora_dense.get(id(dq))
        if w is None:                                   # values are exactly fp16 by the loader's policy
            w = ops.dequant(dq.bufs, dq.meta, torch.float32, True).half()
            w = torch.cat([w, w], dim=0).contiguous()   # stacked twice: see split_fp16
            self._lora_dense[id(dq)] = w
        return w

    def _prep_modes(self, N, lins):
        """Which form each mix row is written in: the scaled fp16 copy when its linear runs on
        the dequant-fused GEMM, else fp32."""
        gemm = lambda dq: dq.kind in ("sb6", "sym") and N > max(self.gemv_max_batch, self.batch_max)
        return [ops.PREP_SCALED if gemm(dq) else ops.PREP_F32 for dq in lins]

    def _block_seq(self, i, L, x, v_first, state):
        B, T, D = x.shape
        H, S = self.n_head, self.head_size
        wkv, ts, cs = state
        N = B * T
        pairs = [(L.w1, L.w2), (L.a1, L.a2), (L.g1, L.g2)] + ([(L.v1, L.v2)] if i > 0 else [])
        # both LoRA products of all branches in two launches of the library's own tensor-core kernels, up
        # to lora_pair_max rows; longer calls (pp512 at batch 16 = 8192 rows) go through a dense fp16 copy
        # and a library GEMM, which is faster there (the own kernels re-stage x per 32 rank columns)
        pair_kernel = N <= self.lora_pair_max and ops.lora_pair_ok(pairs, D)
        if self.fused_prep and N > 8 and D % 2 == 0:
            # LN1 + shift + 6 lerps, each row written once in the form its consumers read
            mr, mk, mv = self._prep_modes(N, (L.Wr, L.Wk, L.Wv))
            lm = ops.PREP_F32 if pair_kernel else ops.PREP_SPLIT
            modes = [mr, lm, mk, mv | (lm if i > 0 else 0), lm, lm]
            (xr, xw, xk, xv, xa, xg), ts = ops.seq_ln_shift_mix_prep(x, L.ln1[0], L.ln1[1], ts, L.x_mix, modes)
            lin, lora = self._linear_rows, self._lora_rows
            f32 = lambda rows: rows.f32
        else:
            xs, ts = ops.seq_ln_shift_mix(x, L.ln1[0], L.ln1[1], ts, L.x_mix)          # LN1 + shift + 6 lerps
            xr, xw, xk, xv, xa, xg = (xs[j].reshape(N, D) for j in range(6))
            lin, lora = self._linear, self._lora_seq
            f32 = lambda rows: rows
        lora2 = lambda dq, t, act=0: self._lora_seq(dq, t, act)
        r, k, v = lin(L.Wr, xr), lin(L.Wk, xk), lin(L.Wv, xv)
        if pair_kernel:
            ys = ops.lora_pair(pairs, [f32(xw), f32(xa), f32(xg)] + ([f32(xv)] if i > 0 else []), [1, 0, 2, 0][:len(pairs)])
            y_w, y_a, g = ys[:3]
            y_v = ys[3] if i > 0 else None
        else:
            y_w = lora2(L.w2, lora(L.w1, xw, 1))
            y_a = lora2(L.a2, lora(L.a1, xa, 0))
            g = lora2(L.g2, lora(L.g1, xg, 2))
            y_v = None if i == 0 else lora2(L.v2, lora(L.v1, xv, 0))
        if i == 0:
            v_first = v
        w, k, v2, na, nb = ops.seq_tmix_pre(k, v, y_w, y_a, y_v, None if i == 0 else v_first, L.w0, L.a0, L.v0,
                                            L.k_k, L.k_a, H)
        r4 = lambda t: t.reshape(B, T, H, S)
        out, wkv = wkv7_infer(r4(r), r4(w), r4(k), r4(v2), r4(na), r4(nb), wkv)
        og = wkv_tail(out, r, k, v2, L.r_k, L.lnx[0], L.lnx[1], g, H, S)
        x = self._linear(L.Wo, og.reshape(N, D), epilogue=_lib.EPI_ADD, resid=x.reshape(N, D).contiguous())
        if self.fused_prep and N > 8 and D % 2 == 0:
            (xk2,), cs = ops.seq_ln_shift_mix_prep(x.reshape(B, T, D), L.ln2[0], L.ln2[1], cs, L.ffn_x_k,
                                                   self._prep_modes(N, (L.Wfk,)))
            h = self._linear_rows(L.Wfk, xk2, epilogue=_lib.EPI_RELU2)
        else:
            xk2, cs = ops.seq_ln_shift_mix(x.reshape(B, T, D), L.ln2[0], L.ln2[1], cs, L.ffn_x_k)     # LN2 + shift + lerp
            h = self._linear(L.Wfk, xk2.reshape(N, D), epilogue=_lib.EPI_RELU2)
        x = self._linear(L.Wfv, h, epilogue=_lib.EPI_ADD, resid=x).reshape(B, T, D)
        return x, v_first, (wkv, ts, cs)

    def _embed(self, idx):
        """Rows of the packed table in the loader's precision fp16(bf16(.))."""
        flat = idx.reshape(-1).clamp(0, self.vocab_size - 1)
        uniq, inv = torch.unique(flat, return_inverse=True)
        if self.emb.kind == "dense":
            rows = self.emb.bufs[0][uniq].float()
        else:
            bufs = [b[uniq].contiguous() if b.numel() and b.shape[0] == self.emb.rows else b
                    for b in self.emb.bufs[:9]] + list(self.emb.bufs[9:])
            meta = list(self.emb.meta)
            meta[2] = uniq.numel()
            bufs[9] = bufs[10] = torch.empty(0, dtype=torch.uint8, device=self.device)
            rows = ops.dequant(bufs, meta, torch.float32, True)
        return rows.half().float()[inv].reshape(*idx.shape, self.n_embd)

    def forward_hidden(self, idx, states):
        idx = torch.as_tensor(idx, device=self.device).long()
        B, T = idx.shape
        states = self._materialize(states, B)
        if self.emb.outliers is None and self.n_embd <= 4096:
            x = ops.seq_embed_ln0(self.emb, idx.clamp(0, self.vocab_size - 1), *self.ln0)     # gather + LN0: one kernel
        else:
            x = F.layer_norm(self._embed(idx), (self.n_embd,), *self.ln0)
        v_first, new_states = None, []
        for i, (L, st) in enumerate(zip(self.blocks, states)):
            x, v_first, st = self._block_seq(i, L, x, v_first, st)
            new_states.append(st)
        if self.n_embd <= 4096:
            return ops.seq_layer_norm(x, *self.ln_out), new_states
        return F.layer_norm(x, (self.n_embd,), *self.ln_out), new_states

    def forward_stateful(self, idx, states, last_only: bool = False, tail_only: int = 0):
        """idx [B, T] -> (logits [B, T | 1 | tail_only, V] fp32, new_states).
        T == 1 updates the given state tensors in place and returns them."""
        idx = torch.as_tensor(idx, device=self.device).long()
        B, T = idx.shape
        if T == 1:
            st = self._materialize(states, B)
            logits = self._decode(idx.reshape(B).contiguous(), st)
            return logits.reshape(B, 1, self.vocab_size), st
        x, new_states = self.forward_hidden(idx, states)
        if last_only:
            x = x[:, -1:]
        elif tail_only and T > tail_only:
            x = x[:, -tail_only:]
        n = x.shape[1]
        logits = self._linear(self.head, x.reshape(B * n, self.n_embd).contiguous())
        return logits.reshape(B, n, self.vocab_size), new_states

    @property
    def step(self):
        return self.forward_stateful

    def __call__(self, idx):
        idx = torch.as_tensor(idx, device=self.device).long()
        return self.forward_stateful(idx, self.init_state(idx.shape[0]))[0]

    # ------------------------------------------------------------------ generation
    def generate(self, idx, n_tokens: int):
        """Greedy decode: prefill ``idx`` [B, T], then ``n_tokens`` argmax steps.
        Returns (tokens [B, n_tokens], states)."""
        idx = torch.as_tensor(idx, device=self.device).long()
        B = idx.shape[0]
        logits, st = self.forward_stateful(idx, self.init_state(B), last_only=True)
        dec = self.decoder(B, states=st, use_graph=False)
        tok = logits[:, -1].argmax(-1)
        out = []
        for _ in range(n_tokens):
            out.append(tok.clone())
            tok = dec.step(tok)
        return torch.stack(out, dim=1), dec.states

    def decoder(self, batch_size: int = 1, states=None, use_graph: bool = True, self_feed: bool = False, groups=None):
        """A ``Decoder``: the whole token of ``batch_size`` streams as one CUDA-graph replay."""
        return Decoder(self, batch_size, states, use_graph, self_feed, groups)

    def decode_groups(self, batch_size: int) -> int:
        """Stream groups whose launch chains run side by side (see ``Decoder``).  Measured on B200
        (1.5B, ms per step, one group / two groups): 64 streams 4.20 / 4.38, 32 streams 3.02 / 3.03,
        16 streams 2.13 / 2.54 with the default two-term linears (which walk 16-token tiles inside one
        launch), 3.57 / 3.8 at 64 streams with RWKVQ_BATCH_FAST=1.  One group is the default."""
        return 1

    @property
    def launches_per_token(self) -> int:
        """Kernels one decoded token launches at batch 1: per layer 2 norm/shift/lerp,
        4 GEMV (r/k/v fused), 2 LoRA, 1 time-mix core; plus embedding, final norm, head, argmax (2)."""
        return self.n_layer * 9 + 5


class Decoder:
    """Token-by-token greedy decoding of B streams with device-resident state.
    ``step(tokens)`` feeds tokens [B] and returns the argmax next tokens [B] (device);
    with ``use_graph`` the whole token (all kernels) is one CUDA-graph replay.

    ``groups`` > 1 splits the streams into that many groups whose launch chains run side by
    side on their own CUDA streams (parallel branches of the captured graph): a chain is a
    sequence of dependent, latency-bound launches none of which fills the GPU, so two or four
    of them overlap; the price is that every group streams the weights itself."""

    def __init__(self, model: QuantRWKV7, batch_size, states=None, use_graph=True, self_feed=False, groups=None):
        self.m, self.B = model, batch_size
        self.self_feed = self_feed        # the replayed graph ends by feeding the argmax back
        st = model.init_state(batch_size) if states is None else states
        self.states = model._materialize(st, batch_size)
        dev = model.device
        self.tokens = torch.zeros(batch_size, dtype=torch.long, device=dev)
        self.next_tokens = torch.zeros(batch_size, dtype=torch.long, device=dev)
        self.logits = torch.empty((batch_size, model.vocab_size), dtype=torch.float32, device=dev)
        if groups is None:
            groups = model.decode_groups(batch_size)
        self.groups = max(1, min(int(groups), batch_size))
        self._bounds = [(g * batch_size // self.groups, (g + 1) * batch_size // self.groups) for g in range(self.groups)]
        # its own workspaces: decoders (and groups) on different streams may overlap
        self._ws = [model._new_workspace(b1 - b0) for b0, b1 in self._bounds]
        self._streams = [torch.cuda.Stream(device=dev) for _ in range(self.groups - 1)]
        self._views = [([tuple(t[b0:b1] for t in st) for st in self.states], self.tokens[b0:b1], self.logits[b0:b1],
                        self.next_tokens[b0:b1]) for b0, b1 in self._bounds]
        self.graph = None
        self.launches_per_step = None
        if use_graph:
            self._capture()

    def _run(self):
        cur = torch.cuda.current_stream()
        for g in range(1, self.groups):                 # fork: the other groups leave the caller's stream here
            st, tok, lg, nxt = self._views[g]
            s = self._streams[g - 1]
            s.wait_stream(cur)
            with torch.cuda.stream(s):
                self.m._decode(tok, st, lg, nxt, self._ws[g])
        st, tok, lg, nxt = self._views[0]
        self.m._decode(tok, st, lg, nxt, self._ws[0])
        for s in self._streams:
            cur.wait_stream(s)                          # join
        if self.self_feed:
            self.tokens.copy_(self.next_tokens)

    def _capture(self):
        snap = QuantRWKV7.clone_state(self.states)
        s = torch.cuda.Stream(device=self.m.device)
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            self._run()                       # warm-up outside capture (lazy attribute set-up)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=s):
                self._run()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        for dst, src in zip(self.states, snap):       # undo the two trial steps
            for d, t in zip(dst, src):
                d.copy_(t)
        self.tokens.zero_()
        self.graph = g

    def step(self, tokens=None):
        if tokens is not None:
            self.tokens.copy_(tokens.reshape(self.B), non_blocking=True)
        if self.graph is not None:
            self.graph.replay()
        else:
            self._run()
        return self.next_tokens

    def feed_back(self):
        """Use the last argmax as the next input without leaving the device."""
        self.tokens.copy_(self.next_tokens)

    def check(self):
        """Synchronise and raise if a bounded device-side wait of a step ran out (the first word of
        a step's workspace then holds the error code)."""
        torch.cuda.synchronize(self.m.device)
        for ws in self._ws:
            _lib.check(int(ws[:4].view(torch.int32).item()), "rwkvq_decode_step(kernel status)")
