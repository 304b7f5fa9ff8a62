"""Stateful fp32 CPU forward of a quantized RWKV-7 (x070) checkpoint.

TEST INFRASTRUCTURE (parity oracle / CPU baseline) -- not a product code path.

Restates, in numpy, the reference's inference model
(backends/metal/quant_model.py) with the math of its PyTorch oracle
(models/rwkv7_ref.py):

  token shift with carried state    quant_model.py:292-301
  time-mix                          quant_model.py:730-784, rwkv7_ref.py:184-234
  WKV-7 recurrence with state in/out  rwkv7_ref.py:244-254 (zero state there),
                                    call site quant_model.py:118-125
  channel-mix                       quant_model.py:803-809, rwkv7_ref.py:257-263
  block / model / last_only / tail_only   quant_model.py:827-836, 964-990

Weight precision policy (quant_model.py:128-154, 245-262): quantized linears
(r/k/v/o, ffn key/value, head) use the exact fp32 ``q*s+m`` of the codec;
everything else is dequantised, rounded to bf16 (reader._dequantize_one), then
to fp16 when 2-D with min(shape) >= 32 (LoRA matrices, embedding, r_k), else
kept fp32.  ``linear_weights="bf16"`` rounds the linears to bf16 as well, which
is what ``RWKV7Ref`` on ``load_dequantized()`` sees; that mode is used to pin
this restatement against the reference forward.

Activations are fp32 throughout (the Metal model additionally rounds the LoRA
matmul outputs to fp16; that is an implementation artefact, not the definition).
"""
from __future__ import annotations

import numpy as np

from . import codec_np as C

F32 = np.float32


def _layer_norm(x, w, b, eps=1e-5):
    mu = x.mean(-1, keepdims=True, dtype=F32)
    xc = x - mu
    var = (xc * xc).mean(-1, keepdims=True, dtype=F32)
    return (xc / np.sqrt(var + F32(eps))) * w + b


def _sigmoid(x):
    return (F32(1) / (F32(1) + np.exp(-x))).astype(F32)


def wkv7_np(r, w, k, v, a, b, state):
    """r,w,k,v,a,b [B,T,H,S] fp32 (w is the decay itself), state [B,H,S,S]
    indexed [value row dv, key column dk].  Per step
        sa = S a;  S = S*diag(w) + sa b^T + v k^T;  y = S r."""
    B, T, H, S = r.shape
    st = np.array(state, dtype=F32, copy=True)
    out = np.empty((B, T, H, S), dtype=F32)
    for t in range(T):
        sa = np.einsum("bhvk,bhk->bhv", st, a[:, t])
        st = st * w[:, t][:, :, None, :] + sa[..., None] * b[:, t][:, :, None, :] \
            + v[:, t][..., None] * k[:, t][:, :, None, :]
        out[:, t] = np.einsum("bhvk,bhk->bhv", st, r[:, t])
    return out, st


class OracleRWKV7:
    def __init__(self, manifest, arrays, linear_weights="exact", matmul=None):
        assert linear_weights in ("exact", "bf16")
        self.man, self.arr = manifest, arrays
        self.L = manifest["n_layer"]
        self.D = manifest["n_embd"]
        self.S = manifest["head_size"]
        self.H = self.D // self.S
        self.V = manifest["vocab_size"]
        self.naming = manifest["naming"]
        assert self.naming in ("world", "custom"), self.naming
        self._lin_mode = linear_weights
        self._mm = matmul or (lambda x, w: x @ w.T)

        self.emb = self._dense("emb.weight")
        self.head = self._linear("head.weight")
        ln0 = "ln0." if self.naming == "custom" else "blocks.0.ln0."     # quant_model.py:856-859
        self.ln0 = (self._dense(ln0 + "weight"), self._dense(ln0 + "bias"))
        self.ln_out = (self._dense("ln_out.weight"), self._dense("ln_out.bias"))
        self.layers = [self._layer(i) for i in range(self.L)]

    # ---- weights
    def _dense(self, key):
        w = C.f32_to_bf16_rne(C.dequant_key(self.man, self.arr, key))
        if w.ndim == 2 and min(w.shape) >= 32:
            w = w.astype(np.float16).astype(F32)
        return np.ascontiguousarray(w, dtype=F32)

    def _linear(self, key):
        w = C.dequant_key(self.man, self.arr, key)
        if self._lin_mode == "bf16":
            w = C.f32_to_bf16_rne(w)
        return np.ascontiguousarray(w, dtype=F32)

    def _layer_custom(self, i):
        """Custom naming (quant_model.py:317-340, 791): tmix./cmix. prefixes, LoRA pairs stored as
        nn.Linear weights [out, in] (no transposition), the w0/a0/v0 vectors as *_lora_B.bias."""
        p, a, f = f"blocks.{i}.", f"blocks.{i}.tmix.", f"blocks.{i}.cmix."
        d = self._dense
        lw = dict(
            ln1=(d(p + "ln1.weight"), d(p + "ln1.bias")),
            ln2=(d(p + "ln2.weight"), d(p + "ln2.bias")),
            x=np.stack([d(a + n).reshape(-1) for n in ("x_r", "x_w", "x_k", "x_v", "x_a", "x_g")]),
            w1=d(a + "w_lora_A.weight"), w2=d(a + "w_lora_B.weight"), w0=d(a + "w_lora_B.bias").reshape(-1),
            a1=d(a + "a_lora_A.weight"), a2=d(a + "a_lora_B.weight"), a0=d(a + "a_lora_B.bias").reshape(-1),
            g1=d(a + "g_lora_A.weight"), g2=d(a + "g_lora_B.weight"),
            k_k=d(a + "k_k").reshape(self.H, self.S), k_a=d(a + "k_a").reshape(self.H, self.S),
            r_k=d(a + "r_k").reshape(self.H, self.S),
            ln_x=(d(a + "ln_x.weight"), d(a + "ln_x.bias")),
            Wr=self._linear(a + "r_proj.weight"), Wk=self._linear(a + "k_proj.weight"),
            Wv=self._linear(a + "v_proj.weight"), Wo=self._linear(a + "o_proj.weight"),
            fx=d(f + "x_k").reshape(-1),
            Wfk=self._linear(f + "key.weight"), Wfv=self._linear(f + "value.weight"))
        if i > 0:
            lw.update(v1=d(a + "v_lora_A.weight"), v2=d(a + "v_lora_B.weight"),
                      v0=d(a + "v_lora_B.bias").reshape(-1))
        return lw

    def _layer(self, i):
        if self.naming == "custom":
            return self._layer_custom(i)
        p, a, f = f"blocks.{i}.", f"blocks.{i}.att.", f"blocks.{i}.ffn."
        d = self._dense
        lw = dict(
            ln1=(d(p + "ln1.weight"), d(p + "ln1.bias")),
            ln2=(d(p + "ln2.weight"), d(p + "ln2.bias")),
            x=np.stack([d(a + n).reshape(-1) for n in ("x_r", "x_w", "x_k", "x_v", "x_a", "x_g")]),
            # stored [in, out]: dequantise first, transpose after (codec.py:514-526)
            w1=d(a + "w1").T, w2=d(a + "w2").T, w0=d(a + "w0").reshape(-1),
            a1=d(a + "a1").T, a2=d(a + "a2").T, a0=d(a + "a0").reshape(-1),
            g1=d(a + "g1").T, g2=d(a + "g2").T,
            k_k=d(a + "k_k").reshape(self.H, self.S), k_a=d(a + "k_a").reshape(self.H, self.S),
            r_k=d(a + "r_k").reshape(self.H, self.S),
            ln_x=(d(a + "ln_x.weight"), d(a + "ln_x.bias")),
            Wr=self._linear(a + "receptance.weight"), Wk=self._linear(a + "key.weight"),
            Wv=self._linear(a + "value.weight"), Wo=self._linear(a + "output.weight"),
            fx=d(f + "x_k").reshape(-1),
            Wfk=self._linear(f + "key.weight"), Wfv=self._linear(f + "value.weight"))
        if i > 0:
            lw.update(v1=d(a + "v1").T, v2=d(a + "v2").T, v0=d(a + "v0").reshape(-1))
        return lw

    # ---- state
    def init_state(self, batch_size=1):
        """[(wkv [B,H,S,S], tmix_shift [B,D] or None, cmix_shift [B,D] or None)] * L;
        a None shift means zeros (quant_model.py:902-908)."""
        return [(np.zeros((batch_size, self.H, self.S, self.S), F32), None, None)
                for _ in range(self.L)]

    @staticmethod
    def _shift(x, prev):
        B, T, D = x.shape
        p = np.zeros((B, 1, D), F32) if prev is None else prev.reshape(B, 1, D)
        return np.concatenate([p, x[:, :-1]], axis=1), x[:, -1].copy()

    # ---- blocks
    def _tmix(self, lw, i, x, v_first, wkv_state, shift):
        B, T, D = x.shape
        H, S = self.H, self.S
        mm = self._mm
        shifted, new_shift = self._shift(x, shift)
        xx = shifted - x
        xr, xw, xk, xv, xa, xg = (x + xx * lw["x"][j] for j in range(6))
        r = mm(xr, lw["Wr"]); k = mm(xk, lw["Wk"]); v = mm(xv, lw["Wv"])
        y_w = mm(np.tanh(mm(xw, lw["w1"])), lw["w2"])
        y_a = mm(mm(xa, lw["a1"]), lw["a2"])
        g = mm(_sigmoid(mm(xg, lw["g1"])), lw["g2"])
        a = _sigmoid(y_a + lw["a0"]).reshape(B, T, H, S)
        w = np.exp(F32(-0.606531) * _sigmoid(y_w + lw["w0"])).astype(F32).reshape(B, T, H, S)
        r4, k4, v4 = r.reshape(B, T, H, S), k.reshape(B, T, H, S), v.reshape(B, T, H, S)
        kk = k4 * lw["k_k"]
        kk = kk / np.sqrt((kk * kk).sum(-1, keepdims=True, dtype=F32) + F32(1e-12))
        k4 = k4 * (F32(1) + (a - F32(1)) * lw["k_a"])
        if i == 0:
            v_first = v4
        else:
            vv = _sigmoid(mm(mm(xv, lw["v1"]), lw["v2"]) + lw["v0"]).reshape(B, T, H, S)
            v4 = v4 + (v_first - v4) * vv
        out, new_state = wkv7_np(r4, w, k4, v4, -kk, kk * a, wkv_state)
        mu = out.mean(-1, keepdims=True, dtype=F32)
        oc = out - mu
        var = (oc * oc).mean(-1, keepdims=True, dtype=F32)
        out = oc / np.sqrt(var + F32(64e-5))
        out = out * lw["ln_x"][0].reshape(H, S) + lw["ln_x"][1].reshape(H, S)
        bonus = (r4 * k4 * lw["r_k"]).sum(-1, keepdims=True, dtype=F32) * v4
        out = ((out + bonus).reshape(B, T, D) * g).astype(F32)
        return mm(out, lw["Wo"]), v_first, new_state, new_shift

    def _cmix(self, lw, x, shift):
        shifted, new_shift = self._shift(x, shift)
        xk = x + (shifted - x) * lw["fx"]
        h = np.maximum(self._mm(xk, lw["Wfk"]), F32(0)) ** 2
        return self._mm(h, lw["Wfv"]), new_shift

    def forward_hidden(self, idx, states, trace=None):
        idx = np.asarray(idx)
        x = _layer_norm(self.emb[idx], *self.ln0).astype(F32)
        v_first, new_states = None, []
        for i, (lw, st) in enumerate(zip(self.layers, states)):
            wkv, ts, cs = st
            h, v_first, wkv, ts = self._tmix(lw, i, _layer_norm(x, *lw["ln1"]).astype(F32),
                                             v_first, wkv, ts)
            x = x + h
            c, cs = self._cmix(lw, _layer_norm(x, *lw["ln2"]).astype(F32), cs)
            x = (x + c).astype(F32)
            new_states.append((wkv, ts, cs))
            if trace is not None:
                trace.append(x.copy())
        return _layer_norm(x, *self.ln_out).astype(F32), new_states

    def forward_stateful(self, idx, states, last_only=False, tail_only=0):
        x, new_states = self.forward_hidden(idx, states)
        if last_only and x.shape[1] > 1:
            x = x[:, -1:]
        elif tail_only and x.shape[1] > tail_only:
            x = x[:, -tail_only:]
        return self._mm(x, self.head), new_states

    def __call__(self, idx):
        return self.forward_stateful(idx, self.init_state(np.asarray(idx).shape[0]))[0]

    def generate(self, idx, n_tokens):
        """Greedy decode: prefill `idx` [B,T] then n_tokens argmax steps."""
        logits, st = self.forward_stateful(idx, self.init_state(np.asarray(idx).shape[0]),
                                           last_only=True)
        toks = []
        for _ in range(n_tokens):
            nxt = logits[:, -1].argmax(-1)
            toks.append(nxt)
            logits, st = self.forward_stateful(nxt[:, None], st)
        return np.stack(toks, axis=1), st
