"""Greedy speculative decoding on the model's small-T path (draft from the stream's own history).

The scheme of the reference's demo (tests/spec_decode_champ.py:89-137): the recurrent state
``S`` covers a prefix of the stream; ``pending`` holds tokens already decided but not yet in
``S``.  A round runs ONE ``step(pending + draft, S, tail_only=len(draft)+1)``: position i of
the tail predicts the token after ``pending + draft[:i]``, so the longest draft prefix that
equals the predictions is accepted together with one more ("bonus") token.  The new state is
taken only when the whole draft was accepted (it then covers exactly ``pending + draft``);
otherwise ``S`` stays and everything accepted joins ``pending``, which a later round, or a
flush of ``pending`` alone, carries into the state.  Output tokens are those of plain greedy
decoding whenever the small-T and single-token paths agree on every argmax.

Any object with the reference's ``step(idx[B,T], states, tail_only=n) -> (logits, states)``
contract works (the CUDA ``QuantRWKV7`` and the CPU oracle alike); sequences (T > 1) must
return fresh state tensors, which is the contract of ``forward_stateful``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, List, Sequence

import numpy as np


def ngram_draft(hist: Sequence[int], k: int, nmax: int = 8, nmin: int = 2) -> List[int]:
    """Up to ``k`` tokens that followed the most recent earlier occurrence of the longest
    suffix of ``hist`` (length ``nmax`` down to ``nmin``) seen before; [] if none."""
    h = list(hist)
    n_hist = len(h)
    for n in range(min(nmax, n_hist - 1), nmin - 1, -1):
        suffix = h[n_hist - n:]
        for start in range(n_hist - n - 1, -1, -1):
            if h[start:start + n] == suffix:
                follow = h[start + n:start + n + k]
                if follow:
                    return follow
    return []


@dataclass
class SpecStats:
    rounds: int = 0
    drafted: int = 0
    accepted: int = 0
    flushes: int = 0
    model_calls: int = 0
    tokens: List[int] = field(default_factory=list)

    @property
    def acceptance(self) -> float:
        return self.accepted / max(self.drafted, 1)

    @property
    def tokens_per_call(self) -> float:
        return len(self.tokens) / max(self.model_calls, 1)


def _argmax_tail(logits) -> np.ndarray:
    """logits [1, n, V] (torch or numpy) -> argmax per position as numpy ints."""
    if hasattr(logits, "argmax") and not isinstance(logits, np.ndarray):
        return logits[0].argmax(-1).cpu().numpy()
    return np.asarray(logits)[0].argmax(-1)


def generate_speculative(model, prompt: Sequence[int], n_tokens: int, k: int = 4, flush: int = 8,
                         draft: Callable[[Sequence[int], int], List[int]] = ngram_draft,
                         to_idx: Callable = None) -> SpecStats:
    """Greedy continuation of one stream, ``n_tokens`` long.  ``k`` = draft length, ``flush`` =
    the number of pending tokens beyond which they are pushed into the state on their own.
    ``to_idx(list_of_lists)`` builds the model's index tensor (default: numpy int64)."""
    to_idx = to_idx or (lambda rows: np.asarray(rows, dtype=np.int64))
    stats = SpecStats()
    states = model.init_state(1)
    logits, states = model.forward_stateful(to_idx([list(prompt)]), states, last_only=True)
    stats.model_calls += 1
    cur = int(_argmax_tail(logits)[-1])
    hist = list(prompt) + [cur]
    out = [cur]
    pending = [cur]                                  # decided, not yet in the state
    while len(out) < n_tokens:
        if len(pending) > flush:
            logits, states = model.forward_stateful(to_idx([pending]), states, tail_only=1)
            stats.model_calls += 1
            nxt = int(_argmax_tail(logits)[-1])
            pending = [nxt]
            hist.append(nxt)
            out.append(nxt)
            stats.flushes += 1
            continue
        d = [int(t) for t in draft(hist, k)]
        x = pending + d
        if len(x) == 1:
            # a single token takes the in-place decode path: copy nothing, the state is kept
            logits, states = model.forward_stateful(to_idx([x]), states, tail_only=1)
            new_states = states
        else:
            logits, new_states = model.forward_stateful(to_idx([x]), states, tail_only=len(d) + 1)
        stats.model_calls += 1
        pred = _argmax_tail(logits)                  # pred[i] follows pending + d[:i]
        m = 0
        while m < len(d) and d[m] == int(pred[m]):
            m += 1
        good = d[:m] + [int(pred[m])]
        out.extend(good)
        hist.extend(good)
        stats.rounds += 1
        stats.accepted += m
        stats.drafted += len(d)
        if m == len(d):                              # the state now covers all of x
            states = new_states
            pending = [good[-1]]
        else:
            pending = pending + good
    stats.tokens = out[:n_tokens]
    return stats
