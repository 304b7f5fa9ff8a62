"""Speculative greedy decoding (history n-gram drafts verified on the small-T path):
semantics of tests/spec_decode_champ.py:89-137 of the reference.  Host logic on CPU against a
model whose predictions depend on everything its state has absorbed, and against the oracle."""
import os

import numpy as np
import pytest

from conftest import GOLDEN
from oracle import codec_np as oc
from oracle.model_np import OracleRWKV7
from rwkv_quant_b200.spec_decode import generate_speculative, ngram_draft


def test_ngram_draft():
    assert ngram_draft([1, 2, 3, 4, 1, 2, 3], 3) == [4, 1, 2]          # longest suffix [1,2,3] seen at 0
    assert ngram_draft([5, 6, 7, 8], 4) == []                             # nothing repeats
    assert ngram_draft([1, 2, 9, 1, 2, 8, 1, 2], 2) == [8, 1]           # the most recent earlier occurrence
    assert ngram_draft([3, 3, 3, 3], 2) == [3]                            # what follows may be shorter than k
    assert ngram_draft([1, 2], 3) == []


class SumModel:
    """next token = a hash of the sum of all absorbed tokens: pseudo-random, so drafts are right
    only now and then, and wrong state handling shows at once."""
    V = 5

    def __init__(self):
        self.calls = []

    def init_state(self, batch_size=1):
        return [np.zeros(1, dtype=np.int64)]

    def forward_stateful(self, idx, states, last_only=False, tail_only=0):
        idx = np.asarray(idx)
        T = idx.shape[1]
        self.calls.append(T)
        run = states[0][0] + np.cumsum(idx[0])
        pred = ((run * 2654435761) >> 9) % self.V
        logits = np.zeros((1, T, self.V), np.float32)
        logits[0, np.arange(T), pred] = 1.0
        if last_only:
            logits = logits[:, -1:]
        elif tail_only:
            logits = logits[:, -tail_only:]
        return logits, [np.array([run[-1]], dtype=np.int64)]       # fresh state, input untouched


def _plain_greedy(model, prompt, n):
    st = model.init_state(1)
    lg, st = model.forward_stateful(np.asarray([prompt]), st, last_only=True)
    out = [int(np.asarray(lg)[0, -1].argmax())]
    while len(out) < n:
        lg, st = model.forward_stateful(np.asarray([[out[-1]]]), st)
        out.append(int(np.asarray(lg)[0, -1].argmax()))
    return out


@pytest.mark.parametrize("k,flush", [(1, 2), (4, 8), (6, 3)])
def test_speculative_equals_greedy_on_state_dependent_model(k, flush):
    prompt = [3, 1, 4, 1, 0, 2, 2, 4]
    want = _plain_greedy(SumModel(), prompt, 300)
    m = SumModel()
    st = generate_speculative(m, prompt, 300, k=k, flush=flush)
    assert st.tokens == want
    assert st.accepted > 0 and st.accepted < st.drafted            # both branches of a round ran
    assert st.model_calls == len(m.calls) and st.model_calls < 300  # fewer passes than tokens
    assert max(m.calls[1:]) <= flush + 1 + k


def test_speculative_equals_greedy_on_oracle():
    man, arr = oc.open_rwkvq(os.path.join(GOLDEN, "toy_compression.rwkvq"))
    model = OracleRWKV7(man, arr)
    prompt = [7, 8, 9, 10] * 5
    want = _plain_greedy(model, prompt, 24)
    st = generate_speculative(model, prompt, 24, k=3, flush=4)
    assert st.tokens == want
    assert st.drafted > 0
