"""SpeculativeDecoder / BatchedDecoder (mirrors of python/torchburn/llm/speculative.py:71-379) driven by
toy decoders on the CPU: the logits of a toy decoder are a fixed pseudo-random function of the WHOLE
token history in its cache, so a token written at a wrong position, a missing cache row or a stale one
changes every later token."""
import random
import zlib

import numpy as np
import pytest

import torchburn_b200.speculative as sp

V = 37


class Toy:
    """step(token, offset) writes the token at `offset` and returns logits that depend on cache[0..offset]."""

    def __init__(self, salt=0, flip_every=0, rows=1):
        self.salt, self.flip_every, self.max_batch = salt, flip_every, rows
        self.cache = [dict() for _ in range(rows)]
        self.steps = 0
        self.verify_calls = 0

    def reset_kv_cache(self):
        for c in self.cache:
            c.clear()

    def _logits(self, row, offset):
        c = self.cache[row]
        hist = [c[i] for i in range(offset + 1)]          # KeyError = a position was never written
        seed = zlib.crc32(np.asarray(hist, np.int64).tobytes()) ^ 0x5bd1e995
        z = np.random.default_rng(seed).standard_normal(V)
        if self.flip_every and (offset % self.flip_every) == self.flip_every - 1:
            z = np.random.default_rng(seed ^ (self.salt + 1)).standard_normal(V)   # the draft disagrees here
        return z.astype(np.float32)

    def step(self, token, offset):
        self.steps += 1
        self.cache[0][offset] = int(token)
        return self._logits(0, offset)

    def prefill_tokens(self, tokens, start=0):
        for i, t in enumerate(tokens):
            self.cache[0][start + i] = int(t)
        return start + len(tokens)


class ToyVerify(Toy):
    def verify_tokens(self, start, tokens):
        self.verify_calls += 1
        return np.stack([self.step(t, start + i) for i, t in enumerate(tokens)])


class ToyBatch(Toy):
    def step_batch(self, tokens, offsets):
        self.steps += 1
        out = []
        for r, (t, o) in enumerate(zip(tokens, offsets)):
            self.cache[r][o] = int(t)
            out.append(self._logits(r, o))
        return np.stack(out)


def greedy(dec, prompt, n):
    dec.reset_kv_cache()
    for i, t in enumerate(prompt[:-1]):
        dec.step(t, i)
    out, tok, off = [], prompt[-1], len(prompt) - 1
    for _ in range(n):
        tok = int(np.argmax(dec.step(tok, off)))
        out.append(tok)
        off += 1
    return out


@pytest.mark.parametrize("K", [1, 3, 4, 7])
@pytest.mark.parametrize("target_cls", [Toy, ToyVerify])
def test_greedy_speculative_equals_target_greedy(K, target_cls):
    prompt = [5, 9, 2, 30]
    want = greedy(Toy(), prompt, 40)
    draft, target = Toy(salt=3, flip_every=3), target_cls()
    spec = sp.SpeculativeDecoder(draft, target, K=K, temperature=0.0)
    got = spec.generate(prompt, max_new_tokens=40)
    assert got == want
    assert spec.rounds < 40 or K == 1              # drafts were accepted: fewer verify rounds than tokens
    if K > 1:
        assert spec.accepted > 0
    if target_cls is ToyVerify:
        assert target.verify_calls == spec.rounds  # one batched call per round
    # a draft that always agrees: every round emits K + 1 tokens
    spec2 = sp.SpeculativeDecoder(Toy(), target_cls(), K=K, temperature=0.0)
    assert spec2.generate(prompt, max_new_tokens=40) == want
    assert spec2.rounds == -(-40 // (K + 1))


def test_speculative_sampling_runs_and_stops_at_eos():
    random.seed(4)
    prompt = [1, 2, 3]
    spec = sp.SpeculativeDecoder(Toy(salt=1, flip_every=2), ToyVerify(), K=4, temperature=0.8, top_k=10, eos_token_id=7)
    out = spec.generate(prompt, max_new_tokens=200)
    assert 0 < len(out) <= 200 and all(0 <= t < V for t in out)
    if 7 in out:
        assert out.index(7) == len(out) - 1
    with pytest.raises(ValueError):
        spec.generate([], 5)
    with pytest.raises(ValueError):
        sp.SpeculativeDecoder(Toy(), Toy(), K=0)
    # single-token prompt
    assert sp.SpeculativeDecoder(Toy(), Toy(), K=3, temperature=0.0).generate([4], 9) == greedy(Toy(), [4], 9)


@pytest.mark.parametrize("one_decoder", [False, True])
def test_batched_decoder_greedy_equals_each_sequence_alone(one_decoder):
    prompts = [[5, 9, 2], [7], [1, 2, 3, 4, 5, 6], [8, 8], [3, 1, 4, 1, 5]]
    made = []

    def factory():
        d = ToyBatch(rows=4) if one_decoder else Toy()
        made.append(d)
        return d

    bd = sp.BatchedDecoder(factory, max_batch=4, temperature=0.0, top_k=0)
    got = bd.generate_batch(prompts, max_new_tokens=12)
    assert got == [greedy(Toy(), p, 12) for p in prompts]
    if one_decoder:
        assert len(made) == 2          # one decoder per chunk (4 + 1 prompts)
    else:
        assert len(made) == len(prompts)
    # eos: a sequence stops at its first eos and the others go on
    eos = got[0][3]
    got2 = sp.BatchedDecoder(factory, max_batch=4, temperature=0.0, top_k=0, eos_token_id=eos).generate_batch(prompts, 12)
    assert got2[0] == got[0][:got[0].index(eos) + 1] if got[0].index(eos) > 0 else got2[0] == []
    for g2, g in zip(got2[1:], got[1:]):
        assert g2 == (g[:g.index(eos) + 1] if eos in g and g.index(eos) > 0 else ([] if eos in g and g.index(eos) == 0 else g))
    with pytest.raises(ValueError):
        bd.generate_batch([[1], []], 3)
