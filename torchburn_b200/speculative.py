"""Speculative decoding and multi-sequence batching over the decoders of this package.

Mirrors python/torchburn/llm/speculative.py:71-379 of the reference: the same two classes, constructor
arguments and methods, so code written against the reference runs unchanged.

``SpeculativeDecoder``: a small draft decoder proposes K tokens, the target decoder checks them
(Leviathan et al. 2023: accept token t with probability min(1, p_target(t) / p_draft(t)); on the first
rejection sample from max(0, p_target - p_draft) renormalised; when all K pass, one more token comes
from the target's next distribution).  With a ``B200QwenDecoder`` built with ``max_batch > 1`` as the
target, the K + 1 positions of a round are ONE batched step (``verify_tokens``): one pass over the
weights instead of K + 1.

``BatchedDecoder``: several prompts with separate KV caches.  The reference creates one decoder per
sequence (``decoder_factory``); here, when the factory's decoder has ``step_batch`` and enough rows, ONE
decoder advances all sequences of a chunk per step (one pass over the weights for the whole chunk).
Decoders without ``step_batch`` are driven one per sequence as in the reference.

Both accept any object with ``prefill(tokens) -> logits``, ``step(token, offset) -> logits`` and
``reset_kv_cache()``.  Randomness comes from ``random`` (seed it for reproducible runs).

Two deliberate differences in position bookkeeping.  The reference feeds the last prompt token a second
time at position len(prompt) (speculative.py:104-127) and, after a round in which every draft passed,
advances the offset by K although K + 1 tokens were emitted (:243-247), so that the bonus token overwrites
the last draft's cache row.  Here every token sits at its own position: the caches hold the prompt without
its last token, that token is the first input of the first round, and the offset advances by the number
of emitted tokens.  With temperature 0 the output therefore equals the target decoder's own greedy
continuation of the prompt (tested).
"""
from __future__ import annotations

import random
from typing import Any, Callable, List, Optional, Sequence

import numpy as np

__all__ = ["SpeculativeDecoder", "BatchedDecoder"]


def _probs(logits, temperature: float, top_k: int = 0) -> np.ndarray:
    """Softmax of logits / temperature; temperature <= 0 is greedy (a one-hot row).  ``top_k`` > 0 keeps
    the k largest logits."""
    z = np.asarray(logits, dtype=np.float64).reshape(-1)
    if not temperature > 0.0:
        p = np.zeros_like(z)
        p[int(np.argmax(z))] = 1.0
        return p
    if 0 < top_k < z.size:
        kth = np.partition(z, z.size - top_k)[z.size - top_k]
        z = np.where(z >= kth, z, -np.inf)
    z = (z - z.max()) / temperature
    e = np.exp(z)
    return e / e.sum()


def _draw(p: np.ndarray) -> int:
    """Inverse-CDF draw (python/torchburn/llm/speculative.py:51-58: first index whose running sum reaches r)."""
    r = random.random()
    i = int(np.searchsorted(np.cumsum(p), r, side="left"))
    return min(i, p.size - 1)


def _prefill(dec, prompt: Sequence[int]) -> np.ndarray:
    """Logits after the last prompt token, by the fastest call the decoder has."""
    if hasattr(dec, "reset_kv_cache"):
        dec.reset_kv_cache()
    if len(prompt) > 1 and hasattr(dec, "prefill_tokens"):
        dec.prefill_tokens(list(prompt[:-1]), 0)
        return np.asarray(dec.step(prompt[-1], len(prompt) - 1))
    if len(prompt) > 1 and hasattr(dec, "prefill"):
        return np.asarray(dec.prefill(list(prompt)))
    out = None
    for i, t in enumerate(prompt):
        out = dec.step(t, i)
    return np.asarray(out)


class SpeculativeDecoder:
    """python/torchburn/llm/speculative.py:71-252."""

    def __init__(self, draft: Any, target: Any, K: int = 4, temperature: float = 1.0, top_k: int = 0,
                 eos_token_id: Optional[int] = None) -> None:
        if K < 1:
            raise ValueError("K must be at least 1")
        self.draft, self.target = draft, target
        self.K, self.temperature, self.top_k, self.eos_token_id = K, temperature, top_k, eos_token_id
        self.rounds = 0          # verify rounds of the last generate()
        self.accepted = 0        # draft tokens accepted in the last generate()

    def _target_rows(self, last: int, offset: int, drafts: List[int]) -> np.ndarray:
        """Target logits at positions offset .. offset + len(drafts): the inputs are the last emitted token
        and then the drafts.  One batched call when the target has verify_tokens."""
        inputs = [last] + drafts
        if hasattr(self.target, "verify_tokens"):
            return np.asarray(self.target.verify_tokens(offset, inputs))
        return np.stack([np.asarray(self.target.step(t, offset + i)) for i, t in enumerate(inputs)])

    def generate(self, prompt_ids: Sequence[int], max_new_tokens: int = 128) -> List[int]:
        """Token ids generated after the prompt (at most ``max_new_tokens``)."""
        prompt = list(prompt_ids)
        if not prompt:
            raise ValueError("empty prompt")
        self.rounds = self.accepted = 0
        # both caches hold the prompt except its last token, which is the first input of the first round
        for dec in (self.draft, self.target):
            dec.reset_kv_cache()
            if len(prompt) > 1:
                if hasattr(dec, "prefill_tokens"):
                    dec.prefill_tokens(prompt[:-1], 0)
                else:
                    for i, t in enumerate(prompt[:-1]):
                        dec.step(t, i)
        out: List[int] = []
        offset = len(prompt) - 1      # position of the next input token
        last = prompt[-1]
        while len(out) < max_new_tokens:
            if self.eos_token_id is not None and out and out[-1] == self.eos_token_id:
                break
            # draft K tokens
            drafts: List[int] = []
            dps: List[np.ndarray] = []
            tok = last
            for i in range(self.K):
                p = _probs(self.draft.step(tok, offset + i), self.temperature, self.top_k)
                tok = _draw(p)
                drafts.append(tok)
                dps.append(p)
                if self.eos_token_id is not None and tok == self.eos_token_id:
                    break
            # the target's distributions at the same positions, and one beyond
            rows = self._target_rows(last, offset, drafts)
            self.rounds += 1
            n_ok = 0
            emitted: List[int] = []
            for i, t in enumerate(drafts):
                tp = _probs(rows[i], self.temperature, self.top_k)
                if random.random() <= min(1.0, tp[t] / (dps[i][t] + 1e-12)):
                    emitted.append(t)
                    n_ok += 1
                    if self.eos_token_id is not None and t == self.eos_token_id:
                        break
                else:
                    rest = np.maximum(tp - dps[i], 0.0)
                    s = rest.sum()
                    emitted.append(_draw(rest / s) if s > 0 else int(np.argmax(tp)))
                    break
            else:
                emitted.append(_draw(_probs(rows[len(drafts)], self.temperature, self.top_k)))
                # the draft model has not seen its own last token yet: its cache must hold it before the next round
                self.draft.step(drafts[-1], offset + len(drafts))
            self.accepted += n_ok
            out.extend(emitted)
            # positions offset .. offset + len(emitted) - 1 now hold [last] + emitted[:-1] in both caches as far as
            # the accepted prefix goes; the last emitted token is the next round's first input and overwrites
            # whatever a rejected draft left at its position
            offset += len(emitted)
            last = emitted[-1]
        return out[:max_new_tokens]


class BatchedDecoder:
    """python/torchburn/llm/speculative.py:296-379."""

    def __init__(self, decoder_factory: Callable[[], Any], max_batch: int = 8, temperature: float = 1.0, top_k: int = 40,
                 eos_token_id: Optional[int] = None) -> None:
        if max_batch < 1:
            raise ValueError("max_batch must be at least 1")
        self.decoder_factory = decoder_factory
        self.max_batch, self.temperature, self.top_k, self.eos_token_id = max_batch, temperature, top_k, eos_token_id

    def generate_batch(self, prompts: Sequence[Sequence[int]], max_new_tokens: int = 128) -> List[List[int]]:
        out: List[List[int]] = []
        for i in range(0, len(prompts), self.max_batch):
            out.extend(self._chunk([list(p) for p in prompts[i:i + self.max_batch]], max_new_tokens))
        return out

    def _pick(self, logits) -> int:
        return _draw(_probs(logits, self.temperature, self.top_k))

    def _chunk(self, prompts: List[List[int]], max_new_tokens: int) -> List[List[int]]:
        if any(not p for p in prompts):
            raise ValueError("empty prompt")
        first = self.decoder_factory()
        rows = getattr(first, "max_batch", 1)
        if hasattr(first, "step_batch") and rows >= len(prompts) and len(prompts) > 1:
            return self._chunk_one_decoder(first, prompts, max_new_tokens)
        decs = [first] + [self.decoder_factory() for _ in prompts[1:]]
        gen: List[List[int]] = [[] for _ in prompts]
        done = [False] * len(prompts)
        for i, (dec, p) in enumerate(zip(decs, prompts)):
            t = self._pick(_prefill(dec, p))
            if self.eos_token_id is not None and t == self.eos_token_id:
                done[i] = True
            else:
                gen[i].append(t)
        for _ in range(max_new_tokens - 1):
            if all(done):
                break
            for i, dec in enumerate(decs):
                if done[i]:
                    continue
                t = self._pick(dec.step(gen[i][-1], len(prompts[i]) + len(gen[i]) - 1))
                gen[i].append(t)
                done[i] = (self.eos_token_id is not None and t == self.eos_token_id) or len(gen[i]) >= max_new_tokens
        return [g[:max_new_tokens] for g in gen]

    def _chunk_one_decoder(self, dec, prompts: List[List[int]], max_new_tokens: int) -> List[List[int]]:
        """All sequences of the chunk as rows of one decoder: a step reads the weights once for every row.
        Finished rows keep stepping on their last token at their last position (their cache row is simply
        rewritten) and their results are dropped."""
        n = len(prompts)
        dec.reset_kv_cache()
        longest = max(len(p) for p in prompts)
        logits = [None] * n
        for pos in range(longest):   # prompts advance together; a shorter one repeats its last token in place
            toks = [p[min(pos, len(p) - 1)] for p in prompts]
            offs = [min(pos, len(p) - 1) for p in prompts]
            res = dec.step_batch(toks, offs)
            for i, p in enumerate(prompts):
                if pos == len(p) - 1:
                    logits[i] = res[i].copy()
        gen: List[List[int]] = [[] for _ in prompts]
        done = [False] * n
        for i in range(n):
            t = self._pick(logits[i])
            if self.eos_token_id is not None and t == self.eos_token_id:
                done[i] = True
            else:
                gen[i].append(t)
        for _ in range(max_new_tokens - 1):
            if all(done):
                break
            toks = [g[-1] if g else p[-1] for g, p in zip(gen, prompts)]
            offs = [len(p) + len(g) - 1 if g else len(p) - 1 for g, p in zip(gen, prompts)]
            res = dec.step_batch(toks, offs)
            for i in range(n):
                if done[i]:
                    continue
                t = self._pick(res[i])
                gen[i].append(t)
                done[i] = (self.eos_token_id is not None and t == self.eos_token_id) or len(gen[i]) >= max_new_tokens
        return [g[:max_new_tokens] for g in gen]
