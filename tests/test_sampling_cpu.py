"""Host-side sampling of the library (no GPU needed) against the oracle's restatement of
sample_logits / apply_repetition_penalty and the reference's own known-answer tests
(tests/parity/decoder.rs:31-61)."""
import ctypes as C

import numpy as np
import pytest


@pytest.fixture(scope="module")
def L():
    from torchburn_b200 import build as tb_build

    tb_build.build()
    import torchburn_b200 as tb

    return tb.lib()


def sample(L, logits, temperature, top_k, top_p, u):
    l = np.ascontiguousarray(logits, dtype=np.float32)
    tok = C.c_int64(-1)
    assert L.tb_sample_logits(l.ctypes.data, l.size, temperature, top_k, top_p, u, C.byref(tok)) == 0
    return int(tok.value)


def test_greedy_sample_is_argmax(L):
    # tests/parity/decoder.rs:31-40
    logits = np.sin(np.arange(4096, dtype=np.float32) * np.float32(0.013)).astype(np.float32)
    logits[1234] = 100.0
    assert sample(L, logits, 0.0, 1, 1.0, 0.3) == 1234
    assert sample(L, logits, 0.7, 1, 1.0, 0.3) == 1234
    assert sample(L, logits, float("nan"), 40, 1.0, 0.3) == 1234
    tied = np.zeros(100, np.float32)
    assert sample(L, tied, 0.0, 1, 1.0, 0.5) == 0  # first maximum wins


def test_sample_within_vocab_and_top_tokens(L):
    # tests/parity/decoder.rs:42-61
    logits = (np.sin(np.arange(151936, dtype=np.float32) * np.float32(0.007)) * 5).astype(np.float32)
    logits[7], logits[88] = 40.0, 39.0
    seen = [sample(L, logits, 0.7, 40, 1.0, u) for u in np.linspace(0.0, 0.999, 64)]
    assert all(0 <= t < logits.size for t in seen)
    assert 7 in seen or 88 in seen


@pytest.mark.parametrize("top_k,top_p,temp", [(40, 1.0, 0.7), (5, 0.9, 1.3), (1000, 0.5, 0.2), (64, 0.0, 1.0), (5000, 1.0, 0.7)])
def test_sampling_matches_oracle_for_every_draw(L, oracle, top_k, top_p, temp):
    rng = np.random.default_rng(top_k)
    vocab = 2048 if top_k < 2048 else 4096  # top_k >= vocab exercises the keep-everything branch
    if top_k == 5000:
        vocab = 4096
    logits = (rng.standard_normal(vocab) * 3).astype(np.float32)
    logits[5] = np.inf  # non-finite logits are treated as -inf
    logits[9] = np.nan
    for u in np.linspace(0.0, 0.9999, 97):
        assert sample(L, logits, temp, top_k, top_p, float(u)) == oracle.sample_logits(logits, temp, top_k, top_p, float(u))


def test_large_top_k_branch_samples_from_the_top_set(L):
    rng = np.random.default_rng(1)
    logits = (rng.standard_normal(20000) * 2).astype(np.float32)
    top = set(np.argsort(logits)[-2000:].tolist())
    for u in np.linspace(0, 0.999, 40):
        assert sample(L, logits, 1.0, 2000, 1.0, float(u)) in top


def test_repetition_penalty_matches_oracle(L, oracle):
    rng = np.random.default_rng(2)
    logits = rng.standard_normal(500).astype(np.float32)
    recent = np.asarray([3, 3, 499, 7, 1000, -1, 7, 42] + list(range(100, 160)), dtype=np.int64)
    for pen in (1.0, 0.5, 1.3):
        got = logits.copy()
        assert L.tb_apply_repetition_penalty(got.ctypes.data, got.size, recent.ctypes.data, recent.size, pen) == 0
        assert np.array_equal(got, oracle.apply_repetition_penalty(logits, recent, pen))


def test_recent_window_keeps_last_64(L):
    buf = np.zeros(64, np.int64)
    n = 0
    for t in range(100):
        n = L.tb_push_recent_window(buf.ctypes.data, n, t)
    assert n == 64 and buf.tolist() == list(range(36, 100))


# ---- speculative acceptance (src/llm/decoder.rs:583-727), host part -------------------------
def _accept(L, rows, toks, probs, temp, top_p, seed):
    rows = np.ascontiguousarray(rows, np.float32); probs = np.ascontiguousarray(probs, np.float32)
    toks = np.ascontiguousarray(toks, np.int64)
    rng = C.c_uint64(seed); acc = C.c_int64(-1); bonus = C.c_int64(-1)
    v = rows.shape[-1]
    assert L.tb_speculative_accept_rows(rows.ctypes.data, v, toks.ctypes.data, toks.size, probs.ctypes.data, temp, top_p,
                                        C.byref(rng), C.byref(acc), C.byref(bonus)) == 0
    return int(acc.value), int(bonus.value), int(rng.value)


def _softmax(x, t=1.0):
    e = np.exp((x - x.max(-1, keepdims=True)) / t)
    return (e / e.sum(-1, keepdims=True)).astype(np.float32)


@pytest.mark.parametrize("temp,top_p,noise", [(1.0, 1.0, 0.3), (0.7, 0.9, 1.5), (1.3, 0.5, 0.0), (0.0, 1.0, 3.0)])
def test_speculative_accept_rows_match_oracle(L, oracle, temp, top_p, noise):
    rng = np.random.default_rng(int(temp * 10) + int(noise * 7))
    k, v = 5, 257
    outcomes = set()
    for seed in range(1, 120):
        target = (rng.standard_normal((k, v)) * 2).astype(np.float32)
        target[0, 3] = np.inf  # non-finite logits count as -inf
        draft = _softmax(target.clip(-50, 50) + noise * rng.standard_normal((k, v)).astype(np.float32), max(temp, 0.5))
        draft[0, 3] = 0.0
        toks = np.array([rng.choice(v, p=d / d.sum()) for d in draft.astype(np.float64)])
        got = _accept(L, target, toks, draft, temp, top_p, seed)
        want = oracle.speculative_accept_rows(target, toks, draft, temp, top_p, seed)
        assert got == want, (seed, got, want)
        assert 0 <= got[0] <= k and 0 <= got[1] < v
        outcomes.add(got[0])
    assert len(outcomes) >= 2 or noise == 0.0  # both the reject and the accept exits were taken


def test_speculative_accept_edge_cases(L, oracle):
    v = 64
    rows = np.linspace(-1, 1, 2 * v, dtype=np.float32).reshape(2, v)
    tp = _softmax(rows)
    # k = 0: nothing to verify (decoder.rs:594-596)
    assert _accept(L, rows[:0].reshape(0, v), [], rows[:0].reshape(0, v), 1.0, 1.0, 9)[:2] == (0, v - 1)
    # the draft puts all its mass where the target has little: rejected, and max(0, p - q) is empty
    # everywhere, so the bonus is the target's most likely token (last of equals)
    probs = tp.copy(); probs[0, 5] = 1.0
    got = _accept(L, rows, [5, 7], probs, 1.0, 1.0, 1234)
    assert got == oracle.speculative_accept_rows(rows, [5, 7], probs, 1.0, 1.0, 1234)
    if got[0] == 0:
        assert got[1] == int(np.flatnonzero(tp[0] == tp[0].max())[-1])
    # draft == target: every proposal is accepted (ratio 1), bonus from the last row's nucleus
    toks = [int(tp[0].argmax()), int(tp[1].argmax())]
    acc, bonus, _ = _accept(L, rows, toks, tp, 1.0, 0.2, 77)
    assert acc == 2 and bonus in set(np.argsort(tp[1])[::-1][:20].tolist())
    assert (acc, bonus) == oracle.speculative_accept_rows(rows, toks, tp, 1.0, 0.2, 77)[:2]
