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
