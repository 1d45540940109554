"""The CPU oracle against (1) outputs of the reference's own Python code
(tests/golden/*.npz, made by tests/golden/make_golden.py) and (2) the
closed-form known-answer cases of the reference's Rust parity tests."""
import os

import numpy as np
import pytest

from helpers import GOLDEN, load_decoder_golden, max_rel_err, rust_test_quantize_grouped


# ---------------------------------------------------------------- quantizer
def _quant_cases():
    z = np.load(os.path.join(GOLDEN, "quantizer_golden.npz"))
    names = sorted({f.split("__")[0] for f in z.files})
    return z, names


@pytest.mark.parametrize("name", _quant_cases()[1])
def test_quantizer_bit_exact_vs_reference_python(oracle, name):
    z, _ = _quant_cases()
    w, g = z[f"{name}__w"], int(z[f"{name}__g"])
    packed, scales = oracle.quantize_int4_grouped(w, g)
    assert np.array_equal(packed, z[f"{name}__packed"]), "packed bytes differ from the reference quantizer"
    assert np.array_equal(scales.view(np.uint32), z[f"{name}__scales"].view(np.uint32)), "scales differ bitwise"


def test_quantizer_rejects_ragged_k(oracle):
    with pytest.raises(ValueError):
        oracle.quantize_int4_grouped(np.zeros((2, 48), np.float32), 32)  # quantization.py:75-79


def test_unpack_all_byte_values(oracle):
    # every byte value at even (low nibble) and odd (high nibble) positions
    packed = np.arange(256, dtype=np.uint8).reshape(8, 32)
    codes = oracle.unpack_codes(packed)
    b = packed.astype(np.int32)
    assert np.array_equal(codes[:, 0::2], (b & 15) - 8)
    assert np.array_equal(codes[:, 1::2], (b >> 4) - 8)


# ------------------------------------------------- Rust parity known answers
def _ref_gemv(x, packed, scales, g):
    """reference_gemv of tests/parity/int4.rs:96-125: exact dequant-dot, f32."""
    n, pc = packed.shape
    k = pc * 2
    lo = (packed & 15).astype(np.int32) - 8
    hi = (packed >> 4).astype(np.int32) - 8
    q = np.stack([lo, hi], axis=2).reshape(n, k).astype(np.float64)
    w = q * np.repeat(scales.astype(np.float64), g, axis=1)
    return (w @ x.astype(np.float64)).astype(np.float32)


@pytest.mark.parametrize("tier", [1, 2, 3])
@pytest.mark.parametrize("g", [64, 32])
def test_int4_rs_gemv_matches_exact_dequant_reference(oracle, tier, g):
    # tests/parity/int4.rs:172-215 (n=64, k=896; budget 1e-3)
    n, k = 64, 896
    i = np.arange(k, dtype=np.float32)
    x = (np.sin(i * np.float32(0.13)) * 2).astype(np.float32)
    j = np.arange(n * k, dtype=np.float32)
    w = (np.cos(j * np.float32(0.29)) * np.float32(1.5)).astype(np.float32)
    packed, scales = rust_test_quantize_grouped(w, k, g)
    oracle.force_tier(tier)
    try:
        out = oracle.gemm_w4a32_grouped(x, packed, scales, None, g)
    finally:
        oracle.force_tier(0)
    assert max_rel_err(out, _ref_gemv(x, packed, scales, g)) < 1e-3


def test_int4_rs_bias_is_added(oracle):
    # tests/parity/int4.rs:303-329
    n, k, g = 16, 64, 64
    x = np.full(k, 0.5, np.float32)
    w = (np.sin(np.arange(n * k, dtype=np.float32) * np.float32(0.23)) * np.float32(0.5)).astype(np.float32)
    packed, scales = rust_test_quantize_grouped(w, k, g)
    bias = (np.arange(n, dtype=np.float32) * np.float32(0.01) + np.float32(0.1)).astype(np.float32)
    out = oracle.gemm_w4a32_grouped(x, packed, scales, bias, g)
    want = _ref_gemv(x, packed, scales, g) + bias
    rel = np.abs(out - want) / np.maximum(np.abs(want), 1e-4)
    assert rel.max() < 1e-2


@pytest.mark.parametrize("g", [64, 32])
def test_dispatch_tiers_exact_tiers_allclose_to_scalar(oracle, g):
    # tests/parity/dispatch_tiers.rs:130-177
    n, k = 256, 896
    x = (np.sin(np.arange(k, dtype=np.float32) * np.float32(0.13)) * 2).astype(np.float32)
    idx = np.arange(n * (k // 2), dtype=np.uint64)
    w = ((idx * np.uint64(2654435761)) % np.uint64(256)).astype(np.uint8).reshape(n, k // 2)
    si = np.arange(n * (k // g), dtype=np.int64)
    scales = (0.5 + ((si * 31) % 97).astype(np.float32) * np.float32(0.01)).astype(np.float32).reshape(n, k // g)
    oracle.force_tier(1)
    scalar = oracle.gemm_w4a32_grouped(x, w, scales, None, g)
    try:
        for tier in (2, 3):
            if oracle.force_tier(tier) != tier:
                continue
            out = oracle.gemm_w4a32_grouped(x, w, scales, None, g)
            assert max_rel_err(out, scalar) < 1e-3
    finally:
        oracle.force_tier(0)


def test_decoder_rs_rms_norm(oracle):
    # tests/parity/decoder.rs:13-29 (n=896, eps 1e-6, rel 1e-4)
    n = 896
    i = np.arange(n, dtype=np.float32)
    x = (np.sin(i * np.float32(0.31)) * 3).astype(np.float32)
    w = (1 + np.float32(0.001) * i).astype(np.float32)
    want = x.astype(np.float64) / np.sqrt((x.astype(np.float64) ** 2).mean() + 1e-6) * w
    for tier in (1, 3):
        oracle.force_tier(tier)
        got = oracle.rms_norm(x, w, 1e-6)
        oracle.force_tier(0)
        assert (np.abs(got - want) / np.maximum(np.abs(want), 1e-6)).max() < 1e-4


def test_scalar_tail_group_is_clamped(oracle):
    # gemv.rs:1606: a group size other than 32/64 takes the scalar loop and
    # clamps the last group to the K that is left.
    rng = np.random.default_rng(3)
    n, k, g = 5, 40, 16  # 3 groups, the last one 8 wide
    packed = rng.integers(0, 256, (n, k // 2), dtype=np.uint8)
    scales = rng.random((n, 3), dtype=np.float32)
    x = rng.standard_normal(k).astype(np.float32)
    out = oracle.gemm_w4a32_grouped(x, packed, scales, None, g)
    lo = (packed & 15).astype(np.int32) - 8
    hi = (packed >> 4).astype(np.int32) - 8
    q = np.stack([lo, hi], axis=2).reshape(n, k).astype(np.float64)
    want = (q * np.repeat(scales, g, axis=1)[:, :k]) @ x
    assert max_rel_err(out, want) < 1e-5


# --------------------------------------- decoder vs the reference's Python model
@pytest.mark.parametrize("fixture,tol", [("decoder_qwen_tiny_g32.npz", 1e-4), ("decoder_llama_tiny_g64.npz", 1e-4)])
@pytest.mark.parametrize("tier", [1, 3])
def test_decoder_step_matches_reference_python_model(oracle, fixture, tol, tier):
    cfg, embed, layers, fnorm, lm_w, lm_s, z = load_decoder_golden(fixture)
    oracle.force_tier(tier)
    try:
        dec = oracle.OracleDecoder(cfg, embed, layers, fnorm, lm_w, lm_s)
        for off, tok in enumerate(z["tokens"]):
            logits = dec.step(int(tok), off)
            err = max_rel_err(logits, z["logits"][off])
            assert err < tol, f"step {off}: logits rel err {err:.2e}"
        assert dec.kv_len() == len(z["tokens"])
        k0, v0 = dec.kv_cache(0)
        T = len(z["tokens"])
        assert max_rel_err(k0[:, :T], z["k_cache_l0"]) < 1e-5  # layout [Hkv, t, d], RoPE'd keys
        assert max_rel_err(v0[:, :T], z["v_cache_l0"]) < 1e-5
    finally:
        oracle.force_tier(0)


def test_decoder_oob_token_or_offset_gives_zero_logits(oracle):
    # decoder.rs:1066-1078
    cfg, embed, layers, fnorm, lm_w, lm_s, z = load_decoder_golden("decoder_qwen_tiny_g32.npz")
    dec = oracle.OracleDecoder(cfg, embed, layers, fnorm, lm_w, lm_s)
    dec.step(3, 0)
    assert np.abs(dec.get_logits()).max() > 0
    assert np.all(dec.step(cfg["vocab_size"], 1) == 0)
    assert np.all(dec.step(3, cfg["max_seq_len"]) == 0)
    assert dec.kv_len() == 1


def test_decoder_prefill_reset_semantics(oracle):
    # decoder.rs:431-477
    cfg, embed, layers, fnorm, lm_w, lm_s, z = load_decoder_golden("decoder_qwen_tiny_g32.npz")
    dec = oracle.OracleDecoder(cfg, embed, layers, fnorm, lm_w, lm_s)
    toks = [int(t) for t in z["tokens"]]
    assert dec.prefill_tokens([], 3) == 3
    assert dec.prefill_tokens(toks, 0) == len(toks)
    assert max_rel_err(dec.get_logits(), z["logits"][-1]) < 1e-4
    with pytest.raises(ValueError):
        dec.prefill_tokens(toks, cfg["max_seq_len"] - 2)
    dec.reset_kv_cache()
    assert dec.kv_len() == 0
    k0, v0 = dec.kv_cache(0)
    assert not k0.any() and not v0.any()
    assert dec.prefill_tokens(toks, 0) == len(toks)
    assert max_rel_err(dec.get_logits(), z["logits"][-1]) < 1e-4
