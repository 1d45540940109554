"""The interleaved v2 weight layout (34-byte blocks, binary16 scales): the library's host functions
and the oracle's restatement against fixtures produced by the reference's own Python code
(tests/golden/make_golden.py: quantize_weight_int4_grouped_v2 / dequantize_int4_grouped_v2) and
the known-answer cases of src/quantization/packed_v2.rs:716-769."""
import ctypes as C
import os

import numpy as np
import pytest

from helpers import GOLDEN


@pytest.fixture(scope="module")
def L():
    from torchburn_b200 import build as tb_build

    tb_build.build()
    import torchburn_b200 as tb

    return tb.lib()


@pytest.fixture(scope="module")
def gold():
    return np.load(os.path.join(GOLDEN, "layout_v2_golden.npz"))


def test_f16_conversion_is_bit_exact_with_torch_half(L, oracle, gold):
    for v, bits, back in zip(gold["f16_inputs"], gold["f16_bits"], gold["f16_back"]):
        for conv in (lambda x: L.tb_f32_to_f16(C.c_float(float(x))), oracle.f32_to_f16):
            assert conv(v) == int(bits), (v, conv(v), bits)
        for conv in (lambda b: L.tb_f16_to_f32(int(b)), oracle.f16_to_f32):
            got = np.float32(conv(bits))
            assert got.tobytes() == np.float32(back).tobytes() or (np.isnan(got) and np.isnan(back)), (v, got, back)
    # every binary16 value survives the round trip through fp32
    for bits in range(0, 1 << 16, 7):
        f = L.tb_f16_to_f32(bits)
        if f == f:
            assert L.tb_f32_to_f16(C.c_float(f)) == bits
            assert np.float32(f).tobytes() == np.float32(oracle.f16_to_f32(bits)).tobytes()


def test_f16_roundtrip_accuracy_known_answers(L):
    # src/quantization/packed_v2.rs:716-741
    for v in (0.0, -0.0, 1.0, -1.0, 0.5, 2.0, 65504.0, -3.75, 1234.5, 1e-4, 6.0e-5, 6.1e-8):
        back = L.tb_f16_to_f32(L.tb_f32_to_f16(C.c_float(v)))
        if v == 0.0:
            assert back == 0.0 and np.signbit(np.float32(back)) == np.signbit(np.float32(v))
        elif abs(v) < 6.1e-5:
            assert abs(back - v) < 6e-8
        else:
            assert abs((back - v) / v) < 6e-4
    assert L.tb_f16_to_f32(L.tb_f32_to_f16(C.c_float(1e6))) == float("inf")
    assert L.tb_f16_to_f32(L.tb_f32_to_f16(C.c_float(-1e6))) == float("-inf")


def test_pack_matches_reference_python_blocks(L, oracle, gold):
    packed, scales, blocked = gold["packed"], gold["scales"], gold["blocked"]
    n, k = packed.shape[0], packed.shape[1] * 2
    out = np.empty_like(blocked)
    assert L.tb_pack_v1_to_v2(packed.ctypes.data, scales.ctypes.data, n, k, out.ctypes.data) == 0
    assert np.array_equal(out, blocked)
    assert np.array_equal(oracle.pack_v1_to_v2(packed, scales), blocked)
    p2, s2 = np.empty_like(packed), np.empty_like(scales)
    assert L.tb_unpack_v2_to_v1(blocked.ctypes.data, n, k, p2.ctypes.data, s2.ctypes.data) == 0
    assert np.array_equal(p2, packed)
    assert np.array_equal(s2, scales.astype(np.float16).astype(np.float32))  # test_parity.py:184
    # dequantised values equal the reference's dequantize_int4_grouped_v2
    codes = oracle.unpack_codes(p2).astype(np.float32)
    assert np.array_equal(codes * np.repeat(s2, 64, axis=1), gold["dequant"])


def test_pack_block_layout_known_answer(L):
    # src/quantization/packed_v2.rs:743-769: lcg bytes, scales 0.01 + i*0.001, n=3, k=128
    seed = 42
    src = []
    for _ in range(3 * 64):
        seed = (seed * 6364136223846793005 + 1442695040888963407) % (1 << 64)
        src.append((seed >> 33) & 0xFF)
    src = np.array(src, np.uint8).reshape(3, 64)
    scales = (0.01 + np.arange(6, dtype=np.float32) * np.float32(0.001)).reshape(3, 2)
    out = np.empty((3, 2 * 34), np.uint8)
    assert L.tb_pack_v1_to_v2(src.ctypes.data, scales.ctypes.data, 3, 128, out.ctypes.data) == 0
    for row in range(3):
        for g in range(2):
            blk = out[row, g * 34:(g + 1) * 34]
            assert np.array_equal(blk[:32], src[row, g * 32:(g + 1) * 32])
            got = L.tb_f16_to_f32(int(blk[32]) | (int(blk[33]) << 8))
            assert abs(got - scales[row, g]) / scales[row, g] < 6e-4


def test_v2_shape_errors(L):
    buf = np.zeros(4096, np.uint8)
    sc = np.zeros(64, np.float32)
    assert L.tb_pack_v1_to_v2(buf.ctypes.data, sc.ctypes.data, 2, 96, buf.ctypes.data) == 2  # TB_ERR_SHAPE
    import torchburn_b200 as tb
    assert "TB_UNSUPPORTED" in tb.last_error()
    assert L.tb_pack_v1_to_v2(None, sc.ctypes.data, 2, 128, buf.ctypes.data) == 1


def test_oracle_v2_gemv_matches_v1_within_f16_tolerance(oracle):
    # src/quantization/packed_v2.rs:771-...: v2 against v1 within the binary16 scale error (budget 5e-3)
    rng = np.random.default_rng(7)
    n, k = 8, 128
    w = rng.integers(0, 256, (n, k // 2), dtype=np.uint8)
    s = (0.002 + rng.integers(0, 1000, (n, k // 64)) * 1e-5).astype(np.float32)
    x = ((rng.integers(0, 2000, k) - 1000) / 500).astype(np.float32)
    v1 = oracle.gemm_w4a32_grouped(x, w, s, None, 64)
    v2 = oracle.gemv_w4a32_v2(x, oracle.pack_v1_to_v2(w, s))
    assert np.abs(v2 - v1).max() / np.abs(v1).max() < 5e-3
