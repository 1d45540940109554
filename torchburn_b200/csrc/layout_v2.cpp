// The interleaved "v2" weight layout: every 64-element group of a row is one 34-byte block,
// 32 bytes of packed nibbles followed by the group's scale as IEEE binary16, little-endian.
// Replaces f32_to_f16 / f16_to_f32 / pack_rows_w4a32_group64_v1_to_v2
// (src/quantization/packed_v2.rs:26-143) and the Python quantize / dequantize of that layout
// (python/torchburn/quantization.py:121-170).  The kernels of this library read the v1 form
// (nibbles [N, K/2] + fp32 scales [N, K/64]); a v2 matrix is unpacked once when a linear is
// created, its scales being exactly the binary16 values - the same numbers the reference's v2
// kernels multiply with, so results agree with them up to fp32 summation order.
#include <cstdint>
#include <cstring>
#include <vector>

#include <cuda_runtime.h>

#include "../../include/torchburn_b200.h"

namespace tb {
tb_status fail(tb_status code, const char* fmt, ...);
}
using tb::fail;

extern "C" {

// Round to nearest even; overflow gives infinity; subnormals keep round-to-nearest-even.
uint16_t tb_f32_to_f16(float v) {
  uint32_t x;
  std::memcpy(&x, &v, 4);
  const uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
  const int exp_abs = (int)((x >> 23) & 0xFF);
  const uint32_t mant = x & 0x007FFFFFu;
  if (exp_abs == 0xFF) return (uint16_t)(sign | (mant == 0 ? 0x7C00u : 0x7E00u));
  const int e = exp_abs - 127;
  if (e > 15) return (uint16_t)(sign | 0x7C00u);
  if (e >= -14) {
    uint32_t h = ((uint32_t)(e + 15) << 10) | (mant >> 13);
    const uint32_t rem = mant & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) ++h;  // a carry into the exponent is correct
    return (uint16_t)(sign | h);
  }
  if (e < -25) return sign;  // underflow to signed zero
  const uint32_t full = mant | 0x00800000u;
  const uint32_t shift = (uint32_t)(-e - 1);
  uint32_t m = full >> shift;
  const uint32_t rem = full & ((1u << shift) - 1u), half = 1u << (shift - 1);
  if (rem > half || (rem == half && (m & 1u))) ++m;
  return (uint16_t)(sign | m);
}

float tb_f16_to_f32(uint16_t bits) {
  const uint32_t sign = (bits >> 15) & 1u, exp = (bits >> 10) & 0x1Fu, mant = bits & 0x3FFu;
  uint32_t out;
  if (exp == 0) {
    if (mant == 0) {
      out = sign << 31;
    } else {  // subnormal: mant * 2^-24, exact in fp32
      const float v = (float)mant * 5.9604644775390625e-08f;
      std::memcpy(&out, &v, 4);
      out |= sign << 31;
    }
  } else if (exp == 0x1F) {
    out = (sign << 31) | 0x7F800000u | (mant ? 0x00400000u : 0u);
  } else {
    out = (sign << 31) | ((exp + 112u) << 23) | (mant << 13);
  }
  float f;
  std::memcpy(&f, &out, 4);
  return f;
}

static tb_status check_v2_shape(const char* who, int64_t n, int64_t k) {
  if (n < 0 || k < 0) return fail(TB_ERR_ARG, "%s: negative shape", who);
  if (k % 64 != 0) return fail(TB_ERR_SHAPE, "TB_UNSUPPORTED: the v2 layout needs k divisible by 64, got %lld", (long long)k);
  return TB_OK;
}

tb_status tb_pack_v1_to_v2(const uint8_t* w_packed, const float* scales, int64_t n, int64_t k, uint8_t* blocks) {
  if (tb_status s = check_v2_shape("tb_pack_v1_to_v2", n, k)) return s;
  if (n * k == 0) return TB_OK;
  if (!w_packed || !scales || !blocks) return fail(TB_ERR_ARG, "tb_pack_v1_to_v2: null operand");
  const int64_t ng = k / 64;
  for (int64_t r = 0; r < n; ++r)
    for (int64_t g = 0; g < ng; ++g) {
      uint8_t* dst = blocks + (r * ng + g) * 34;
      std::memcpy(dst, w_packed + r * (k / 2) + g * 32, 32);
      const uint16_t h = tb_f32_to_f16(scales[r * ng + g]);
      dst[32] = (uint8_t)(h & 0xFF);
      dst[33] = (uint8_t)(h >> 8);
    }
  return TB_OK;
}

tb_status tb_unpack_v2_to_v1(const uint8_t* blocks, int64_t n, int64_t k, uint8_t* w_packed, float* scales) {
  if (tb_status s = check_v2_shape("tb_unpack_v2_to_v1", n, k)) return s;
  if (n * k == 0) return TB_OK;
  if (!w_packed || !scales || !blocks) return fail(TB_ERR_ARG, "tb_unpack_v2_to_v1: null operand");
  const int64_t ng = k / 64;
  for (int64_t r = 0; r < n; ++r)
    for (int64_t g = 0; g < ng; ++g) {
      const uint8_t* src = blocks + (r * ng + g) * 34;
      std::memcpy(w_packed + r * (k / 2) + g * 32, src, 32);
      scales[r * ng + g] = tb_f16_to_f32((uint16_t)(src[32] | (src[33] << 8)));
    }
  return TB_OK;
}

tb_status tb_linear_create_v2(tb_linear** out, const uint8_t* blocks, const float* bias, int64_t n, int64_t k,
                              tb_space space) {
  if (!out) return fail(TB_ERR_ARG, "tb_linear_create_v2: null out");
  *out = nullptr;
  if (tb_status s = check_v2_shape("tb_linear_create_v2", n, k)) return s;
  if (!blocks || n < 1 || k < 64) return fail(TB_ERR_ARG, "tb_linear_create_v2: bad arguments");
  const size_t nb = (size_t)n * (size_t)(k / 64) * 34;
  std::vector<uint8_t> host_blocks, w;
  std::vector<float> sc, hb;
  try {
    w.resize((size_t)n * (size_t)(k / 2));
    sc.resize((size_t)n * (size_t)(k / 64));
    if (space == TB_DEVICE) {
      host_blocks.resize(nb);
      if (bias) hb.resize((size_t)n);
    }
  } catch (...) {
    return fail(TB_ERR_OOM, "tb_linear_create_v2: host allocation failed");
  }
  if (space == TB_DEVICE) {
    if (cudaMemcpy(host_blocks.data(), blocks, nb, cudaMemcpyDeviceToHost) != cudaSuccess ||
        (bias && cudaMemcpy(hb.data(), bias, sizeof(float) * (size_t)n, cudaMemcpyDeviceToHost) != cudaSuccess))
      return fail(TB_ERR_CUDA, "tb_linear_create_v2: copy from the device failed: %s", cudaGetErrorString(cudaGetLastError()));
    blocks = host_blocks.data();
    if (bias) bias = hb.data();
  }
  if (tb_status s = tb_unpack_v2_to_v1(blocks, n, k, w.data(), sc.data())) return s;
  return tb_linear_create(out, w.data(), sc.data(), bias, n, k, 64, TB_HOST);
}

}  // extern "C"
