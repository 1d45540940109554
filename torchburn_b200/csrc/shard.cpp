// Host-side weight sharding for tensor parallelism: pure byte slicing of the
// packed INT4 matrices and their scales.  The reference has no multi-device
// code; the layout is the Megatron one (column-parallel = split output rows,
// row-parallel = split input columns on group boundaries).
#include <cstring>

#include "../../include/torchburn_b200.h"

namespace tb {
tb_status fail(tb_status code, const char* fmt, ...);
}
using tb::fail;

extern "C" {

tb_status tb_shard_rows(const uint8_t* packed, const float* scales, int64_t n, int64_t k,
                        int32_t g, int64_t row0, int64_t rows, uint8_t* packed_out, float* scales_out) {
  if (!packed || !scales || !packed_out || !scales_out) return fail(TB_ERR_ARG, "tb_shard_rows: null argument");
  if (g <= 0 || k <= 0 || k % g != 0 || (k & 1)) return fail(TB_ERR_SHAPE, "tb_shard_rows: k=%lld, group_size=%d", (long long)k, g);
  if (row0 < 0 || rows < 0 || row0 + rows > n) return fail(TB_ERR_SHAPE, "tb_shard_rows: rows [%lld, %lld) outside [0, %lld)", (long long)row0, (long long)(row0 + rows), (long long)n);
  memcpy(packed_out, packed + row0 * (k / 2), (size_t)rows * (k / 2));
  memcpy(scales_out, scales + row0 * (k / g), sizeof(float) * (size_t)rows * (k / g));
  return TB_OK;
}

tb_status tb_shard_cols(const uint8_t* packed, const float* scales, int64_t n, int64_t k,
                        int32_t g, int64_t col0, int64_t cols, uint8_t* packed_out, float* scales_out) {
  if (!packed || !scales || !packed_out || !scales_out) return fail(TB_ERR_ARG, "tb_shard_cols: null argument");
  if (g <= 0 || k <= 0 || k % g != 0 || (g & 1)) return fail(TB_ERR_SHAPE, "tb_shard_cols: k=%lld, group_size=%d", (long long)k, g);
  if (col0 < 0 || cols < 0 || col0 + cols > k || col0 % g != 0 || cols % g != 0)
    return fail(TB_ERR_SHAPE, "tb_shard_cols: columns [%lld, %lld) must lie in [0, %lld) on group boundaries (%d)", (long long)col0, (long long)(col0 + cols), (long long)k, g);
  for (int64_t r = 0; r < n; ++r) {
    memcpy(packed_out + r * (cols / 2), packed + r * (k / 2) + col0 / 2, (size_t)(cols / 2));
    memcpy(scales_out + r * (cols / g), scales + r * (k / g) + col0 / g, sizeof(float) * (size_t)(cols / g));
  }
  return TB_OK;
}

tb_status tb_shard_qkv(const uint8_t* packed, const float* scales, const float* bias, int64_t hidden,
                       int32_t num_heads, int32_t num_kv_heads, int32_t head_dim, int32_t g,
                       int32_t rank, int32_t size, uint8_t* packed_out, float* scales_out, float* bias_out) {
  if (!packed || !scales || !packed_out || !scales_out) return fail(TB_ERR_ARG, "tb_shard_qkv: null argument");
  if (size <= 0 || rank < 0 || rank >= size || num_heads % size || num_kv_heads % size)
    return fail(TB_ERR_ARG, "tb_shard_qkv: rank %d of %d does not divide %d q / %d kv heads", rank, size, num_heads, num_kv_heads);
  if (g <= 0 || hidden % g != 0) return fail(TB_ERR_SHAPE, "tb_shard_qkv: hidden=%lld, group_size=%d", (long long)hidden, g);
  const int64_t bpr = hidden / 2, spr = hidden / g;
  const int64_t q_rows = (int64_t)num_heads * head_dim, kv_rows = (int64_t)num_kv_heads * head_dim;
  const int64_t ql = q_rows / size, kvl = kv_rows / size;
  const int64_t src0[3] = {rank * ql, q_rows + rank * kvl, q_rows + kv_rows + rank * kvl};
  const int64_t cnt[3] = {ql, kvl, kvl};
  int64_t dst = 0;
  for (int part = 0; part < 3; ++part) {
    memcpy(packed_out + dst * bpr, packed + src0[part] * bpr, (size_t)cnt[part] * bpr);
    memcpy(scales_out + dst * spr, scales + src0[part] * spr, sizeof(float) * (size_t)cnt[part] * spr);
    if (bias && bias_out) memcpy(bias_out + dst, bias + src0[part], sizeof(float) * (size_t)cnt[part]);
    dst += cnt[part];
  }
  return TB_OK;
}

}  // extern "C"
