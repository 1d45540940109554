// Small kernels around the projections: RMSNorm, embedding gather, greedy
// argmax, and the INT4 group quantizer.
#include "tb_common.cuh"

namespace tb {

namespace {

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// fast_rms_norm, src/quantization/fused_ops.rs:1066-1117: one CTA per row.
__global__ void __launch_bounds__(256) rms_norm_kernel(const float* __restrict__ x,
                                                       const float* __restrict__ w,
                                                       float* __restrict__ out, int64_t n, float eps) {
  __shared__ float s_part[8];
  const float* xr = x + (int64_t)blockIdx.x * n;
  float* orow = out + (int64_t)blockIdx.x * n;
  float ss = 0.f;
  for (int64_t i = threadIdx.x; i < n; i += blockDim.x) ss = fmaf(xr[i], xr[i], ss);
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += s_part[i];
  const float inv = 1.0f / sqrtf(tot / (float)n + eps);
  for (int64_t i = threadIdx.x; i < n; i += blockDim.x) orow[i] = (xr[i] * inv) * w[i];
}

__global__ void __launch_bounds__(256) embed_gather_kernel(const float* __restrict__ table,
                                                           const int32_t* __restrict__ tokens,
                                                           const int32_t* __restrict__ offsets,
                                                           float* __restrict__ x,
                                                           int32_t* __restrict__ eff_offsets,
                                                           int64_t vocab, int64_t hidden,
                                                           int64_t max_seq_len) {
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.y;
  const int tok = tokens[b], off = offsets[b];
  const bool ok = tok >= 0 && tok < vocab && off >= 0 && off < max_seq_len;
  if (blockIdx.x == 0 && threadIdx.x == 0) eff_offsets[b] = ok ? off : -1;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;  // float4 index
  if (i < hidden / 4) {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (ok) v = reinterpret_cast<const float4*>(table + (int64_t)tok * hidden)[i];
    reinterpret_cast<float4*>(x + (int64_t)b * hidden)[i] = v;
  }
}

// Greedy branch of sample_logits, src/llm/decoder.rs:895-906: the first maximum wins.
// Several CTAs per row: each folds its slice into a 64-bit key (order-preserving image of the
// float in the high word, ~index in the low word, so the maximum key is the largest value at
// the smallest index) with atomicMax; the last CTA of the row publishes the token and resets
// the row's key and ticket for the next launch.
__device__ __forceinline__ unsigned int orderable(float v) {
  const unsigned int u = __float_as_uint(v);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__global__ void __launch_bounds__(256) argmax_kernel(const float* __restrict__ logits, int64_t vocab,
                                                     int32_t* __restrict__ out_tokens,
                                                     int32_t* __restrict__ next_offsets,
                                                     int32_t* __restrict__ hist,
                                                     int32_t* __restrict__ hist_pos,
                                                     unsigned long long* __restrict__ keys,
                                                     int* __restrict__ tickets) {
  __shared__ unsigned long long s_key[8];
  const int b = blockIdx.y;
  const float* row = logits + (int64_t)b * vocab;
  unsigned long long best = 0ull;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < vocab; i += (int64_t)gridDim.x * blockDim.x) {
    const float v = row[i];
    if (v == v) {  // NaN never wins (the reference compares with >)
      const unsigned long long k = ((unsigned long long)orderable(v) << 32) | (unsigned long long)(0xFFFFFFFFu - (unsigned int)i);
      best = k > best ? k : best;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
    best = other > best ? other : best;
  }
  if ((threadIdx.x & 31) == 0) s_key[threadIdx.x >> 5] = best;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w) best = s_key[w] > best ? s_key[w] : best;
    atomicMax(&keys[b], best);
    __threadfence();
    if (atomicAdd(&tickets[b], 1) == (int)gridDim.x - 1) {
      __threadfence();
      const unsigned long long k = atomicExch(&keys[b], 0ull);
      tickets[b] = 0;
      const int tok = k == 0ull ? 0 : (int)(0xFFFFFFFFu - (unsigned int)(k & 0xFFFFFFFFull));
      out_tokens[b] = tok;
      if (next_offsets) next_offsets[b] += 1;
      if (hist && b == 0) hist[(*hist_pos)++] = tok;
    }
  }
}

// quantize_weight_int4_grouped, python/torchburn/quantization.py:85-96.  One warp per
// 32 consecutive elements of a row; a group of G elements spans G/32 adjacent warps' worth
// of data, so the group maximum is taken over G/32 loads by the same warp.
template <int G>
__global__ void __launch_bounds__(256) quantize_int4_kernel(const float* __restrict__ w, int64_t n,
                                                            int64_t k, uint8_t* __restrict__ packed,
                                                            float* __restrict__ scales) {
  constexpr int PER = G / 32;  // elements per lane
  const int lane = threadIdx.x & 31;
  const int64_t ng = k / G;
  const int64_t gid = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);  // group id
  if (gid >= n * ng) return;
  const int64_t row = gid / ng, g = gid - row * ng;
  const float* src = w + row * k + g * G;
  float v[PER];
  float mx = 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    v[i] = src[i * 32 + lane];
    mx = fmaxf(mx, fabsf(v[i]));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  const float s = fmaxf(__fdiv_rn(mx, 7.0f), 1e-8f);  // clamp(max/7, min=1e-8)
  if (lane == 0) scales[gid] = s;
  uint8_t* dst = packed + row * (k >> 1) + g * (G >> 1);
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    float q = rintf(__fdiv_rn(v[i], s));  // torch.round: half to even
    q = fminf(fmaxf(q, -8.0f), 7.0f);
    const unsigned u = (unsigned)((int)q + 8) & 0xFu;
    const unsigned hi = __shfl_down_sync(0xffffffffu, u, 1);
    if ((lane & 1) == 0) dst[(i * 32 + lane) >> 1] = (uint8_t)(u | (hi << 4));
  }
}

}  // namespace

tb_status launch_rms_norm(const float* x, const float* w, float* out, int64_t m, int64_t n,
                          float eps, cudaStream_t stream) {
  if (!x || !w || !out) return fail(TB_ERR_ARG, "rms_norm: null operand");
  if (m < 1 || n < 1) return fail(TB_ERR_SHAPE, "rms_norm: empty shape");
  rms_norm_kernel<<<(unsigned)m, 256, 0, stream>>>(x, w, out, n, eps);
  TB_CUDA_TRY(cudaGetLastError());
  return TB_OK;
}

tb_status launch_embed_gather(const float* table, const int32_t* tokens, const int32_t* offsets,
                              float* x, int32_t* eff_offsets, int batch, int64_t vocab,
                              int64_t hidden, int64_t max_seq_len, bool pdl, cudaStream_t stream) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)((hidden / 4 + 255) / 256), (unsigned)batch);
  cfg.blockDim = dim3(256);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  TB_CUDA_TRY(cudaLaunchKernelEx(&cfg, embed_gather_kernel, table, tokens, offsets, x, eff_offsets,
                                 vocab, hidden, max_seq_len));
  return TB_OK;
}

tb_status launch_argmax(const float* logits, int64_t vocab, int batch, int32_t* out_tokens,
                        int32_t* next_offsets, int32_t* hist, int32_t* hist_pos, void* scratch,
                        cudaStream_t stream) {
  unsigned long long* keys = static_cast<unsigned long long*>(scratch);
  int* tickets = reinterpret_cast<int*>(keys + batch);
  int ctas = (int)((vocab + 4095) / 4096);
  if (ctas > 64) ctas = 64;
  argmax_kernel<<<dim3((unsigned)ctas, (unsigned)batch), 256, 0, stream>>>(logits, vocab, out_tokens, next_offsets, hist, hist_pos, keys, tickets);
  TB_CUDA_TRY(cudaGetLastError());
  return TB_OK;
}

tb_status launch_quantize_int4(const float* w, int64_t n, int64_t k, int g, uint8_t* packed,
                               float* scales, cudaStream_t stream) {
  if (!w || !packed || !scales) return fail(TB_ERR_ARG, "quantize: null operand");
  if (n < 1 || k < 1) return fail(TB_ERR_SHAPE, "quantize: empty shape");
  if (g != 32 && g != 64 && g != 128)
    return fail(TB_ERR_SHAPE, "TB_UNSUPPORTED: group_size %d (supported: 32, 64, 128)", g);
  if (k % g != 0)
    return fail(TB_ERR_SHAPE, "Weight dimension K=%lld must be divisible by group_size=%d", (long long)k, g);
  const int64_t groups = n * (k / g);
  const unsigned blocks = (unsigned)((groups + 7) / 8);
  if (g == 32) quantize_int4_kernel<32><<<blocks, 256, 0, stream>>>(w, n, k, packed, scales);
  else if (g == 64) quantize_int4_kernel<64><<<blocks, 256, 0, stream>>>(w, n, k, packed, scales);
  else quantize_int4_kernel<128><<<blocks, 256, 0, stream>>>(w, n, k, packed, scales);
  TB_CUDA_TRY(cudaGetLastError());
  return TB_OK;
}

}  // namespace tb
