// Grouped INT4 W4A32 matrix-vector products for sm_100a.
//
// y[m, j] = sum_g scales[j, g] * sum_{i in g} x[m, i] * code(w[j, i])      (m <= 8)
//
// Replaces gemv_w4a32_grouped / gemm_w4a32_grouped (src/quantization/gemv.rs:1514-1725),
// the SwiGLU neuron pair (src/quantization/gemv/swiglu.rs:205-289, src/llm/decoder.rs:1280-1328)
// and, through the fused prologue/epilogue, fast_rms_norm (src/quantization/fused_ops.rs:1066-1117)
// and the residual adds of the decoder step (src/llm/decoder.rs:1230-1232, 1345-1347).
//
// Shape of the computation: HBM-bound streaming of packed nibbles, no tensor
// cores.  One lane owns one 32-element block of K per step: it loads the
// block's 16 packed bytes with a single 128-bit load (a warp reads 512
// contiguous bytes of a row), keeps the block's 32 activations in registers
// and reuses them for R rows, multiplies the block sum by the group scale and
// accumulates; rows are finished with warp shuffles.
//
// Nibble -> fp32 without integer-to-float conversion instructions: the nibble
// is masked in place and OR-ed into the mantissa of 2^23, so the register
// holds 2^23 + code4 * 16^p exactly (p = position of the nibble in the word);
// subtracting 2^23 + 8 * 16^p leaves (code4 - 8) * 16^p, and the activation
// was pre-multiplied by 16^-p when it was staged in shared memory.  All of
// these scalings are by powers of two, so every product is the bit-exact
// fp32 product x * (code4 - 8) the reference computes.
#include <mutex>
#include <vector>

#include "tb_common.cuh"
#include "w4_math.cuh"

namespace tb {

namespace {

constexpr int kMaxM = 8;

struct GemvParams {
  const float* x;
  const uint8_t* w[2];
  const float* scales[2];
  const float* bias[2];
  const float* norm_w;
  const float* resid;
  float* out;
  float* x_normed_out;
  float eps;
  int n;        // output rows
  int k;        // input features
  int nb32;     // k / 32
  int gshift;   // log2(group_size / 32)
  int ng;       // groups per row
  int kc;       // activations staged per chunk (multiple of 1024 or == k rounded up)
};

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ __forceinline__ uint4 ldg_stream(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::128B.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ float ldg_stream_f(const float* p) {
  float v;
  asm volatile("ld.global.nc.L1::no_allocate.f32 %0, [%1];" : "=f"(v) : "l"(p));
  return v;
}

// Multipliers 16^-p for the 8 nibbles of a 32-bit word (element e sits at bits
// [4e, 4e+4); elements 5..7 are reached through word >> 12, see dot8()).
__device__ __forceinline__ float prescale_of(int e) {
  // p(e) = {0,1,2,3,4,2,3,4}
  const int p = (e < 5) ? e : e - 3;
  return __int_as_float((127 - 4 * p) << 23);
}

// sum_{e<8} x'[e] * (code4(word, e) - 8) * 16^p(e), with x' pre-scaled by 16^-p(e).
__device__ __forceinline__ float dot8(uint32_t w, const float4 xa, const float4 xb, float acc) {
  constexpr uint32_t kMagic = 0x4B000000u;  // 2^23
  const uint32_t w2 = w >> 12;
  const float f0 = __uint_as_float((w & 0x0000000Fu) | kMagic) - 8388616.0f;    // 2^23 + 8
  const float f1 = __uint_as_float((w & 0x000000F0u) | kMagic) - 8388736.0f;    // 2^23 + 8*16
  const float f2 = __uint_as_float((w & 0x00000F00u) | kMagic) - 8390656.0f;    // 2^23 + 8*256
  const float f3 = __uint_as_float((w & 0x0000F000u) | kMagic) - 8421376.0f;    // 2^23 + 8*4096
  const float f4 = __uint_as_float((w & 0x000F0000u) | kMagic) - 8912896.0f;    // 2^23 + 8*65536
  const float f5 = __uint_as_float((w2 & 0x00000F00u) | kMagic) - 8390656.0f;
  const float f6 = __uint_as_float((w2 & 0x0000F000u) | kMagic) - 8421376.0f;
  const float f7 = __uint_as_float((w2 & 0x000F0000u) | kMagic) - 8912896.0f;
  acc = fmaf(f0, xa.x, acc);
  acc = fmaf(f1, xa.y, acc);
  acc = fmaf(f2, xa.z, acc);
  acc = fmaf(f3, xa.w, acc);
  acc = fmaf(f4, xb.x, acc);
  acc = fmaf(f5, xb.y, acc);
  acc = fmaf(f6, xb.z, acc);
  acc = fmaf(f7, xb.w, acc);
  return acc;
}

__device__ __forceinline__ float dot32(const uint4 wv, const float4 (&xr)[8]) {
  float a = dot8(wv.x, xr[0], xr[1], 0.f);
  float b = dot8(wv.y, xr[2], xr[3], 0.f);
  a = dot8(wv.z, xr[4], xr[5], a);
  b = dot8(wv.w, xr[6], xr[7], b);
  return a + b;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// EPI: 0 = plain (+bias, +resid), 1 = SwiGLU of two matrices sharing x.
// M activation rows, R weight rows per warp, WARPS warps per CTA,
// XMODE: 0 = fp32 products, 1 = integer products (see above).
template <int M, int R, int WARPS, int EPI, bool NORM, int XMODE>
__global__ void __launch_bounds__(WARPS * 32) w4_gemv_kernel(const GemvParams p) {
  constexpr int NW = (EPI == 1) ? 2 : 1;
  constexpr int XV = XMODE == 1 ? 7 : 8;  // 16-byte vectors of staged x per block
  extern __shared__ uint4 xs[];  // XMODE 0: [M][kc/4] float4, XOR-swizzled per block
                                 // XMODE 1: [M][7][kc/32] (vector-major, block-minor)
  __shared__ float s_red[kMaxM][WARPS];

  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int row0 = (blockIdx.x * WARPS + warp) * R;
  const int64_t bpr = (int64_t)p.k >> 1;
  const int iters = (p.nb32 + 31) >> 5;
  const int iters_per_chunk = p.kc >> 10;
  const int cb = p.kc >> 5;  // blocks per chunk

  // Row pointers; rows past the end are clamped for the loads and masked at the store.
  const uint8_t* wrow[NW][R];
  const float* srow[NW][R];
#pragma unroll
  for (int q = 0; q < NW; ++q)
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int row = min(row0 + r, p.n - 1);
      wrow[q][r] = p.w[q] + (int64_t)row * bpr;
      srow[q][r] = p.scales[q] + (int64_t)row * p.ng;
    }

  uint4 wv[NW][R];
  float sc[NW][R];
  auto load_tile = [&](int it, uint4 (&wt)[NW][R], float (&st)[NW][R]) {
    const int b = min(it * 32 + lane, p.nb32 - 1);
#pragma unroll
    for (int q = 0; q < NW; ++q)
#pragma unroll
      for (int r = 0; r < R; ++r) {
        wt[q][r] = ldg_stream(reinterpret_cast<const uint4*>(wrow[q][r]) + b);
        st[q][r] = ldg_stream_f(srow[q][r] + (b >> p.gshift));
      }
  };
  // The weights do not depend on the previous kernel: start streaming them
  // before waiting for it (programmatic dependent launch).
  load_tile(0, wv, sc);
  pdl_wait();
  pdl_launch_dependents();

  // Fused RMSNorm prologue: rms = sqrt(sum(x^2)/k + eps); x_n = (x * (1/rms)) * norm_w.
  float inv_rms[M];
  if (NORM) {
#pragma unroll
    for (int m = 0; m < M; ++m) {
      float ss = 0.f;
      const float4* xg = reinterpret_cast<const float4*>(p.x + (int64_t)m * p.k);
      for (int i = threadIdx.x; i < (p.k >> 2); i += WARPS * 32) {
        const float4 v = xg[i];
        ss = fmaf(v.x, v.x, ss);
        ss = fmaf(v.y, v.y, ss);
        ss = fmaf(v.z, v.z, ss);
        ss = fmaf(v.w, v.w, ss);
      }
      ss = warp_sum(ss);
      if (lane == 0) s_red[m][warp] = ss;
    }
    __syncthreads();
#pragma unroll
    for (int m = 0; m < M; ++m) {
      float tot = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) tot += s_red[m][w];
      const float rms = sqrtf(tot / (float)p.k + p.eps);
      inv_rms[m] = 1.0f / rms;
    }
  }

  float acc[NW][M][R];
#pragma unroll
  for (int q = 0; q < NW; ++q)
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
      for (int r = 0; r < R; ++r) acc[q][m][r] = 0.f;

  const int kc4 = p.kc >> 2;
  for (int it = 0; it < iters; ++it) {
    if (it % iters_per_chunk == 0) {
      // Stage the next chunk of activations.
      if (it != 0) __syncthreads();
      const int k0 = it << 10;
      if (XMODE == 0) {
        // normalise, pre-scale by 16^-p, swizzle
        float4* xs4 = reinterpret_cast<float4*>(xs);
        const int kn4 = min(p.kc, p.k - k0) >> 2;
#pragma unroll
        for (int m = 0; m < M; ++m) {
          const float4* xg = reinterpret_cast<const float4*>(p.x + (int64_t)m * p.k + k0);
          for (int i = threadIdx.x; i < kn4; i += WARPS * 32) {
            float4 v = xg[i];
            if (NORM) {
              const float4 nw = reinterpret_cast<const float4*>(p.norm_w + k0)[i];
              v.x = (v.x * inv_rms[m]) * nw.x;
              v.y = (v.y * inv_rms[m]) * nw.y;
              v.z = (v.z * inv_rms[m]) * nw.z;
              v.w = (v.w * inv_rms[m]) * nw.w;
              if (p.x_normed_out != nullptr && blockIdx.x == 0)
                reinterpret_cast<float4*>(p.x_normed_out + (int64_t)m * p.k + k0)[i] = v;
            }
            const int e0 = (i & 1) * 4;  // position of v.x inside its 8-element word
            v.x *= prescale_of(e0 + 0);
            v.y *= prescale_of(e0 + 1);
            v.z *= prescale_of(e0 + 2);
            v.w *= prescale_of(e0 + 3);
            const int blk = i >> 3, j = i & 7;
            xs4[m * kc4 + blk * 8 + (j ^ (blk & 7))] = v;
          }
        }
      } else {
        // normalise, then one thread per block: 24-bit fixed point digits
        const int nblk = min(p.kc, p.k - k0) >> 5;
#pragma unroll 1
        for (int m = 0; m < M; ++m) {
          for (int blk = threadIdx.x; blk < nblk; blk += WARPS * 32) {
            const float4* xg = reinterpret_cast<const float4*>(p.x + (int64_t)m * p.k + k0) + blk * 8;
            float v[32];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              float4 t = xg[j];
              if (NORM) {
                const float4 nw = reinterpret_cast<const float4*>(p.norm_w + k0)[blk * 8 + j];
                t.x = (t.x * inv_rms[m]) * nw.x;
                t.y = (t.y * inv_rms[m]) * nw.y;
                t.z = (t.z * inv_rms[m]) * nw.z;
                t.w = (t.w * inv_rms[m]) * nw.w;
                if (p.x_normed_out != nullptr && blockIdx.x == 0)
                  reinterpret_cast<float4*>(p.x_normed_out + (int64_t)m * p.k + k0)[blk * 8 + j] = t;
              }
              v[4 * j + 0] = t.x; v[4 * j + 1] = t.y; v[4 * j + 2] = t.z; v[4 * j + 3] = t.w;
            }
            uint32_t dig[24];
            float sx;
            int S, s8hi, s8lo;
            quantize_part_int<32>(v, abs_max<32>(v), dig, sx, S);
            split_offset(S, s8hi, s8lo);
            uint4* dst = xs + (size_t)m * 7 * cb + blk;
#pragma unroll
            for (int j = 0; j < 6; ++j)
              dst[j * cb] = make_uint4(dig[4 * j], dig[4 * j + 1], dig[4 * j + 2], dig[4 * j + 3]);
            dst[6 * cb] = make_uint4(__float_as_uint(sx), (uint32_t)s8hi, (uint32_t)s8lo, 0u);
          }
        }
      }
      __syncthreads();
    }
    uint4 wn[NW][R];
    float sn[NW][R];
    if (it + 1 < iters) load_tile(it + 1, wn, sn);

    const int bl = (it % iters_per_chunk) * 32 + lane;  // block index inside the chunk
    if (it * 32 + lane < p.nb32) {
      if (XMODE == 0) {
        const float4* xs4 = reinterpret_cast<const float4*>(xs);
#pragma unroll
        for (int m = 0; m < M; ++m) {
          float4 xr[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) xr[j] = xs4[m * kc4 + bl * 8 + (j ^ (bl & 7))];
#pragma unroll
          for (int q = 0; q < NW; ++q)
#pragma unroll
            for (int r = 0; r < R; ++r)
              acc[q][m][r] = fmaf(dot32(wv[q][r], xr), sc[q][r], acc[q][m][r]);
        }
      } else {
#pragma unroll
        for (int m = 0; m < M; ++m) {
          uint32_t xq[24];
          const uint4* src = xs + (size_t)m * 7 * cb + bl;
#pragma unroll
          for (int j = 0; j < 6; ++j) {
            const uint4 t = src[j * cb];
            xq[4 * j] = t.x; xq[4 * j + 1] = t.y; xq[4 * j + 2] = t.z; xq[4 * j + 3] = t.w;
          }
          const uint4 tail = src[6 * cb];
          const float sx = __uint_as_float(tail.x);
          const int s8hi = (int)tail.y, s8lo = (int)tail.z;
#pragma unroll
          for (int q = 0; q < NW; ++q)
#pragma unroll
            for (int r = 0; r < R; ++r) {
              const uint32_t w4[4] = {wv[q][r].x, wv[q][r].y, wv[q][r].z, wv[q][r].w};
              const float d = sx * idot_words_off<4>(w4, xq, s8hi, s8lo);
              acc[q][m][r] = fmaf(d, sc[q][r], acc[q][m][r]);
            }
        }
      }
    }
    if (it + 1 < iters) {
#pragma unroll
      for (int q = 0; q < NW; ++q)
#pragma unroll
        for (int r = 0; r < R; ++r) {
          wv[q][r] = wn[q][r];
          sc[q][r] = sn[q][r];
        }
    }
  }

#pragma unroll
  for (int q = 0; q < NW; ++q)
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
      for (int r = 0; r < R; ++r) acc[q][m][r] = warp_sum(acc[q][m][r]);

  if (lane == 0) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int row = row0 + r;
      if (row >= p.n) continue;
#pragma unroll
      for (int m = 0; m < M; ++m) {
        float v;
        if (EPI == 1) {
          const float g = acc[0][m][r] + (p.bias[0] ? p.bias[0][row] : 0.f);
          const float u = acc[1][m][r] + (p.bias[1] ? p.bias[1][row] : 0.f);
          v = (g / (1.0f + expf(-g))) * u;  // src/llm/decoder.rs:1319-1322
        } else {
          v = acc[0][m][r] + (p.bias[0] ? p.bias[0][row] : 0.f);
          if (p.resid) v = p.resid[(int64_t)m * p.n + row] + v;
        }
        p.out[(int64_t)m * p.n + row] = v;
      }
    }
  }
}

// Tuning state (process-wide): product mode and an optional forced launch shape.
int g_xmode = 1;
int g_mma_enabled = 1;
int g_force_r = 0, g_force_warps = 0;

template <int M, int R, int WARPS, int EPI, bool NORM, int XMODE>
tb_status launch_cfg(const GemvParams& p, bool pdl, cudaStream_t stream) {
  auto kern = w4_gemv_kernel<M, R, WARPS, EPI, NORM, XMODE>;
  const size_t smem = XMODE == 1 ? (size_t)M * 7 * (p.kc >> 5) * sizeof(uint4) : (size_t)M * p.kc * sizeof(float);
  static thread_local size_t configured[64] = {0};
  int dev = 0;
  TB_CUDA_TRY(cudaGetDevice(&dev));
  // static + dynamic shared memory above 48 KB needs the opt-in, so opt in from 32 KB up
  if (smem > 32 * 1024 && (dev >= 64 || configured[dev] < smem)) {
    TB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    if (dev < 64) configured[dev] = smem;
  }
  const int rows_per_cta = R * WARPS;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)((p.n + rows_per_cta - 1) / rows_per_cta));
  cfg.blockDim = dim3(WARPS * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  TB_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, p));
  return TB_OK;
}

template <int M, int EPI, bool NORM, int XMODE>
tb_status launch_m(const GemvParams& p, bool pdl, cudaStream_t stream) {
  // Rows per warp: more rows amortise the activation reads from shared memory and keep
  // more loads in flight; fewer rows give more warps when the matrix is small.
  const int sms = sm_count();
  if constexpr (M == 1) {
    int r = 0, w = 8;
    if (g_force_r > 0) {
      r = g_force_r;
      w = g_force_warps > 0 ? g_force_warps : 8;
    } else if (EPI == 1) {
      r = ((int64_t)p.n >= (int64_t)sms * 64) ? 2 : 1;
    } else {
      r = ((int64_t)p.n >= (int64_t)sms * 128) ? 4 : ((int64_t)p.n >= (int64_t)sms * 32 ? 2 : 1);
      if (r == 1) w = 4;
    }
    if (EPI == 1 && r == 4) r = 2;
    if (w == 4) {
      if (r == 1) return launch_cfg<M, 1, 4, EPI, NORM, XMODE>(p, pdl, stream);
      if (r == 2) return launch_cfg<M, 2, 4, EPI, NORM, XMODE>(p, pdl, stream);
      if constexpr (EPI == 0) return launch_cfg<M, 4, 4, EPI, NORM, XMODE>(p, pdl, stream);
    }
    if (r == 1) return launch_cfg<M, 1, 8, EPI, NORM, XMODE>(p, pdl, stream);
    if (r == 2) return launch_cfg<M, 2, 8, EPI, NORM, XMODE>(p, pdl, stream);
    if constexpr (EPI == 0) return launch_cfg<M, 4, 8, EPI, NORM, XMODE>(p, pdl, stream);
    return launch_cfg<M, 2, 8, EPI, NORM, XMODE>(p, pdl, stream);
  } else if constexpr (EPI == 1) {
    return launch_cfg<M, 1, 8, EPI, NORM, XMODE>(p, pdl, stream);
  } else {
    return launch_cfg<M, 2, 8, EPI, NORM, XMODE>(p, pdl, stream);
  }
}

template <int EPI, bool NORM, int XMODE>
tb_status launch_x(int m, const GemvParams& p, bool pdl, cudaStream_t stream) {
  switch (m) {
    case 1: return launch_m<1, EPI, NORM, XMODE>(p, pdl, stream);
    case 2: return launch_m<2, EPI, NORM, XMODE>(p, pdl, stream);
    case 3: return launch_m<3, EPI, NORM, XMODE>(p, pdl, stream);
    case 4: return launch_m<4, EPI, NORM, XMODE>(p, pdl, stream);
    case 5: return launch_m<5, EPI, NORM, XMODE>(p, pdl, stream);
    case 6: return launch_m<6, EPI, NORM, XMODE>(p, pdl, stream);
    case 7: return launch_m<7, EPI, NORM, XMODE>(p, pdl, stream);
    case 8: return launch_m<8, EPI, NORM, XMODE>(p, pdl, stream);
  }
  return fail(TB_ERR_SHAPE, "w4 gemv: m=%d outside 1..8", m);
}

template <int EPI, bool NORM>
tb_status launch_epi(int m, const GemvParams& p, bool pdl, cudaStream_t stream) {
  // The fp32 product path is kept for M = 1 (A/B measurements, exact-fp32 option).
  if (g_xmode == 0 && m == 1) return launch_m<1, EPI, NORM, 0>(p, pdl, stream);
  return launch_x<EPI, NORM, 1>(m, p, pdl, stream);
}

}  // namespace

void set_gemv_tuning(int xmode, int rows_per_warp, int warps) {
  g_mma_enabled = xmode == 2 ? 0 : 1;  // 2: integer products on CUDA cores for every M
  set_tc5_enabled(xmode == 3 ? 0 : 1);  // 3: the mma.sync integer kernel also for M > 16
  g_xmode = xmode != 0 ? 1 : 0;
  g_force_r = rows_per_warp;
  g_force_warps = warps;
}

// Workspace of the products with several activation rows (digit form of x, partial sums and tickets of the K
// split) for callers that bring none: one block per (device, stream), kept between calls and grown when a call
// needs more.  Calls on one stream are ordered, so they can share it; calls on different streams get different
// blocks.  Without it every call would allocate, clear and free stream-ordered memory - three extra nodes when
// the calls are captured into a CUDA graph.  Nothing is allocated while the stream is being captured: a call
// that then finds no block large enough takes stream-ordered memory for its own duration, as before.
namespace {
struct Workspace { int dev; cudaStream_t stream; void* ptr; size_t bytes; };
std::mutex g_ws_mu;
std::vector<Workspace> g_ws;

void* workspace_for(cudaStream_t stream, size_t bytes) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess) { cudaGetLastError(); return nullptr; }
  std::lock_guard<std::mutex> lock(g_ws_mu);
  Workspace* e = nullptr;
  for (Workspace& w : g_ws)
    if (w.dev == dev && w.stream == stream) { e = &w; break; }
  if (e && e->bytes >= bytes) return e->ptr;
  if (cap != cudaStreamCaptureStatusNone) return nullptr;
  if (e) {  // grow: earlier calls on the stream may still use the old block
    if (cudaStreamSynchronize(stream) != cudaSuccess) return nullptr;
    cudaFree(e->ptr);
    e->ptr = nullptr;
    e->bytes = 0;
  } else {
    g_ws.push_back(Workspace{dev, stream, nullptr, 0});
    e = &g_ws.back();
  }
  void* p = nullptr;
  if (cudaMalloc(&p, bytes) != cudaSuccess) { cudaGetLastError(); return nullptr; }
  if (cudaMemsetAsync(p, 0, 4096, stream) != cudaSuccess) { cudaGetLastError(); cudaFree(p); return nullptr; }  // the tickets start at zero; every launch leaves them zero
  e->ptr = p;
  e->bytes = bytes;
  return p;
}
}  // namespace

void release_workspaces() {
  std::lock_guard<std::mutex> lock(g_ws_mu);
  int cur = 0;
  cudaGetDevice(&cur);
  for (Workspace& w : g_ws) {
    if (!w.ptr) continue;
    cudaSetDevice(w.dev);
    cudaDeviceSynchronize();
    cudaFree(w.ptr);
  }
  g_ws.clear();
  cudaSetDevice(cur);
}

// Kernels one launch_w4_gemv call starts for these operands (the same choices as below).
static bool few_rows_narrow(const GemvArgs& a) {
  // Three or four rows of a narrow matrix: the CUDA-core kernel beats the tensor-core rows kernel, whose cost
  // hardly depends on the row count below 8 (graph-timed, K = 4096: N = 4096 at 3 / 4 / 5 rows 11.7 / 13.9 /
  // 16.0 us against 19.3; N = 6144 at 3 / 4 rows 18.2 / 21.4 against 23.0; the wide gate/up pair never).
  // Every CTA of that kernel prepares all rows of x itself (with a fused RMSNorm: twice over them), so it is
  // kept to four rows, three with the norm.
  return a.m >= 3 && a.m <= (a.norm_w ? 3 : 4) && a.w2 == nullptr && a.k <= 4096 && (int64_t)a.m * a.n <= 24576;
}
int w4_gemv_launches(const GemvArgs& a) {
  if (w4_stream_supported(a)) return 1;
  if (a.m >= 2 && g_mma_enabled && !few_rows_narrow(a) && ((a.k / 2) % 16) == 0)
    return 2 * ((a.m + 63) / 64);   // per pass of up to 64 rows: the activation pre-pass + the product
  return (a.m + kMaxM - 1) / kMaxM;
}

// Rows of x beyond 8 are processed in slices of up to 8 (the weights are
// streamed once per slice).
tb_status launch_w4_gemv(const GemvArgs& a, cudaStream_t stream) {
  if (!a.x || !a.w || !a.scales || !a.out) return fail(TB_ERR_ARG, "w4 gemv: null operand");
  if (a.m < 1 || a.n < 1 || a.k < 1) return fail(TB_ERR_SHAPE, "w4 gemv: empty shape m=%d n=%lld k=%lld", a.m, (long long)a.n, (long long)a.k);
  if (a.g != 32 && a.g != 64 && a.g != 128)
    return fail(TB_ERR_SHAPE, "TB_UNSUPPORTED: group_size %d (supported: 32, 64, 128)", a.g);
  if (a.k % a.g != 0) return fail(TB_ERR_SHAPE, "TB_UNSUPPORTED: k=%lld not a multiple of group_size %d", (long long)a.k, a.g);
  if (a.n > (1ll << 30) || a.k > (1ll << 24)) return fail(TB_ERR_SHAPE, "w4 gemv: shape too large");
  if ((reinterpret_cast<uintptr_t>(a.w) & 15) || (reinterpret_cast<uintptr_t>(a.x) & 15) ||
      (a.w2 && (reinterpret_cast<uintptr_t>(a.w2) & 15)) ||
      (a.norm_w && (reinterpret_cast<uintptr_t>(a.norm_w) & 15)))
    return fail(TB_ERR_ARG, "w4 gemv: x, w and norm_w must be 16-byte aligned");
  const bool swiglu = a.w2 != nullptr;
  if (swiglu && !a.scales2) return fail(TB_ERR_ARG, "w4 gemv: swiglu needs scales2");

  GemvParams p;
  p.w[0] = a.w; p.w[1] = a.w2;
  p.scales[0] = a.scales; p.scales[1] = a.scales2;
  p.bias[0] = a.bias; p.bias[1] = a.bias2;
  p.norm_w = a.norm_w;
  p.eps = a.eps;
  p.n = (int)a.n;
  p.k = (int)a.k;
  p.nb32 = (int)(a.k / 32);
  p.gshift = a.g == 32 ? 0 : (a.g == 64 ? 1 : 2);
  p.ng = (int)(a.k / a.g);
  const int k_pad = (int)((a.k + 1023) / 1024 * 1024);

  if (w4_stream_supported(a)) return launch_w4_stream(a, stream);
  if (a.x_ss8 || a.out_scaled || a.out_ss8)
    return fail(TB_ERR_UNSUPPORTED, "TB_UNSUPPORTED: the split RMSNorm needs the persistent M = 1 kernel for this shape");
  if (a.m >= 2 && g_mma_enabled && !few_rows_narrow(a) && ((a.k / 2) % 16) == 0) {
    const bool tc5 = w4_tc5_supported(a);   // more than 16 rows: tcgen05, operand images behind the ticket header
    if (a.xq_scratch) return tc5 ? launch_w4_tc5(a, static_cast<char*>(a.xq_scratch) + 4096, stream) : launch_w4_mma(a, a.xq_scratch, stream);
    const size_t need = w4_mma_scratch_bytes(a.m < 64 ? a.m : 64, a.k);
    if (void* ws = workspace_for(stream, need)) return tc5 ? launch_w4_tc5(a, static_cast<char*>(ws) + 4096, stream) : launch_w4_mma(a, ws, stream);
    void* tmp = nullptr;
    TB_CUDA_TRY(cudaMallocAsync(&tmp, need, stream));
    TB_CUDA_TRY(cudaMemsetAsync(tmp, 0, 4096, stream));  // the tickets of the K split
    const tb_status s = tc5 ? launch_w4_tc5(a, static_cast<char*>(tmp) + 4096, stream) : launch_w4_mma(a, tmp, stream);
    cudaFreeAsync(tmp, stream);
    return s;
  }

  for (int m0 = 0; m0 < a.m; m0 += kMaxM) {
    const int mc = a.m - m0 < kMaxM ? a.m - m0 : kMaxM;
    p.x = a.x + (int64_t)m0 * a.k;
    p.out = a.out + (int64_t)m0 * a.n;
    p.resid = a.resid ? a.resid + (int64_t)m0 * a.n : nullptr;
    p.x_normed_out = a.x_normed_out ? a.x_normed_out + (int64_t)m0 * a.k : nullptr;
    // Whole K staged at once while it fits comfortably; otherwise 4096 per chunk.
    p.kc = ((size_t)mc * k_pad * sizeof(float) <= 96 * 1024) ? k_pad : (mc <= 4 ? 4096 : 2048);
    tb_status s;
    const bool pdl = a.pdl && m0 == 0;
    if (swiglu)
      s = a.norm_w ? launch_epi<1, true>(mc, p, pdl, stream) : launch_epi<1, false>(mc, p, pdl, stream);
    else
      s = a.norm_w ? launch_epi<0, true>(mc, p, pdl, stream) : launch_epi<0, false>(mc, p, pdl, stream);
    if (s != TB_OK) return s;
  }
  return TB_OK;
}

}  // namespace tb
