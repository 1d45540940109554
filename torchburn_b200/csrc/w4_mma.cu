// Grouped INT4 W4A32 products for several activation rows (2 <= M <= 64 per pass) on the
// tensor cores, with exact integer arithmetic.
//
// Replaces gemm_w4a32_grouped (src/quantization/gemv.rs:1690-1725: M independent GEMVs) and
// fused_swiglu_mlp_batched (src/quantization/fused_ops.rs:1267-1319) for M > 1.
//
// Step 1 (quantize_x_kernel): every 32-element block of every activation row becomes three
// byte digits of a 24-bit block-fixed-point number (see w4_math.cuh), optionally after the
// fused RMSNorm, stored in the fragment order the MMA wants.
// Step 2 (w4_mma_kernel): per 32-element block of K one mma.sync.m16n8k32 per digit multiplies
// 16 weight rows (nibbles kept as unsigned bytes: two AND/shift per 32-bit word, no
// conversion) with 8 activation rows; the three int32 results are combined and scaled by
// scale[row, group] * sx[m, block] in fp32.  The per-group scale forces that promotion once
// per 32 elements of K, which - not the tensor pipe - bounds the kernel for M >= 32; the
// weights are still read from HBM exactly once per pass of up to 64 activation rows.
#include "tb_common.cuh"
#include "w4_math.cuh"

namespace tb {

namespace {

constexpr int kTileWords = 208;  // per (block, 8 activation rows): 6 x 32 digit words + 8 sx + 8 corr

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ------------------------------------------------------------------------------------------
// x [M, K] fp32 -> xq [K/32][Mt][208] words, Mt = ceil(M/8).  Tile layout: word
// ((d' * 4 + t) * 8 + g) holds digit word d' (0..2 even elements digit 0..2, 3..5 odd elements)
// of 8-element word t of the block, for activation row 8*mt + g; then sx[8], corr[8].
// One CTA per activation row (rows >= M are written as zeros).
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) quantize_x_kernel(const float* __restrict__ x, const float* __restrict__ norm_w,
                                                         float eps, uint32_t* __restrict__ xq, int m_rows, int k,
                                                         int mt_total, float* __restrict__ x_normed_out) {
  __shared__ float s_part[4];
  pdl_wait();
  pdl_launch_dependents();  // after the own wait: completion stays transitive along the chain
  const int m = blockIdx.x;
  const int nb32 = k >> 5;
  const int mt = m >> 3, g = m & 7;
  const bool live = m < m_rows;
  float inv_rms = 1.f;
  if (norm_w != nullptr && live) {
    float ss = 0.f;
    const float4* xr = reinterpret_cast<const float4*>(x + (int64_t)m * k);
    for (int i = threadIdx.x; i < (k >> 2); i += blockDim.x) {
      const float4 v = xr[i];
      ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) tot += s_part[i];
    inv_rms = 1.0f / sqrtf(tot / (float)k + eps);
  }
  // blockIdx.y selects a slice of 128 blocks of K
  for (int blk = blockIdx.y * 128 + threadIdx.x; blk < min(nb32, (int)(blockIdx.y + 1) * 128); blk += blockDim.x) {
    float v[32];
    if (live) {
      const float4* xr = reinterpret_cast<const float4*>(x + (int64_t)m * k) + blk * 8;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float4 t = xr[j];
        if (norm_w != nullptr) {
          const float4 nw = reinterpret_cast<const float4*>(norm_w)[blk * 8 + j];
          t.x = (t.x * inv_rms) * nw.x; t.y = (t.y * inv_rms) * nw.y;
          t.z = (t.z * inv_rms) * nw.z; t.w = (t.w * inv_rms) * nw.w;
          if (x_normed_out != nullptr) reinterpret_cast<float4*>(x_normed_out + (int64_t)m * k)[blk * 8 + j] = t;
        }
        v[4 * j] = t.x; v[4 * j + 1] = t.y; v[4 * j + 2] = t.z; v[4 * j + 3] = t.w;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = 0.f;
    }
    uint32_t dig[24];
    float sx, corr;
    quantize_block(v, dig, sx, corr);
    if (!live) { sx = 0.f; corr = 0.f; }
    uint32_t* tile = xq + ((size_t)blk * mt_total + mt) * kTileWords;
#pragma unroll
    for (int t = 0; t < 4; ++t)
#pragma unroll
      for (int d = 0; d < 6; ++d) tile[(d * 4 + t) * 8 + g] = dig[t * 6 + d];
    tile[192 + g] = __float_as_uint(sx);
    tile[200 + g] = __float_as_uint(corr);
  }
}

__device__ __forceinline__ void mma_u8u8(int (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_u8s8(int (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

struct MmaParams {
  const uint32_t* xq;     // [nb32][mt_total][208]
  const uint8_t* w[2];
  const float* scales[2];
  const float* bias[2];
  const float* resid;
  float* out;
  int m, n, k, nb32, gshift, ng, mt_total;
  int pdl;             // launched with programmatic stream serialization
  int ksplit;          // CTAs that share a row tile and split K (1 = none)
  float* ksplit_part;  // gridDim.y > 1: partial sums [y][x][row tile][activation tile][4][32]
  int* ksplit_cnt;     // gridDim.y > 1: one ticket per blockIdx.x, zero before the first launch, left zero
};

// ------------------------------------------------------------------------------------------
// Every warp keeps 16 weight rows for ALL activation tiles (MT tiles of 8 activation rows,
// accumulators in registers), WR such warps stand side by side and WK warps split the blocks
// of K of each stage, so that a CTA covers 16 * WR rows and the digit tiles of a stage - which
// every warp needs - are fetched once per 16 * WR rows.  With 64 activation rows the digits
// are 13 times the bytes of the weights they meet.  Scales ride in the stage too (no global
// load inside the K loop); three cp.async stages.
// ------------------------------------------------------------------------------------------
template <int MT, int WR, int WK, int EPI, int KC, int NS = 3>
__global__ void __launch_bounds__(32 * WR * WK) w4_mma_rows_kernel(const MmaParams p) {
  constexpr int NW = EPI == 1 ? 2 : 1;
  constexpr int NT = 32 * WR * WK;        // threads
  constexpr int RC = 16 * WR;             // weight rows per CTA
  constexpr int WROW = KC * 4 + 4;        // words per staged weight row (16 bytes of padding)
  constexpr int SROW = KC + 1;            // staged scales per row (padded)
  constexpr int PD = NS - 1;              // chunks requested ahead
  extern __shared__ __align__(16) uint32_t sm[];
  // stage layout: weights [NW][RC][WROW] | scales [NW][RC][SROW] | digits [KC][MT][208]
  constexpr int W_WORDS = NW * RC * WROW;
  constexpr int S_WORDS = (NW * RC * SROW + 3) & ~3;
  constexpr int X_WORDS = KC * MT * kTileWords;
  constexpr int STAGE = W_WORDS + S_WORDS + X_WORDS;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int wr = warp / WK, wk = warp % WK;
  const int row_base = blockIdx.x * RC;
  const int64_t bpr = (int64_t)p.k >> 1;
  const int nchunks_all = (p.nb32 + KC - 1) / KC;
  // gridDim.y CTAs share a row tile and split the chunks of K (narrow matrices at many activation rows)
  const int ch_lo = (int)(((long long)nchunks_all * blockIdx.y) / gridDim.y);
  const int ch_hi = (int)(((long long)nchunks_all * (blockIdx.y + 1)) / gridDim.y);
  const int nchunks = ch_hi - ch_lo;
  const int gsh = p.gshift;

  // weights and scales of a stage (static data: may be requested before the dependency wait)
  auto issue_w = [&](int chunk, int stage) {
    uint32_t* ws = sm + stage * STAGE;
    float* ss = reinterpret_cast<float*>(ws + W_WORDS);
    const int b0 = (ch_lo + chunk) * KC;
    for (int i = tid; i < NW * RC * KC; i += NT) {
      const int q = i / (RC * KC), r = (i / KC) % RC, c = i % KC;
      const int row = min(row_base + r, p.n - 1);
      const int blk = min(b0 + c, p.nb32 - 1);
      cp_async16(ws + (q * RC + r) * WROW + c * 4, p.w[q] + (int64_t)row * bpr + (int64_t)blk * 16);
      // one scale per (row, block); blocks of one group repeat the value
      asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(ss + (q * RC + r) * SROW + c)),
                   "l"(p.scales[q] + (int64_t)row * p.ng + (blk >> gsh))
                   : "memory");
    }
  };
  // digit tiles of a stage (written by the kernel ahead); closes the stage's copy group
  auto issue_x = [&](int chunk, int stage) {
    uint32_t* xs = sm + stage * STAGE + W_WORDS + S_WORDS;
    const int b0 = (ch_lo + chunk) * KC;
    for (int i = tid; i < KC * MT * (kTileWords / 4); i += NT) {
      const int piece = i % (kTileWords / 4), tile = i / (kTileWords / 4);
      const int c = tile / MT, mt = tile % MT;
      const int blk = min(b0 + c, p.nb32 - 1);
      const int mtg = min(mt, p.mt_total - 1);
      cp_async16(xs + (c * MT + mt) * kTileWords + piece * 4, p.xq + ((size_t)blk * p.mt_total + mtg) * kTileWords + piece * 4);
    }
    cp_async_commit();
  };
  auto issue = [&](int chunk, int stage) {
    issue_w(chunk, stage);
    issue_x(chunk, stage);
  };

  float acc[NW][MT][4];
#pragma unroll
  for (int q = 0; q < NW; ++q)
#pragma unroll
    for (int nt = 0; nt < MT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[q][nt][i] = 0.f;

#pragma unroll
  for (int i = 0; i < PD; ++i)
    if (i < nchunks) issue_w(i, i);
  pdl_wait();
  pdl_launch_dependents();
#pragma unroll
  for (int i = 0; i < PD; ++i)
    if (i < nchunks) issue_x(i, i);
  for (int ch = 0; ch < nchunks; ++ch) {
    if (ch + PD < nchunks) issue(ch + PD, (ch + PD) % NS);
    const int pend = min(PD, nchunks - 1 - ch);   // copy groups that may stay in flight while chunk ch is used
    if (pend >= 5) cp_async_wait<5>();
    else if (pend == 4) cp_async_wait<4>();
    else if (pend == 3) cp_async_wait<3>();
    else if (pend == 2) cp_async_wait<2>();
    else if (pend == 1) cp_async_wait<1>();
    else cp_async_wait<0>();
    __syncthreads();
    const uint32_t* ws = sm + (ch % NS) * STAGE;
    const float* ss = reinterpret_cast<const float*>(ws + W_WORDS);
    const uint32_t* xs = ws + W_WORDS + S_WORDS;
#pragma unroll
    for (int cc = 0; cc < KC / WK; ++cc) {
      const int c = cc * WK + wk;          // this warp's blocks of the stage
      const int blk = (ch_lo + ch) * KC + c;
      if (blk < p.nb32) {
#pragma unroll
        for (int q = 0; q < NW; ++q) {
          const uint32_t w0 = ws[(q * RC + wr * 16 + g) * WROW + c * 4 + t];
          const uint32_t w1 = ws[(q * RC + wr * 16 + g + 8) * WROW + c * 4 + t];
          const uint32_t a[4] = {w0 & 0x0F0F0F0Fu, w1 & 0x0F0F0F0Fu, (w0 >> 4) & 0x0F0F0F0Fu, (w1 >> 4) & 0x0F0F0F0Fu};
          const float s0 = ss[(q * RC + wr * 16 + g) * SROW + c];
          const float s1 = ss[(q * RC + wr * 16 + g + 8) * SROW + c];
#pragma unroll
          for (int nt = 0; nt < MT; ++nt) {
            const uint32_t* tile = xs + (c * MT + nt) * kTileWords;
            int c0[4] = {0, 0, 0, 0}, c1[4] = {0, 0, 0, 0}, c2[4] = {0, 0, 0, 0};
            mma_u8u8(c0, a, tile[(0 * 4 + t) * 8 + g], tile[(3 * 4 + t) * 8 + g]);
            mma_u8u8(c1, a, tile[(1 * 4 + t) * 8 + g], tile[(4 * 4 + t) * 8 + g]);
            mma_u8s8(c2, a, tile[(2 * 4 + t) * 8 + g], tile[(5 * 4 + t) * 8 + g]);
            const float2 sx = *reinterpret_cast<const float2*>(tile + 192 + 2 * t);
            const float2 cr = *reinterpret_cast<const float2*>(tile + 200 + 2 * t);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float f = fmaf(65536.0f, (float)c2[i], (float)(c0[i] + (c1[i] << 8)));
              const float d = fmaf((i & 1) ? sx.y : sx.x, f, (i & 1) ? cr.y : cr.x);
              acc[q][nt][i] = fmaf(d, (i & 2) ? s1 : s0, acc[q][nt][i]);
            }
          }
        }
      }
    }
    __syncthreads();
  }

  if (WK > 1) {
    // the WK warps of a row tile cover disjoint blocks of K: sum them in shared memory
    float* red = reinterpret_cast<float*>(sm);
    constexpr int PER = NW * MT * 4;
#pragma unroll
    for (int q = 0; q < NW; ++q)
#pragma unroll
      for (int nt = 0; nt < MT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) red[(warp * PER + (q * MT + nt) * 4 + i) * 32 + lane] = acc[q][nt][i];
    __syncthreads();
    if (wk == 0) {
#pragma unroll
      for (int q = 0; q < NW; ++q)
#pragma unroll
        for (int nt = 0; nt < MT; ++nt)
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < WK; ++w) v += red[((wr * WK + w) * PER + (q * MT + nt) * 4 + i) * 32 + lane];
            acc[q][nt][i] = v;
          }
    }
  }
  if (gridDim.y > 1) {
    // K split over CTAs (single matrix only): every CTA writes its sums, the last one of the row tile
    // to arrive (ticket) adds all of them in the order of blockIdx.y - the same order whichever CTA
    // is last - and goes on to the epilogue.
    __shared__ int s_last;
    const size_t slot = ((size_t)blockIdx.x * WR + wr) * MT * 128;
    const size_t per_y = (size_t)gridDim.x * WR * MT * 128;
    if (wk == 0) {
#pragma unroll
      for (int nt = 0; nt < MT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) p.ksplit_part[blockIdx.y * per_y + slot + (nt * 4 + i) * 32 + lane] = acc[0][nt][i];
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = atomicAdd(&p.ksplit_cnt[blockIdx.x], 1) == (int)gridDim.y - 1;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (tid == 0) p.ksplit_cnt[blockIdx.x] = 0;  // ready for the next launch
    if (wk == 0) {
#pragma unroll
      for (int nt = 0; nt < MT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float v = 0.f;
          for (int y = 0; y < (int)gridDim.y; ++y) v += __ldcg(p.ksplit_part + y * per_y + slot + (nt * 4 + i) * 32 + lane);
          acc[0][nt][i] = v;
        }
    }
  }
  if (wk != 0) return;
  // accumulator i: row (g + 8 * (i >> 1)), activation row (tile * 8 + 2 * t + (i & 1))
#pragma unroll
  for (int nt = 0; nt < MT; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int row = row_base + wr * 16 + g + 8 * (i >> 1);
      const int m = nt * 8 + 2 * t + (i & 1);
      if (row >= p.n || m >= p.m) continue;
      float v;
      if (EPI == 1) {
        const float gg = acc[0][nt][i] + (p.bias[0] ? p.bias[0][row] : 0.f);
        const float uu = acc[NW - 1][nt][i] + (p.bias[1] ? p.bias[1][row] : 0.f);
        v = (gg / (1.0f + expf(-gg))) * uu;  // src/quantization/fused_ops.rs:1305-1311
      } else {
        v = acc[0][nt][i] + (p.bias[0] ? p.bias[0][row] : 0.f);
        if (p.resid) v = p.resid[(int64_t)m * p.n + row] + v;
      }
      p.out[(int64_t)m * p.n + row] = v;
    }
}

template <int MT, int WR, int WK, int EPI, int KC, int NS = 3>
tb_status launch_rows_cfg(const MmaParams& p, cudaStream_t stream) {
  constexpr int NW = EPI == 1 ? 2 : 1;
  constexpr int RC = 16 * WR;
  constexpr size_t stage_words = (size_t)NW * RC * (KC * 4 + 4) + (((size_t)NW * RC * (KC + 1) + 3) & ~(size_t)3) + (size_t)KC * MT * kTileWords;
  constexpr size_t red_words = WK > 1 ? (size_t)WR * WK * NW * MT * 4 * 32 : 0;
  constexpr size_t smem = sizeof(uint32_t) * (NS * stage_words > red_words ? NS * stage_words : red_words);
  static_assert(smem <= 200 * 1024, "stage too large");
  auto kern = w4_mma_rows_kernel<MT, WR, WK, EPI, KC, NS>;
  static thread_local bool configured[64] = {false};
  int dev = 0;
  TB_CUDA_TRY(cudaGetDevice(&dev));
  if (smem > 32 * 1024 && (dev >= 64 || !configured[dev])) {
    TB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    if (dev < 64) configured[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)((p.n + RC - 1) / RC), (unsigned)(EPI == 0 && p.ksplit > 1 ? p.ksplit : 1));
  cfg.blockDim = dim3(32 * WR * WK);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = p.pdl ? 1 : 0;
  TB_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, p));
  return TB_OK;
}

template <int MT, int EPI, int KC>
tb_status launch_rows_mt(const MmaParams& p, cudaStream_t stream) {
  // rows per CTA so that the grid is about one CTA per SM or more; narrow matrices split K over warps
  const int per_sm = p.n / sm_count();
  // Up to 16 activation rows (MT <= 2), graph-timed on the Llama-3-8B shapes at 8 / 16 rows: CTAs of 64 weight
  // rows with 8 warps (4 side by side, K of a stage split in two) against CTAs of 32 rows with 4 warps: gate/up
  // pair 42.7 / 61.9 us against 46.5 / 71.8; the K = 14336 projection 33.2 (K split over 4 CTAs) / 44.0 against
  // 40.1 / 49.4.  Only where 64-row CTAs still cover every SM: the narrow projections and the shards of a
  // tensor-parallel rank stay with 32-row CTAs of 8 warps (N = 4096, K = 4096 at 8 rows: 19.7 against 24.8 us).
  // A fourth stage, stages of 128 elements of K and CTAs of 16 or 128 rows were measured too: none is faster.
  // More than 16 rows (reached only with the tcgen05 kernel switched off): the digit traffic decides.
  if (MT <= 2) {
    const int ctas64 = ((p.n + 63) / 64) * (EPI == 0 && p.ksplit > 1 ? p.ksplit : 1);
    if (ctas64 >= sm_count()) return launch_rows_cfg<MT, 4, 2, EPI, KC>(p, stream);
    return launch_rows_cfg<MT, 2, 4, EPI, KC>(p, stream);
  }
  if (MT != 4 && per_sm >= 64) return launch_rows_cfg<MT, 2, 2, EPI, KC>(p, stream);
  return launch_rows_cfg<MT, 2, 4, EPI, KC>(p, stream);
}

template <int EPI>
tb_status launch_rows_epi(const MmaParams& p, cudaStream_t stream) {
  if (p.mt_total <= 1) return launch_rows_mt<1, EPI, 8>(p, stream);
  if (p.mt_total <= 2) return launch_rows_mt<2, EPI, 8>(p, stream);
  if (p.mt_total <= 4) return launch_rows_mt<4, EPI, 4>(p, stream);
  return launch_rows_mt<8, EPI, 4>(p, stream);
}

}  // namespace

// Scratch layout: [tickets of the K split, 4096 bytes - zero before the first use, left zero] [digit tiles]
// [partial sums of the K split].
constexpr size_t kSplitHeader = 4096;
constexpr int kSplitMaxN = 8192, kSplitMax = 4;
constexpr size_t kSplitPartBytes = (size_t)kSplitMax * (kSplitMaxN / 16) * 8 * 128 * sizeof(float);
static size_t digit_bytes(int m, int64_t k) {
  const int mt = (m + 7) / 8;
  return (((size_t)(k / 32) * mt * kTileWords * sizeof(uint32_t)) + 255) & ~(size_t)255;
}
size_t w4_mma_scratch_bytes(int m, int64_t k) {
  const size_t own = digit_bytes(m, k) + kSplitPartBytes, tc5 = w4_tc5_scratch_bytes(m, k);
  return kSplitHeader + (own > tc5 ? own : tc5);
}

// Up to 64 activation rows per pass; `scratch` holds w4_mma_scratch_bytes(min(m, 64), k) and its first
// 4096 bytes are zero (the decoder clears its block once; a temporary block is cleared per call).
tb_status launch_w4_mma(const GemvArgs& a, void* scratch, cudaStream_t stream) {
  if (a.k % 32 != 0 || (reinterpret_cast<uintptr_t>(a.w) & 15) || (a.w2 && (reinterpret_cast<uintptr_t>(a.w2) & 15)) ||
      ((a.k / 2) % 16) != 0)
    return fail(TB_ERR_ARG, "w4 mma: k must be a multiple of 32 and the weights 16-byte aligned");
  for (int m0 = 0; m0 < a.m; m0 += 64) {
    const int mc = a.m - m0 < 64 ? a.m - m0 : 64;
    const int mt = (mc + 7) / 8;
    const bool pdl = a.pdl;
    {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3((unsigned)(mt * 8), (unsigned)((a.k / 32 + 127) / 128));
      cfg.blockDim = dim3(128);
      cfg.stream = stream;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[0].val.programmaticStreamSerializationAllowed = 1;
      cfg.attrs = attr;
      cfg.numAttrs = pdl ? 1 : 0;
      TB_CUDA_TRY(cudaLaunchKernelEx(&cfg, quantize_x_kernel, a.x + (int64_t)m0 * a.k, a.norm_w, a.eps,
                                     reinterpret_cast<uint32_t*>(static_cast<char*>(scratch) + kSplitHeader), mc, (int)a.k, mt,
                                     a.x_normed_out ? a.x_normed_out + (int64_t)m0 * a.k : (float*)nullptr));
    }
    MmaParams p;
    p.xq = reinterpret_cast<const uint32_t*>(static_cast<char*>(scratch) + kSplitHeader);
    // Narrow single matrices at many activation rows: 32-row CTAs alone leave SMs idle, so 2 or 4 CTAs
    // share a row tile and split K (deterministic sum by the last one to finish).
    int ksplit = 1;
    if (!a.w2 && (mt >= 2 || a.k >= 8192) && a.n <= kSplitMaxN && a.n / 32 < sm_count() && a.k >= 4096) ksplit = a.k >= 8192 ? 4 : 2;
    p.ksplit = ksplit;
    p.ksplit_cnt = reinterpret_cast<int*>(scratch);
    p.ksplit_part = reinterpret_cast<float*>(static_cast<char*>(scratch) + kSplitHeader + digit_bytes(mc, a.k));
    p.w[0] = a.w; p.w[1] = a.w2;
    p.scales[0] = a.scales; p.scales[1] = a.scales2;
    p.bias[0] = a.bias; p.bias[1] = a.bias2;
    p.resid = a.resid ? a.resid + (int64_t)m0 * a.n : nullptr;
    p.out = a.out + (int64_t)m0 * a.n;
    p.m = mc; p.n = (int)a.n; p.k = (int)a.k; p.nb32 = (int)(a.k / 32);
    p.gshift = a.g == 32 ? 0 : (a.g == 64 ? 1 : 2);
    p.ng = (int)(a.k / a.g);
    p.mt_total = mt;
    p.pdl = pdl ? 1 : 0;
    tb_status s = a.w2 ? launch_rows_epi<1>(p, stream) : launch_rows_epi<0>(p, stream);
    if (s != TB_OK) return s;
  }
  return TB_OK;
}

}  // namespace tb
