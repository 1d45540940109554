// Persistent, K-stationary grouped-INT4 GEMV for one activation row (M = 1).
//
// Same arithmetic as w4_gemv.cu (gemv_w4a32_grouped, src/quantization/gemv.rs:1514-1684;
// SwiGLU pair src/quantization/gemv/swiglu.rs:205-289; fused fast_rms_norm
// src/quantization/fused_ops.rs:1066-1117), laid out for B200:
//
//  * One CTA per SM (or two), alive for the whole matrix.  Lane (warp w, lane l) owns the
//    32-element block w*32+l of K for the entire kernel: its activations are turned into
//    integer digits once and stay in registers, so the inner loop reads no activations.
//  * A producer warp streams the CTA's rows through a ring of shared-memory stages with
//    bulk asynchronous copies (cp.async.bulk, completion on mbarriers).  Rows are contiguous
//    in memory, so a stage is one linear copy of RS rows of packed nibbles plus one of their
//    scales.  The ring starts filling before the previous kernel has finished
//    (programmatic dependent launch); only the activations wait for it.
//  * Consumers take one 128-bit shared-memory load per row and lane, multiply with dp4a,
//    and finish 32 rows at a time with a transposing butterfly (31 shuffles for 32 rows)
//    and one cross-warp sum; the 32 results of a tile are written with one coalesced store.
//
// HBM-bound: algorithmic bytes per launch = n*k/2 + n*(k/g)*4 (+ the vectors).
#include "tb_common.cuh"
#include "w4_math.cuh"

namespace tb {

namespace {

constexpr int kRingBytesMax = 96 * 1024;  // leaves room for the next kernel's CTA on the same SM
constexpr int kMaxStages = 8;
constexpr long long kWaitCycles = 4000000000ll;  // ~2 s: a wait that long means a lost copy

__device__ int g_stream_fault = 0;

struct StreamParams {
  const float* x;
  const uint8_t* w[2];
  const float* scales[2];
  const float* bias[2];
  const float* norm_w;
  const float* resid;
  float* out;
  float* x_normed_out;
  const float* x_ss8;        // not null: x is already multiplied by the norm weights, x_ss8[i] = sum of squares of
                             // the un-weighted elements 8i..8i+7; the row sums are divided by the rms at the end
  float* out_scaled;         // optional second output out * out_scale_w (the next kernel's pre-weighted x)
  const float* out_scale_w;
  float* out_ss8;            // optional: sums of squares of out over groups of 8 rows
  float eps;
  int n, k, nb32, gshift, ng;
  int nwarps;        // consumer warps per group = ceil(k / EPL / 32)
  int groups;        // always 1 (see the kernel comment)
  int stages;        // ring depth
  int stage_bytes;   // bytes of one stage
  int rounds;        // ceil(n / 8): the unit of work distribution (8 rows)
  unsigned long long* tl;  // timestamps of this launch or null
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst_smem)),
      "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
// Bounded wait; returns false (and raises the abort flag) when the limit ran out or another
// thread already gave up.  Nobody spins forever: after an abort every wait returns at once.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  const uint32_t addr = smem_u32(bar);
  const long long t0 = clock64();
  for (uint32_t i = 0;; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(addr), "r"(parity)
        : "memory");
    if (ok) return true;
    if ((i & 255) == 255) {
      if (*abort_flag) return false;
      if (clock64() - t0 > kWaitCycles) {
        *abort_flag = 1;
        return false;
      }
    }
  }
}

__device__ __forceinline__ void consumer_barrier(int threads) {
  asm volatile("bar.sync 1, %0;" ::"r"(threads) : "memory");
}

// Sum over the 32 lanes of p[j], delivered to lane j (31 shuffles).
__device__ __forceinline__ float transpose_reduce(float (&p)[32], int lane) {
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) {
    const bool hi = (lane & off) != 0;
#pragma unroll
    for (int j = 0; j < off; ++j) {
      const float send = hi ? p[j] : p[j + off];
      const float keep = hi ? p[j + off] : p[j];
      p[j] = keep + __shfl_xor_sync(0xffffffffu, send, off);
    }
  }
  return p[0];
}

// Same idea for 8 values: three transposing steps leave one row per lane (row = lane >> 2),
// two plain steps finish the sum over the four lanes that share it (9 shuffles for 8 rows).
__device__ __forceinline__ float transpose_reduce8(float (&p)[8], int lane) {
#pragma unroll
  for (int step = 0; step < 3; ++step) {
    const int off = 16 >> step, half = 4 >> step;
    const bool hi = (lane & off) != 0;
#pragma unroll
    for (int j = 0; j < half; ++j) {
      const float send = hi ? p[j] : p[j + half];
      const float keep = hi ? p[j + half] : p[j];
      p[j] = keep + __shfl_xor_sync(0xffffffffu, send, off);
    }
  }
  float v = p[0];
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  return v;
}

// RS rows per stage (8 % RS == 0); EPI 0 plain / 1 SwiGLU; NORM fused RMSNorm of x;
// EPL elements of K owned by one lane (32 = a whole block, 16 = half a block).
//
// The consumer warps of a CTA together cover all of K (lane l of warp w owns elements
// [(w*32+l)*EPL, +EPL)) and observe every stage of the ring in order, which keeps the mbarrier
// phase parities unambiguous (p.groups is always 1).  Work is handed out in rounds of 8 rows:
// every CTA gets a contiguous, balanced share, so no CTA waits for a straggler tile.
template <int RS, int EPI, bool NORM, int EPL>
__global__ void __launch_bounds__(512) w4_stream_kernel(const StreamParams p) {
  constexpr int NW = EPI == 1 ? 2 : 1;
  constexpr int TR = 8;            // rows per round
  constexpr int SPR = TR / RS;     // stages per round
  constexpr int NWD = EPL / 8;     // 32-bit weight words per lane and row
  extern __shared__ __align__(128) unsigned char ring[];
  __shared__ uint64_t full[kMaxStages], empty[kMaxStages];
  __shared__ float s_part[2][NW][16][33];  // [buffer][matrix][consumer warp][row] (padded)
  __shared__ float s_ss[16];
  __shared__ int s_abort;
  __shared__ int s_waited;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nwarps = p.nwarps, groups = p.groups;
  const bool is_producer = warp == nwarps * groups;
  const int row_bytes = p.k >> 1, srow_bytes = p.ng * 4;
  // Contiguous, balanced share of the 8-row rounds: the first `rem` CTAs take one more.
  const int base_rounds = p.rounds / (int)gridDim.x, rem_rounds = p.rounds % (int)gridDim.x;
  const int my_rounds = base_rounds + ((int)blockIdx.x < rem_rounds ? 1 : 0);
  const int round0 = (int)blockIdx.x * base_rounds + min((int)blockIdx.x, rem_rounds);
  const int total_stages = my_rounds * SPR;

  if (tid == 0) {
    s_abort = 0;
    s_waited = 0;
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], nwarps);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    tl_mark(p.tl, (int)blockIdx.x, 0);
    if (blockIdx.x == 0) tl_header(p.tl, 1, (int)gridDim.x);
  }
  __syncthreads();

  if (is_producer) {
    // ---------------- producer: one lane feeds the ring ----------------
    // The producer must not signal launch_dependents: the next kernel may only start once
    // this grid's consumers are past their griddepcontrol.wait, i.e. once everything before
    // this kernel has completed (kernels further down the chain rely on that).
    if (lane == 0) {
      for (int i = 0; i < total_stages; ++i) {
        const int s = i % p.stages, round = i / p.stages;
        if (round > 0 && !mbar_wait(&empty[s], (uint32_t)(round - 1) & 1u, &s_abort)) break;
        if (i == 0) tl_mark(p.tl, (int)blockIdx.x, 6);
        if (i == total_stages - 1) tl_mark(p.tl, (int)blockIdx.x, 7);
        const int row0 = (round0 + i / SPR) * TR + (i % SPR) * RS;
        const int cnt = max(0, min(RS, p.n - row0));
        unsigned char* dst = ring + (size_t)s * p.stage_bytes;
        if (cnt == 0) {  // nothing to fetch for this stage: complete the phase by hand
          mbar_arrive(&full[s]);
          continue;
        }
        const uint32_t wb = (uint32_t)cnt * row_bytes, sb = (uint32_t)cnt * srow_bytes;
        mbar_expect_tx(&full[s], NW * (wb + sb));
#pragma unroll
        for (int q = 0; q < NW; ++q) {
          unsigned char* d = dst + (size_t)q * RS * (row_bytes + srow_bytes);
          bulk_g2s(d, p.w[q] + (int64_t)row0 * row_bytes, wb, &full[s]);
          bulk_g2s(d + (size_t)RS * row_bytes, p.scales[q] + (int64_t)row0 * p.ng, sb, &full[s]);
        }
      }
      {
        // All of this CTA's HBM requests are out: the next kernel may start filling its ring
        // (launch_dependents is signalled here, after the last stage was requested).
        // Only after the consumers are past their griddepcontrol.wait (completion must stay
        // transitive along the chain of kernels); bounded like every other wait.
        const long long t0 = clock64();
        while (*reinterpret_cast<volatile int*>(&s_waited) == 0 && clock64() - t0 < kWaitCycles) {}
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
      }
    }
    return;
  }

  // ---------------- consumers ----------------
  // Everything below reads the previous kernel's output.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (tid == 0) *reinterpret_cast<volatile int*>(&s_waited) = 1;
  if (tid == 0) tl_mark(p.tl, (int)blockIdx.x, 1);

  const int grp = warp / nwarps, gw = warp - grp * nwarps;
  const int part = gw * 32 + lane;                 // index of this lane's EPL-element slice of K
  const bool has_part = part * EPL < p.k;
  const int blk = (part * EPL) >> 5;
  const int group_threads = nwarps * 32;
  uint32_t dig[NWD * 6];
  float sx = 0.f;
  int s8hi = 0, s8lo = 0;   // 8 * sum of this lane's digits-as-integers: the offset of the codes
  float inv_rms = 1.f;
  {
    float v[EPL];
    // The norm weights travel together with x: one trip to L2 instead of two in a row.
    float4 nwv[NORM ? EPL / 4 : 1];
    if (NORM && has_part) {
      const float4* nw = reinterpret_cast<const float4*>(p.norm_w) + part * (EPL / 4);
#pragma unroll
      for (int j = 0; j < EPL / 4; ++j) nwv[j] = __ldg(nw + j);
    }
    if (has_part) {
      const float4* xg = reinterpret_cast<const float4*>(p.x) + part * (EPL / 4);
#pragma unroll
      for (int j = 0; j < EPL / 4; ++j) {
        const float4 t = xg[j];
        v[4 * j] = t.x; v[4 * j + 1] = t.y; v[4 * j + 2] = t.z; v[4 * j + 3] = t.w;
      }
    } else {
#pragma unroll
      for (int j = 0; j < EPL; ++j) v[j] = 0.f;
    }
    if (NORM) {
      // rms = sqrt(sum(x^2)/k + eps).  The product with 1/rms is applied to the finished row
      // sums (the projection is linear); the norm weights are folded into x here.
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < EPL; ++j) ss = fmaf(v[j], v[j], ss);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if (lane == 0) s_ss[warp] = ss;
      asm volatile("bar.sync %0, %1;" ::"r"(1 + grp), "r"(group_threads) : "memory");
      float tot = 0.f;
      for (int w = 0; w < nwarps; ++w) tot += s_ss[grp * nwarps + w];
      inv_rms = 1.0f / sqrtf(tot / (float)p.k + p.eps);
      if (has_part) {
#pragma unroll
        for (int j = 0; j < EPL / 4; ++j) {
          const float4 t = nwv[j];
          if (p.x_normed_out != nullptr && blockIdx.x == 0 && grp == 0)
            reinterpret_cast<float4*>(p.x_normed_out)[part * (EPL / 4) + j] =
                make_float4((v[4 * j] * inv_rms) * t.x, (v[4 * j + 1] * inv_rms) * t.y,
                            (v[4 * j + 2] * inv_rms) * t.z, (v[4 * j + 3] * inv_rms) * t.w);
          v[4 * j] *= t.x; v[4 * j + 1] *= t.y; v[4 * j + 2] *= t.z; v[4 * j + 3] *= t.w;
        }
      }
    }
    float amax = abs_max<EPL>(v);
    if (EPL == 16) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));  // the block's other half
    int S;
    quantize_part_int<EPL>(v, amax, dig, sx, S);
    split_offset(S, s8hi, s8lo);
    if (!has_part) { sx = 0.f; s8hi = 0; s8lo = 0; }
  }

  if (!NORM && p.x_ss8 != nullptr && gw == 0) {
    // RMSNorm with pre-weighted x: only the warp that writes the results needs 1/rms, and only
    // at the end, so these loads stay off the path to the first product.  Fixed summation
    // order (lane-sequential, then a butterfly): every CTA computes the same value.
    float ss = 0.f;
    const int n8 = p.k >> 3;
    for (int i = lane * 4; i < n8; i += 128) {
      const float4 t = *reinterpret_cast<const float4*>(p.x_ss8 + i);
      ss += (t.x + t.y) + (t.z + t.w);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    inv_rms = 1.0f / sqrtf(ss / (float)p.k + p.eps);
  }
  if (tid == 0) tl_mark(p.tl, (int)blockIdx.x, 2);
  const int sidx = blk >> p.gshift;
  int buf = 0;
#pragma unroll 1
  for (int rd = 0; rd < my_rounds; ++rd) {
    float pa[NW][TR];
    // The round that ends with an epilogue: its per-row operands (bias, residual, next norm's
    // weight) are requested now, so that they have arrived when the row sums are complete.
    float pre_b0 = 0.f, pre_b1 = 0.f, pre_res = 0.f, pre_sw = 0.f;
    if (gw == 0 && ((rd & 3) == 3 || rd == my_rounds - 1)) {
      const int row = (round0 + (rd & ~3)) * TR + lane;
      if (lane < ((rd & 3) + 1) * TR && row < p.n) {
        if (p.bias[0]) pre_b0 = p.bias[0][row];
        if (EPI == 1 && p.bias[1]) pre_b1 = p.bias[1][row];
        if (EPI == 0 && p.resid) pre_res = p.resid[row];
        if (p.out_scaled != nullptr) pre_sw = p.out_scale_w[row];
      }
    }
#pragma unroll
    for (int ss = 0; ss < SPR; ++ss) {
      const int it = rd * SPR + ss;
      const int s = it % p.stages;
      const bool ok = mbar_wait(&full[s], (uint32_t)(it / p.stages) & 1u, &s_abort);
      if (tid == 0 && it == 0) tl_mark(p.tl, (int)blockIdx.x, 3);
      if (tid == 0 && it == my_rounds * SPR - 1) tl_mark(p.tl, (int)blockIdx.x, 4);
      const unsigned char* st = ring + (size_t)s * p.stage_bytes;
#pragma unroll
      for (int q = 0; q < NW; ++q) {
        const unsigned char* base = st + (size_t)q * RS * (row_bytes + srow_bytes);
#pragma unroll
        for (int r = 0; r < RS; ++r) {
          float val = 0.f;
          if (has_part && ok) {
            uint32_t wv[NWD];
            const unsigned char* wp = base + (size_t)r * row_bytes + part * (EPL / 2);
            if (EPL == 32) {
              const uint4 t4 = *reinterpret_cast<const uint4*>(wp);
              wv[0] = t4.x; wv[1] = t4.y; wv[NWD - 2] = t4.z; wv[NWD - 1] = t4.w;
            } else {
              const uint2 t2 = *reinterpret_cast<const uint2*>(wp);
              wv[0] = t2.x; wv[1] = t2.y;
            }
            const float sc = *reinterpret_cast<const float*>(base + (size_t)RS * row_bytes + (size_t)r * srow_bytes + sidx * 4);
            val = sc * (sx * idot_words_off<NWD>(wv, dig, s8hi, s8lo));
          }
          pa[q][ss * RS + r] = val;
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);
    }
    // ---- 8 rows done for this lane's slice of K: sum over the warp's lanes ----
    const int slot = rd & 3;
#pragma unroll
    for (int q = 0; q < NW; ++q) {
      const float v = transpose_reduce8(pa[q], lane);
      if ((lane & 3) == 0) s_part[buf][q][warp][slot * TR + (lane >> 2)] = v;
    }
    if (slot != 3 && rd != my_rounds - 1) continue;
    // ---- up to 32 rows gathered: sum over the warps, epilogue, one coalesced store ----
    asm volatile("bar.sync %0, %1;" ::"r"(1 + grp), "r"(group_threads) : "memory");
    float v_out = 0.f;  // this lane's finished row (0 when it has none): input of the sums of squares
    if (gw == 0 && lane < (slot + 1) * TR) {
      const int row = (round0 + (rd & ~3)) * TR + lane;
      float acc[NW];
#pragma unroll
      for (int q = 0; q < NW; ++q) {
        float a = 0.f;
        for (int w = 0; w < nwarps; ++w) a += s_part[buf][q][grp * nwarps + w][lane];
        acc[q] = a * inv_rms;
      }
      if (row < p.n) {
        float v;
        if (EPI == 1) {
          const float g = acc[0] + pre_b0;
          const float u = acc[NW - 1] + pre_b1;
          v = (g / (1.0f + expf(-g))) * u;  // src/llm/decoder.rs:1319-1322
        } else {
          v = acc[0] + pre_b0;
          if (p.resid) v = pre_res + v;
        }
        p.out[row] = v;
        if (p.out_scaled != nullptr) p.out_scaled[row] = v * pre_sw;
        v_out = v;
      }
    }
    if (p.out_ss8 != nullptr && gw == 0) {
      float sq = v_out * v_out;
      sq += __shfl_xor_sync(0xffffffffu, sq, 1);
      sq += __shfl_xor_sync(0xffffffffu, sq, 2);
      sq += __shfl_xor_sync(0xffffffffu, sq, 4);
      const int row = (round0 + (rd & ~3)) * TR + lane;
      if ((lane & 7) == 0 && lane < (slot + 1) * TR && row < p.n) p.out_ss8[row >> 3] = sq;
    }
    buf ^= 1;
  }
  if (tid == 0) tl_mark(p.tl, (int)blockIdx.x, 5);
  if (s_abort && tid == 0) atomicExch(&g_stream_fault, 1);
}

// ---------------------------------------------------------------------------------------------
// The same kernel for TWO activation rows (two sequences of a batch, or a draft token and its
// predecessor in a speculative verify): a lane keeps the digits of its block of K for both rows and
// multiplies every weight word it loads with both, so the rows cost one pass over the weights.
// Measured on the Llama-3-8B shapes against the tensor-core rows kernel at 2 rows: gate/up pair 28.9
// against 42.3 us, K = 14336 projection 19.9 against 33.0, QKV 11.7 against 22.9, o_proj 9.8 against
// 19.5.  Four rows per lane were built and measured too (~200-250 registers, one or two CTAs of 5 warps
// per SM): 90 us for the pair, slower than the tensor-core kernel, so three rows and more stay there.
// A kernel of its own, with its own parameter block: the single-row kernel above is sensitive to both
// (the same source with a row count as template parameter cost it 9% on the gate/up pair).
// ---------------------------------------------------------------------------------------------
struct RowsParams {
  const float* x;            // [m, k]
  const uint8_t* w[2];
  const float* scales[2];
  const float* bias[2];
  const float* norm_w;
  const float* resid;        // [m, n] or null
  float* out;                // [m, n]
  float* x_normed_out;       // [m, k] or null
  float eps;
  int m;                     // activation rows of this launch (<= MR; the rest are zeros)
  int n, k, nb32, gshift, ng;
  int nwarps, groups, stages, stage_bytes, rounds;
  unsigned long long* tl;
};

template <int RS, int EPI, bool NORM, int MR>
__global__ void __launch_bounds__(512) w4_stream_rows_kernel(const RowsParams p) {
  constexpr int EPL = 32;
  constexpr int NW = EPI == 1 ? 2 : 1;
  constexpr int MW = 16;   // consumer warps the partial sums are sized for
  constexpr int TR = 8;            // rows per round
  constexpr int SPR = TR / RS;     // stages per round
  constexpr int NWD = EPL / 8;     // 32-bit weight words per lane and row
  extern __shared__ __align__(128) unsigned char ring[];
  __shared__ uint64_t full[kMaxStages], empty[kMaxStages];
  __shared__ float s_part[2][NW][MR][MW][33];  // [buffer][matrix][activation row][consumer warp][row] (padded)
  __shared__ float s_ss[MR][16];
  __shared__ int s_abort;
  __shared__ int s_waited;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nwarps = p.nwarps, groups = p.groups;
  const bool is_producer = warp == nwarps * groups;
  const int row_bytes = p.k >> 1, srow_bytes = p.ng * 4;
  // Contiguous, balanced share of the 8-row rounds: the first `rem` CTAs take one more.
  const int base_rounds = p.rounds / (int)gridDim.x, rem_rounds = p.rounds % (int)gridDim.x;
  const int my_rounds = base_rounds + ((int)blockIdx.x < rem_rounds ? 1 : 0);
  const int round0 = (int)blockIdx.x * base_rounds + min((int)blockIdx.x, rem_rounds);
  const int total_stages = my_rounds * SPR;

  if (tid == 0) {
    s_abort = 0;
    s_waited = 0;
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], nwarps);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    tl_mark(p.tl, (int)blockIdx.x, 0);
    if (blockIdx.x == 0) tl_header(p.tl, 1, (int)gridDim.x);
  }
  __syncthreads();

  if (is_producer) {
    // ---------------- producer: one lane feeds the ring ----------------
    // The producer must not signal launch_dependents: the next kernel may only start once
    // this grid's consumers are past their griddepcontrol.wait, i.e. once everything before
    // this kernel has completed (kernels further down the chain rely on that).
    if (lane == 0) {
      for (int i = 0; i < total_stages; ++i) {
        const int s = i % p.stages, round = i / p.stages;
        if (round > 0 && !mbar_wait(&empty[s], (uint32_t)(round - 1) & 1u, &s_abort)) break;
        if (i == 0) tl_mark(p.tl, (int)blockIdx.x, 6);
        if (i == total_stages - 1) tl_mark(p.tl, (int)blockIdx.x, 7);
        const int row0 = (round0 + i / SPR) * TR + (i % SPR) * RS;
        const int cnt = max(0, min(RS, p.n - row0));
        unsigned char* dst = ring + (size_t)s * p.stage_bytes;
        if (cnt == 0) {  // nothing to fetch for this stage: complete the phase by hand
          mbar_arrive(&full[s]);
          continue;
        }
        const uint32_t wb = (uint32_t)cnt * row_bytes, sb = (uint32_t)cnt * srow_bytes;
        mbar_expect_tx(&full[s], NW * (wb + sb));
#pragma unroll
        for (int q = 0; q < NW; ++q) {
          unsigned char* d = dst + (size_t)q * RS * (row_bytes + srow_bytes);
          bulk_g2s(d, p.w[q] + (int64_t)row0 * row_bytes, wb, &full[s]);
          bulk_g2s(d + (size_t)RS * row_bytes, p.scales[q] + (int64_t)row0 * p.ng, sb, &full[s]);
        }
      }
      {
        // All of this CTA's HBM requests are out: the next kernel may start filling its ring
        // (launch_dependents is signalled here, after the last stage was requested).
        // Only after the consumers are past their griddepcontrol.wait (completion must stay
        // transitive along the chain of kernels); bounded like every other wait.
        const long long t0 = clock64();
        while (*reinterpret_cast<volatile int*>(&s_waited) == 0 && clock64() - t0 < kWaitCycles) {}
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
      }
    }
    return;
  }

  // ---------------- consumers ----------------
  // Everything below reads the previous kernel's output.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (tid == 0) *reinterpret_cast<volatile int*>(&s_waited) = 1;
  if (tid == 0) tl_mark(p.tl, (int)blockIdx.x, 1);

  const int grp = warp / nwarps, gw = warp - grp * nwarps;
  const int part = gw * 32 + lane;                 // index of this lane's EPL-element slice of K
  const bool has_part = part * EPL < p.k;
  const int blk = (part * EPL) >> 5;
  const int group_threads = nwarps * 32;
  uint32_t dig[MR][NWD * 6];
  float sx[MR];
  int s8hi[MR], s8lo[MR];   // 8 * sum of this lane's digits-as-integers: the offset of the codes
  float inv_rms[MR];
#pragma unroll
  for (int m = 0; m < MR; ++m) { sx[m] = 0.f; s8hi[m] = 0; s8lo[m] = 0; inv_rms[m] = 1.f; }
  {
    // Several rows: the sums of squares of every row first (one barrier for all of them), then row after
    // row is read again (it is in L1/L2 by now), weighted and turned into digits, so that only one row's
    // elements are live at a time.  Rows from p.m on are zeros.
    auto load_row = [&](int m, float (&v)[EPL]) {
      if (has_part && m < p.m) {
        const float4* xg = reinterpret_cast<const float4*>(p.x + (int64_t)m * p.k) + part * (EPL / 4);
#pragma unroll
        for (int j = 0; j < EPL / 4; ++j) {
          const float4 t = xg[j];
          v[4 * j] = t.x; v[4 * j + 1] = t.y; v[4 * j + 2] = t.z; v[4 * j + 3] = t.w;
        }
      } else {
#pragma unroll
        for (int j = 0; j < EPL; ++j) v[j] = 0.f;
      }
    };
    if (NORM) {
#pragma unroll
      for (int m = 0; m < MR; ++m) {
        float v[EPL];
        load_row(m, v);
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < EPL; ++j) ss = fmaf(v[j], v[j], ss);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (lane == 0) s_ss[m][warp] = ss;
      }
      asm volatile("bar.sync %0, %1;" ::"r"(1 + grp), "r"(group_threads) : "memory");
#pragma unroll
      for (int m = 0; m < MR; ++m) {
        float tot = 0.f;
        for (int w = 0; w < nwarps; ++w) tot += s_ss[m][grp * nwarps + w];
        inv_rms[m] = 1.0f / sqrtf(tot / (float)p.k + p.eps);
      }
    }
#pragma unroll
    for (int m = 0; m < MR; ++m) {
      float v[EPL];
      load_row(m, v);
      if (NORM && has_part) {
        const float4* nw = reinterpret_cast<const float4*>(p.norm_w) + part * (EPL / 4);
#pragma unroll
        for (int j = 0; j < EPL / 4; ++j) {
          const float4 t = __ldg(nw + j);
          if (p.x_normed_out != nullptr && blockIdx.x == 0 && grp == 0 && m < p.m)
            reinterpret_cast<float4*>(p.x_normed_out + (int64_t)m * p.k)[part * (EPL / 4) + j] =
                make_float4((v[4 * j] * inv_rms[m]) * t.x, (v[4 * j + 1] * inv_rms[m]) * t.y,
                            (v[4 * j + 2] * inv_rms[m]) * t.z, (v[4 * j + 3] * inv_rms[m]) * t.w);
          v[4 * j] *= t.x; v[4 * j + 1] *= t.y; v[4 * j + 2] *= t.z; v[4 * j + 3] *= t.w;
        }
      }
      float amax = abs_max<EPL>(v);
      if (EPL == 16) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      int S;
      quantize_part_int<EPL>(v, amax, dig[m], sx[m], S);
      split_offset(S, s8hi[m], s8lo[m]);
      if (!has_part) { sx[m] = 0.f; s8hi[m] = 0; s8lo[m] = 0; }
    }
  }

  if (tid == 0) tl_mark(p.tl, (int)blockIdx.x, 2);
  const int sidx = blk >> p.gshift;
  int buf = 0;
#pragma unroll 1
  for (int rd = 0; rd < my_rounds; ++rd) {
    float pa[NW][MR][TR];
    // The round that ends with an epilogue: its per-row operands (bias, residual, next norm's
    // weight) are requested now, so that they have arrived when the row sums are complete.
    float pre_b0 = 0.f, pre_b1 = 0.f;
    if (gw == 0 && ((rd & 3) == 3 || rd == my_rounds - 1)) {
      const int row = (round0 + (rd & ~3)) * TR + lane;
      if (lane < ((rd & 3) + 1) * TR && row < p.n) {
        if (p.bias[0]) pre_b0 = p.bias[0][row];
        if (EPI == 1 && p.bias[1]) pre_b1 = p.bias[1][row];
      }
    }
#pragma unroll
    for (int ss = 0; ss < SPR; ++ss) {
      const int it = rd * SPR + ss;
      const int s = it % p.stages;
      const bool ok = mbar_wait(&full[s], (uint32_t)(it / p.stages) & 1u, &s_abort);
      if (tid == 0 && it == 0) tl_mark(p.tl, (int)blockIdx.x, 3);
      if (tid == 0 && it == my_rounds * SPR - 1) tl_mark(p.tl, (int)blockIdx.x, 4);
      const unsigned char* st = ring + (size_t)s * p.stage_bytes;
#pragma unroll
      for (int q = 0; q < NW; ++q) {
        const unsigned char* base = st + (size_t)q * RS * (row_bytes + srow_bytes);
#pragma unroll
        for (int r = 0; r < RS; ++r) {
          if (has_part && ok) {
            uint32_t wv[NWD];
            const unsigned char* wp = base + (size_t)r * row_bytes + part * (EPL / 2);
            if (EPL == 32) {
              const uint4 t4 = *reinterpret_cast<const uint4*>(wp);
              wv[0] = t4.x; wv[1] = t4.y; wv[NWD - 2] = t4.z; wv[NWD - 1] = t4.w;
            } else {
              const uint2 t2 = *reinterpret_cast<const uint2*>(wp);
              wv[0] = t2.x; wv[1] = t2.y;
            }
            const float sc = *reinterpret_cast<const float*>(base + (size_t)RS * row_bytes + (size_t)r * srow_bytes + sidx * 4);
#pragma unroll
            for (int m = 0; m < MR; ++m) pa[q][m][ss * RS + r] = sc * (sx[m] * idot_words_off<NWD>(wv, dig[m], s8hi[m], s8lo[m]));
          } else {
#pragma unroll
            for (int m = 0; m < MR; ++m) pa[q][m][ss * RS + r] = 0.f;
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);
    }
    // ---- 8 rows done for this lane's slice of K: sum over the warp's lanes ----
    const int slot = rd & 3;
#pragma unroll
    for (int q = 0; q < NW; ++q)
#pragma unroll
      for (int m = 0; m < MR; ++m) {
        const float v = transpose_reduce8(pa[q][m], lane);
        if ((lane & 3) == 0) s_part[buf][q][m][warp][slot * TR + (lane >> 2)] = v;
      }
    if (slot != 3 && rd != my_rounds - 1) continue;
    // ---- up to 32 rows gathered: sum over the warps, epilogue, one coalesced store ----
    asm volatile("bar.sync %0, %1;" ::"r"(1 + grp), "r"(group_threads) : "memory");
    if (gw == 0 && lane < (slot + 1) * TR) {
      const int row = (round0 + (rd & ~3)) * TR + lane;
#pragma unroll
      for (int m = 0; m < MR; ++m) {
        float acc[NW];
#pragma unroll
        for (int q = 0; q < NW; ++q) {
          float a = 0.f;
          for (int w = 0; w < nwarps; ++w) a += s_part[buf][q][m][grp * nwarps + w][lane];
          acc[q] = a * inv_rms[m];
        }
        if (row < p.n && m < p.m) {
          float v;
          if (EPI == 1) {
            const float g = acc[0] + pre_b0;
            const float u = acc[NW - 1] + pre_b1;
            v = (g / (1.0f + expf(-g))) * u;  // src/llm/decoder.rs:1319-1322
          } else {
            v = acc[0] + pre_b0;
            if (p.resid) v = p.resid[(int64_t)m * p.n + row] + v;
          }
          p.out[(int64_t)m * p.n + row] = v;
        }
      }
    }
    buf ^= 1;
  }
  if (tid == 0) tl_mark(p.tl, (int)blockIdx.x, 5);
  if (s_abort && tid == 0) atomicExch(&g_stream_fault, 1);
}

int g_stream_enabled = 1;
int g_ctas_per_sm = 0;
int g_ring_kb = 0;
int g_force_epl = 0, g_force_groups = 0;

template <int RS, int EPI, bool NORM, int EPL>
tb_status launch_rs(const StreamParams& p, int grid, size_t smem, bool pdl, cudaStream_t stream) {
  auto kern = w4_stream_kernel<RS, EPI, NORM, EPL>;
  static thread_local size_t configured[64] = {0};
  int dev = 0;
  TB_CUDA_TRY(cudaGetDevice(&dev));
  // static + dynamic shared memory above 48 KB needs the opt-in, so opt in from 32 KB up
  if (smem > 32 * 1024 && (dev >= 64 || configured[dev] < smem)) {
    TB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    if (dev < 64) configured[dev] = smem;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3((unsigned)(p.nwarps * p.groups + 1) * 32);
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

template <int EPI, bool NORM, int EPL>
tb_status launch_en(int rs, const StreamParams& p, int grid, size_t smem, bool pdl, cudaStream_t stream) {
  switch (rs) {
    case 1: return launch_rs<1, EPI, NORM, EPL>(p, grid, smem, pdl, stream);
    case 2: return launch_rs<2, EPI, NORM, EPL>(p, grid, smem, pdl, stream);
    case 4: return launch_rs<4, EPI, NORM, EPL>(p, grid, smem, pdl, stream);
    case 8: return launch_rs<8, EPI, NORM, EPL>(p, grid, smem, pdl, stream);
  }
  return fail(TB_ERR_ARG, "w4 stream: rows per stage %d", rs);
}

template <int EPL>
tb_status launch_epl(bool swiglu, bool norm, int rs, const StreamParams& p, int grid, size_t smem, bool pdl,
                     cudaStream_t stream) {
  if (swiglu) return norm ? launch_en<1, true, EPL>(rs, p, grid, smem, pdl, stream) : launch_en<1, false, EPL>(rs, p, grid, smem, pdl, stream);
  return norm ? launch_en<0, true, EPL>(rs, p, grid, smem, pdl, stream) : launch_en<0, false, EPL>(rs, p, grid, smem, pdl, stream);
}

template <int RS, int EPI, bool NORM>
tb_status launch_rows_rs(const RowsParams& p, int grid, size_t smem, bool pdl, cudaStream_t stream) {
  auto kern = w4_stream_rows_kernel<RS, EPI, NORM, 2>;
  static thread_local size_t configured[64] = {0};
  int dev = 0;
  TB_CUDA_TRY(cudaGetDevice(&dev));
  // static + dynamic shared memory above 48 KB needs the opt-in (17 KB are static here), so opt in from 16 KB up
  if (smem > 16 * 1024 && (dev >= 64 || configured[dev] < smem)) {
    TB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    if (dev < 64) configured[dev] = smem;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3((unsigned)(p.nwarps + 1) * 32);
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

template <int EPI, bool NORM>
tb_status launch_rows_en(int rs, const RowsParams& p, int grid, size_t smem, bool pdl, cudaStream_t stream) {
  switch (rs) {
    case 1: return launch_rows_rs<1, EPI, NORM>(p, grid, smem, pdl, stream);
    case 2: return launch_rows_rs<2, EPI, NORM>(p, grid, smem, pdl, stream);
    case 4: return launch_rows_rs<4, EPI, NORM>(p, grid, smem, pdl, stream);
    case 8: return launch_rows_rs<8, EPI, NORM>(p, grid, smem, pdl, stream);
  }
  return fail(TB_ERR_ARG, "w4 stream: rows per stage %d", rs);
}

// Two activation rows: same ring sizing as the single-row launch, a whole block of K per lane.
tb_status launch_w4_stream_rows(const GemvArgs& a, cudaStream_t stream) {
  RowsParams p;
  p.x = a.x;
  p.w[0] = a.w; p.w[1] = a.w2;
  p.scales[0] = a.scales; p.scales[1] = a.scales2;
  p.bias[0] = a.bias; p.bias[1] = a.bias2;
  p.norm_w = a.norm_w; p.resid = a.resid; p.out = a.out; p.x_normed_out = a.x_normed_out;
  p.eps = a.eps;
  p.m = a.m;
  p.tl = timeline_next_block();
  p.n = (int)a.n; p.k = (int)a.k; p.nb32 = (int)(a.k / 32);
  p.gshift = a.g == 32 ? 0 : (a.g == 64 ? 1 : 2);
  p.ng = (int)(a.k / a.g);
  p.rounds = (p.n + 7) / 8;
  const int cps = g_ctas_per_sm > 0 ? g_ctas_per_sm : (p.k >= 8192 ? 1 : 3);
  int grid = sm_count() * cps;
  if (grid > p.rounds) grid = p.rounds;
  p.nwarps = (p.nb32 + 31) / 32;
  p.groups = 1;
  const int nw = a.w2 ? 2 : 1;
  const int per_row = nw * (p.k / 2 + p.ng * 4);
  const int ring_budget = g_ring_kb > 0 ? g_ring_kb * 1024 : (cps >= 3 ? 40 * 1024 : kRingBytesMax / cps);
  int rs = 8;
  while (rs > 1 && (rs * per_row > 20 * 1024 || rs * per_row * 3 > ring_budget)) rs >>= 1;
  p.stage_bytes = rs * per_row;
  p.stages = ring_budget / p.stage_bytes;
  if (p.stages > kMaxStages) p.stages = kMaxStages;
  if (p.stages < 2) p.stages = 2;
  const size_t smem = (size_t)p.stages * p.stage_bytes;
  if (smem > 180 * 1024) return fail(TB_ERR_UNSUPPORTED, "w4 stream: a row of %d bytes does not fit the ring", per_row);
  if (a.w2) return a.norm_w ? launch_rows_en<1, true>(rs, p, grid, smem, a.pdl, stream) : launch_rows_en<1, false>(rs, p, grid, smem, a.pdl, stream);
  return a.norm_w ? launch_rows_en<0, true>(rs, p, grid, smem, a.pdl, stream) : launch_rows_en<0, false>(rs, p, grid, smem, a.pdl, stream);
}

}  // namespace

void set_stream_tuning(int enabled, int ctas_per_sm, int ring_kb, int epl, int groups) {
  g_stream_enabled = enabled;
  g_ctas_per_sm = ctas_per_sm;
  g_ring_kb = ring_kb;
  g_force_epl = epl;
  g_force_groups = groups;
}

// Non-zero after a bulk copy was declared lost by one of the bounded waits.
int stream_fault_flag() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_stream_fault, sizeof(int)) != cudaSuccess) return -1;
  return v;
}

// True when the persistent kernel can take this product (M = 1, bulk-copy alignment rules).
bool w4_stream_supported(const GemvArgs& a) {
  if (!g_stream_enabled || a.m < 1 || a.m > 2) return false;
  // two rows: no split RMSNorm (its operands belong to one vector)
  if (a.m == 2 && (a.x_ss8 || a.out_scaled || a.out_ss8)) return false;
  // narrow K leaves most of a CTA's lanes without work: the per-row-tile kernels are faster there
  if (a.k % 32 != 0 || a.k < 2048 || a.k > 32 * 32 * 15) return false;  // at most 15 consumer warps + the producer
  const int64_t ng = a.k / a.g;
  if ((ng * 4) % 16 != 0) return false;  // a row of scales must be a whole number of 16-byte units
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (!al16(a.w) || !al16(a.scales) || !al16(a.x)) return false;
  if (a.w2 && (!al16(a.w2) || !al16(a.scales2))) return false;
  if (a.norm_w && !al16(a.norm_w)) return false;
  if (a.x_ss8 && (a.norm_w || !al16(a.x_ss8) || a.k % 32 != 0)) return false;
  if ((a.out_scaled != nullptr) != (a.out_scale_w != nullptr)) return false;
  return true;
}

tb_status launch_w4_stream(const GemvArgs& a, cudaStream_t stream) {
  if (a.m == 2) return launch_w4_stream_rows(a, stream);
  StreamParams p;
  p.x = a.x;
  p.w[0] = a.w; p.w[1] = a.w2;
  p.scales[0] = a.scales; p.scales[1] = a.scales2;
  p.bias[0] = a.bias; p.bias[1] = a.bias2;
  p.norm_w = a.norm_w; p.resid = a.resid; p.out = a.out; p.x_normed_out = a.x_normed_out;
  p.x_ss8 = a.x_ss8; p.out_scaled = a.out_scaled; p.out_scale_w = a.out_scale_w; p.out_ss8 = a.out_ss8;
  p.eps = a.eps;
  p.tl = timeline_next_block();
  // Dependents may start once this CTA's last HBM request is out (measured: start, that point and
  // the end of the kernel differ by < 1% on the decode step; the early start helps small kernels).
  p.n = (int)a.n; p.k = (int)a.k; p.nb32 = (int)(a.k / 32);
  p.gshift = a.g == 32 ? 0 : (a.g == 64 ? 1 : 2);
  p.ng = (int)(a.k / a.g);
  p.rounds = (p.n + 7) / 8;
  // K split: half a block per lane in the latency regime (few tiles per CTA: more lanes work
  // on each row), a whole block per lane in the throughput regime (fewer instructions per
  // element); wide K runs one CTA per SM with twice the ring.
  int cps = g_ctas_per_sm > 0 ? g_ctas_per_sm : (p.k >= 8192 ? 1 : 3);
  int grid = sm_count() * cps;
  if (grid > p.rounds) grid = p.rounds;
  const int rounds_per_cta = (p.rounds + grid - 1) / grid;
  // half a block per lane only up to K = 4096: beyond, 14 consumer warps per CTA cost more than they bring
  // (N = 4096, K = 7168: 13.6 us against 10.4 us with a whole block per lane)
  int epl = (rounds_per_cta <= 4 && p.nb32 <= 128) ? 16 : 32;
  if (g_force_epl == 16 || g_force_epl == 32) epl = g_force_epl;
  p.nwarps = (p.k / epl + 31) / 32;
  if (p.nwarps > 15) { epl = 32; p.nwarps = (p.nb32 + 31) / 32; }
  // One consumer group: every consumer warp observes every stage of the ring in order,
  // which is what keeps the mbarrier phase parities unambiguous.
  p.groups = 1;
  const int nw = a.w2 ? 2 : 1;
  const int per_row = nw * (p.k / 2 + p.ng * 4);
  // Stage: at most ~20 KB; ring: as many stages as fit the budget (2..8).
  const int ring_budget = g_ring_kb > 0 ? g_ring_kb * 1024 : (cps >= 3 ? 40 * 1024 : kRingBytesMax / cps);
  int rs = 8;
  while (rs > 1 && (rs * per_row > 20 * 1024 || rs * per_row * 3 > ring_budget)) rs >>= 1;
  p.stage_bytes = rs * per_row;
  p.stages = ring_budget / p.stage_bytes;
  if (p.stages > kMaxStages) p.stages = kMaxStages;
  if (p.stages < 2) p.stages = 2;
  const size_t smem = (size_t)p.stages * p.stage_bytes;
  if (smem > 200 * 1024) return fail(TB_ERR_UNSUPPORTED, "w4 stream: a row of %d bytes does not fit the ring", per_row);
  const bool swiglu = a.w2 != nullptr;
  const bool pdl = a.pdl;
  if (epl == 16) return launch_epl<16>(swiglu, a.norm_w != nullptr, rs, p, grid, smem, pdl, stream);
  return launch_epl<32>(swiglu, a.norm_w != nullptr, rs, p, grid, smem, pdl, stream);
}

}  // namespace tb
