// GQA decode attention over the fp32 KV cache: RoPE + KV append + split-K
// flash-decode + merge, one launch.
//
// Replaces steps C-E of RustQwenDecoder::step_internal (src/llm/decoder.rs:1127-1213;
// rope_apply_head :28-68) and the wgpu shaders rope_append.wgsl / attn_decode.wgsl.
//
// The reference walks the sequence serially per q head with a two-pass softmax.
// Here the positions [0, offset] of every (sequence, kv head) are divided evenly
// among the CTAs of a grid row, whatever the current length, so that every SM
// streams its share.  Inside a CTA one producer lane feeds a ring of shared-memory
// stages with bulk asynchronous copies (32 K rows + 32 V rows per stage, contiguous
// in the [Hkv, S, d] cache) and the consumer warps score the rows for all q heads
// that share the kv head, keep an online softmax and accumulate the weighted V -
// each K/V row is read from HBM once per step and the bytes in flight do not
// depend on registers or occupancy.  Every CTA writes an un-normalised partial
// (max, sum, weighted V) to scratch; the last CTA of a (sequence, kv head) to
// finish - found with a ticket counter - rescales and sums the partials.  The
// result equals the two-pass softmax up to fp32 rounding.  HBM-bound:
// algorithmic bytes = 2 * Hkv * (offset+1) * d * 4 per sequence and layer.
#include <atomic>

#include "tb_common.cuh"

namespace tb {

namespace {

#ifndef TB_ATTN_CW
#define TB_ATTN_CW 4
#endif
constexpr int kCW = TB_ATTN_CW;        // consumer warps per CTA
constexpr int kCT = kCW * 32;          // consumer threads
constexpr int kThreads = kCT + 32;     // + the producer warp
constexpr int kStageRows = 32;         // K rows (and V rows) per ring stage
constexpr int kWR = kStageRows / kCW;  // rows of a stage that one consumer warp owns (8)
constexpr int kRG = kWR / 4;           // groups of 4 rows per warp and stage (2)
constexpr int kMaxGq = 8;              // q heads per kv head
constexpr int kMaxStages = 8;
constexpr int kChunkRows = 512;        // positions whose scores are held in shared memory at a time
constexpr size_t kCounterBytes = 16384;  // 4096 tickets: (sequence, kv head) pairs of a launch
constexpr int kSeqCap = 32768;         // src/llm/decoder.rs:1180
constexpr long long kWaitCycles = 4000000000ll;  // ~2 s: a wait that long means a lost copy

__device__ int g_attn_fault = 0;

struct AttnParams {
  const float* qkv;
  float* k_cache;
  float* v_cache;
  const float* cos_t;
  const float* sin_t;
  const int32_t* offsets;
  float* out;
  float* part_o;    // [b, Hq, nc, D]
  float* part_ml;   // [b, Hq, nc, 2]
  int* counters;    // [b, Hkv] tickets
  float* qkv_rot_out;
  int num_heads, num_kv_heads, gq;
  int fixed_per;    // positions per CTA when forced, else 0: divide the current length evenly
  int nc;           // CTAs per (sequence, kv head) = gridDim.x
  int stages;       // ring depth
  int max_parts;    // upper bound of CTAs of a (sequence, kv head) that take positions
  int region_floats;  // floats of the ring region (also holds the combine / merge buffers)
  int64_t max_seq_len;
  int per_call_tables;
  int shared_cache;   // every row of the batch is a position of ONE sequence: sequence 0's cache, rows appended beforehand
  float scale;
  unsigned long long* tl;  // timestamps of this launch or null
};

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ---- mbarrier + bulk async copy (TMA engine, linear form) ----
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
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
// Barrier among the consumer threads only (the producer warp leaves early).
__device__ __forceinline__ void consumer_barrier() {
  asm volatile("bar.sync 1, %0;" ::"r"(kCT) : "memory");
}

// rotate-half with separately rounded products, src/llm/decoder.rs:40-66:
//   o[i]      = x[i]*cos[i]          - x[i+half]*sin[i]
//   o[i+half] = x[i+half]*cos[i+half] + x[i]*sin[i+half]
__device__ __forceinline__ float rope_elem(const float* x, const float* c, const float* s, int i,
                                           int half) {
  if (i < half) return __fsub_rn(__fmul_rn(x[i], c[i]), __fmul_rn(x[i + half], s[i]));
  return __fadd_rn(__fmul_rn(x[i], c[i]), __fmul_rn(x[i - half], s[i]));
}

// Shared memory (floats): q_s [gq][D] | kv_new [2][D] | S [kChunkRows + 1][GQM] | region.  The
// region is the ring (stages * 32 * D) while rows stream in; afterwards it holds w_acc
// [kCW][gq][D] for the combine and, in the CTA that merges, wts [gq][nc] | ml [gq] | a tile of
// partials.  Every part starts on a 16-byte boundary (float4 accesses).
__host__ __device__ inline size_t up4(size_t v) { return (v + 3) & ~(size_t)3; }
__host__ __device__ inline size_t attn_fixed_floats(int D, int gq, int gqm) {
  return up4((size_t)gq * D) + 2 * (size_t)D + up4((size_t)(kChunkRows + 1) * gqm);
}
inline size_t attn_region_floats(int D, int gq, int nc, int stages) {
  const size_t ring = (size_t)stages * kStageRows * D;
  const size_t comb = (size_t)kCW * gq * D;
  const size_t merge = up4((size_t)gq * nc) + up4(gq) + (size_t)gq * D;
  size_t r = ring > comb ? ring : comb;
  return r > merge ? r : merge;
}

// Sums over the 8 lanes that share a K row.  In: v[i] for i < V, this lane's partial sums.
// Out: v[j] for j < max(1, V/8) holds the complete sum of index
//   idx = sum_t bit_t(l8) * (V >> (t+1)) + j      (t over the halving steps),
// so the V sums end up spread over the 8 lanes instead of replicated in all of them.
template <int V>
__device__ __forceinline__ void spread_reduce8(float (&v)[V], int l8) {
  if (V >= 2) {
    const bool hi = (l8 & 1) != 0;
#pragma unroll
    for (int j = 0; j < V / 2; ++j) {
      const float send = hi ? v[j] : v[j + V / 2];
      const float keep = hi ? v[j + V / 2] : v[j];
      v[j] = keep + __shfl_xor_sync(0xffffffffu, send, 1);
    }
  } else {
    v[0] += __shfl_xor_sync(0xffffffffu, v[0], 1);
  }
  if (V >= 4) {
    const bool hi = (l8 & 2) != 0;
#pragma unroll
    for (int j = 0; j < V / 4; ++j) {
      const float send = hi ? v[j] : v[j + V / 4];
      const float keep = hi ? v[j + V / 4] : v[j];
      v[j] = keep + __shfl_xor_sync(0xffffffffu, send, 2);
    }
  } else {
    v[0] += __shfl_xor_sync(0xffffffffu, v[0], 2);
  }
  if (V >= 8) {
    const bool hi = (l8 & 4) != 0;
#pragma unroll
    for (int j = 0; j < V / 8; ++j) {
      const float send = hi ? v[j] : v[j + V / 8];
      const float keep = hi ? v[j + V / 8] : v[j];
      v[j] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
    }
  } else {
    v[0] += __shfl_xor_sync(0xffffffffu, v[0], 4);
  }
}

// Scores of up to 8 rows (K rows in shared memory at kb) against the q heads of this kv head.
// Lanes work 8 to a row (4 rows at a time, two such groups); spread_reduce8 leaves every
// (row, head) sum in one lane, which scales it, stores it at S[(srow0 + row) * GQM + head] and
// folds it into its running maximum lmax.
template <int D, int GQM, bool QREG>
__device__ __forceinline__ void score_rows(const float* __restrict__ kb, int nr, int srow0, int gq, float scale,
                                           const float4 (&qreg)[QREG ? GQM : 1][D / 32],
                                           const float* __restrict__ q_s, float* __restrict__ S,
                                           float (&lmax)[kRG * GQM >= 8 ? kRG * GQM / 8 : 1], int lane) {
  constexpr int F4 = D / 32;   // float4 per lane and row (8 lanes per row)
  constexpr int CPR = D / 4;   // float4 columns per row
  constexpr int V = kRG * GQM;
  constexpr int NV = V >= 8 ? V / 8 : 1;
  constexpr int HSTEPS = V >= 8 ? 3 : (V == 4 ? 2 : (V == 2 ? 1 : 0));
  const int l8 = lane & 7, rsub = lane >> 3;
  float v[V];
#pragma unroll
  for (int rg = 0; rg < kRG; ++rg) {
    const int row = rg * 4 + rsub;
    float4 kf[F4];
#pragma unroll
    for (int i = 0; i < F4; ++i)
      kf[i] = row < nr ? reinterpret_cast<const float4*>(kb)[row * CPR + l8 + 8 * i] : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int g = 0; g < GQM; ++g) {
      float a0 = 0.f, a1 = 0.f;
      if (g < gq) {
#pragma unroll
        for (int i = 0; i < F4; ++i) {
          const float4 qv = QREG ? qreg[QREG ? g : 0][i] : reinterpret_cast<const float4*>(q_s)[g * CPR + l8 + 8 * i];
          a0 = fmaf(qv.x, kf[i].x, a0);
          a1 = fmaf(qv.y, kf[i].y, a1);
          a0 = fmaf(qv.z, kf[i].z, a0);
          a1 = fmaf(qv.w, kf[i].w, a1);
        }
      }
      v[rg * GQM + g] = a0 + a1;
    }
  }
  spread_reduce8<V>(v, l8);
  int idx0 = 0;
#pragma unroll
  for (int t = 0; t < HSTEPS; ++t) idx0 += ((l8 >> t) & 1) * (V >> (t + 1));
  if (l8 < V) {  // for V < 8 the sums are replicated over the unused lane bits: one copy writes
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int idx = idx0 + j;
      const int rg = idx / GQM, g = idx % GQM;
      const int row = rg * 4 + rsub;
      if (row < nr) {  // rows past nr are neither stored (S ends after the chunk) nor read
        const float sc = v[j] * scale;
        S[(srow0 + row) * GQM + g] = sc;
        lmax[j] = fmaxf(lmax[j], sc);
      }
    }
  }
}

// acc[g] += sum over up to 8 rows of p[row][g] * V[row][:], one float4 column per lane.
template <int D, int GQM>
__device__ __forceinline__ void weigh_rows(const float* __restrict__ vb, int nr, int srow0,
                                           const float* __restrict__ S, float4 (&acc)[GQM], int lane) {
  constexpr int CPR = D / 4;
  constexpr int RPL = 32 / CPR;  // rows per warp-wide V load
  const int vc4 = lane % CPR, vrs = lane / CPR;
#pragma unroll
  for (int j = 0; j < kWR / RPL; ++j) {
    const int r = j * RPL + vrs;
    if (r < nr) {
      const float4 vv = reinterpret_cast<const float4*>(vb)[r * CPR + vc4];
      float pg[GQM];
      if (GQM >= 4) {
#pragma unroll
        for (int q4 = 0; q4 < GQM / 4; ++q4) {
          const float4 t = reinterpret_cast<const float4*>(S + (srow0 + r) * GQM)[q4];
          pg[q4 * 4 + 0] = t.x; pg[q4 * 4 + 1] = t.y; pg[q4 * 4 + 2] = t.z; pg[q4 * 4 + 3] = t.w;
        }
      } else {
#pragma unroll
        for (int g = 0; g < GQM; ++g) pg[g] = S[(srow0 + r) * GQM + g];
      }
#pragma unroll
      for (int g = 0; g < GQM; ++g) {
        acc[g].x = fmaf(pg[g], vv.x, acc[g].x);
        acc[g].y = fmaf(pg[g], vv.y, acc[g].y);
        acc[g].z = fmaf(pg[g], vv.z, acc[g].z);
        acc[g].w = fmaf(pg[g], vv.w, acc[g].w);
      }
    }
  }
}

// One CTA = one share of the positions of one (sequence, kv head).  The share is walked in
// chunks of at most kChunkRows positions; for every chunk the producer lane streams the K
// rows and then the V rows through the ring (32 rows per stage).  The consumer warps score the
// K stages as they land (8 rows of a stage per warp) into S, the CTA then takes the exact
// maximum and the exponentials of the chunk (a two-pass softmax inside the chunk; the running
// max / sum / weighted V are rescaled only between chunks), and the V stages are weighted as
// they land.  No softmax dependency sits inside either streaming loop.
// Two CTAs per SM is what the grid is sized for; telling the compiler so costs nothing (159 registers)
// and measured 1% on the whole step.  With a bound of one CTA it takes 187 registers and the step is 8% slower.
#ifndef TB_ATTN_MIN_CTAS
#define TB_ATTN_MIN_CTAS 2
#endif
#define TB_ATTN_BOUNDS __launch_bounds__(kThreads, TB_ATTN_MIN_CTAS)
template <int D, int GQM>
__global__ void TB_ATTN_BOUNDS attn_decode_kernel(const AttnParams p) {
  constexpr int F4 = D / 32;
  constexpr int CPR = D / 4;
  constexpr bool QREG = GQM * F4 <= 16 && kCW == 4;
  constexpr int V = kRG * GQM;
  constexpr int NV = V >= 8 ? V / 8 : 1;
  constexpr int HSTEPS = V >= 8 ? 3 : (V == 4 ? 2 : (V == 2 ? 1 : 0));
  static_assert(D == 32 || D == 64 || D == 128, "head_dim");

  extern __shared__ __align__(128) float smem[];
  __shared__ __align__(8) uint64_t full[kMaxStages];
  __shared__ __align__(8) uint64_t empty[kMaxStages];
  __shared__ float s_wmax[kCW][kMaxGq], s_wsum[kCW][kMaxGq], s_ml[2][kMaxGq];
  __shared__ int s_abort;
  __shared__ int s_last;

  const int gq = p.gq;
  float* q_s = smem;
  float* kv_new = q_s + up4((size_t)gq * D);
  float* S = kv_new + 2 * D;                             // [(kChunkRows + 1)][GQM]
  float* region = S + up4((size_t)(kChunkRows + 1) * GQM);

  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int qkv_dim = (p.num_heads + 2 * p.num_kv_heads) * D;

  if (tid == 0) {
    s_abort = 0;
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], kCW);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const int cta_lin = (int)(blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z));
  if (tid < kMaxGq) {  // an empty share: weight 0 in any merge
    s_ml[0][tid] = -INFINITY;
    s_ml[1][tid] = 0.f;
  }
  if (tid == 0) {
    tl_mark(p.tl, cta_lin, 0);
    if (cta_lin == 0) tl_header(p.tl, 2, (int)(gridDim.x * gridDim.y * gridDim.z));
  }

  // Before griddepcontrol.wait only data from at least two kernels back may be touched: the
  // offsets (written at the start of the step) and the cache rows of earlier steps.  The kernel
  // directly ahead produces qkv and nothing else, and it signals its dependents only after its
  // own wait, so everything older is complete when this code runs.  The plan and the whole
  // K/V stream therefore start while that kernel is still draining; only the q-dependent
  // work waits.
  const int off = p.offsets[b];
  const bool seq_ok = off >= 0 && (int64_t)off < p.max_seq_len;
  const int t_end = seq_ok ? min(off + 1, kSeqCap) : 0;  // attend to [0, t_end)
  int per = p.fixed_per;
  if (per <= 0) {
    const int parts = min(p.nc, p.max_parts);  // more partials than this cost more in the merge than they save
    per = (t_end + parts - 1) / parts;
    per = max(kStageRows, (per + kStageRows - 1) & ~(kStageRows - 1));
  }
  const int nvalid = (t_end + per - 1) / per;   // CTAs of this grid row that have positions
  const int t0 = split * per;
  const bool active = t0 < t_end;
  const int rows = active ? min(per, t_end - t0) : 0;
  // The CTA that holds position `off` appends the new k (rotated) and v to the cache.  That
  // row is the last one of its range; it is taken from shared memory, not from the cache.
  const bool has_new = active && off >= t0 && off < t0 + rows;
  const int ring_rows = rows - (has_new ? 1 : 0);
  const int nchunks = active ? max(1, (ring_rows + kChunkRows - 1) / kChunkRows) : 0;
  const int cache_seq = p.shared_cache ? 0 : b;
  float* kc = p.k_cache + ((int64_t)cache_seq * p.num_kv_heads + kvh) * p.max_seq_len * D;
  float* vc = p.v_cache + ((int64_t)cache_seq * p.num_kv_heads + kvh) * p.max_seq_len * D;
  const int stage_floats = kStageRows * D;

  if (warp == kCW) {
    // ---------------- producer: one lane feeds the ring ----------------
    if (lane == 0) {
      int i = 0;
      bool lost = false;
      for (int c = 0; c < nchunks && !lost; ++c) {
        const int cr0 = c * kChunkRows;
        const int crn = min(kChunkRows, ring_rows - cr0);
        const int nt = (crn + kStageRows - 1) / kStageRows;
        for (int pass = 0; pass < 2 && !lost; ++pass) {
          const float* src = (pass == 0 ? kc : vc) + (int64_t)(t0 + cr0) * D;
          for (int t = 0; t < nt; ++t, ++i) {
            const int s = i % p.stages, round = i / p.stages;
            if (round > 0 && !mbar_wait(&empty[s], (uint32_t)(round - 1) & 1u, &s_abort)) { lost = true; break; }
            if (i == 0) tl_mark(p.tl, cta_lin, 6);
            const int nr = min(kStageRows, crn - t * kStageRows);
            const uint32_t bytes = (uint32_t)nr * D * sizeof(float);
            mbar_expect_tx(&full[s], bytes);
            bulk_g2s(region + (size_t)s * stage_floats, src + (int64_t)t * kStageRows * D, bytes, &full[s]);
          }
        }
      }
      tl_mark(p.tl, cta_lin, 7);
    }
    return;
  }

  // ---------------- consumers ----------------
  pdl_wait();
  pdl_launch_dependents();
  if (tid == 0) tl_mark(p.tl, cta_lin, 1);
  const float* qkv_b = p.qkv + (int64_t)b * qkv_dim;
  if (active) {
    const float* cs = p.cos_t + (p.per_call_tables ? (int64_t)b * D : (int64_t)off * D);
    const float* sn = p.sin_t + (p.per_call_tables ? (int64_t)b * D : (int64_t)off * D);
    // q heads of this kv head, rotated, into shared memory.  All loads are issued first, then the
    // arithmetic: with load and arithmetic interleaved per element the q vector was ready 2 us later.
    constexpr int QIT = kMaxGq * 128 / kCT;
    float xa[QIT], xb[QIT], ca[QIT], sa[QIT];
#pragma unroll
    for (int k = 0; k < QIT; ++k) {
      const int i = tid + k * kCT;
      if (i < gq * D) {
        const int g = i / D, e = i - g * D;
        const float* xh = qkv_b + (int64_t)(kvh * gq + g) * D;
        xa[k] = xh[e];
        xb[k] = xh[e < D / 2 ? e + D / 2 : e - D / 2];
        ca[k] = cs[e];
        sa[k] = sn[e];
      }
    }
#pragma unroll
    for (int k = 0; k < QIT; ++k) {
      const int i = tid + k * kCT;
      if (i < gq * D) {
        const int g = i / D, e = i - g * D;
        // rotate-half with separately rounded products (rope_elem)
        const float v = e < D / 2 ? __fsub_rn(__fmul_rn(xa[k], ca[k]), __fmul_rn(xb[k], sa[k]))
                                  : __fadd_rn(__fmul_rn(xa[k], ca[k]), __fmul_rn(xb[k], sa[k]));
        q_s[g * D + e] = v;
        if (p.qkv_rot_out && split == 0)
          p.qkv_rot_out[(int64_t)b * qkv_dim + (int64_t)(kvh * gq + g) * D + e] = v;
      }
    }
    if (has_new) {
      const float* kx = qkv_b + (int64_t)p.num_heads * D + (int64_t)kvh * D;
      const float* vx = kx + (int64_t)p.num_kv_heads * D;
      for (int e = tid; e < D; e += kCT) {
        const float kr = rope_elem(kx, cs, sn, e, D / 2);
        const float vr = vx[e];
        if (!p.shared_cache) {   // shared cache: rope_append_rows_kernel wrote every row before this launch
          kc[(int64_t)off * D + e] = kr;
          vc[(int64_t)off * D + e] = vr;
        }
        kv_new[e] = kr;
        kv_new[D + e] = vr;
        if (p.qkv_rot_out) {
          float* o = p.qkv_rot_out + (int64_t)b * qkv_dim + (int64_t)p.num_heads * D + (int64_t)kvh * D;
          o[e] = kr;
          o[(int64_t)p.num_kv_heads * D + e] = vr;
        }
      }
    }
    consumer_barrier();
    if (tid == 0) tl_mark(p.tl, cta_lin, 2);

    const int l8 = lane & 7;
    float4 qreg[QREG ? GQM : 1][F4];
    if (QREG) {
#pragma unroll
      for (int g = 0; g < GQM; ++g)
#pragma unroll
        for (int i = 0; i < F4; ++i)
          qreg[QREG ? g : 0][i] = g < gq ? reinterpret_cast<const float4*>(q_s)[g * CPR + l8 + 8 * i]
                                         : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    int idx0 = 0;
#pragma unroll
    for (int t = 0; t < HSTEPS; ++t) idx0 += ((l8 >> t) & 1) * (V >> (t + 1));
    float m_run[GQM], l_run[GQM];
    float4 acc[GQM];
#pragma unroll
    for (int g = 0; g < GQM; ++g) {
      m_run[g] = -INFINITY;
      l_run[g] = 0.f;
      acc[g] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    const int g_t = tid % GQM;  // the head whose exponentials this thread takes in the softmax pass

    int it = 0;  // stages consumed so far (same order as the producer's)
#pragma unroll 1
    for (int c = 0; c < nchunks; ++c) {
      const int cr0 = c * kChunkRows;
      const int crn = min(kChunkRows, ring_rows - cr0);
      const int nt = (crn + kStageRows - 1) / kStageRows;
      const bool new_here = has_new && c == nchunks - 1;
      if (c > 0) consumer_barrier();  // the previous chunk's weights in S have been used
      // ---- K stages: scores into S ----
      float lmax[NV];
#pragma unroll
      for (int j = 0; j < NV; ++j) lmax[j] = -INFINITY;
#pragma unroll 1
      for (int t = 0; t < nt; ++t, ++it) {
        const int s = it % p.stages;
        const bool ok = mbar_wait(&full[s], (uint32_t)(it / p.stages) & 1u, &s_abort);
        if (tid == 0 && it == 0) tl_mark(p.tl, cta_lin, 3);
        const int nr = min(kWR, crn - t * kStageRows - warp * kWR);
        if (ok && nr > 0)
          score_rows<D, GQM, QREG>(region + (size_t)s * stage_floats + (size_t)warp * kWR * D, nr,
                                   t * kStageRows + warp * kWR, gq, p.scale, qreg, q_s, S, lmax, lane);
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);
      }
      if (new_here && warp == 0) score_rows<D, GQM, QREG>(kv_new, 1, crn, gq, p.scale, qreg, q_s, S, lmax, lane);
      // the warp's maximum per head: the rows sit in lane bits 3-4 and (row group) bit 0
#pragma unroll
      for (int j = 0; j < NV; ++j) {
        float mx = lmax[j];
        if (kRG == 2) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
        const int idx = idx0 + j;
        if (lane < 8 && l8 < V && idx / GQM == 0) s_wmax[warp][idx % GQM] = mx;
      }
      consumer_barrier();
      // ---- exact softmax statistics of the chunk; S becomes the weights ----
      float resc[GQM];
      float m_t = 0.f;
#pragma unroll
      for (int g = 0; g < GQM; ++g) {
        float mc = s_wmax[0][g];
#pragma unroll
        for (int w = 1; w < kCW; ++w) mc = fmaxf(mc, s_wmax[w][g]);
        const float m_new = fmaxf(m_run[g], mc);      // finite for every real head: the chunk has a row
        resc[g] = expf(m_run[g] - m_new);              // exp(-inf) = 0 for the first chunk
        m_run[g] = m_new;
        if (g == g_t) m_t = m_new;
      }
      const int n_s = (crn + (new_here ? 1 : 0)) * GQM;
      float ls = 0.f;
      for (int i = tid; i < n_s; i += kCT) {
        const float e = expf(S[i] - m_t);
        S[i] = e;
        ls += e;
      }
#pragma unroll
      for (int o = GQM; o < 32; o <<= 1) ls += __shfl_xor_sync(0xffffffffu, ls, o);
      if (lane < GQM) s_wsum[warp][lane] = ls;
      consumer_barrier();
#pragma unroll
      for (int g = 0; g < GQM; ++g) {
        float t = s_wsum[0][g];
#pragma unroll
        for (int w = 1; w < kCW; ++w) t += s_wsum[w][g];
        l_run[g] = l_run[g] * resc[g] + t;
        if (c > 0) { acc[g].x *= resc[g]; acc[g].y *= resc[g]; acc[g].z *= resc[g]; acc[g].w *= resc[g]; }
      }
      // ---- V stages: weighted sum ----
#pragma unroll 1
      for (int t = 0; t < nt; ++t, ++it) {
        const int s = it % p.stages;
        const bool ok = mbar_wait(&full[s], (uint32_t)(it / p.stages) & 1u, &s_abort);
        const int nr = min(kWR, crn - t * kStageRows - warp * kWR);
        if (ok && nr > 0)
          weigh_rows<D, GQM>(region + (size_t)s * stage_floats + (size_t)warp * kWR * D, nr,
                             t * kStageRows + warp * kWR, S, acc, lane);
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);
      }
      if (new_here && warp == 0) weigh_rows<D, GQM>(kv_new + D, 1, crn, S, acc, lane);
    }

    // ---- this CTA's partial: the warps' weighted V summed, with the share's max and sum ----
    consumer_barrier();  // every warp is done with the ring
    if (tid == 0) tl_mark(p.tl, cta_lin, 4);
    float* w_acc = region;
#pragma unroll
    for (int g = 0; g < GQM; ++g) {
      if (g < gq) {
#pragma unroll
        for (int o = CPR; o < 32; o <<= 1) {  // lanes that share a column (head_dim < 128)
          acc[g].x += __shfl_xor_sync(0xffffffffu, acc[g].x, o);
          acc[g].y += __shfl_xor_sync(0xffffffffu, acc[g].y, o);
          acc[g].z += __shfl_xor_sync(0xffffffffu, acc[g].z, o);
          acc[g].w += __shfl_xor_sync(0xffffffffu, acc[g].w, o);
        }
        if (lane < CPR) reinterpret_cast<float4*>(w_acc + ((size_t)warp * gq + g) * D)[lane] = acc[g];
        if (tid == 0) { s_ml[0][g] = m_run[g]; s_ml[1][g] = l_run[g]; }
      }
    }
    consumer_barrier();
    for (int i = tid; i < gq * D; i += kCT) {
      const int g = i / D, e = i - g * D;
      float o = 0.f;
#pragma unroll
      for (int w = 0; w < kCW; ++w) o += w_acc[((size_t)w * gq + g) * D + e];
      const int h = kvh * gq + g;
      p.part_o[(((int64_t)b * p.num_heads + h) * p.nc + split) * D + e] = o;
      if (e == 0) {
        float* dst = p.part_ml + (((int64_t)b * p.num_heads + h) * p.nc + split) * 2;
        dst[0] = s_ml[0][g];
        dst[1] = s_ml[1][g];
      }
    }
  }

  // ---- ticket: the last CTA of this (sequence, kv head) merges the partials ----
  __threadfence();
  consumer_barrier();
  if (tid == 0) {
    if (s_abort) atomicExch(&g_attn_fault, 1);
    const int ticket = atomicAdd(&p.counters[b * p.num_kv_heads + kvh], 1);
    s_last = (ticket == (int)gridDim.x - 1);
  }
  consumer_barrier();
  if (tid == 0 && !s_last) tl_mark(p.tl, cta_lin, 5);
  if (!s_last) return;
  __threadfence();
  if (tid == 0) p.counters[b * p.num_kv_heads + kvh] = 0;  // ready for the next launch
  if (tid == 0) tl_mark(p.tl, cta_lin, 6);

  const int h0 = kvh * gq;
  if (nvalid == 0) {
    for (int i = tid; i < gq * D; i += kCT) p.out[((int64_t)b * p.num_heads + h0) * D + i] = 0.f;
    return;
  }
  // Layout of the region now: wts [gq][nc] | ml [gq] | tile [gq][cc][D], cc partials at a time.
  float* wts = region;
  float* ml = wts + up4((size_t)gq * p.nc);
  float* tile = ml + up4(gq);
  const int cc = (int)min((int64_t)nvalid, (int64_t)(p.region_floats - (tile - region)) / ((int64_t)gq * D));
  const float* po = p.part_o + ((int64_t)b * p.num_heads + h0) * p.nc * D;
  // Request the first tile of partials (asynchronous copies, no registers held) before the
  // weights are worked out, so that both trips to L2 overlap.
  auto request_tile = [&](int c0, int n) {
    for (int i = tid; i < gq * n * CPR; i += kCT) {
      const int g = i / (n * CPR), r = i - g * (n * CPR);  // r = chunk-in-tile * CPR + column
      const float* src = po + ((int64_t)g * p.nc + c0) * D + (int64_t)r * 4;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(tile + ((size_t)g * cc) * D + (size_t)r * 4)),
                   "l"(src)
                   : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  // The (max, sum) pairs are requested first - they gate the weights - then the tile.
  float2 mlv[2][2];
#pragma unroll
  for (int hs = 0; hs < 2; ++hs)
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int g = warp + hs * kCW, c = lane + 32 * k;
      mlv[hs][k] = (g < gq && c < nvalid)
                       ? __ldcg(reinterpret_cast<const float2*>(p.part_ml + (((int64_t)b * p.num_heads + h0 + g) * p.nc + c) * 2))
                       : make_float2(-INFINITY, 0.f);
    }
  request_tile(0, min(cc, nvalid));
  // weights of every partial: one warp per q head
#pragma unroll
  for (int hs = 0; hs < 2; ++hs) {
    const int g = warp + hs * kCW;
    if (g >= gq) continue;
    const float* pml = p.part_ml + ((int64_t)b * p.num_heads + h0 + g) * p.nc * 2;
    float mx = fmaxf(mlv[hs][0].x, mlv[hs][1].x);
    for (int c = lane + 64; c < nvalid; c += 32) mx = fmaxf(mx, __ldcg(pml + c * 2));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float tot = 0.f;
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int c = lane + 32 * k;
      if (c < nvalid) {
        const float w = expf(mlv[hs][k].x - mx);
        wts[g * p.nc + c] = w;
        tot = fmaf(mlv[hs][k].y, w, tot);
      }
    }
    for (int c = lane + 64; c < nvalid; c += 32) {
      const float w = expf(__ldcg(pml + c * 2) - mx);
      wts[g * p.nc + c] = w;
      tot = fmaf(__ldcg(pml + c * 2 + 1), w, tot);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
    if (lane == 0) ml[g] = 1.0f / fmaxf(tot, 1e-30f);  // src/llm/decoder.rs:1203
  }
  // Each thread owns float4 outputs o = tid, tid + kCT, ... of the gq * CPR in this kv head.
  constexpr int OPT = (GQM * CPR + kCT - 1) / kCT;
  float4 acc[OPT];
#pragma unroll
  for (int k = 0; k < OPT; ++k) acc[k] = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int c0 = 0; c0 < nvalid; c0 += cc) {
    const int n = min(cc, nvalid - c0);
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    consumer_barrier();  // the tile and (first time) the weights are in shared memory
    if (tid == 0) tl_mark(p.tl, cta_lin, 7);
#pragma unroll
    for (int k = 0; k < OPT; ++k) {
      const int o = tid + k * kCT;
      if (o < gq * CPR) {
        const int g = o / CPR, col = o - g * CPR;
        const float4* t4 = reinterpret_cast<const float4*>(tile + ((size_t)g * cc) * D) + col;
        const float* w = wts + g * p.nc + c0;
        for (int c = 0; c < n; ++c) {
          const float4 v = t4[c * CPR];
          const float wc = w[c];
          acc[k].x = fmaf(wc, v.x, acc[k].x);
          acc[k].y = fmaf(wc, v.y, acc[k].y);
          acc[k].z = fmaf(wc, v.z, acc[k].z);
          acc[k].w = fmaf(wc, v.w, acc[k].w);
        }
      }
    }
    if (c0 + cc < nvalid) {
      consumer_barrier();  // everybody is done with the tile before it is overwritten
      request_tile(c0 + cc, min(cc, nvalid - c0 - cc));
    }
  }
#pragma unroll
  for (int k = 0; k < OPT; ++k) {
    const int o = tid + k * kCT;
    if (o < gq * CPR) {
      const int g = o / CPR, col = o - g * CPR;
      const float r = ml[g];
      reinterpret_cast<float4*>(p.out + ((int64_t)b * p.num_heads + h0 + g) * D)[col] =
          make_float4(acc[k].x * r, acc[k].y * r, acc[k].z * r, acc[k].w * r);
    }
  }
  if (tid == 0) tl_mark(p.tl, cta_lin, 5);
}

int g_chunk_override = 0;
int g_ctas_per_sm = 0;   // 0 = automatic (2)
int g_ring_stages = 0;   // 0 = automatic

struct AttnLayout {
  int fixed_per;  // 0 = divide the current length evenly among the nc CTAs
  int nc;         // CTAs per (sequence, kv head)
  int stages;
  size_t part_o, part_ml;
};

// Upper bound of CTAs per (sequence, kv head) that the scratch block is sized for.
int max_splits(int64_t max_seq_len) {
  const int64_t cap = max_seq_len < kSeqCap ? max_seq_len : kSeqCap;
  return (int)((cap + 31) / 32);
}

AttnLayout attn_layout(int batch, int num_heads, int num_kv_heads, int head_dim, int64_t max_seq_len) {
  AttnLayout L;
  const int64_t cap = max_seq_len < kSeqCap ? max_seq_len : kSeqCap;
  const int64_t cols = (int64_t)batch * num_kv_heads;
  // Ring depth: 96 KB of stages for head_dim 128 (two CTAs per SM), fewer bytes for narrower heads.
  const int cps = g_ctas_per_sm > 0 ? g_ctas_per_sm : 2;
  L.stages = head_dim == 128 ? 6 : 8;
  if (cps == 1 && L.stages < 8) L.stages = 8;
  if (g_ring_stages > 0) L.stages = g_ring_stages;
  if (L.stages > kMaxStages) L.stages = kMaxStages;
  if (g_chunk_override > 0) {
    L.fixed_per = g_chunk_override;
    L.nc = (int)((cap + L.fixed_per - 1) / L.fixed_per);
  } else {
    // two resident CTAs per SM, all of them busy whatever the current length
    L.fixed_per = 0;
    int64_t nc = ((int64_t)cps * sm_count()) / cols;
    const int64_t most = (cap + kStageRows - 1) / kStageRows;
    if (nc > most) nc = most;
    if (nc < 1) nc = 1;
    L.nc = (int)nc;
  }
  auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
  L.part_o = up((size_t)batch * num_heads * L.nc * head_dim * sizeof(float));
  L.part_ml = up((size_t)batch * num_heads * L.nc * 2 * sizeof(float));
  return L;
}

}  // namespace

void set_attention_chunk_override(int tc) { g_chunk_override = tc; }
void set_attention_tuning(int ctas_per_sm, int stages) {
  g_ctas_per_sm = ctas_per_sm;
  g_ring_stages = stages;
}

int attention_fault_flag() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_attn_fault, sizeof(int)) != cudaSuccess) return -1;
  return v;
}

// Scratch = ticket counters + partials.  The counters must be zero before the first launch; every
// launch leaves them zero again.  They sit at the START of the block, in a region of fixed size: their
// place must not depend on the batch of a launch, or the partials of a launch with many rows would land
// on the counters that a later launch with fewer rows expects to be zero.
size_t attention_scratch_bytes(int batch, int num_heads, int num_kv_heads, int head_dim,
                               int64_t max_seq_len) {
  // sized for the largest number of CTAs per (sequence, kv head) any setting can ask for
  const int nc = max_splits(max_seq_len);
  auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
  return kCounterBytes + up((size_t)batch * num_heads * nc * head_dim * sizeof(float)) +
         up((size_t)batch * num_heads * nc * 2 * sizeof(float));
}

size_t attention_counters_offset(int batch, int num_heads, int num_kv_heads, int head_dim,
                                 int64_t max_seq_len, size_t* counter_bytes) {
  (void)batch; (void)num_heads; (void)num_kv_heads; (void)head_dim; (void)max_seq_len;
  if (counter_bytes) *counter_bytes = kCounterBytes;
  return 0;
}

template <int D, int GQM>
static tb_status launch_attn(const AttnParams& p, const cudaLaunchConfig_t& cfg) {
  if (cfg.dynamicSmemBytes > 32 * 1024)
    TB_CUDA_TRY(cudaFuncSetAttribute(attn_decode_kernel<D, GQM>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)cfg.dynamicSmemBytes));
  TB_CUDA_TRY(cudaLaunchKernelEx(&cfg, attn_decode_kernel<D, GQM>, p));
  return TB_OK;
}

template <int D>
static tb_status launch_attn_d(const AttnParams& p, const cudaLaunchConfig_t& cfg, int gqm) {
  switch (gqm) {
    case 1: return launch_attn<D, 1>(p, cfg);
    case 2: return launch_attn<D, 2>(p, cfg);
    case 4: return launch_attn<D, 4>(p, cfg);
    default: return launch_attn<D, 8>(p, cfg);
  }
}

// Several positions of ONE sequence in a batch (speculative verify): row r of qkv is position offsets[r]
// of sequence 0.  Its k (rotated) and v are appended to sequence 0's cache here, for all rows, BEFORE the
// attention launch, which then only reads the cache (row r attends to [0, offsets[r]], so it also reads
// the rows of its predecessors in the batch).  grid (rows, kv heads), head_dim threads.
__global__ void rope_append_rows_kernel(const float* __restrict__ qkv, float* __restrict__ k_cache, float* __restrict__ v_cache,
                                        const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                        const int32_t* __restrict__ offsets, int num_heads, int num_kv_heads, int D,
                                        int64_t max_seq_len) {
  const int b = blockIdx.x, kvh = blockIdx.y, e = threadIdx.x;
  const int off = offsets[b];
  if (off < 0 || (int64_t)off >= max_seq_len || off >= kSeqCap) return;   // the attention kernel writes zeros for such a row
  const int64_t qkv_dim = (int64_t)(num_heads + 2 * num_kv_heads) * D;
  const float* kx = qkv + (int64_t)b * qkv_dim + (int64_t)num_heads * D + (int64_t)kvh * D;
  const float* vx = kx + (int64_t)num_kv_heads * D;
  const float* cs = cos_t + (int64_t)off * D;
  const float* sn = sin_t + (int64_t)off * D;
  const int64_t at = ((int64_t)kvh * max_seq_len + off) * D + e;
  k_cache[at] = rope_elem(kx, cs, sn, e, D / 2);
  v_cache[at] = vx[e];
}

tb_status launch_rope_append_rows(const AttnArgs& a, cudaStream_t stream) {
  if (!a.qkv || !a.k_cache || !a.v_cache || !a.cos_t || !a.sin_t || !a.offsets || a.per_call_tables)
    return fail(TB_ERR_ARG, "rope_append_rows: null operand or per-call tables");
  rope_append_rows_kernel<<<dim3((unsigned)a.batch, (unsigned)a.num_kv_heads), a.head_dim, 0, stream>>>(
      a.qkv, a.k_cache, a.v_cache, a.cos_t, a.sin_t, a.offsets, a.num_heads, a.num_kv_heads, a.head_dim, a.max_seq_len);
  TB_CUDA_TRY(cudaGetLastError());
  return TB_OK;
}

tb_status launch_attention_decode(const AttnArgs& a, cudaStream_t stream) {
  if (!a.qkv || !a.k_cache || !a.v_cache || !a.cos_t || !a.sin_t || !a.offsets || !a.out || !a.scratch)
    return fail(TB_ERR_ARG, "attention: null operand");
  if (a.num_kv_heads <= 0 || a.num_heads % a.num_kv_heads != 0)
    return fail(TB_ERR_ARG, "num_heads (%d) must be divisible by num_kv_heads (%d) for GQA", a.num_heads, a.num_kv_heads);
  const int gq = a.num_heads / a.num_kv_heads;
  if (gq > kMaxGq) return fail(TB_ERR_UNSUPPORTED, "TB_UNSUPPORTED: %d q heads per kv head (max %d)", gq, kMaxGq);
  if (a.head_dim != 32 && a.head_dim != 64 && a.head_dim != 128)
    return fail(TB_ERR_UNSUPPORTED, "TB_UNSUPPORTED: head_dim %d (supported: 32, 64, 128)", a.head_dim);
  if (a.batch < 1 || a.max_seq_len < 1) return fail(TB_ERR_SHAPE, "attention: empty shape");
  if (a.max_seq_len > kSeqCap)  // beyond it a new row would neither be appended nor attended to
    return fail(TB_ERR_UNSUPPORTED, "TB_UNSUPPORTED: max_seq_len %lld (attention covers at most %d positions)", (long long)a.max_seq_len, kSeqCap);
  if ((reinterpret_cast<uintptr_t>(a.k_cache) | reinterpret_cast<uintptr_t>(a.v_cache)) & 15)
    return fail(TB_ERR_ARG, "attention: the KV caches must be 16-byte aligned");

  AttnLayout L = attn_layout(a.batch, a.num_heads, a.num_kv_heads, a.head_dim, a.max_seq_len);
  if (L.fixed_per && (L.fixed_per < 64 || L.fixed_per > 512 || (L.fixed_per & (L.fixed_per - 1))))
    return fail(TB_ERR_ARG, "attention: chunk %d is not a power of two in [64, 512]", L.fixed_per);
  if (L.nc > max_splits(a.max_seq_len)) return fail(TB_ERR_SHAPE, "attention: %d splits exceed the scratch layout", L.nc);
  size_t cbytes = 0;
  const size_t coff = attention_counters_offset(a.batch, a.num_heads, a.num_kv_heads, a.head_dim, a.max_seq_len, &cbytes);
  const int gqm = gq <= 1 ? 1 : (gq <= 2 ? 2 : (gq <= 4 ? 4 : 8));
  const int D = a.head_dim;
  AttnParams p;
  p.qkv = a.qkv; p.k_cache = a.k_cache; p.v_cache = a.v_cache;
  p.cos_t = a.cos_t; p.sin_t = a.sin_t; p.offsets = a.offsets; p.out = a.out;
  char* base = static_cast<char*>(a.scratch);
  if (((size_t)a.batch * a.num_kv_heads + 1) * sizeof(int) > cbytes)
    return fail(TB_ERR_UNSUPPORTED, "TB_UNSUPPORTED: attention: %d x %d (sequence, kv head) pairs exceed the ticket block", a.batch, a.num_kv_heads);
  p.counters = reinterpret_cast<int*>(base + coff);
  p.part_o = reinterpret_cast<float*>(base + coff + cbytes);
  p.part_ml = reinterpret_cast<float*>(base + coff + cbytes + L.part_o);
  p.qkv_rot_out = a.q_rot_out;
  p.num_heads = a.num_heads; p.num_kv_heads = a.num_kv_heads; p.gq = gq;
  p.fixed_per = L.fixed_per; p.nc = L.nc; p.stages = L.stages;
  p.max_parts = 48;
  // two CTAs per SM when the ring can be cut to make room (wide heads with many q heads per kv head)
  int stages = L.stages;
  while (stages > 3 && 2 * (sizeof(float) * (attn_fixed_floats(D, gq, gqm) + attn_region_floats(D, gq, L.nc, stages)) + 2048) > 227 * 1024)
    --stages;
  p.stages = stages;
  const size_t region = attn_region_floats(D, gq, L.nc, stages);
  p.region_floats = (int)region;
  p.max_seq_len = a.max_seq_len;
  p.per_call_tables = a.per_call_tables ? 1 : 0;
  p.shared_cache = a.shared_cache ? 1 : 0;
  p.scale = 1.0f / sqrtf((float)a.head_dim);
  p.tl = timeline_next_block();

  const size_t smem = sizeof(float) * (attn_fixed_floats(D, gq, gqm) + region);
  if (smem > 200 * 1024) return fail(TB_ERR_UNSUPPORTED, "TB_UNSUPPORTED: attention needs %zu bytes of shared memory", smem);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)L.nc, (unsigned)a.num_kv_heads, (unsigned)a.batch);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (a.pdl) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  if (D == 128) return launch_attn_d<128>(p, cfg, gqm);
  if (D == 64) return launch_attn_d<64>(p, cfg, gqm);
  return launch_attn_d<32>(p, cfg, gqm);
}

// ---------------------------------------------------------------------------
// Attention without any allocation.  The partials and ticket counters of the kernel above
// normally live in scratch memory that the caller allocates.  Some callers cannot allocate:
// a serving process whose device memory was carved up completely at start-up, code that runs
// while another thread is capturing a CUDA graph (an allocation there breaks the capture), or a
// latency-critical loop in which a cudaMalloc would stall every stream of the device.  For
// them the same kernel runs on a fixed block of device memory that is part of this library's
// image: every GPU that loads the library holds these 8 MiB until the process exits.
// ---------------------------------------------------------------------------
constexpr size_t kStaticScratchBytes = 8u << 20;
static __device__ __align__(256) unsigned char g_static_attn_scratch[kStaticScratchBytes];

size_t static_attention_scratch_capacity() { return kStaticScratchBytes; }

// In host code the array's name is only a handle for the runtime, not an address a kernel
// could use; the device address is looked up once per device, with that device current.
tb_status static_attention_scratch(void** ptr) {
  static std::atomic<void*> cached[64];   // several host threads may make their first call at once
  int dev = 0;
  TB_CUDA_TRY(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64) {
    void* c = cached[dev].load(std::memory_order_relaxed);
    if (c) {
      *ptr = c;
      return TB_OK;
    }
  }
  void* p = nullptr;
  cudaError_t e = cudaGetSymbolAddress(&p, g_static_attn_scratch);
  if (e != cudaSuccess || p == nullptr)
    return fail(TB_ERR_CUDA, "cudaGetSymbolAddress(static attention scratch) failed: %s", cudaGetErrorString(e));
  if (dev >= 0 && dev < 64) cached[dev].store(p, std::memory_order_relaxed);
  *ptr = p;
  return TB_OK;
}

}  // namespace tb
