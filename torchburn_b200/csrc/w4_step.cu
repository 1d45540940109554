// One decode step (batch 1) as ONE persistent cooperative kernel.
//
// The reference records the whole token into one command stream (src/wgpu/decode.rs:239-289)
// and runs the layer as one fused routine on the CPU (step_internal, src/llm/decoder.rs:1051-1374;
// fused_transformer_layer_step_w4a32, src/quantization/fused_transformer.rs:16-376).  On B200 a
// chain of 160 dependent launches loses more time between the kernels (launch gap, refill of a
// cold pipeline, activation broadcast) than inside them.  Here one CTA per SM stays alive for the
// whole step and walks a list of phases:
//
//   per layer   QKV projection -> attention over this layer's cache -> merge of the split-K
//               partials -> O projection + residual -> gate/up + SwiGLU -> down + residual
//   at the end  lm_head
//
//  * A producer warp streams the CTA's share of every phase through ONE ring of shared-memory
//    stages (cp.async.bulk, mbarrier completion).  Weights and the cache rows of earlier steps do
//    not depend on this step's activations, so the producer runs ahead of the consumers across
//    phase boundaries: while the grid waits at a barrier and re-loads the activations, the ring
//    already holds the first ~160 KB per SM of the next phase and HBM never goes idle.
//  * Phases are separated by a grid-wide barrier (one atomic per CTA, acquire polling).  Every
//    wait in the kernel - mbarriers and the grid barrier - is bounded; when one runs out the
//    kernel raises a fault word, every later wait returns at once and the kernel ends.
//  * Projections keep the arithmetic of the single-launch kernels: a lane owns 32 consecutive
//    elements of K as integer digits in registers (w4_math.cuh), rows are reduced with a
//    transposing butterfly, RMSNorm is split (producers write x * w_norm and sums of squares,
//    consumers divide the finished row sums by the rms).
//  * Attention: the positions [0, offset] of each kv head are divided evenly among grid/Hkv CTAs;
//    K tiles then V tiles of 32 rows go through the same ring; a warp scores 8 rows for 2 q heads
//    (q in registers), exact softmax inside chunks of 512 positions, partials (max, sum,
//    weighted V) to scratch; the merge phase turns them into the attention output.
//
// HBM-bound: algorithmic bytes per step = all weights + scales + the KV rows read.
#include "tb_common.cuh"
#include "w4_math.cuh"

namespace tb {

namespace {

constexpr int kCW = 15;                   // consumer warps (with the producer warp: 4 warps per SM sub-partition)
constexpr int kCT = kCW * 32;             // consumer threads
constexpr int kThreads = kCT + 32;        // + the producer warp
constexpr int kStages = 8;                // ring depth
constexpr int kStageBytes = 20480;        // one stage
constexpr int kMaxK = 14336;              // activations staged per phase (also the attention work area)
constexpr int kXBufBytes = kMaxK * 4;
constexpr int kPartFloats = 2 * 2 * kCW * 33;   // [buffer][matrix][warp][row]
constexpr int kSmemBytes = kStages * kStageBytes + kXBufBytes + kPartFloats * 4;   // + kBarBytes of barriers
constexpr int kBarBytes = 2 * kStages * 8 + 16;
#ifndef TB_STEP_BATCH
#define TB_STEP_BATCH 8
#endif
constexpr int kBatch = TB_STEP_BATCH;     // rows of a round whose loads a lane issues before the products
constexpr int kAttnRows = 32;             // K (or V) rows per ring stage
constexpr int kChunkRows = 512;           // positions whose scores are held in shared memory at a time
constexpr int kMaxSplits = 64;            // partials per head the merge reads with two loads per lane
constexpr int kSeqCap = 32768;            // src/llm/decoder.rs:1180
constexpr long long kWaitCyclesDefault = 4000000000ll;  // ~2 s

__device__ int g_step_fault = 0;

struct StepParams {
  const StepPhase* phases;
  int nphases;
  unsigned* sync;
  int* host_fault;
  const float* qkv;
  float* attn;
  const float* cos_t;
  const float* sin_t;
  const int32_t* offsets;
  float* part_o;
  float* part_ml;
  int num_heads, num_kv_heads, gq, parts, nc;
  long long max_seq_len;
  float scale;
  long long wait_cycles;
  int debug;                // test hook: bit 0 = consume the stages without multiplying
  // tensor parallel (tp_size 1: none of it is used)
  int tp_rank, tp_size, tp_hidden, n_exchanges;
  uint2* tp_recv[8];
  float* tp_logits[8];
  uint32_t* tp_flags[8];
  uint32_t* tp_epoch;
  uint32_t epoch_base;      // copy of *tp_epoch taken when the kernel starts (in the shared copy of the parameters)
  unsigned long long* tl;   // optional timestamps (step_mark)
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
// Bounded wait.  Returns false once the limit ran out here or anywhere else in the CTA (s_abort)
// or in the grid (g_step_fault): after the first failure nobody waits any more.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* s_abort, long long limit) {
  const uint32_t addr = smem_u32(bar);
  long long t0 = 0;
  for (uint32_t i = 0;; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(addr), "r"(parity)
        : "memory");
    if (ok) return true;
    if ((i & 127) == 127) {
      if (*s_abort) return false;
      if (t0 == 0) t0 = clock64();
      else if (clock64() - t0 > limit || *reinterpret_cast<volatile int*>(&g_step_fault)) {
        *s_abort = 1;
        atomicExch(&g_step_fault, 1);
        return false;
      }
    }
  }
}

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kCT) : "memory"); }
__device__ __forceinline__ void group_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// All consumer threads of all CTAs.  Writes made before it by any consumer thread of the grid are
// visible after it to every consumer thread (bar.sync orders the CTA's threads before thread 0's
// release; thread 0's acquire is ordered before the CTA's threads by the second bar.sync).
// The arrivals are spread over four counters (CTA number mod 4) so that they do not queue on one
// address; a waiter reads all four with one 16-byte load.  `round` counts the barriers so far.
__device__ __forceinline__ void grid_barrier(unsigned* counters, unsigned round, volatile int* s_abort, long long limit,
                                             int tid) {
  consumer_sync();
  if (tid == 0) {
    // release: the CTA's writes (ordered before this by the bar.sync) become visible before the count
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(counters + (blockIdx.x & 3)) : "memory");
    if (!*s_abort) {
      const unsigned g = gridDim.x;
      const unsigned t0c = round * ((g + 3) >> 2), t1c = round * ((g + 2) >> 2), t2c = round * ((g + 1) >> 2), t3c = round * (g >> 2);
      long long t0 = 0;
      for (uint32_t i = 0;; ++i) {
        unsigned c0, c1, c2, c3;
        asm volatile("ld.relaxed.gpu.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(c0), "=r"(c1), "=r"(c2), "=r"(c3) : "l"(counters) : "memory");
        if (c0 >= t0c && c1 >= t1c && c2 >= t2c && c3 >= t3c) break;
        if ((i & 31) == 31) {
          if (t0 == 0) t0 = clock64();
          else if (clock64() - t0 > limit || *reinterpret_cast<volatile int*>(&g_step_fault)) {
            *s_abort = 1;
            atomicExch(&g_step_fault, 1);
            break;
          }
        }
      }
    }
    __threadfence();
  }
  consumer_sync();
}

// Optional timestamps of one CTA (the first one): for phase ph, slot 0 = start, 1 = activations
// ready, 2 = end of the phase's work (the barrier wait is the gap to the next start).
__device__ __forceinline__ void step_mark(const StepParams& p, int ph, int slot, int tid) {
  if (p.tl != nullptr && blockIdx.x == 0 && tid == 0) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    p.tl[ph * 4 + slot] = t;
  }
}

// Sum over the 32 lanes of 8 values: three transposing steps leave one row per lane
// (row = lane >> 2), two plain steps finish the sum over the four lanes that share it.
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

// sum_i q_i * (nibble_i - 8) for one 32-element block as (hi, lo): value = 65536 * hi + lo.
// The -8 offset is taken in the integer domain (s8hi = 8 * (S >> 16), s8lo = 8 * (S & 0xFFFF) with
// S = sum_i q_i), so no large terms cancel in floating point.
__device__ __forceinline__ float idot_block(const uint4 wv, const uint32_t (&xq)[24], int s8hi, int s8lo) {
  const uint32_t w[4] = {wv.x, wv.y, wv.z, wv.w};
  // the accumulators start at the offset term; d0 and d1 wrap modulo 2^32, their combination is exact
  uint32_t d0 = (uint32_t)(-s8lo), d1 = 0;
  int d2 = -s8hi;
#pragma unroll
  for (int wd = 0; wd < 4; ++wd) {
    const uint32_t t = w[wd] & 0x0F0F0F0Fu;
    const uint32_t u = (w[wd] >> 4) & 0x0F0F0F0Fu;
    d0 = dp4a_uu(t, xq[wd * 6 + 0], d0);
    d1 = dp4a_uu(t, xq[wd * 6 + 1], d1);
    d2 = dp4a_us(t, xq[wd * 6 + 2], d2);
    d0 = dp4a_uu(u, xq[wd * 6 + 3], d0);
    d1 = dp4a_uu(u, xq[wd * 6 + 4], d1);
    d2 = dp4a_us(u, xq[wd * 6 + 5], d2);
  }
  const int lo = (int)(d0 + (d1 << 8));   // |lo| < 2^26
  return fmaf(65536.0f, (float)d2, (float)lo);
}

// Balanced, contiguous share of `rounds` 8-row rounds for CTA `cta` of `grid`; the CTAs that take
// one round more rotate with `rot` from phase to phase, so the bytes per CTA even out over a layer.
__device__ __forceinline__ void round_share(int rounds, int grid, int cta, int rot, int& round0, int& my_rounds) {
  int idx = cta - rot;
  if (idx < 0) idx += grid;
  const int base = rounds / grid, rem = rounds - base * grid;
  my_rounds = base + (idx < rem ? 1 : 0);
  round0 = idx * base + min(idx, rem);
}

// The positions one CTA takes in an attention phase.
struct AttnPlan {
  int kvh, split, t0, rows, ring_rows, nchunks, nvalid, off;
  bool active, has_new;
};
__device__ __forceinline__ AttnPlan attn_plan(const StepParams& p, int cta) {
  AttnPlan a;
  a.off = p.offsets[0];
  const bool seq_ok = a.off >= 0 && (long long)a.off < p.max_seq_len;
  const int t_end = seq_ok ? min(a.off + 1, kSeqCap) : 0;
  int per = (t_end + p.nc - 1) / p.nc;
  per = max(8, (per + 7) & ~7);
  a.nvalid = (t_end + per - 1) / per;
  a.kvh = cta / p.nc;
  a.split = cta - a.kvh * p.nc;
  a.t0 = a.split * per;
  a.active = a.kvh < p.num_kv_heads && a.t0 < t_end;
  a.rows = a.active ? min(per, t_end - a.t0) : 0;
  a.has_new = a.active && a.off >= a.t0 && a.off < a.t0 + a.rows;
  a.ring_rows = a.rows - (a.has_new ? 1 : 0);
  a.nchunks = a.active ? max(1, (a.ring_rows + kChunkRows - 1) / kChunkRows) : 0;
  return a;
}

// ------------------------------------------------------------------------------------------
// Producer: one lane walks the same phase list and feeds the ring.
// ------------------------------------------------------------------------------------------
template <int D>
__device__ __forceinline__ void producer_loop(const StepParams& p, unsigned char* ring, uint64_t* full, uint64_t* empty,
                                              volatile int* s_abort, const int lane) {
  // Lane s of the producer warp owns ring slot s: it requests every stage that lands there
  // (global stage numbers s, s + 8, ...).  Eight lanes work out addresses and wait for their
  // slots side by side, so one slow slot does not hold back the requests for the others.
  if (lane >= kStages) return;
  const int cta = (int)blockIdx.x, grid = (int)gridDim.x;
  const long long wait_limit = p.wait_cycles;
  const int nphases = p.nphases;
  const StepPhase* phases = p.phases;
  unsigned char* dst = ring + (size_t)lane * kStageBytes;
  uint64_t* my_full = &full[lane];
  uint64_t* my_empty = &empty[lane];
  uint32_t base = 0;    // global number of the first stage of the current phase (or chunk pass)
  uint32_t uses = 0;    // stages this lane has requested so far
  auto acquire = [&]() -> bool {  // the slot is free again
    const bool ok = uses == 0 ? !*s_abort : mbar_wait(my_empty, (uses - 1u) & 1u, s_abort, wait_limit);
    ++uses;
    return ok;
  };
  for (int ph = 0; ph < nphases; ++ph) {
    const StepPhase* d = phases + ph;
    const int kind = __ldg(&d->kind);
    if (kind == 0) {
      const int n = __ldg(&d->n), k = __ldg(&d->k), ng = __ldg(&d->ng), rs = __ldg(&d->rs), nw = __ldg(&d->nw);
      const int row_bytes = k >> 1, srow_bytes = ng * 4;
      const uint8_t* w0 = d->w[0];
      const uint8_t* w1 = d->w[1];
      const float* s0 = d->sc[0];
      const float* s1 = d->sc[1];
      int round0, my_rounds;
      round_share((n + 7) >> 3, grid, cta, __ldg(&d->rot), round0, my_rounds);
      const int rs_shift = rs == 8 ? 3 : (rs == 4 ? 2 : 1);
      const int nst = (my_rounds * 8) >> rs_shift;
      for (int i = (int)((lane - base) & (kStages - 1)); i < nst; i += kStages) {
        if (!acquire()) return;
        const int row0 = round0 * 8 + i * rs;
        const int cnt = max(0, min(rs, n - row0));
        if (cnt == 0) {  // nothing to fetch: complete the phase of the barrier by hand
          mbar_arrive(my_full);
          continue;
        }
        const uint32_t wb = (uint32_t)cnt * row_bytes, sb = (uint32_t)cnt * srow_bytes;
        mbar_expect_tx(my_full, nw * (wb + sb));
        bulk_g2s(dst, w0 + (int64_t)row0 * row_bytes, wb, my_full);
        bulk_g2s(dst + (size_t)rs * row_bytes, s0 + (int64_t)row0 * ng, sb, my_full);
        if (nw == 2) {
          unsigned char* d2 = dst + (size_t)rs * (row_bytes + srow_bytes);
          bulk_g2s(d2, w1 + (int64_t)row0 * row_bytes, wb, my_full);
          bulk_g2s(d2 + (size_t)rs * row_bytes, s1 + (int64_t)row0 * ng, sb, my_full);
        }
      }
      base += (uint32_t)nst;
    } else if (kind == 1) {
      const AttnPlan a = attn_plan(p, cta);
      if (!a.active) continue;
      const float* kc = d->k_cache + (int64_t)a.kvh * p.max_seq_len * D;
      const float* vc = d->v_cache + (int64_t)a.kvh * p.max_seq_len * D;
      for (int c = 0; c < a.nchunks; ++c) {
        const int cr0 = c * kChunkRows;
        const int crn = min(kChunkRows, a.ring_rows - cr0);
        const int nt = (crn + kAttnRows - 1) / kAttnRows;
        // the chunk's K tiles, then its V tiles: 2 * nt stages
        for (int i = (int)((lane - base) & (kStages - 1)); i < 2 * nt; i += kStages) {
          if (!acquire()) return;
          const int pass = i >= nt ? 1 : 0, t = i - pass * nt;
          const float* src = (pass == 0 ? kc : vc) + (int64_t)(a.t0 + cr0 + t * kAttnRows) * D;
          const int nr = min(kAttnRows, crn - t * kAttnRows);
          const uint32_t bytes = (uint32_t)nr * D * sizeof(float);
          mbar_expect_tx(my_full, bytes);
          bulk_g2s(dst, src, bytes, my_full);
        }
        base += (uint32_t)(2 * nt);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------
// Projection phase (consumers).  out[j] = sum_g scales[j,g] * sum_{i in g} x[i] * code(w[j,i])
// (gemv_w4a32_grouped, src/quantization/gemv.rs:1514-1684; SwiGLU pair
// src/quantization/gemv/swiglu.rs:205-289; fast_rms_norm src/quantization/fused_ops.rs:1066-1117).
// ------------------------------------------------------------------------------------------
// Dynamic shared memory: ring | activations / attention work area | partial row sums | barriers.
// Every routine takes its pointers from the one extern array, so the compiler addresses it as
// shared memory (32-bit addresses, no generic loads).
struct Shared {
  unsigned char* ring;
  float* xbuf;
  float* part;
  uint64_t* full;
  uint64_t* empty;
  volatile int* s_abort;
};
__device__ __forceinline__ Shared shared_layout() {
  extern __shared__ __align__(128) unsigned char smem[];
  Shared sh;
  sh.ring = smem;
  sh.xbuf = reinterpret_cast<float*>(smem + kStages * kStageBytes);
  sh.part = reinterpret_cast<float*>(smem + kStages * kStageBytes + kXBufBytes);
  sh.full = reinterpret_cast<uint64_t*>(smem + kSmemBytes);
  sh.empty = sh.full + kStages;
  sh.s_abort = reinterpret_cast<volatile int*>(sh.empty + kStages);
  return sh;
}

// What a lane carries from the prologue of a projection phase into its rounds.
struct LaneX {
  uint32_t dig[24];   // digits of this lane's 32 activations
  float sx;           // their scale (0 for a lane without a block)
  int s8hi, s8lo;     // 8 * sum(q) split at bit 16: the -8 offset of the codes
  float inv_rms;      // 1 / rms of the un-weighted activations (1 when the phase has no norm)
};

// The rounds of one projection phase.  One code path for every stage shape: a round is 8 rows of
// each matrix, spread over 8 / rs consecutive stages; a lane takes them in batches of kBatch rows
// (loads first, then the products: that many independent rows in flight).
__device__ __forceinline__ uint32_t gemv_rounds(const StepPhase& d, const StepParams& p, uint32_t it,
                                                const int tid, const int ph, const LaneX& X) {
  const Shared sh = shared_layout();
  const int lane = tid & 31, warp = tid >> 5;
  const int K = d.k, nb = K >> 5;
  const int KW = (nb + 31) >> 5;          // warps that cover K, one 32-element block per lane
  const int RG = kCW / KW;                // groups of KW warps; a group takes every RG-th round
  const int kw = warp % KW, rg = warp / KW;
  const bool wactive = rg < RG;
  const int part = kw * 32 + lane;
  const bool has_part = wactive && part < nb;
  const int row_bytes = K >> 1, srow_bytes = d.ng * 4;
  const int n = d.n, NW = d.nw, RS = d.rs;
  const int SPR = 8 / RS;                 // stages per round (rs >= 2: at most 4)
  const int rs_shift = RS == 8 ? 3 : (RS == 4 ? 2 : 1);
  const int mat_bytes = RS * (row_bytes + srow_bytes);
  const long long wait_limit = p.wait_cycles;
  const float sx = X.sx, inv_rms = X.inv_rms;
  const int s8hi = X.s8hi, s8lo = X.s8lo;

  int round0, my_rounds;
  round_share((n + 7) >> 3, (int)gridDim.x, (int)blockIdx.x, d.rot, round0, my_rounds);
  const int my_g_rounds = wactive ? (my_rounds - rg + RG - 1) / RG : 0;   // rounds rd = rg, rg + RG, ...
  // byte offsets of this lane's 16 bytes of nibbles in a row and of its scale in a row of scales
  // (lanes past the end of K read block 0 and discard the product)
  const int pofs = has_part ? part * 16 : 0;
  const int sofs = RS * row_bytes + (has_part ? (part >> d.gshift) * 4 : 0);
  int gr = 0, buf = 0, next_mine = rg;
  float* s_part = sh.part;
#pragma unroll 1
  for (int rd = 0; rd < my_rounds; ++rd, it += (uint32_t)SPR) {
    const bool mine = wactive && rd == next_mine;
    float pre_b0 = 0.f, pre_b1 = 0.f, pre_res = 0.f, pre_sw = 0.f;
    if (mine && kw == 0 && ((gr & 3) == 3 || gr == my_g_rounds - 1)) {
      // this round ends with an epilogue: request its per-row operands now
      const int j = lane >> 3, r = lane & 7;
      const int row = (round0 + ((gr & ~3) + j) * RG + rg) * 8 + r;
      if (j <= (gr & 3) && row < n) {
        if (d.bias[0]) pre_b0 = __ldg(d.bias[0] + row);
        if (NW == 2 && d.bias[1]) pre_b1 = __ldg(d.bias[1] + row);
        if (NW == 1 && d.resid) pre_res = __ldcg(d.resid + row);
        if (d.out_scaled != nullptr) pre_sw = __ldg(d.out_scale_w + row);
      }
    }
    bool ok = true;
#pragma unroll 1
    for (int ss = 0; ss < SPR; ++ss) {
      const uint32_t is = it + (uint32_t)ss;
      ok = mbar_wait(&sh.full[is % kStages], (is / kStages) & 1u, sh.s_abort, wait_limit) && ok;
    }
    if (mine && !(p.debug & 1)) {
#pragma unroll 1
      for (int q = 0; q < NW; ++q) {
        float pa[8];
#pragma unroll
        for (int hb = 0; hb < 8 / kBatch; ++hb) {
          uint4 wv[kBatch];
          float sc[kBatch];
#pragma unroll
          for (int j = 0; j < kBatch; ++j) {
            const int row = hb * kBatch + j;                       // row of the round
            const uint32_t is = it + (uint32_t)(row >> rs_shift);
            const unsigned char* base = sh.ring + (size_t)(is % kStages) * kStageBytes + q * mat_bytes;
            const int r = row & (RS - 1);                     // row inside its stage
            wv[j] = *reinterpret_cast<const uint4*>(base + r * row_bytes + pofs);
            sc[j] = *reinterpret_cast<const float*>(base + r * srow_bytes + sofs);
          }
#pragma unroll
          for (int j = 0; j < kBatch; ++j) {
            const float val = (sc[j] * sx) * idot_block(wv[j], X.dig, s8hi, s8lo);
            pa[hb * kBatch + j] = (has_part && ok) ? val : 0.f;
          }
        }
        const float v = transpose_reduce8(pa, lane);
        if ((lane & 3) == 0) s_part[((buf * 2 + q) * kCW + warp) * 33 + (gr & 3) * 8 + (lane >> 2)] = v;
      }
    }
    __syncwarp();
    if (lane == 0) {
#pragma unroll 1
      for (int ss = 0; ss < SPR; ++ss) mbar_arrive(&sh.empty[(it + (uint32_t)ss) % kStages]);
    }
    if (!mine) continue;
    next_mine += RG;
    const int slot = gr & 3;
    ++gr;
    if (slot != 3 && gr != my_g_rounds) continue;
    // ---- up to 32 rows of this group gathered: sum over its warps, epilogue, store ----
    if (KW > 1) group_sync(2 + rg, KW * 32);
    else __syncwarp();
    if (kw == 0) {
      const int j = lane >> 3, r = lane & 7;
      const int row = (round0 + (((gr - 1) & ~3) + j) * RG + rg) * 8 + r;
      const bool valid = j <= slot && row < n;
      float v_out = 0.f;
      if (valid) {
        float a0 = 0.f, a1 = 0.f;
        for (int w = 0; w < KW; ++w) a0 += s_part[((buf * 2 + 0) * kCW + rg * KW + w) * 33 + lane];
        if (NW == 2)
          for (int w = 0; w < KW; ++w) a1 += s_part[((buf * 2 + 1) * kCW + rg * KW + w) * 33 + lane];
        float v;
        if (NW == 2) {
          const float g = a0 * inv_rms + pre_b0;
          const float u = a1 * inv_rms + pre_b1;
          v = (g / (1.0f + expf(-g))) * u;  // src/llm/decoder.rs:1319-1322
        } else {
          v = a0 * inv_rms + pre_b0;
          if (d.resid) v = pre_res + v;
        }
        if (d.tp_mode == 0) {
          d.out[row] = v;
          if (d.out_scaled != nullptr) d.out_scaled[row] = v * pre_sw;
        } else if (d.tp_mode == 1) {
          // this rank's partial row into every rank's receive area, tagged with the exchange number
          const uint32_t e = p.epoch_base + (uint32_t)d.xi;
          const size_t at = ((size_t)(e & 1u) * p.tp_size + p.tp_rank) * p.tp_hidden + row;
          for (int q = 0; q < p.tp_size; ++q)
            asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p.tp_recv[q] + at), "r"(__float_as_uint(v)), "r"(e + 1u) : "memory");
        } else {
          for (int q = 0; q < p.tp_size; ++q) p.tp_logits[q][(size_t)d.xi + row] = v;
        }
        v_out = v;
      }
      if (d.out_ss8 != nullptr) {
        float sq = v_out * v_out;
        sq += __shfl_xor_sync(0xffffffffu, sq, 1);
        sq += __shfl_xor_sync(0xffffffffu, sq, 2);
        sq += __shfl_xor_sync(0xffffffffu, sq, 4);
        if (r == 0 && valid) d.out_ss8[row >> 3] = sq;
      }
    }
    buf ^= 1;
  }
  return it;
}

// One projection phase: prologue (activations -> digits), then the rounds.
__device__ __forceinline__ uint32_t gemv_phase(const StepPhase& d, const StepParams& p, uint32_t it,
                                               const int tid, const int ph) {
  const Shared sh = shared_layout();
  const int lane = tid & 31, warp = tid >> 5;
  const int K = d.k, nb = K >> 5;
  const int KW = (nb + 31) >> 5;
  const int RG = kCW / KW;
  const int kw = warp % KW, rg = warp / KW;
  const bool wactive = rg < RG;
  const int part = kw * 32 + lane;
  const bool has_part = wactive && part < nb;

  // ---- activations: coalesced load into shared memory (128-byte rows, 16-byte chunks swizzled) ----
  {
    const float4* xg = reinterpret_cast<const float4*>(d.x);
    const int nf4 = K >> 2;
    constexpr int XIT = (kMaxK / 4 + kCT - 1) / kCT;
    float4 t[XIT];
#pragma unroll
    for (int j = 0; j < XIT; ++j) {
      const int f = tid + j * kCT;
      t[j] = f < nf4 ? __ldcg(xg + f) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int j = 0; j < XIT; ++j) {
      const int f = tid + j * kCT;
      if (f < nf4) {
        const int r = f >> 3, c = f & 7;
        reinterpret_cast<float4*>(sh.xbuf)[r * 8 + (c ^ (r & 7))] = t[j];
      }
    }
  }
  LaneX X;
  // RMSNorm with pre-weighted x: the warps that write results need 1/rms, and only at the end.
  // Fixed summation order: every CTA computes the same value.
  X.inv_rms = 1.f;
  if (d.x_ss8 != nullptr && wactive && kw == 0) {
    float ss = 0.f;
    const int n8 = K >> 3;
    for (int i0 = lane * 4; i0 < n8; i0 += 512) {   // four independent loads per trip: one trip for K <= 4096
      float4 t4[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        t4[j] = i0 + j * 128 < n8 ? __ldcg(reinterpret_cast<const float4*>(d.x_ss8 + i0 + j * 128)) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int j = 0; j < 4; ++j) ss += (t4[j].x + t4[j].y) + (t4[j].z + t4[j].w);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    X.inv_rms = 1.0f / sqrtf(ss / (float)K + d.eps);
  }
  consumer_sync();
  {
    // the block maximum first, then the two halves one after the other (fewer live registers)
    const float4* xs = reinterpret_cast<const float4*>(sh.xbuf) + (has_part ? part : 0) * 8;
    const int sw = part & 7;
    float amax = 0.f;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const float4 t4 = xs[c ^ sw];
      amax = fmaxf(fmaxf(amax, fmaxf(fabsf(t4.x), fabsf(t4.y))), fmaxf(fabsf(t4.z), fabsf(t4.w)));
    }
    int S = 0;
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      float v[16];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float4 t4 = xs[(hf * 4 + c) ^ sw];
        v[4 * c] = t4.x; v[4 * c + 1] = t4.y; v[4 * c + 2] = t4.z; v[4 * c + 3] = t4.w;
      }
      uint32_t dh[12];
      int Sh;
      quantize_part_int<16>(v, amax, dh, X.sx, Sh);
#pragma unroll
      for (int c = 0; c < 12; ++c) X.dig[hf * 12 + c] = dh[c];
      S += Sh;
    }
    X.s8hi = 8 * (S >> 16);
    X.s8lo = 8 * (S & 0xFFFF);
    if (!has_part) { X.sx = 0.f; X.s8hi = 0; X.s8lo = 0; }
  }
  step_mark(p, ph, 1, tid);
  return gemv_rounds(d, p, it, tid, ph, X);
}

// ------------------------------------------------------------------------------------------
// Attention phase (consumers).  RoPE + KV append + this CTA's share of the positions
// (src/llm/decoder.rs:1127-1213, rope_apply_head :28-68).
// ------------------------------------------------------------------------------------------

// Sums over the 8 lanes that share a K row: v[0..3] in, the complete sum of index
// (l8 & 1) * 2 + ((l8 >> 1) & 1) out in v[0] (replicated over bit 2 of l8).
__device__ __forceinline__ float spread_reduce4(float (&v)[4], int l8) {
  {
    const bool hi = (l8 & 1) != 0;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const float send = hi ? v[j] : v[j + 2];
      const float keep = hi ? v[j + 2] : v[j];
      v[j] = keep + __shfl_xor_sync(0xffffffffu, send, 1);
    }
  }
  {
    const bool hi = (l8 & 2) != 0;
    const float send = hi ? v[0] : v[1];
    const float keep = hi ? v[1] : v[0];
    v[0] = keep + __shfl_xor_sync(0xffffffffu, send, 2);
  }
  v[0] += __shfl_xor_sync(0xffffffffu, v[0], 4);
  return v[0];
}

// Scores of up to 8 rows (at kb, in shared memory) against this warp's two q heads.  Lanes work
// 8 to a row, 4 rows at a time; each (row, head) sum ends in one lane, which scales it, stores it
// at S[(srow0 + row) * gqp + g0 + head] and folds it into lmax.
template <int D>
__device__ __forceinline__ void score_rows2(const float* __restrict__ kb, int nr, int srow0, int gqp, int g0, float scale,
                                            const float4 (&qreg)[2][D / 32], float* __restrict__ S, float& lmax, int lane) {
  constexpr int F4 = D / 32, CPR = D / 4;
  const int l8 = lane & 7, rsub = lane >> 3;
  float v[4];
#pragma unroll
  for (int rgp = 0; rgp < 2; ++rgp) {
    const int row = rgp * 4 + rsub;
    float4 kf[F4];
#pragma unroll
    for (int i = 0; i < F4; ++i)
      kf[i] = row < nr ? reinterpret_cast<const float4*>(kb)[row * CPR + l8 + 8 * i] : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int g = 0; g < 2; ++g) {
      float a0 = 0.f, a1 = 0.f;
#pragma unroll
      for (int i = 0; i < F4; ++i) {
        a0 = fmaf(qreg[g][i].x, kf[i].x, a0);
        a1 = fmaf(qreg[g][i].y, kf[i].y, a1);
        a0 = fmaf(qreg[g][i].z, kf[i].z, a0);
        a1 = fmaf(qreg[g][i].w, kf[i].w, a1);
      }
      v[rgp * 2 + g] = a0 + a1;
    }
  }
  const float sum = spread_reduce4(v, l8);
  const int idx = (l8 & 1) * 2 + ((l8 >> 1) & 1);
  const int row = (idx >> 1) * 4 + rsub, g = idx & 1;
  if (l8 < 4 && row < nr) {
    const float sc = sum * scale;
    S[(srow0 + row) * gqp + g0 + g] = sc;
    lmax = fmaxf(lmax, sc);
  }
}

// acc[g] += sum over up to 8 rows of S[row][g0 + g] * V[row][:], one float4 column per lane.
template <int D>
__device__ __forceinline__ void weigh_rows2(const float* __restrict__ vb, int nr, int srow0, int gqp, int g0,
                                            const float* __restrict__ S, float4 (&acc)[2], int lane) {
  constexpr int CPR = D / 4, RPL = 32 / CPR;
  const int vc4 = lane % CPR, vrs = lane / CPR;
#pragma unroll
  for (int j = 0; j < 8 / RPL; ++j) {
    const int r = j * RPL + vrs;
    if (r < nr) {
      const float4 vv = reinterpret_cast<const float4*>(vb)[r * CPR + vc4];
      const float2 pg = *reinterpret_cast<const float2*>(S + (srow0 + r) * gqp + g0);
      acc[0].x = fmaf(pg.x, vv.x, acc[0].x); acc[0].y = fmaf(pg.x, vv.y, acc[0].y);
      acc[0].z = fmaf(pg.x, vv.z, acc[0].z); acc[0].w = fmaf(pg.x, vv.w, acc[0].w);
      acc[1].x = fmaf(pg.y, vv.x, acc[1].x); acc[1].y = fmaf(pg.y, vv.y, acc[1].y);
      acc[1].z = fmaf(pg.y, vv.z, acc[1].z); acc[1].w = fmaf(pg.y, vv.w, acc[1].w);
    }
  }
}

template <int D>
__device__ __forceinline__ uint32_t attn_phase(const StepPhase& d, const StepParams& p, uint32_t it, const int tid,
                                               const int ph) {
  const Shared sh = shared_layout();
  constexpr int F4 = D / 32, CPR = D / 4;
  const int lane = tid & 31, warp = tid >> 5;
  const AttnPlan a = attn_plan(p, (int)blockIdx.x);
  if (!a.active) return it;   // CTA-uniform: no stage was issued for this CTA either
  const int gq = p.gq, parts = p.parts, gqp = 2 * parts;
  const long long wait_limit = p.wait_cycles;
  const float qk_scale = p.scale;
  // work area (floats), every part 16-byte aligned
  float* q_s = sh.xbuf;                                   // [gqp][D]
  float* kv_new = q_s + gqp * D;                          // [2][D]
  float* S = kv_new + 2 * D;                              // [kChunkRows + 1][gqp]
  float* w_acc = S + (((kChunkRows + 1) * gqp + 3) & ~3);   // [kCW][2][D]
  float* s_wmax = w_acc + kCW * 2 * D;                    // [kCW][2]
  float* s_wsum = s_wmax + kCW * 2;                       // [kCW][8]
  float* s_m = s_wsum + kCW * 8;                          // [8] running maximum
  float* s_l = s_m + 8;                                   // [8] running sum
  float* s_resc = s_l + 8;                                // [8] rescale factor of this chunk

  const int off = a.off, kvh = a.kvh;
  float* kc = d.k_cache + (int64_t)kvh * p.max_seq_len * D;
  float* vc = d.v_cache + (int64_t)kvh * p.max_seq_len * D;
  const float* cs = p.cos_t + (int64_t)off * D;
  const float* sn = p.sin_t + (int64_t)off * D;
  {
    // q heads of this kv head, rotated (rotate-half with separately rounded products,
    // src/llm/decoder.rs:40-66); all loads first, then the arithmetic
    constexpr int QIT = (8 * D + kCT - 1) / kCT;
    float xa[QIT], xb[QIT], ca[QIT], sa[QIT];
#pragma unroll
    for (int k = 0; k < QIT; ++k) {
      const int i = tid + k * kCT;
      if (i < gq * D) {
        const int g = i / D, e = i - g * D;
        const float* xh = p.qkv + (int64_t)(kvh * gq + g) * D;
        xa[k] = __ldcg(xh + e);
        xb[k] = __ldcg(xh + (e < D / 2 ? e + D / 2 : e - D / 2));
        ca[k] = __ldg(cs + e);
        sa[k] = __ldg(sn + e);
      }
    }
#pragma unroll
    for (int k = 0; k < QIT; ++k) {
      const int i = tid + k * kCT;
      if (i < gq * D) {
        const int e = i % D;
        q_s[i] = e < D / 2 ? __fsub_rn(__fmul_rn(xa[k], ca[k]), __fmul_rn(xb[k], sa[k]))
                           : __fadd_rn(__fmul_rn(xa[k], ca[k]), __fmul_rn(xb[k], sa[k]));
      } else if (i < gqp * D) {
        q_s[i] = 0.f;   // the padding head of an odd group
      }
    }
    if (a.has_new && tid < D) {
      const float* kx = p.qkv + (int64_t)p.num_heads * D + (int64_t)kvh * D;
      const float* vx = kx + (int64_t)p.num_kv_heads * D;
      const int e = tid, e2 = e < D / 2 ? e + D / 2 : e - D / 2;
      const float ke = __ldcg(kx + e), ko = __ldcg(kx + e2);
      const float c = __ldg(cs + e), s_ = __ldg(sn + e);
      const float kr = e < D / 2 ? __fsub_rn(__fmul_rn(ke, c), __fmul_rn(ko, s_)) : __fadd_rn(__fmul_rn(ke, c), __fmul_rn(ko, s_));
      const float vr = __ldcg(vx + e);
      kc[(int64_t)off * D + e] = kr;
      vc[(int64_t)off * D + e] = vr;
      kv_new[e] = kr;
      kv_new[D + e] = vr;
    }
    if (tid < 8) { s_m[tid] = -INFINITY; s_l[tid] = 0.f; }
  }
  consumer_sync();
  step_mark(p, ph, 1, tid);

  // warp roles: a team of rsl * parts warps takes one stage: rsl slices of RW rows x `parts` head pairs
  const int rsl = parts == 1 ? 4 : 2, RW = kAttnRows / rsl;
  const int tsz = rsl * parts, nteams = kCW / tsz;
  const int team = warp / tsz, wi = warp - team * tsz;   // warps past the last whole team have no stage
  const int pid = wi % parts, rslice = wi / parts;
  const int g0 = pid * 2;
  const int l8 = lane & 7;
  float4 qreg[2][F4];
#pragma unroll
  for (int g = 0; g < 2; ++g)
#pragma unroll
    for (int i = 0; i < F4; ++i) qreg[g][i] = reinterpret_cast<const float4*>(q_s)[(g0 + g) * CPR + l8 + 8 * i];
  float4 acc[2];
  acc[0] = make_float4(0.f, 0.f, 0.f, 0.f);
  acc[1] = make_float4(0.f, 0.f, 0.f, 0.f);
  const int g_t = tid % gqp;   // the head whose exponentials this thread takes in the softmax pass

#pragma unroll 1
  for (int c = 0; c < a.nchunks; ++c) {
    const int cr0 = c * kChunkRows;
    const int crn = min(kChunkRows, a.ring_rows - cr0);
    const int nt = (crn + kAttnRows - 1) / kAttnRows;
    const bool new_here = a.has_new && c == a.nchunks - 1;
    if (c > 0) consumer_sync();  // the previous chunk's weights in S have been used
    // ---- K stages: scores into S ----
    float lmax = -INFINITY;
#pragma unroll 1
    for (int t = 0; t < nt; ++t, ++it) {
      const int s = (int)(it % kStages);
      const bool ok = mbar_wait(&sh.full[s], (it / kStages) & 1u, sh.s_abort, wait_limit);
      if (ok && (t % nteams) == team) {
        for (int r0 = rslice * RW; r0 < (rslice + 1) * RW; r0 += 8) {
          const int nr = min(8, crn - t * kAttnRows - r0);
          if (nr > 0)
            score_rows2<D>(reinterpret_cast<const float*>(sh.ring + (size_t)s * kStageBytes) + (size_t)r0 * D, nr,
                           t * kAttnRows + r0, gqp, g0, qk_scale, qreg, S, lmax, lane);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh.empty[s]);
    }
    if (new_here && team == 0 && rslice == 0) score_rows2<D>(kv_new, 1, crn, gqp, g0, qk_scale, qreg, S, lmax, lane);
    if (c == 0) step_mark(p, ph, 3, tid);
    {
      // the warp's maximum per head: row group in lane bit 0, head in bit 1, row in bits 3-4
      float mx = lmax;
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
      if (lane == 0) s_wmax[warp * 2 + 0] = mx;
      if (lane == 2) s_wmax[warp * 2 + 1] = mx;
    }
    consumer_sync();
    if (tid < gqp) {   // exact statistics of the chunk, one thread per head
      const int hp = tid >> 1, hg = tid & 1;
      float mc = -INFINITY;
      for (int w = 0; w < kCW; ++w)
        if ((w % tsz) % parts == hp) mc = fmaxf(mc, s_wmax[w * 2 + hg]);
      const float m_old = s_m[tid];
      const float m_new = fmaxf(m_old, mc);
      const float resc = m_new == -INFINITY ? 1.f : expf(m_old - m_new);  // exp(-inf) = 0 for the first chunk
      s_m[tid] = m_new;
      s_resc[tid] = resc;
      s_l[tid] *= resc;
    }
    consumer_sync();
    {
      const float m_t = s_m[g_t];
      const int n_s = (crn + (new_here ? 1 : 0)) * gqp;
      float ls = 0.f;
      for (int i = tid; i < n_s; i += kCT) {
        const float e = expf(S[i] - m_t);
        S[i] = e;
        ls += e;
      }
      for (int o = gqp; o < 32; o <<= 1) ls += __shfl_xor_sync(0xffffffffu, ls, o);
      if (lane < gqp) s_wsum[warp * 8 + lane] = ls;
      if (c > 0) {
        const float r0 = s_resc[g0], r1 = s_resc[g0 + 1];
        acc[0].x *= r0; acc[0].y *= r0; acc[0].z *= r0; acc[0].w *= r0;
        acc[1].x *= r1; acc[1].y *= r1; acc[1].z *= r1; acc[1].w *= r1;
      }
    }
    consumer_sync();
    if (tid < gqp) {
      float tsum = 0.f;
      for (int w = 0; w < kCW; ++w) tsum += s_wsum[w * 8 + tid];
      s_l[tid] += tsum;
    }
    // ---- V stages: weighted sum ----
#pragma unroll 1
    for (int t = 0; t < nt; ++t, ++it) {
      const int s = (int)(it % kStages);
      const bool ok = mbar_wait(&sh.full[s], (it / kStages) & 1u, sh.s_abort, wait_limit);
      if (ok && (t % nteams) == team) {
        for (int r0 = rslice * RW; r0 < (rslice + 1) * RW; r0 += 8) {
          const int nr = min(8, crn - t * kAttnRows - r0);
          if (nr > 0)
            weigh_rows2<D>(reinterpret_cast<const float*>(sh.ring + (size_t)s * kStageBytes) + (size_t)r0 * D, nr,
                           t * kAttnRows + r0, gqp, g0, S, acc, lane);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh.empty[s]);
    }
    if (new_here && team == 0 && rslice == 0) weigh_rows2<D>(kv_new + D, 1, crn, gqp, g0, S, acc, lane);
  }

  // ---- this CTA's partial: the warps' weighted V summed, with the share's max and sum ----
#pragma unroll
  for (int g = 0; g < 2; ++g) {
#pragma unroll
    for (int o = CPR; o < 32; o <<= 1) {  // lanes that share a column (head_dim < 128)
      acc[g].x += __shfl_xor_sync(0xffffffffu, acc[g].x, o);
      acc[g].y += __shfl_xor_sync(0xffffffffu, acc[g].y, o);
      acc[g].z += __shfl_xor_sync(0xffffffffu, acc[g].z, o);
      acc[g].w += __shfl_xor_sync(0xffffffffu, acc[g].w, o);
    }
    if (lane < CPR) reinterpret_cast<float4*>(w_acc + ((size_t)warp * 2 + g) * D)[lane] = acc[g];
  }
  consumer_sync();
  for (int i = tid; i < gq * D; i += kCT) {
    const int g = i / D, e = i - g * D;
    const int hp = g >> 1, hg = g & 1;
    float o = 0.f;
    for (int w = 0; w < kCW; ++w)
      if ((w % tsz) % parts == hp) o += w_acc[((size_t)w * 2 + hg) * D + e];
    const int h = kvh * gq + g;
    p.part_o[((int64_t)h * p.nc + a.split) * D + e] = o;
    if (e == 0) {
      float* dst = p.part_ml + ((int64_t)h * p.nc + a.split) * 2;
      dst[0] = s_m[g];
      dst[1] = s_l[g];
    }
  }
  return it;
}

// Merge phase: out[h] = sum_c exp(m_c - max) * o_c / max(sum_c exp(m_c - max) * l_c, 1e-30)
// (the two-pass softmax of src/llm/decoder.rs:1185-1210 over the split positions).  One warp per
// float4 of the output, one partial per lane (two for more than 32 splits).
template <int D>
__device__ __forceinline__ void merge_phase(const StepParams& p, const int tid) {
  constexpr int CPR = D / 4;
  const int lane = tid & 31, warp = tid >> 5;
  const AttnPlan a = attn_plan(p, 0);
  const int nvalid = a.nvalid;
  const int total = p.num_heads * CPR;
  for (int o = (int)blockIdx.x * kCW + warp; o < total; o += (int)gridDim.x * kCW) {
    const int h = o / CPR, col = o - h * CPR;
    float m[2], l[2];
    float4 v[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int c = lane + 32 * k;
      m[k] = -INFINITY; l[k] = 0.f; v[k] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (c < nvalid) {
        const float2 ml = __ldcg(reinterpret_cast<const float2*>(p.part_ml + ((int64_t)h * p.nc + c) * 2));
        m[k] = ml.x; l[k] = ml.y;
        v[k] = __ldcg(reinterpret_cast<const float4*>(p.part_o + ((int64_t)h * p.nc + c) * D) + col);
      }
    }
    float mx = fmaxf(m[0], m[1]);
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, s));
    float tot = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      if (m[k] != -INFINITY) {
        const float w = expf(m[k] - mx);
        tot = fmaf(l[k], w, tot);
        acc.x = fmaf(v[k].x, w, acc.x); acc.y = fmaf(v[k].y, w, acc.y);
        acc.z = fmaf(v[k].z, w, acc.z); acc.w = fmaf(v[k].w, w, acc.w);
      }
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) {
      tot += __shfl_xor_sync(0xffffffffu, tot, s);
      acc.x += __shfl_xor_sync(0xffffffffu, acc.x, s);
      acc.y += __shfl_xor_sync(0xffffffffu, acc.y, s);
      acc.z += __shfl_xor_sync(0xffffffffu, acc.z, s);
      acc.w += __shfl_xor_sync(0xffffffffu, acc.w, s);
    }
    if (lane == 0) {
      const float r = 1.0f / fmaxf(tot, 1e-30f);   // src/llm/decoder.rs:1203
      reinterpret_cast<float4*>(p.attn + (int64_t)h * D)[col] =
          (nvalid == 0 || mx == -INFINITY) ? make_float4(0.f, 0.f, 0.f, 0.f) : make_float4(acc.x * r, acc.y * r, acc.z * r, acc.w * r);
    }
  }
}

// Exchange phase (tensor parallel): x[r] += sum over the ranks of their partial row r, plus the
// next norm's pre-weighted copy and the sums of squares.  A warp takes 8 rows; lane (s, r) polls
// the entries of sources s, s + 4 for row r until they carry this exchange's number (the
// producing projection stored them straight into this rank's receive area), the four lanes of a
// row are added in a fixed order - the same on every rank, so every rank holds the same x.
__device__ __forceinline__ void exch_phase(const StepPhase& d, const StepParams& p, const int tid, volatile int* s_abort) {
  const int lane = tid & 31, warp = tid >> 5;
  const int H = d.n, size = p.tp_size;
  const uint32_t e = p.epoch_base + (uint32_t)d.xi;
  const uint2* base = p.tp_recv[p.tp_rank] + (size_t)(e & 1u) * size * p.tp_hidden;
  const long long limit = p.wait_cycles;
  for (int o = (int)blockIdx.x + warp * (int)gridDim.x; o < (H >> 3); o += (int)gridDim.x * kCW) {
    const int row = o * 8 + (lane & 7);
    float sum = 0.f;
    for (int src = lane >> 3; src < size; src += 4) {
      const uint2* at = base + (size_t)src * p.tp_hidden + row;
      uint32_t v0, v1;
      long long t0 = 0;
      for (uint32_t spin = 0;; ++spin) {
        asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v0), "=r"(v1) : "l"(at) : "memory");
        if (v1 == e + 1u) break;
        if ((spin & 63) == 63) {
          if (*s_abort) { v0 = 0u; break; }
          if (t0 == 0) t0 = clock64();
          else if (clock64() - t0 > limit || *reinterpret_cast<volatile int*>(&g_step_fault)) {
            *s_abort = 1;
            atomicExch(&g_step_fault, 1);
            v0 = 0u;
            break;
          }
        }
      }
      sum += __uint_as_float(v0);
    }
    sum += __shfl_xor_sync(0xffffffffu, sum, 8);
    sum += __shfl_xor_sync(0xffffffffu, sum, 16);
    float xv = 0.f;
    if (lane < 8) {
      xv = __ldcg(d.resid + row) + sum;
      d.out[row] = xv;
      if (d.out_scaled != nullptr) d.out_scaled[row] = xv * __ldg(d.out_scale_w + row);
    }
    if (d.out_ss8 != nullptr) {
      float sq = xv * xv;
      sq += __shfl_xor_sync(0xffffffffu, sq, 1);
      sq += __shfl_xor_sync(0xffffffffu, sq, 2);
      sq += __shfl_xor_sync(0xffffffffu, sq, 4);
      if (lane == 0) d.out_ss8[o] = sq;
    }
  }
}

template <int D>
__global__ void __launch_bounds__(kThreads, 1) w4_step_kernel(const StepParams kp) {
  __shared__ __align__(16) StepPhase s_desc[2];
  __shared__ __align__(16) StepParams s_params;   // the phase routines read the parameters from here
  const StepParams& p = s_params;
  const Shared sh = shared_layout();
  uint64_t* full = sh.full;
  uint64_t* empty = sh.empty;

  const int tid = threadIdx.x, warp = tid >> 5;
  if (tid == 0) {
    s_params = kp;
    if (kp.tp_size > 1) s_params.epoch_base = *kp.tp_epoch;
    *sh.s_abort = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], kCW);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (tid < kStepPhaseWords) reinterpret_cast<int4*>(&s_desc[0])[tid] = __ldg(reinterpret_cast<const int4*>(kp.phases) + tid);
  __syncthreads();

  if (warp == kCW) {
    producer_loop<D>(p, sh.ring, full, empty, sh.s_abort, tid & 31);
    return;
  }

  uint32_t it = 0;
  unsigned round = 0;
#pragma unroll 1
  for (int ph = 0; ph < p.nphases; ++ph) {
    const StepPhase& d = s_desc[ph & 1];
    step_mark(p, ph, 0, tid);
    if (ph + 1 < p.nphases && tid < kStepPhaseWords)   // the next descriptor travels while this phase runs
      reinterpret_cast<int4*>(&s_desc[(ph + 1) & 1])[tid] = __ldg(reinterpret_cast<const int4*>(p.phases + ph + 1) + tid);
    if (d.kind == 0) {
      it = gemv_phase(d, p, it, tid, ph);
    } else if (d.kind == 1) {
      it = attn_phase<D>(d, p, it, tid, ph);
    } else if (d.kind == 2) {
      merge_phase<D>(p, tid);
    } else {
      exch_phase(d, p, tid, sh.s_abort);
    }
    step_mark(p, ph, 2, tid);
    // (a projection whose rows go to the ranks' receive areas is followed by the exchange phase,
    // which waits on those rows themselves: no barrier in between)
    if ((ph + 1 < p.nphases || p.tp_size > 1) && !(d.kind == 0 && d.tp_mode == 1)) {
      ++round;
      grid_barrier(p.sync, round, sh.s_abort, p.wait_cycles, tid);
    } else {
      // no grid barrier here, but the CTA's warps must all be done with this phase's descriptor
      // before the next phase's first threads overwrite the other descriptor slot
      consumer_sync();
    }
  }
  // The last CTA to leave puts the barrier words back to zero for the next launch (every CTA has
  // passed its last barrier by the time it takes an exit ticket).
  if (p.tp_size > 1 && blockIdx.x == 0 && tid == 0) {
    // Every CTA of this rank has stored its logit rows into every rank's copy (the barrier above).
    // Tell the peers, then wait until every peer has told us: the logits are complete everywhere.
    const uint32_t fin = p.epoch_base + (uint32_t)p.n_exchanges + 1u;
    __threadfence_system();
    for (int q = 0; q < p.tp_size; ++q)
      asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.tp_flags[q] + p.tp_rank), "r"(fin) : "memory");
    const long long limit = p.wait_cycles;
    for (int src = 0; src < p.tp_size && !*sh.s_abort; ++src) {
      long long t0 = 0;
      for (uint32_t spin = 0;; ++spin) {
        uint32_t v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p.tp_flags[p.tp_rank] + src) : "memory");
        if (v == fin) break;
        if ((spin & 63) == 63) {
          if (t0 == 0) t0 = clock64();
          else if (clock64() - t0 > limit || *reinterpret_cast<volatile int*>(&g_step_fault)) {
            *sh.s_abort = 1;
            atomicExch(&g_step_fault, 1);
            break;
          }
        }
      }
    }
  }
  consumer_sync();
  if (tid == 0) {
    if (*sh.s_abort && p.host_fault != nullptr) {
      *reinterpret_cast<volatile int*>(p.host_fault) = 1;
      __threadfence_system();
    }
    if (atomicAdd(p.sync + 4, 1u) == gridDim.x - 1) {
      p.sync[0] = 0u; p.sync[1] = 0u; p.sync[2] = 0u; p.sync[3] = 0u;
      p.sync[4] = 0u;
      if (p.tp_size > 1) *p.tp_epoch = p.epoch_base + (uint32_t)p.n_exchanges + 1u;
      __threadfence();
    }
  }
}

// The two bounded waits of the step kernel on conditions that nothing fulfils: an mbarrier phase
// nobody completes and a grid barrier one arrival short.  With a short limit both must give up,
// raise the fault word and let the kernel end (one CTA of one warp; nothing else is touched).
__global__ void __launch_bounds__(32) wait_probe_kernel(unsigned* counters, long long limit, int* out) {
  __shared__ __align__(8) uint64_t bar;
  __shared__ int s_abort;
  if (threadIdx.x == 0) {
    s_abort = 0;
    mbar_init(&bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  if (threadIdx.x == 0) {
    const bool a = mbar_wait(&bar, 0u, &s_abort, limit);            // nobody arrives on `bar`
    out[0] = a ? 0 : 1;
    s_abort = 0;
    // a lone CTA waits for a second arrival that never comes (round 1 of a grid of "2")
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(counters) : "memory");
    long long t0 = clock64();
    bool gave_up = false;
    while (ld_acquire_gpu(counters) < 2u) {
      if (clock64() - t0 > limit) { gave_up = true; atomicExch(&g_step_fault, 1); break; }
    }
    out[1] = gave_up ? 1 : 0;
  }
}

// x = table[token]; xn = x * norm_w; ss8: one CTA (the vector is a few thousand floats).
__global__ void __launch_bounds__(1024) step_embed_kernel(const float* __restrict__ table, const int32_t* __restrict__ tokens,
                                                          const int32_t* __restrict__ offsets,
                                                          const float* __restrict__ norm_w, float* __restrict__ x,
                                                          float* __restrict__ xn, float* __restrict__ ss8,
                                                          int32_t* __restrict__ eff_offsets, int64_t vocab, int64_t hidden,
                                                          int64_t max_seq_len) {
  const int tok = tokens[0], off = offsets[0];
  const bool ok = tok >= 0 && tok < vocab && off >= 0 && off < max_seq_len;
  if (threadIdx.x == 0) eff_offsets[0] = ok ? off : -1;
  // a thread takes 8 consecutive elements: one entry of ss8
  for (int64_t i = threadIdx.x; i < hidden / 8; i += blockDim.x) {
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
    if (ok) {
      a = reinterpret_cast<const float4*>(table + (int64_t)tok * hidden)[2 * i];
      b = reinterpret_cast<const float4*>(table + (int64_t)tok * hidden)[2 * i + 1];
    }
    const float4 wa = reinterpret_cast<const float4*>(norm_w)[2 * i], wb = reinterpret_cast<const float4*>(norm_w)[2 * i + 1];
    reinterpret_cast<float4*>(x)[2 * i] = a;
    reinterpret_cast<float4*>(x)[2 * i + 1] = b;
    reinterpret_cast<float4*>(xn)[2 * i] = make_float4(a.x * wa.x, a.y * wa.y, a.z * wa.z, a.w * wa.w);
    reinterpret_cast<float4*>(xn)[2 * i + 1] = make_float4(b.x * wb.x, b.y * wb.y, b.z * wb.z, b.w * wb.w);
    // the order of the producers' butterfly over 8 rows: ((0+1)+(2+3)) + ((4+5)+(6+7))
    const float s01 = a.x * a.x + a.y * a.y, s23 = a.z * a.z + a.w * a.w;
    const float s45 = b.x * b.x + b.y * b.y, s67 = b.z * b.z + b.w * b.w;
    ss8[i] = (s01 + s23) + (s45 + s67);
  }
}

long long g_wait_cycles = 0;
int g_step_debug = 0;

}  // namespace

void set_step_wait_limit(long long cycles) { g_wait_cycles = cycles; }
void set_step_debug(int flags) { g_step_debug = flags; }

int step_fault_flag() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_step_fault, sizeof(int)) != cudaSuccess) return -1;
  return v;
}

// Test hook: see wait_probe_kernel.  Returns TB_ERR_TIMEOUT when both waits gave up as they
// must (and clears the fault word they raised), TB_ERR_CUDA on any other outcome.
tb_status step_wait_probe(long long limit_cycles) {
  if (limit_cycles < 1000 || limit_cycles > 2000000000ll) return fail(TB_ERR_ARG, "wait probe: limit of %lld cycles is outside [1e3, 2e9]", limit_cycles);
  unsigned* ctr = nullptr;
  int* out = nullptr;
  TB_CUDA_TRY(cudaMalloc((void**)&ctr, 64));
  cudaError_t e = cudaMalloc((void**)&out, 64);
  if (e != cudaSuccess) { cudaFree(ctr); return fail(TB_ERR_OOM, "wait probe: %s", cudaGetErrorString(e)); }
  cudaMemset(ctr, 0, 64);
  cudaMemset(out, 0xff, 64);
  wait_probe_kernel<<<1, 32>>>(ctr, limit_cycles, out);
  int h[2] = {-1, -1};
  e = cudaMemcpy(h, out, sizeof(h), cudaMemcpyDeviceToHost);
  const int flag = step_fault_flag();
  const int zero = 0;
  cudaMemcpyToSymbol(g_step_fault, &zero, sizeof(int));
  cudaFree(ctr);
  cudaFree(out);
  if (e != cudaSuccess) return fail(TB_ERR_CUDA, "wait probe: %s", cudaGetErrorString(e));
  if (h[0] == 1 && h[1] == 1 && flag == 1)
    return fail(TB_ERR_TIMEOUT, "a bounded device-side wait ran out (probe: both waits gave up after %lld cycles)", limit_cycles);
  return fail(TB_ERR_CUDA, "wait probe: unexpected outcome (mbarrier %d, grid barrier %d, fault word %d)", h[0], h[1], flag);
}

int w4_step_rows_per_stage(int64_t k, int g, int nw) {
  const int64_t per_row = (int64_t)nw * (k / 2 + (k / g) * 4);
  int rs = 8;
  while (rs > 1 && rs * per_row > kStageBytes) rs >>= 1;
  return rs >= 2 && rs * per_row <= kStageBytes ? rs : 0;   // at most 4 stages per 8-row round
}

bool w4_step_supports(int64_t n, int64_t k, int g, int nw) {
  if (n < 1 || k < 32 || k % 32 != 0 || k > kMaxK) return false;
  if (g != 32 && g != 64 && g != 128) return false;
  if (k % g != 0) return false;
  if (((k / g) * 4) % 16 != 0 || (k / 2) % 16 != 0) return false;  // bulk copies move whole 16-byte units
  const int kw = (int)((k / 32 + 31) / 32);
  if (kw > kCW) return false;
  return w4_step_rows_per_stage(k, g, nw) > 0;
}

int w4_step_attn_split(int grid, int num_kv_heads) {
  if (num_kv_heads < 1 || grid < num_kv_heads) return 0;
  int nc = grid / num_kv_heads;
  return nc > kMaxSplits ? kMaxSplits : nc;
}

template <int D>
static int step_grid_for() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  if (dev >= 0 && dev < 64 && cached[dev] != 0) return cached[dev] < 0 ? 0 : cached[dev];
  int grid = 0, per_sm = 0;
  auto kern = w4_step_kernel<D>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes + kBarBytes) == cudaSuccess &&
      cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kThreads, kSmemBytes + kBarBytes) == cudaSuccess && per_sm >= 1) {
    int coop = 0;
    cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev);
    if (coop) grid = sm_count();
  }
  cudaGetLastError();
  if (dev >= 0 && dev < 64) cached[dev] = grid > 0 ? grid : -1;
  return grid;
}

int w4_step_grid() { return step_grid_for<128>(); }

tb_status launch_w4_step(const StepProgram& g, cudaStream_t stream) {
  if (!g.phases || g.nphases < 1 || !g.sync) return fail(TB_ERR_ARG, "step kernel: empty program");
  if (g.head_dim != 64 && g.head_dim != 128) return fail(TB_ERR_UNSUPPORTED, "TB_UNSUPPORTED: step kernel: head_dim %d", g.head_dim);
  const int grid = g.head_dim == 128 ? step_grid_for<128>() : step_grid_for<64>();
  if (grid <= 0 || grid != g.grid) return fail(TB_ERR_UNSUPPORTED, "TB_UNSUPPORTED: step kernel: grid %d, program laid out for %d", grid, g.grid);
  StepParams p;
  p.phases = g.phases; p.nphases = g.nphases; p.sync = g.sync; p.host_fault = g.host_fault;
  p.qkv = g.qkv; p.attn = g.attn; p.cos_t = g.cos_t; p.sin_t = g.sin_t; p.offsets = g.offsets;
  p.part_o = g.part_o; p.part_ml = g.part_ml;
  p.num_heads = g.num_heads; p.num_kv_heads = g.num_kv_heads;
  p.gq = g.num_kv_heads > 0 ? g.num_heads / g.num_kv_heads : 1;
  p.parts = p.gq <= 2 ? 1 : (p.gq <= 4 ? 2 : 4);
  p.nc = g.nc;
  p.max_seq_len = g.max_seq_len;
  p.scale = 1.0f / sqrtf((float)g.head_dim);
  p.wait_cycles = g_wait_cycles > 0 ? g_wait_cycles : kWaitCyclesDefault;
  p.debug = g_step_debug;
  p.tp_rank = g.tp.rank; p.tp_size = g.tp.size; p.tp_hidden = g.tp.hidden; p.n_exchanges = g.n_exchanges;
  for (int r = 0; r < 8; ++r) { p.tp_recv[r] = g.tp.recv[r]; p.tp_logits[r] = g.tp.logits[r]; p.tp_flags[r] = g.tp.flags[r]; }
  p.tp_epoch = g.tp.epoch; p.epoch_base = 0;
  p.tl = timeline_next_block();
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kSmemBytes + kBarBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (g.head_dim == 128) TB_CUDA_TRY(cudaLaunchKernelEx(&cfg, w4_step_kernel<128>, p));
  else TB_CUDA_TRY(cudaLaunchKernelEx(&cfg, w4_step_kernel<64>, p));
  return TB_OK;
}

// One projection through the step kernel's code path (a program of a single phase): out = W x,
// or silu(W x) * (W2 x) when w2 is given.  For tests and profiling of that path at any shape.
tb_status launch_w4_step_gemv(const GemvArgs& a, cudaStream_t stream) {
  const int nw = a.w2 ? 2 : 1;
  if (a.m != 1 || !w4_step_supports(a.n, a.k, a.g, nw)) return fail(TB_ERR_UNSUPPORTED, "TB_UNSUPPORTED: step kernel projection [%lld, %lld] group %d", (long long)a.n, (long long)a.k, a.g);
  if (a.norm_w) return fail(TB_ERR_UNSUPPORTED, "TB_UNSUPPORTED: step kernel projection takes pre-weighted activations (x_ss8), not norm weights");
  const int grid = w4_step_grid();
  if (grid <= 0) return fail(TB_ERR_UNSUPPORTED, "TB_UNSUPPORTED: the step kernel cannot run on this device");
  StepPhase q;
  q.kind = 0; q.n = (int)a.n; q.k = (int)a.k; q.ng = (int)(a.k / a.g); q.gshift = a.g == 32 ? 0 : (a.g == 64 ? 1 : 2);
  q.nw = nw; q.rs = w4_step_rows_per_stage(a.k, a.g, nw); q.rot = 0; q.eps = a.eps;
  q.w[0] = a.w; q.sc[0] = a.scales; q.bias[0] = a.bias; q.w[1] = a.w2; q.sc[1] = a.scales2; q.bias[1] = a.bias2;
  q.x = a.x; q.x_ss8 = a.x_ss8; q.resid = a.resid; q.out = a.out;
  q.out_scaled = a.out_scaled; q.out_scale_w = a.out_scale_w; q.out_ss8 = a.out_ss8;
  // the phase descriptor and the barrier words live in one small allocation of the stream's pool
  char* blk = nullptr;
  TB_CUDA_TRY(cudaMallocAsync((void**)&blk, 512, stream));
  TB_CUDA_TRY(cudaMemsetAsync(blk + 256, 0, 64, stream));
  TB_CUDA_TRY(cudaMemcpyAsync(blk, &q, sizeof(q), cudaMemcpyHostToDevice, stream));
  StepProgram g;
  g.phases = reinterpret_cast<const StepPhase*>(blk); g.nphases = 1; g.grid = grid;
  g.sync = reinterpret_cast<unsigned*>(blk + 256);
  g.head_dim = 128; g.num_heads = 1; g.num_kv_heads = 1; g.nc = 1; g.max_seq_len = 1;
  const tb_status st = launch_w4_step(g, stream);
  cudaFreeAsync(blk, stream);
  return st;
}

tb_status launch_step_embed(const float* table, const int32_t* tokens, const int32_t* offsets, const float* norm_w,
                            float* x, float* xn, float* ss8, int32_t* eff_offsets, int64_t vocab, int64_t hidden,
                            int64_t max_seq_len, cudaStream_t stream) {
  if (hidden % 8 != 0) return fail(TB_ERR_SHAPE, "step embed: hidden %lld is not a multiple of 8", (long long)hidden);
  step_embed_kernel<<<1, 1024, 0, stream>>>(table, tokens, offsets, norm_w, x, xn, ss8, eff_offsets, vocab, hidden, max_seq_len);
  TB_CUDA_TRY(cudaGetLastError());
  return TB_OK;
}

}  // namespace tb
