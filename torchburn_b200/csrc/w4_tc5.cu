// Batched grouped-INT4 product for more than 16 activation rows on the 5th-generation tensor
// cores (tcgen05): out[m, j] = sum_g scale[j, g] * sum_{k in g} x[m, k] * code(w[j, k])  (+ bias,
// + residual, or the SwiGLU of a gate/up pair).  gemm_w4a32_grouped, src/quantization/gemv.rs:
// 1690-1725; fused_swiglu_mlp_batched, src/quantization/fused_ops.rs:1267-1319.
//
// The 4-bit codes are exact in bf16, so the weights enter the tensor core as they are and the
// scale is applied OUTSIDE it, once per group: every group of K gets a fresh fp32 accumulator
// in tensor memory, which the epilogue warps read back, multiply by scale[row, group] and add
// to their registers while the next groups are being multiplied.  The fp32 activations are
// split once per call (pre-pass, with the fused RMSNorm) into three bf16 pieces x1 + x2 + x3
// (8 + 8 + 8 mantissa bits); the three products share one accumulator.  Products of a 4-bit
// code and an 8-bit piece are exact and the tensor core adds them in fp32.
//
// The weights are the M = 128 side of the MMA (a CTA owns 128 weight rows), the activation
// rows its N = 16..64.  A weight row lives in one LANE of tensor memory: the thread that
// dequantises row r writes its codes with tcgen05.st straight from registers (A operand from
// tensor memory), so the weights pass through shared memory only as packed nibbles (the per-thread
// copy ring), never in operand form.  The activation pieces
// arrive as ready-made 128-byte-swizzled K-major images by bulk copy.
//
//   unpacking    4 or 8 warps, 128 threads per team (thread = weight row; two teams take every other
//                stage): the nibbles of the thread's row stream into the thread's own shared-memory
//                ring with cp.async, eight 64-element chunks ahead; the thread unpacks a chunk into
//                its stage of tensor memory
//   epilogue     8 warps: two teams of 128 threads (thread = weight row, a team = half of the activation
//                rows): per group tcgen05.ld of the accumulator, acc += scale * sum; at the
//                end bias / residual / SwiGLU and the stores (atomic adds when K is split)
//   issue        4 warps, one lane each issues MMAs: issuing a tcgen05.mma costs its thread about 50 cycles
//                whatever its size (measured), six times the arithmetic of a 128 x 16 x 16 MMA, but
//                several warps issue side by side.  With four accumulator slots issuer i owns slot i and
//                takes every group of K whose number is i modulo 4; with two slots (a pair at 48 or 64
//                rows) issuer i owns slot i & 1 and matrix i >> 1.  An issuer commits its MMAs to the
//                "group done" and "stage free" barriers.  The first of them also allocates tensor memory.
// The bulk copies of the activation images are issued by the first thread of an unpacking team.
//
// Every wait is bounded.  No cluster features, no multicast.
#include <cuda_bf16.h>

#include "tb_common.cuh"

namespace tb {

namespace {

constexpr int kTileN = 128;     // weight rows per CTA (the MMA's M)
constexpr int kKC = 64;         // K elements per stage: one 128-byte row of bf16
constexpr int kMaxStages = 8;    // one matrix: 8 stages, a pair: 4 (tensor memory: 32 columns of codes per stage and matrix)
constexpr int kPieces = 3;      // bf16 pieces of an activation
constexpr int kAhead = 8;       // chunks of nibbles in flight per weight row
constexpr int kTmemCols = 512;
constexpr int kMinRows = 17;     // up to 16 activation rows the integer mma.sync kernel is as fast or faster (measured)
constexpr long long kWaitCycles = 4000000000ll;  // ~2 s

__device__ int g_tc5_fault = 0;

struct Tc5Params {
  const uint8_t* w[2];
  const float* scales[2];
  const float* bias[2];
  const float* resid;
  float* out;
  const unsigned char* xq;   // per 64-element chunk of K: kPieces images of [mp rows x 128 B], swizzled
  int m, mp;                 // activation rows, padded to a multiple of 16
  int n, k, ng, g;
  int ksplit, kper;          // CTAs that share a row tile, K elements of each
  int pair;                  // gate/up pair with the SwiGLU epilogue
  int slots;                 // accumulator slots in tensor memory
  int stages;                // stage ring: 8 for one matrix, 4 for a pair
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
// Bounded wait: false (and the abort word raised) when the limit ran out here or elsewhere in the CTA.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* s_abort) {
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
      else if (clock64() - t0 > kWaitCycles) {
        *s_abort = 1;
        atomicExch(&g_tc5_fault, 1);
        return false;
      }
    }
  }
}
// Ready already (the usual case for the issuing thread)?  One instruction, no loop.
__device__ __forceinline__ bool mbar_ready(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __noinline__ bool mbar_wait_slow(uint64_t* bar, uint32_t parity, volatile int* s_abort) { return mbar_wait(bar, parity, s_abort); }
__device__ __forceinline__ bool mbar_wait_fast(uint64_t* bar, uint32_t parity, volatile int* s_abort) {
  return mbar_ready(bar, parity) ? true : mbar_wait_slow(bar, parity, s_abort);
}
// The same for a whole warp.  ONE lane polls: hundreds of threads polling the same barriers keep the
// barrier unit so busy that the arrivals they are waiting for queue up behind their own polls.  The other
// lanes take the answer (one answer for all lanes keeps warp-wide instructions converged) and the
// ordering from the warp barrier.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, volatile int* s_abort) {
  bool ok = true;
  if ((threadIdx.x & 31) == 0) ok = mbar_wait_fast(bar, parity, s_abort);
  __syncwarp();
  return __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile of 128-byte rows with the 128-byte swizzle.
// Lower word: start address in 16-byte units (bits 0-13), leading offset 1 (bits 16-29, unused
// with a swizzle).  Upper word: 1024 bytes between groups of 8 rows (bits 32-45, in 16-byte
// units), descriptor version 1 (bits 46-47), layout type 2 = SWIZZLE_128B (bits 61-63).
// D (tensor memory, fp32) (+)= A (tensor memory, bf16) * B (shared memory, bf16)^T
// b_lo: the lower word of B's shared-memory descriptor (see above); the upper word is the same for every tile.
// ACC 0: overwrite the accumulator, 1: add to it, 2: decided at run time by `acc`.
template <int ACC>
__device__ __forceinline__ void mma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t idesc, uint32_t acc = 0) {
  constexpr uint32_t kDescHi = (uint32_t)(1024 >> 4) | (1u << 14) | (2u << 29);
  if (ACC == 2) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        ".reg .b64 bd;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 bd, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], bd, %4, p;\n\t"
        "}\n" ::"r"(d_tmem),
        "r"(a_tmem), "r"(b_lo), "r"(kDescHi), "r"(idesc), "r"(acc)
        : "memory");
  } else {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        ".reg .b64 bd;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 bd, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], bd, %4, p;\n\t"
        "}\n" ::"r"(d_tmem),
        "r"(a_tmem), "r"(b_lo), "r"(kDescHi), "r"(idesc), "n"(ACC)
        : "memory");
  }
}
// Arrives on `bar` once every MMA issued so far by this thread has finished.
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// 8 consecutive 32-bit columns of this thread's lane of tensor memory (no wait).
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]),
               "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}

// 8 nibbles -> four bf16 pairs holding the codes (nibble - 8) of elements (0,4) (1,5) (2,6) (3,7):
// 0x4300 | nibble is the bf16 number 128 + nibble, and 136 is subtracted exactly.  The activation
// images use the same order of K inside every 8 elements.
__device__ __forceinline__ void unpack8(uint32_t word, uint32_t* out4) {
  const __nv_bfloat162 off = __floats2bfloat162_rn(136.f, 136.f);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint32_t v = ((word >> (4 * i)) & 0x000F000Fu) | 0x43004300u;
    __nv_bfloat162 b = __hsub2(*reinterpret_cast<__nv_bfloat162*>(&v), off);
    out4[i] = *reinterpret_cast<uint32_t*>(&b);
  }
}

struct IssueCtx {
  uint64_t *full_a, *full_b, *empty, *acc_full, *acc_empty, *drained;   // drained: one per issuer
  volatile int* s_abort;
  uint32_t tmem, a_cols, acc_base, acc_cols, b_lo0, stage16, piece16, mp, idesc;
  int nchunks, slots, nw, stages, qsplit;
};

// One MMA-issuing thread.  With four accumulator slots issuer i owns slot i and takes the groups of K whose
// number is i modulo 4, both matrices of a pair.  With two slots (a pair at 48 or 64 activation rows) four
// issuers still work: issuer i owns slot i & 1 and only matrix i >> 1 (QSPLIT); the slot's "group done" barrier
// then counts two commits.  SPG (K16 steps per group: 2, 4 or 8) is a template parameter so that the unrolled
// body knows at compile time where a group starts and ends; descriptors are a constant upper word and a lower
// word that only takes additions.  An issuer skips the stages that hold none of its groups; a stage's "free"
// barrier counts the issuers that do work in it.
template <int SPG, int NW, bool QSPLIT>
__device__ __forceinline__ void issue_loop(const IssueCtx& x, const uint32_t me) {
  const uint32_t nslots = (uint32_t)x.slots;
  const uint32_t my_slot = QSPLIT ? (me & 1u) : me;
  const int q0 = QSPLIT ? (int)(me >> 1) : 0, q1 = QSPLIT ? q0 + 1 : NW;
  const uint32_t d_base = x.tmem + x.acc_base + my_slot * x.acc_cols;
  uint64_t* my_full = &x.acc_full[my_slot];
  uint64_t* my_empty = &x.acc_empty[my_slot];
  const uint32_t stage_mask = (uint32_t)x.stages - 1, stage_shift = x.stages == 8 ? 3u : 2u;
  uint32_t visits = 0;   // groups this issuer has started
  bool ok = true;
  for (int c = 0; c < x.nchunks && ok; ++c) {
    {  // first and last group of this stage: is one of them mine?
      const uint32_t g0 = ((uint32_t)c * (kKC / 16)) / SPG, g1 = ((uint32_t)c * (kKC / 16) + 3) / SPG;
      if ((g0 & (nslots - 1)) != my_slot && (g1 & (nslots - 1)) != my_slot) continue;
    }
    const uint32_t s = (uint32_t)c & stage_mask, par = ((uint32_t)c >> stage_shift) & 1u;
    ok = mbar_wait_fast(&x.full_a[s], par, x.s_abort) && mbar_wait_fast(&x.full_b[s], par, x.s_abort);
    if (!ok) break;
    tc_fence_after();
    const uint32_t b_lo = x.b_lo0 + s * x.stage16;
    const uint32_t a_base = x.tmem + s * x.a_cols;
#pragma unroll
    for (int ks = 0; ks < kKC / 16; ++ks) {   // 16 bf16 = 32 bytes of a row = 8 columns of tensor memory per MMA
      const uint32_t t = (uint32_t)c * (kKC / 16) + ks;            // K16 step of this CTA
      const uint32_t gi = SPG == 2 ? t >> 1 : (SPG == 4 ? t >> 2 : t >> 3);
      if ((gi & (nslots - 1)) != my_slot) continue;
      // SPG 2: groups start at ks 0 and 2; SPG 4: at ks 0; SPG 8: at ks 0 of every other chunk
      const bool starts = SPG == 2 ? (ks % 2 == 0) : (SPG == 4 ? ks == 0 : (ks == 0 && (c & 1) == 0));
      const bool ends = SPG == 2 ? (ks % 2 == 1) : (SPG == 4 ? ks == 3 : (ks == 3 && (c & 1) == 1));
      if (starts) {
        if (visits > 0) {          // the epilogue must have read this slot's previous sums
          ok = mbar_wait_fast(my_empty, (visits - 1u) & 1u, x.s_abort);
          if (!ok) break;
          tc_fence_after();
        }
        ++visits;
      }
#pragma unroll
      for (int pc = 0; pc < kPieces; ++pc)
#pragma unroll
        for (int q = 0; q < NW; ++q) {
          if (q < q0 || q >= q1) continue;
          const uint32_t d = d_base + (uint32_t)q * x.mp, a = a_base + (uint32_t)(q * 32 + ks * 8);
          const uint32_t b = b_lo + (uint32_t)(ks * 2) + (uint32_t)pc * x.piece16;
          if (pc > 0) mma_bf16_ts<1>(d, a, b, x.idesc);
          else if (SPG == 8 && ks == 0) mma_bf16_ts<2>(d, a, b, x.idesc, (uint32_t)(c & 1));
          else if ((SPG == 2 && ks % 2 == 0) || (SPG == 4 && ks == 0)) mma_bf16_ts<0>(d, a, b, x.idesc);
          else mma_bf16_ts<1>(d, a, b, x.idesc);
        }
      if (ends) mma_commit(my_full);
    }
    mma_commit(&x.empty[s]);   // the stage is free once every issuer's MMAs have read it
  }
  // nothing may still be running on the tensor core when the tensor memory is given back
  mma_commit(&x.drained[me]);
  mbar_wait_fast(&x.drained[me], 0u, x.s_abort);
}

// MP: activation rows padded to a multiple of 16; NW: 1 matrix or a gate/up pair.  Template parameters keep
// each variant's loops exactly as long as they need to be (the roles' loop bodies must stay in the
// instruction cache) and its accumulator registers as few.
// DW: unpacking warps, 4 or 8 (two teams that take every other stage; 20 warps leave 96 registers per thread, which
// the single-matrix variants fit).
template <int MP, int NW, int DW>
__global__ void __launch_bounds__((DW + 12) * 32, 1) w4_tc5_kernel(const Tc5Params p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t full_a[kMaxStages], full_b[kMaxStages], empty[kMaxStages], acc_full[4], acc_empty[4], drained[4];
  __shared__ uint32_t s_tmem;
  __shared__ int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b_bytes = kPieces * MP * 128;             // the images of the activations per stage
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int n0 = (int)blockIdx.x * kTileN;
  const int k0 = (int)blockIdx.y * p.kper;
  const int nchunks = p.kper / kKC;
  const int ngroups = p.kper / p.g;
  const int slots = p.slots;
  constexpr int kStages = NW == 1 ? 8 : 4;
  const bool qsplit = NW == 2 && slots == 2;   // two slots: the four issuers split by matrix as well
  // tensor memory columns: [stage][matrix] 32 columns of codes (64 bf16), then [slot][matrix] mp columns of sums
  const uint32_t a_cols = 32u * NW, acc_base = kStages * a_cols, acc_cols = (uint32_t)(MP * NW);

  if (tid == 0) {
    s_abort = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_a[s], 4);    // one lane of each unpacking warp
      mbar_init(&full_b[s], 1);
      mbar_init(&empty[s], (p.g == 32 ? 2u : 1u) * (qsplit ? 2u : 1u));   // the issuers of the stage's groups commit to it
    }
    for (int s = 0; s < 4; ++s) {
      mbar_init(&acc_full[s], qsplit ? 2u : 1u);
      mbar_init(&acc_empty[s], 8);  // one lane of each epilogue warp
    }
    for (int s = 0; s < 4; ++s) mbar_init(&drained[s], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  constexpr int kIssue0 = DW + 8;   // first issuing warp
  if (warp == kIssue0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem;

  if (warp >= kIssue0) {
    // ---------------- MMA issue ----------------
    if (lane == 0 && (warp - kIssue0 < slots || qsplit)) {
      IssueCtx x;
      x.full_a = full_a; x.full_b = full_b; x.empty = empty; x.acc_full = acc_full; x.acc_empty = acc_empty; x.drained = drained;
      x.s_abort = &s_abort;
      x.tmem = tmem; x.a_cols = a_cols; x.acc_base = acc_base; x.acc_cols = acc_cols;
      x.b_lo0 = (smem_u32(smem) >> 4) | (1u << 16);
      x.stage16 = (uint32_t)b_bytes >> 4;
      x.piece16 = (uint32_t)(MP * 128) >> 4;
      x.mp = (uint32_t)MP;
      // instruction descriptor: fp32 accumulator, bf16 x bf16, B K-major, N = mp, M = 128
      x.idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(MP >> 3) << 17) | ((uint32_t)(kTileN >> 4) << 24);
      x.nchunks = nchunks; x.slots = slots; x.nw = NW; x.stages = kStages; x.qsplit = qsplit ? 1 : 0;
      const uint32_t me = (uint32_t)(warp - kIssue0);
      if (NW == 2 && qsplit) {
        if (p.g == 32) issue_loop<2, NW, NW == 2>(x, me);
        else if (p.g == 64) issue_loop<4, NW, NW == 2>(x, me);
        else issue_loop<8, NW, NW == 2>(x, me);
      } else {
        if (p.g == 32) issue_loop<2, NW, false>(x, me);
        else if (p.g == 64) issue_loop<4, NW, false>(x, me);
        else issue_loop<8, NW, false>(x, me);
      }
    }
  } else if (warp < DW) {
    // ---------------- unpacking: thread = weight row; with 8 warps two teams take every other stage ----------------
    constexpr int TS = DW / 4;                 // teams
    constexpr int PD = kAhead / TS - 1;        // own chunks in flight
    const int team = warp >> 2, row = tid & 127;
    const int j = n0 + row;
    const bool live = j < p.n;
    const size_t roff = (size_t)(live ? j : 0) * (size_t)(p.k >> 1) + (size_t)(k0 >> 1);
    const uint8_t* w0 = p.w[0] + roff;
    const uint8_t* w1 = (NW == 2 ? p.w[1] : p.w[0]) + roff;
    const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    // the thread's ring: [slot][matrix][row][32 bytes], the two 16-byte halves swapped for rows 4..7 of
    // every 8 so that a quarter warp touches every bank once
    const uint32_t ring = smem_u32(smem + (size_t)kStages * b_bytes);
    const uint32_t flip = (uint32_t)((row >> 2) & 1) * 16u;
    auto slot_addr = [&](int c, int q) { return ring + (uint32_t)(((c % kAhead) * NW + q) * kTileN + row) * 32u; };
    auto fetch = [&](int c) {
      if (live && c < nchunks) {
        for (int q = 0; q < NW; ++q) {
          const uint8_t* src = (q ? w1 : w0) + (size_t)c * 32;
          const uint32_t dst = slot_addr(c, q);
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + flip), "l"(src) : "memory");
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + (flip ^ 16u)), "l"(src + 16) : "memory");
        }
      }
      asm volatile("cp.async.commit_group;" ::: "memory");   // one group per chunk, empty ones included
    };
    for (int i = 0; i < PD; ++i) fetch(team + i * TS);
    for (int c = team; c < nchunks; c += TS) {
      fetch(c + PD * TS);
      asm volatile("cp.async.wait_group %0;" ::"n"(PD) : "memory");   // chunk c has landed
      const int s = c % kStages;
      if (c >= kStages && !mbar_wait_warp(&empty[s], (uint32_t)(c / kStages - 1) & 1u, &s_abort)) break;
      if (row == 0) {   // the stage's activation images: one bulk copy
        mbar_expect_tx(&full_b[s], (uint32_t)b_bytes);
        bulk_g2s(smem + (size_t)s * b_bytes, p.xq + (size_t)(k0 / kKC + c) * b_bytes, (uint32_t)b_bytes, &full_b[s]);
      }
      tc_fence_after();
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        if (q < NW) {
          const uint32_t src = slot_addr(c, q);
#pragma unroll
          for (int h = 0; h < 2; ++h) {   // 32 elements = 16 columns per 16 bytes of nibbles
            uint32_t wd[4] = {0x88888888u, 0x88888888u, 0x88888888u, 0x88888888u};  // code 0 for rows past n
            if (live)
              asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(wd[0]), "=r"(wd[1]), "=r"(wd[2]), "=r"(wd[3]) : "r"(src + ((uint32_t)h * 16u ^ flip)));
            uint32_t v[16];
#pragma unroll
            for (int t = 0; t < 4; ++t) unpack8(wd[t], &v[4 * t]);
            const uint32_t col = lane_base + (uint32_t)s * a_cols + (uint32_t)q * 32u + (uint32_t)h * 16u;
            const uint32_t lo[8] = {v[0], v[1], v[2], v[3], v[4], v[5], v[6], v[7]};
            const uint32_t hi[8] = {v[8], v[9], v[10], v[11], v[12], v[13], v[14], v[15]};
            tmem_st8(col, lo);
            tmem_st8(col + 8, hi);
          }
        }
      }
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&full_a[s]);
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
  } else {
    // ---------------- per-group scaling and the epilogue: thread = weight row, team = half of the activation rows ----------------
    const int team = (warp - DW) >> 2, row = tid & 127;
    const int j = n0 + row;
    const bool live = j < p.n;
    const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    constexpr int half = MP >> 1;               // 8, 16, 24 or 32 activation rows per team
    constexpr int units = half >> 3;            // in blocks of 8 columns
    const int cb = team * half;
    const float* s0 = p.scales[0] + (size_t)(live ? j : 0) * p.ng + k0 / p.g;
    const float* s1 = (NW == 2 ? p.scales[1] : p.scales[0]) + (size_t)(live ? j : 0) * p.ng + k0 / p.g;
    float acc[NW][half];
#pragma unroll
    for (int q = 0; q < NW; ++q)
#pragma unroll
      for (int i = 0; i < half; ++i) acc[q][i] = 0.f;
    bool ok = true;
    // Four slots and 32-element groups: TWO groups (one 64-element stage) per visit - one wait for both slots, all
    // their loads in flight at once (64 registers at most), one hand-back.  The fixed cost of a visit (barrier,
    // tcgen05.ld latency, fences, arrival: ~400 cycles whatever the number of activation rows) is what bounds
    // the kernel at few rows; the groups of a stage finish together anyway.
    const bool two_per_visit = slots == 4 && p.g == 32;
    if constexpr (units * NW <= 4) {
      if (two_per_visit) {
        float2 sa = live ? __ldg(reinterpret_cast<const float2*>(s0)) : make_float2(0.f, 0.f);
        float2 sb = (live && NW == 2) ? __ldg(reinterpret_cast<const float2*>(s1)) : make_float2(0.f, 0.f);
        for (int gi = 0; gi < ngroups && ok; gi += 2) {
          const float2 ca = sa, cb2 = sb;
          if (gi + 2 < ngroups) {
            sa = live ? __ldg(reinterpret_cast<const float2*>(s0 + gi + 2)) : make_float2(0.f, 0.f);
            if (NW == 2) sb = live ? __ldg(reinterpret_cast<const float2*>(s1 + gi + 2)) : make_float2(0.f, 0.f);
          }
          const int slot = gi & 3;   // 0 or 2: this visit takes slots slot and slot + 1
          const uint32_t par = (uint32_t)(gi >> 2) & 1u;
          ok = mbar_wait_warp(&acc_full[slot], par, &s_abort) && mbar_wait_warp(&acc_full[slot + 1], par, &s_abort);
          if (!ok) break;
          tc_fence_after();
          const uint32_t d = lane_base + acc_base + (uint32_t)slot * acc_cols + (uint32_t)cb;
          uint32_t r[2][NW][units][8];
#pragma unroll
          for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int q = 0; q < NW; ++q)
#pragma unroll
              for (int u = 0; u < units; ++u) tmem_ld8(d + (uint32_t)h * acc_cols + (uint32_t)(q * MP + u * 8), r[h][q][u]);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          tc_fence_before();
          __syncwarp();
          if (lane == 0) { mbar_arrive(&acc_empty[slot]); mbar_arrive(&acc_empty[slot + 1]); }
#pragma unroll
          for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int q = 0; q < NW; ++q) {
              const float cq = q ? (h ? cb2.y : cb2.x) : (h ? ca.y : ca.x);
#pragma unroll
              for (int u = 0; u < units; ++u)
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[q][u * 8 + i] = fmaf(cq, __uint_as_float(r[h][q][u][i]), acc[q][u * 8 + i]);
            }
        }
      }
    }
    float sc0 = live ? __ldg(s0) : 0.f, sc1 = (live && NW == 2) ? __ldg(s1) : 0.f;
    for (int gi = 0; gi < ngroups && !(two_per_visit && units * NW <= 4); ++gi) {
      const float c0 = sc0, c1 = sc1;
      if (gi + 1 < ngroups) {
        sc0 = live ? __ldg(s0 + gi + 1) : 0.f;
        if (NW == 2) sc1 = live ? __ldg(s1 + gi + 1) : 0.f;
      }
      const int slot = gi % slots;
      ok = mbar_wait_warp(&acc_full[slot], (uint32_t)(gi / slots) & 1u, &s_abort);
      if (!ok) break;
      tc_fence_after();
      const uint32_t d = lane_base + acc_base + (uint32_t)slot * acc_cols + (uint32_t)cb;
      if constexpr (units * NW <= 4) {
        // every load of the group is in flight at once (32 registers at most)
        uint32_t r[NW][units][8];
#pragma unroll
        for (int q = 0; q < NW; ++q)
#pragma unroll
          for (int u = 0; u < units; ++u) tmem_ld8(d + (uint32_t)(q * MP + u * 8), r[q][u]);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[slot]);   // the slot's sums are in registers: hand it back before the arithmetic
#pragma unroll
        for (int q = 0; q < NW; ++q) {
          const float cq = q ? c1 : c0;
#pragma unroll
          for (int u = 0; u < units; ++u)
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[q][u * 8 + i] = fmaf(cq, __uint_as_float(r[q][u][i]), acc[q][u * 8 + i]);
        }
      } else {
#pragma unroll
        for (int q = 0; q < NW; ++q) {
          uint32_t r[units][8];
#pragma unroll
          for (int u = 0; u < units; ++u) tmem_ld8(d + (uint32_t)(q * MP + u * 8), r[u]);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          if (q == NW - 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[slot]);
          }
          const float cq = q ? c1 : c0;
#pragma unroll
          for (int u = 0; u < units; ++u)
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[q][u * 8 + i] = fmaf(cq, __uint_as_float(r[u][i]), acc[q][u * 8 + i]);
        }
      }
    }
    if (ok && live) {
      const float b0 = (p.bias[0] && blockIdx.y == 0) ? __ldg(p.bias[0] + j) : 0.f;
      const float b1 = (NW == 2 && p.bias[1]) ? __ldg(p.bias[1] + j) : 0.f;
#pragma unroll
      for (int i = 0; i < half; ++i) {
        const int mrow = cb + i;
        if (mrow < p.m) {
          float v;
          if (NW == 2) {
            const float gg = acc[0][i] + b0, uu = acc[NW - 1][i] + b1;
            v = (gg / (1.0f + expf(-gg))) * uu;   // src/llm/decoder.rs:1319-1322
          } else {
            v = acc[0][i] + b0;
            if (p.resid && blockIdx.y == 0) v += p.resid[(size_t)mrow * p.n + j];
          }
          float* dst = p.out + (size_t)mrow * p.n + j;
          if (p.ksplit > 1) atomicAdd(dst, v);
          else *dst = v;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kIssue0) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
}

// Activations -> kPieces bf16 images per 64-element chunk of K (with the fused RMSNorm).  Inside
// every 8 elements the order is 0 4 1 5 2 6 3 7, the order in which the codes leave a 32-bit
// word of nibbles.  grid (mp rows, ceil(k / 2048)); rows past m are zero.
__global__ void __launch_bounds__(256) tc5_prep_kernel(const float* __restrict__ x, const float* __restrict__ norm_w, float eps,
                                                       unsigned char* __restrict__ xq, int m, int mp, int k) {
  __shared__ float s_part[8];
  const int row = blockIdx.x, tid = threadIdx.x;
  float inv = 1.f;
  if (norm_w != nullptr && row < m) {   // fast_rms_norm, src/quantization/fused_ops.rs:1066-1117
    const float* xr = x + (size_t)row * k;
    float ss = 0.f;
    for (int i = tid; i < k; i += 256) ss = fmaf(xr[i], xr[i], ss);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((tid & 31) == 0) s_part[tid >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += s_part[i];
    inv = 1.0f / sqrtf(tot / (float)k + eps);
  }
  // one thread = 8 consecutive elements = one 16-byte piece of an image row
  const int e = (int)blockIdx.y * 2048 + tid * 8;
  if (e >= k) return;
  float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (row < m) {
    const float4 a = *reinterpret_cast<const float4*>(x + (size_t)row * k + e);
    const float4 b = *reinterpret_cast<const float4*>(x + (size_t)row * k + e + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    if (norm_w != nullptr) {
      const float4 na = *reinterpret_cast<const float4*>(norm_w + e);
      const float4 nb = *reinterpret_cast<const float4*>(norm_w + e + 4);
      const float nw[8] = {na.x, na.y, na.z, na.w, nb.x, nb.y, nb.z, nb.w};
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = (v[i] * inv) * nw[i];
    }
  }
  uint32_t img[kPieces][4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {   // the pair (i, i + 4)
    float r0 = v[i], r1 = v[i + 4];
#pragma unroll
    for (int pc = 0; pc < kPieces; ++pc) {
      uint32_t h0, h1;
      if (pc + 1 < kPieces) {     // the upper 16 bits are a bf16 number; the remainder is exact
        h0 = __float_as_uint(r0) & 0xFFFF0000u;
        h1 = __float_as_uint(r1) & 0xFFFF0000u;
        r0 -= __uint_as_float(h0);
        r1 -= __uint_as_float(h1);
      } else {                    // the last piece is rounded
        h0 = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(r0)) << 16;
        h1 = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(r1)) << 16;
      }
      img[pc][i] = (h0 >> 16) | h1;
    }
  }
  const int c = e >> 6, jp = (e >> 3) & 7;
  unsigned char* dst = xq + (size_t)c * (kPieces * mp * 128) + row * 128 + ((jp ^ (row & 7)) * 16);
#pragma unroll
  for (int pc = 0; pc < kPieces; ++pc)
    *reinterpret_cast<uint4*>(dst + (size_t)pc * mp * 128) = make_uint4(img[pc][0], img[pc][1], img[pc][2], img[pc][3]);
}

int g_tc5_enabled = 1;

}  // namespace

void set_tc5_enabled(int on) { g_tc5_enabled = on; }

int tc5_fault_flag() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_tc5_fault, sizeof(int)) != cudaSuccess) return -1;
  return v;
}

size_t w4_tc5_scratch_bytes(int m, int64_t k) {
  const int mp = ((m < 64 ? m : 64) + 15) & ~15;
  return (size_t)((k + kKC - 1) / kKC) * kPieces * mp * 128;
}

bool w4_tc5_supported(const GemvArgs& a) {
  if (!g_tc5_enabled || a.m < kMinRows) return false;
  if (a.k % 128 != 0 || a.n < 1 || (a.g != 32 && a.g != 64 && a.g != 128)) return false;
  if (a.x_ss8 || a.out_scaled || a.out_ss8 || a.x_normed_out) return false;
  if ((reinterpret_cast<uintptr_t>(a.w) & 15) || (a.w2 && (reinterpret_cast<uintptr_t>(a.w2) & 15))) return false;
  return true;
}

tb_status launch_w4_tc5(const GemvArgs& a, void* scratch, cudaStream_t stream) {
  if (!w4_tc5_supported(a)) return fail(TB_ERR_UNSUPPORTED, "TB_UNSUPPORTED: tcgen05 product: m=%d n=%lld k=%lld", a.m, (long long)a.n, (long long)a.k);
  const bool pair = a.w2 != nullptr;
  const int tiles = (int)((a.n + kTileN - 1) / kTileN);
  for (int m0 = 0; m0 < a.m; m0 += 64) {
    const int mc = a.m - m0 < 64 ? a.m - m0 : 64;
    const int mp = (mc + 15) & ~15;
    Tc5Params p;
    p.w[0] = a.w; p.w[1] = a.w2; p.scales[0] = a.scales; p.scales[1] = a.scales2; p.bias[0] = a.bias; p.bias[1] = a.bias2;
    // residual in place (out == resid) with K split: the partial sums are added onto the residual where it lies
    const bool in_place = a.resid != nullptr && a.resid == a.out;
    p.resid = a.resid ? a.resid + (size_t)m0 * a.n : nullptr;
    p.out = a.out + (size_t)m0 * a.n;
    p.xq = static_cast<const unsigned char*>(scratch);
    p.m = mc; p.mp = mp; p.n = (int)a.n; p.k = (int)a.k; p.ng = (int)(a.k / a.g); p.g = a.g;
    p.pair = pair ? 1 : 0;
    // narrow matrices: several CTAs share a row tile and split K (the SwiGLU needs whole sums: no split)
    int ksplit = 1;
    if (!pair) {
      const int want = sm_count() / tiles;
      for (int s = want; s >= 2; --s)
        if ((a.k / 128) % s == 0) { ksplit = s; break; }
    }
    p.ksplit = ksplit;
    p.kper = (int)(a.k / ksplit);
    const int nw = pair ? 2 : 1;
    const int stages = nw == 1 ? 8 : 4;
    p.stages = stages;
    const int slots = (kTmemCols - stages * 32 * nw) / (mp * nw);
    p.slots = slots >= 4 ? 4 : 2;   // a power of two (the issuing thread masks and shifts)
    const size_t smem = (size_t)stages * kPieces * mp * 128 + (size_t)kAhead * nw * kTileN * 32 + 1024;
    void (*kern)(const Tc5Params) = nullptr;
    int threads = 16 * 32;
    switch (mp * 2 + (pair ? 1 : 0)) {
      case 32: kern = w4_tc5_kernel<16, 1, 8>; threads = 20 * 32; break;
      case 33: kern = w4_tc5_kernel<16, 2, 8>; threads = 20 * 32; break;
      case 64: kern = w4_tc5_kernel<32, 1, 8>; threads = 20 * 32; break;
      case 65: kern = w4_tc5_kernel<32, 2, 4>; break;
      case 96: kern = w4_tc5_kernel<48, 1, 8>; threads = 20 * 32; break;
      case 97: kern = w4_tc5_kernel<48, 2, 4>; break;
      case 128: kern = w4_tc5_kernel<64, 1, 8>; threads = 20 * 32; break;
      default: kern = w4_tc5_kernel<64, 2, 4>; break;
    }
    TB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    tc5_prep_kernel<<<dim3((unsigned)mp, (unsigned)((a.k + 2047) / 2048)), 256, 0, stream>>>(
        a.x + (size_t)m0 * a.k, a.norm_w, a.eps, static_cast<unsigned char*>(scratch), mc, mp, (int)a.k);
    TB_CUDA_TRY(cudaGetLastError());
    if (ksplit > 1 && in_place) p.resid = nullptr;
    else if (ksplit > 1) TB_CUDA_TRY(cudaMemsetAsync(p.out, 0, sizeof(float) * (size_t)mc * a.n, stream));
    kern<<<dim3((unsigned)tiles, (unsigned)ksplit), threads, smem, stream>>>(p);
    TB_CUDA_TRY(cudaGetLastError());
  }
  return TB_OK;
}

}  // namespace tb
