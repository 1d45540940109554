// GQA decode attention over the fp32 KV cache: RoPE + KV append + split-K
// flash-decode + merge, one launch.
//
// Replaces steps C-E of RustQwenDecoder::step_internal (src/llm/decoder.rs:1127-1213;
// rope_apply_head :28-68) and the wgpu shaders rope_append.wgsl / attn_decode.wgsl.
//
// The reference walks the sequence serially per q head with a two-pass softmax.
// Here the sequence of every (sequence, kv head) is cut into chunks of `tc`
// positions, one CTA per chunk (each warp streaming its own rows straight into registers); the CTA serves all q heads that share the kv
// head, so each K/V row is read from HBM once per step.  Every CTA writes an
// un-normalised partial (max, sum, weighted V) to scratch; the last CTA of a
// (sequence, kv head) to finish - found with a ticket counter - rescales and
// sums the partials.  The result equals the two-pass softmax up to fp32
// rounding.  HBM-bound: algorithmic bytes = 2 * Hkv * (offset+1) * d * 4 per
// sequence and layer.
#include "tb_common.cuh"

namespace tb {

namespace {

constexpr int kAttnWarps = 8;
constexpr int kAttnThreads = kAttnWarps * 32;
constexpr int kMaxGq = 8;         // q heads per kv head
constexpr int kSeqCap = 32768;    // src/llm/decoder.rs:1180
constexpr uint32_t kWaitLimit = 1u << 22;  // mbarrier polls before a tile load is declared lost

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
  int* counters;    // [b, Hkv] tickets, then one error word
  int* err;
  float* qkv_rot_out;
  int num_heads, num_kv_heads, gq;
  int tc, nc;
  int64_t max_seq_len;
  int per_call_tables;
  float scale;
  PrefetchList prefetch;
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
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst_smem)),
      "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
// Bounded wait for phase `parity`; false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t addr = smem_u32(bar);
  for (uint32_t i = 0; i < kWaitLimit; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(addr), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
}

// rotate-half with separately rounded products, src/llm/decoder.rs:40-66:
//   o[i]      = x[i]*cos[i]          - x[i+half]*sin[i]
//   o[i+half] = x[i+half]*cos[i+half] + x[i]*sin[i+half]
__device__ __forceinline__ float rope_elem(const float* x, const float* c, const float* s, int i,
                                           int half) {
  if (i < half) return __fsub_rn(__fmul_rn(x[i], c[i]), __fmul_rn(x[i + half], s[i]));
  return __fadd_rn(__fmul_rn(x[i], c[i]), __fmul_rn(x[i - half], s[i]));
}

// Shared memory (floats): q_s [gq][D] | kv_new [2][D] | w_acc [8][gq][D] | w_ml [8][gq][2] |
// wts [gq][nc] | red [1024*gq] | ml [2*gq]   (the last three are used by the merge).  Every
// region starts on a 16-byte boundary (float4 accesses).
__host__ __device__ inline size_t attn_smem_floats(int D, int nc, int gq) {
  return (size_t)gq * D + 2 * D + (size_t)kAttnWarps * gq * D + (size_t)((kAttnWarps * gq * 2 + 3) & ~3) +
         (size_t)((gq * nc + 3) & ~3) + (size_t)1024 * gq + 2 * gq;
}

__device__ __forceinline__ float4 ldg_stream_f4(const float4* p) {
  float4 v;
  asm volatile("ld.global.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p));
  return v;
}

// One CTA = one chunk of tc positions of one (sequence, kv head).  Inside the CTA every warp is
// on its own: in each pass it takes 8 rows of the chunk, loads their K and V rows straight into
// registers (all 16 KB requested before anything is consumed), scores them for the gq query
// heads (8 lanes per row, shuffle reduction), keeps an online softmax (running max / sum) and
// accumulates the weighted V with one float4 column per lane.  No block-wide barrier sits in
// that loop; the warps meet once to combine their (max, sum, acc) triples.
template <int D>
__global__ void __launch_bounds__(kAttnThreads, 2) attn_decode_kernel(const AttnParams p) {
  constexpr int F4 = D / 32;        // float4 per lane and row in the score phase (8 lanes per row)
  constexpr int CPR = D / 4;        // float4 columns per row
  constexpr int RPL = 32 / CPR;     // rows per warp-wide load in the V phase
  constexpr int VL = 8 / RPL;       // V loads per lane and pass
  constexpr int SL = kAttnThreads / CPR;  // chunk slices in the merge
  static_assert(D == 32 || D == 64 || D == 128, "head_dim");

  extern __shared__ __align__(128) float smem[];
  const int gq = p.gq, tc = p.tc;
  float* q_s = smem;
  float* kv_new = q_s + gq * D;
  float* w_acc = kv_new + 2 * D;
  float* w_ml = w_acc + (size_t)kAttnWarps * gq * D;
  float* wts = w_ml + ((kAttnWarps * gq * 2 + 3) & ~3);
  float* red = wts + (((size_t)gq * p.nc + 3) & ~(size_t)3);
  float* ml = red + 1024 * gq;
  __shared__ int s_last;

  const int chunk = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int qkv_dim = (p.num_heads + 2 * p.num_kv_heads) * D;

  if (tid == 32)
    prefetch_l2_slice(p.prefetch, (int)(blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z)),
                      (int)(gridDim.x * gridDim.y * gridDim.z));
  pdl_wait();
  pdl_launch_dependents();

  const int off = p.offsets[b];
  const bool seq_ok = off >= 0 && (int64_t)off < p.max_seq_len;
  const int t_end = seq_ok ? min(off + 1, kSeqCap) : 0;  // attend to [0, t_end)
  const int t0 = chunk * tc;
  const int nvalid_chunks = (t_end + tc - 1) / tc;
  const bool active = t0 < t_end;
  const int rows = active ? min(tc, t_end - t0) : 0;
  float* kc = p.k_cache + ((int64_t)b * p.num_kv_heads + kvh) * p.max_seq_len * D;
  float* vc = p.v_cache + ((int64_t)b * p.num_kv_heads + kvh) * p.max_seq_len * D;
  const float* qkv_b = p.qkv + (int64_t)b * qkv_dim;

  if (active) {
    const float* cs = p.cos_t + (p.per_call_tables ? (int64_t)b * D : (int64_t)off * D);
    const float* sn = p.sin_t + (p.per_call_tables ? (int64_t)b * D : (int64_t)off * D);
    // q heads of this kv head, rotated, into shared memory.
    for (int i = tid; i < gq * D; i += kAttnThreads) {
      const int g = i / D, e = i - g * D;
      const float* xh = qkv_b + (int64_t)(kvh * gq + g) * D;
      const float v = rope_elem(xh, cs, sn, e, D / 2);
      q_s[g * D + e] = v;
      if (p.qkv_rot_out && chunk == 0)
        p.qkv_rot_out[(int64_t)b * qkv_dim + (int64_t)(kvh * gq + g) * D + e] = v;
    }
    // The chunk that holds position `off` appends the new k (rotated) and v to the cache and
    // keeps a copy: its rows are read below while that store may still be in flight.
    const int new_row = off - t0;  // in [0, tc) only for that chunk
    if (new_row >= 0 && new_row < tc) {
      const float* kx = qkv_b + (int64_t)p.num_heads * D + (int64_t)kvh * D;
      const float* vx = kx + (int64_t)p.num_kv_heads * D;
      for (int e = tid; e < D; e += kAttnThreads) {
        const float kr = rope_elem(kx, cs, sn, e, D / 2);
        const float vr = vx[e];
        kc[(int64_t)off * D + e] = kr;
        vc[(int64_t)off * D + e] = vr;
        kv_new[e] = kr;
        kv_new[D + e] = vr;
        if (p.qkv_rot_out) {
          float* o = p.qkv_rot_out + (int64_t)b * qkv_dim + (int64_t)p.num_heads * D + (int64_t)kvh * D;
          o[e] = kr;
          o[(int64_t)p.num_kv_heads * D + e] = vr;
        }
      }
    }
    __syncthreads();

    const int l8 = lane & 7, rsub = lane >> 3;   // score phase: 8 lanes per row, 4 rows per group
    const int vc4 = lane % CPR, vrs = lane / CPR; // V phase: one float4 column per lane
    float m_run[kMaxGq], l_run[kMaxGq];
    float4 acc[kMaxGq];
#pragma unroll
    for (int g = 0; g < kMaxGq; ++g) {
      m_run[g] = -INFINITY;
      l_run[g] = 0.f;
      acc[g] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (int base = warp * 8; base < rows; base += kAttnWarps * 8) {
      // ---- request the 8 K rows and 8 V rows of this pass ----
      float4 kreg[2][F4];
      float4 vreg[VL];
#pragma unroll
      for (int rg = 0; rg < 2; ++rg) {
        const int r = base + rg * 4 + rsub;
        const float4* krow = reinterpret_cast<const float4*>(kc + (int64_t)(t0 + (r < rows ? r : 0)) * D);
#pragma unroll
        for (int i = 0; i < F4; ++i) kreg[rg][i] = ldg_stream_f4(krow + l8 + 8 * i);
      }
#pragma unroll
      for (int j = 0; j < VL; ++j) {
        const int r = base + j * RPL + vrs;
        vreg[j] = ldg_stream_f4(reinterpret_cast<const float4*>(vc + (int64_t)(t0 + (r < rows ? r : 0)) * D) + vc4);
      }
      // the freshly appended row comes from shared memory
      if (new_row >= base && new_row < base + 8) {
#pragma unroll
        for (int rg = 0; rg < 2; ++rg)
          if (base + rg * 4 + rsub == new_row) {
#pragma unroll
            for (int i = 0; i < F4; ++i) kreg[rg][i] = reinterpret_cast<const float4*>(kv_new)[l8 + 8 * i];
          }
#pragma unroll
        for (int j = 0; j < VL; ++j)
          if (base + j * RPL + vrs == new_row) vreg[j] = reinterpret_cast<const float4*>(kv_new + D)[vc4];
      }
      // ---- scores: sg[rg][g] = (q_g . k_row) * scale, identical in the row's 8 lanes ----
      float sg[2][kMaxGq];
#pragma unroll
      for (int rg = 0; rg < 2; ++rg) {
        const bool rv = base + rg * 4 + rsub < rows;
#pragma unroll
        for (int g = 0; g < kMaxGq; ++g) {
          float a = 0.f;
          if (g < gq) {
            const float4* q4 = reinterpret_cast<const float4*>(q_s + g * D);
#pragma unroll
            for (int i = 0; i < F4; ++i) {
              const float4 qv = q4[l8 + 8 * i];
              a = fmaf(qv.x, kreg[rg][i].x, a);
              a = fmaf(qv.y, kreg[rg][i].y, a);
              a = fmaf(qv.z, kreg[rg][i].z, a);
              a = fmaf(qv.w, kreg[rg][i].w, a);
            }
            a += __shfl_xor_sync(0xffffffffu, a, 1);
            a += __shfl_xor_sync(0xffffffffu, a, 2);
            a += __shfl_xor_sync(0xffffffffu, a, 4);
          }
          sg[rg][g] = rv ? a * p.scale : -INFINITY;
        }
      }
      // ---- online softmax over the pass's 8 rows, then the weighted V ----
#pragma unroll
      for (int g = 0; g < kMaxGq; ++g) {
        if (g < gq) {
          float mx = fmaxf(sg[0][g], sg[1][g]);
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
          const float m_new = fmaxf(m_run[g], mx);  // finite: the pass has at least one valid row
          const float resc = expf(m_run[g] - m_new); // exp(-inf) = 0 on the first pass
          const float e0 = expf(sg[0][g] - m_new), e1 = expf(sg[1][g] - m_new);
          float ps = (l8 == 0) ? e0 + e1 : 0.f;      // each row counted once
          ps += __shfl_xor_sync(0xffffffffu, ps, 8);
          ps += __shfl_xor_sync(0xffffffffu, ps, 16);
          ps += __shfl_xor_sync(0xffffffffu, ps, 1);
          ps += __shfl_xor_sync(0xffffffffu, ps, 2);
          ps += __shfl_xor_sync(0xffffffffu, ps, 4);
          l_run[g] = l_run[g] * resc + ps;
          m_run[g] = m_new;
          acc[g].x *= resc; acc[g].y *= resc; acc[g].z *= resc; acc[g].w *= resc;
#pragma unroll
          for (int j = 0; j < VL; ++j) {
            const int r8 = j * RPL + vrs;                 // row of this lane's V load within the pass
            const float pw = __shfl_sync(0xffffffffu, (j * RPL) / 4 == 0 ? e0 : e1, (r8 & 3) * 8);
            acc[g].x = fmaf(pw, vreg[j].x, acc[g].x);
            acc[g].y = fmaf(pw, vreg[j].y, acc[g].y);
            acc[g].z = fmaf(pw, vreg[j].z, acc[g].z);
            acc[g].w = fmaf(pw, vreg[j].w, acc[g].w);
          }
        }
      }
    }
    // lanes that share a column (head_dim < 128) add up their rows
#pragma unroll
    for (int g = 0; g < kMaxGq; ++g) {
      if (g < gq) {
#pragma unroll
        for (int o = CPR; o < 32; o <<= 1) {
          acc[g].x += __shfl_xor_sync(0xffffffffu, acc[g].x, o);
          acc[g].y += __shfl_xor_sync(0xffffffffu, acc[g].y, o);
          acc[g].z += __shfl_xor_sync(0xffffffffu, acc[g].z, o);
          acc[g].w += __shfl_xor_sync(0xffffffffu, acc[g].w, o);
        }
        if (lane < CPR) reinterpret_cast<float4*>(w_acc + ((size_t)warp * gq + g) * D)[lane] = acc[g];
        if (lane == 0) {
          w_ml[(warp * gq + g) * 2 + 0] = m_run[g];
          w_ml[(warp * gq + g) * 2 + 1] = l_run[g];
        }
      }
    }
    __syncthreads();
    // ---- combine the 8 warps: the chunk's partial (max, sum, weighted V) ----
    for (int i = tid; i < gq * D; i += kAttnThreads) {
      const int g = i / D, e = i - g * D;
      float mx = -INFINITY;
#pragma unroll
      for (int w = 0; w < kAttnWarps; ++w) mx = fmaxf(mx, w_ml[(w * gq + g) * 2]);
      float o = 0.f, l = 0.f;
#pragma unroll
      for (int w = 0; w < kAttnWarps; ++w) {
        const float mw = w_ml[(w * gq + g) * 2];
        const float f = mw == -INFINITY ? 0.f : expf(mw - mx);  // warps without rows contribute nothing
        o = fmaf(w_acc[((size_t)w * gq + g) * D + e], f, o);
        l = fmaf(w_ml[(w * gq + g) * 2 + 1], f, l);
      }
      const int h = kvh * gq + g;
      p.part_o[(((int64_t)b * p.num_heads + h) * p.nc + chunk) * D + e] = o;
      if (e == 0) {
        float* dst = p.part_ml + (((int64_t)b * p.num_heads + h) * p.nc + chunk) * 2;
        dst[0] = mx;
        dst[1] = l;
      }
    }
  }

  // ---- ticket: the last CTA of this (sequence, kv head) merges the partials ----
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int ticket = atomicAdd(&p.counters[b * p.num_kv_heads + kvh], 1);
    s_last = (ticket == (int)gridDim.x - 1);
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  if (tid == 0) p.counters[b * p.num_kv_heads + kvh] = 0;  // ready for the next launch

  const int h0 = kvh * gq;
  if (nvalid_chunks == 0) {
    for (int i = tid; i < gq * D; i += kAttnThreads) p.out[((int64_t)b * p.num_heads + h0) * D + i] = 0.f;
    return;
  }
  // weights of every chunk: warp g owns q head g
  if (warp < gq) {
    const float* pml = p.part_ml + ((int64_t)b * p.num_heads + h0 + warp) * p.nc * 2;
    float mx = -INFINITY;
    for (int c = lane; c < nvalid_chunks; c += 32) mx = fmaxf(mx, __ldcg(pml + c * 2));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float tot = 0.f;
    for (int c = lane; c < nvalid_chunks; c += 32) {
      const float w = expf(__ldcg(pml + c * 2) - mx);
      wts[warp * p.nc + c] = w;
      tot = fmaf(__ldcg(pml + c * 2 + 1), w, tot);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
    if (lane == 0) ml[warp] = 1.0f / fmaxf(tot, 1e-30f);  // src/llm/decoder.rs:1203
  }
  __syncthreads();
  {
    const int c4 = tid % CPR, sl = tid / CPR;
    float4 acc[kMaxGq];
#pragma unroll
    for (int g = 0; g < kMaxGq; ++g) acc[g] = make_float4(0.f, 0.f, 0.f, 0.f);
    const float4* po = reinterpret_cast<const float4*>(p.part_o + ((int64_t)b * p.num_heads + h0) * p.nc * D);
    for (int c = sl; c < nvalid_chunks; c += SL) {
#pragma unroll
      for (int g = 0; g < kMaxGq; ++g) {
        if (g < gq) {
          const float4 v = __ldcg(po + ((int64_t)g * p.nc + c) * CPR + c4);
          const float w = wts[g * p.nc + c];
          acc[g].x = fmaf(w, v.x, acc[g].x);
          acc[g].y = fmaf(w, v.y, acc[g].y);
          acc[g].z = fmaf(w, v.z, acc[g].z);
          acc[g].w = fmaf(w, v.w, acc[g].w);
        }
      }
    }
#pragma unroll
    for (int g = 0; g < kMaxGq; ++g)
      if (g < gq) reinterpret_cast<float4*>(red + ((size_t)sl * gq + g) * D)[c4] = acc[g];
  }
  __syncthreads();
  for (int i = tid; i < gq * D; i += kAttnThreads) {
    const int g = i / D, e = i - g * D;
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < SL; ++w) s += red[((size_t)w * gq + g) * D + e];
    p.out[((int64_t)b * p.num_heads + h0 + g) * D + e] = s * ml[g];
  }
}

int pick_chunk(int batch, int num_kv_heads, int gq, int head_dim, int64_t max_seq_len) {
  // The smallest chunk (a multiple of the 64 rows one pass of a CTA covers) for which the
  // whole grid is resident at once (two CTAs per SM), so that no CTA waits for a second wave.
  (void)gq; (void)head_dim;
  const int64_t cols = (int64_t)batch * num_kv_heads;
  const int64_t cap = max_seq_len < kSeqCap ? max_seq_len : kSeqCap;
  int tc = 64;
  while (tc < 512 && cols * ((cap + tc - 1) / tc) > (int64_t)2 * sm_count()) tc <<= 1;
  return tc;
}

int g_chunk_override = 0;

struct AttnLayout {
  int tc, nc;
  size_t part_o, part_ml;
};

AttnLayout attn_layout(int batch, int num_heads, int num_kv_heads, int head_dim, int64_t max_seq_len) {
  AttnLayout L;
  const int gq = num_heads / num_kv_heads;
  L.tc = g_chunk_override > 0 ? g_chunk_override : pick_chunk(batch, num_kv_heads, gq, head_dim, max_seq_len);
  const int64_t cap = max_seq_len < kSeqCap ? max_seq_len : kSeqCap;
  L.nc = (int)((cap + L.tc - 1) / L.tc);
  auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
  L.part_o = up((size_t)batch * num_heads * L.nc * head_dim * sizeof(float));
  L.part_ml = up((size_t)batch * num_heads * L.nc * 2 * sizeof(float));
  return L;
}

}  // namespace

void set_attention_chunk_override(int tc) { g_chunk_override = tc; }

// Scratch = partials + ticket counters.  The counters must be zero before the
// first launch; every launch leaves them zero again.
size_t attention_scratch_bytes(int batch, int num_heads, int num_kv_heads, int head_dim,
                               int64_t max_seq_len) {
  // sized for the smallest chunk so that a later override cannot outgrow it
  const int64_t cap = max_seq_len < kSeqCap ? max_seq_len : kSeqCap;
  const int nc = (int)((cap + 31) / 32);
  auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
  return up((size_t)batch * num_heads * nc * head_dim * sizeof(float)) +
         up((size_t)batch * num_heads * nc * 2 * sizeof(float)) +
         up(((size_t)batch * num_kv_heads + 1) * sizeof(int));
}

size_t attention_counters_offset(int batch, int num_heads, int num_kv_heads, int head_dim,
                                 int64_t max_seq_len, size_t* counter_bytes) {
  const size_t total = attention_scratch_bytes(batch, num_heads, num_kv_heads, head_dim, max_seq_len);
  const size_t cb = (((size_t)batch * num_kv_heads + 1) * sizeof(int) + 255) & ~(size_t)255;
  if (counter_bytes) *counter_bytes = cb;
  return total - cb;
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

  const AttnLayout L = attn_layout(a.batch, a.num_heads, a.num_kv_heads, a.head_dim, a.max_seq_len);
  size_t cbytes = 0;
  const size_t coff = attention_counters_offset(a.batch, a.num_heads, a.num_kv_heads, a.head_dim, a.max_seq_len, &cbytes);
  AttnParams p;
  p.qkv = a.qkv; p.k_cache = a.k_cache; p.v_cache = a.v_cache;
  p.cos_t = a.cos_t; p.sin_t = a.sin_t; p.offsets = a.offsets; p.out = a.out;
  char* base = static_cast<char*>(a.scratch);
  p.part_o = reinterpret_cast<float*>(base);
  p.part_ml = reinterpret_cast<float*>(base + L.part_o);
  p.counters = reinterpret_cast<int*>(base + coff);
  p.err = p.counters + (size_t)a.batch * a.num_kv_heads;
  p.qkv_rot_out = a.q_rot_out;
  p.num_heads = a.num_heads; p.num_kv_heads = a.num_kv_heads; p.gq = gq;
  p.tc = L.tc; p.nc = L.nc;
  p.max_seq_len = a.max_seq_len;
  p.per_call_tables = a.per_call_tables ? 1 : 0;
  p.scale = 1.0f / sqrtf((float)a.head_dim);
  p.prefetch = a.prefetch;

  const int D = a.head_dim;
  if (L.tc < 64 || L.tc > 512 || (L.tc & (L.tc - 1)))
    return fail(TB_ERR_ARG, "attention: chunk %d is not a power of two in [64, 512]", L.tc);
  const size_t smem = sizeof(float) * attn_smem_floats(D, L.nc, gq);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)L.nc, (unsigned)a.num_kv_heads, (unsigned)a.batch);
  cfg.blockDim = dim3(kAttnThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = a.pdl ? 1 : 0;
  auto set_smem = [&](auto kern) -> cudaError_t {
    if (smem > 32 * 1024)
      return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return cudaSuccess;
  };
  if (D == 128) {
    TB_CUDA_TRY(set_smem(attn_decode_kernel<128>));
    TB_CUDA_TRY(cudaLaunchKernelEx(&cfg, attn_decode_kernel<128>, p));
  } else if (D == 64) {
    TB_CUDA_TRY(set_smem(attn_decode_kernel<64>));
    TB_CUDA_TRY(cudaLaunchKernelEx(&cfg, attn_decode_kernel<64>, p));
  } else {
    TB_CUDA_TRY(set_smem(attn_decode_kernel<32>));
    TB_CUDA_TRY(cudaLaunchKernelEx(&cfg, attn_decode_kernel<32>, p));
  }
  return TB_OK;
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
  static void* cached[64] = {nullptr};
  int dev = 0;
  TB_CUDA_TRY(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && cached[dev]) {
    *ptr = cached[dev];
    return TB_OK;
  }
  void* p = nullptr;
  cudaError_t e = cudaGetSymbolAddress(&p, g_static_attn_scratch);
  if (e != cudaSuccess || p == nullptr)
    return fail(TB_ERR_CUDA, "cudaGetSymbolAddress(static attention scratch) failed: %s", cudaGetErrorString(e));
  if (dev >= 0 && dev < 64) cached[dev] = p;
  *ptr = p;
  return TB_OK;
}

}  // namespace tb
