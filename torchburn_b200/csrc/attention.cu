// GQA decode attention over the fp32 KV cache: RoPE + KV append + split-K
// flash-decode + merge, one launch.
//
// Replaces steps C-E of RustQwenDecoder::step_internal (src/llm/decoder.rs:1127-1213;
// rope_apply_head :28-68) and the wgpu shaders rope_append.wgsl / attn_decode.wgsl.
//
// The reference walks the sequence serially per q head with a two-pass softmax.
// Here the sequence of every (sequence, kv head) is cut into chunks of `tc`
// positions, one CTA per chunk; the CTA serves all q heads that share the kv
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

// Shared memory (floats): K tile [tc][D] | V tile [tc][D] | q_s [gq][D] | sc [gq][tc] |
// red [1024 * gq] | ml [2 * gq].  The merge reuses the K|V tiles for its weights [gq][nc].
__host__ __device__ inline size_t attn_smem_floats(int D, int tc, int gq) {
  return (size_t)2 * tc * D + (size_t)gq * D + (size_t)gq * tc + (size_t)1024 * gq + 2 * gq;
}

template <int D>
__global__ void __launch_bounds__(kAttnThreads) attn_decode_kernel(const AttnParams p) {
  constexpr int F4 = D / 32;        // float4 per lane in the score phase (8 lanes per row)
  constexpr int CPR = D / 4;        // float4 columns per row
  constexpr int RPL = 32 / CPR;     // rows per warp load in the V phase
  constexpr int SL = kAttnThreads / CPR;  // chunk slices in the merge
  static_assert(D == 32 || D == 64 || D == 128, "head_dim");
  static_assert(kAttnWarps * RPL == SL, "the V-phase and merge reductions share one buffer");

  extern __shared__ __align__(128) float smem[];
  const int gq = p.gq, tc = p.tc;
  float* k_s = smem;
  float* v_s = k_s + (size_t)tc * D;
  float* q_s = v_s + (size_t)tc * D;
  float* sc = q_s + gq * D;
  float* red = sc + gq * tc;
  float* ml = red + 1024 * gq;
  __shared__ uint64_t bar[2];
  __shared__ int s_last;

  const int chunk = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int qkv_dim = (p.num_heads + 2 * p.num_kv_heads) * D;

  // The offsets were produced before the previous kernel could start, so the K/V tiles
  // (written by earlier steps) can be requested while that kernel is still draining.
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
  bool loads_ok = true;

  if (active) {
    if (tid == 0) {
      mbar_init(&bar[0], 1);
      mbar_init(&bar[1], 1);
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      const uint32_t bytes = (uint32_t)rows * D * sizeof(float);
      mbar_expect_tx(&bar[0], bytes);
      bulk_g2s(k_s, kc + (int64_t)t0 * D, bytes, &bar[0]);
      mbar_expect_tx(&bar[1], bytes);
      bulk_g2s(v_s, vc + (int64_t)t0 * D, bytes, &bar[1]);
    }
  }
  pdl_wait();
  pdl_launch_dependents();

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
    __syncthreads();  // q_s ready; mbarrier inits visible to every thread
    loads_ok = mbar_wait(&bar[0], 0);
    // The chunk that holds position `off` appends the new k (rotated) and v: to the cache in
    // global memory and over whatever the bulk copy fetched for that row.
    const bool has_new = off >= t0 && off < t0 + tc;
    if (has_new) {
      loads_ok = mbar_wait(&bar[1], 0) && loads_ok;
      const float* kx = qkv_b + (int64_t)p.num_heads * D + (int64_t)kvh * D;
      const float* vx = kx + (int64_t)p.num_kv_heads * D;
      for (int e = tid; e < D; e += kAttnThreads) {
        const float kr = rope_elem(kx, cs, sn, e, D / 2);
        const float vr = vx[e];
        kc[(int64_t)off * D + e] = kr;
        vc[(int64_t)off * D + e] = vr;
        k_s[(off - t0) * D + e] = kr;
        v_s[(off - t0) * D + e] = vr;
        if (p.qkv_rot_out) {
          float* o = p.qkv_rot_out + (int64_t)b * qkv_dim + (int64_t)p.num_heads * D + (int64_t)kvh * D;
          o[e] = kr;
          o[(int64_t)p.num_kv_heads * D + e] = vr;
        }
      }
      __syncthreads();
    }

    // ---- scores: 8 lanes per row, each lane F4 float4 (columns l8 + 8*i) ----
    {
      const int l8 = lane & 7, rsub = lane >> 3;
      for (int r = warp * 4 + rsub; r < tc; r += kAttnWarps * 4) {
        const bool rv = r < rows;
        float4 kv4[F4];
        const float4* krow = reinterpret_cast<const float4*>(k_s + (size_t)(rv ? r : 0) * D);
#pragma unroll
        for (int i = 0; i < F4; ++i) kv4[i] = krow[l8 + 8 * i];
        for (int g = 0; g < gq; ++g) {
          const float4* q4 = reinterpret_cast<const float4*>(q_s + g * D);
          float a = 0.f;
#pragma unroll
          for (int i = 0; i < F4; ++i) {
            const float4 qv = q4[l8 + 8 * i];
            a = fmaf(qv.x, kv4[i].x, a);
            a = fmaf(qv.y, kv4[i].y, a);
            a = fmaf(qv.z, kv4[i].z, a);
            a = fmaf(qv.w, kv4[i].w, a);
          }
          a += __shfl_xor_sync(0xffffffffu, a, 1);
          a += __shfl_xor_sync(0xffffffffu, a, 2);
          a += __shfl_xor_sync(0xffffffffu, a, 4);
          if (l8 == 0) sc[g * tc + r] = rv ? a * p.scale : -INFINITY;
        }
      }
    }
    __syncthreads();
    // ---- chunk-local softmax numerators: warp g owns q head g ----
    if (warp < gq) {
      float mx = -INFINITY;
      for (int t = lane; t < tc; t += 32) mx = fmaxf(mx, sc[warp * tc + t]);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      float sum = 0.f;
      for (int t = lane; t < tc; t += 32) {
        const float e = expf(sc[warp * tc + t] - mx);  // exp(-inf) = 0 for masked rows
        sc[warp * tc + t] = e;
        sum += e;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      if (lane == 0) {
        ml[warp * 2 + 0] = mx;
        ml[warp * 2 + 1] = sum;
      }
    }
    if (!has_new) loads_ok = mbar_wait(&bar[1], 0) && loads_ok;
    __syncthreads();
    // ---- weighted V: lane owns float4 column c of row (step*RPL + rs) ----
    {
      const int c = lane % CPR, rs = lane / CPR;
      float4 acc[kMaxGq];
#pragma unroll
      for (int g = 0; g < kMaxGq; ++g) acc[g] = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int r = warp * RPL + rs; r < rows; r += kAttnWarps * RPL) {
        const float4 v4 = reinterpret_cast<const float4*>(v_s + (size_t)r * D)[c];
#pragma unroll
        for (int g = 0; g < kMaxGq; ++g) {
          if (g < gq) {
            const float w = sc[g * tc + r];
            acc[g].x = fmaf(w, v4.x, acc[g].x);
            acc[g].y = fmaf(w, v4.y, acc[g].y);
            acc[g].z = fmaf(w, v4.z, acc[g].z);
            acc[g].w = fmaf(w, v4.w, acc[g].w);
          }
        }
      }
#pragma unroll
      for (int g = 0; g < kMaxGq; ++g)
        if (g < gq) reinterpret_cast<float4*>(red + ((size_t)(warp * RPL + rs) * gq + g) * D)[c] = acc[g];
    }
    __syncthreads();
    for (int i = tid; i < gq * D; i += kAttnThreads) {
      const int g = i / D, e = i - g * D;
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < SL; ++w) s += red[((size_t)w * gq + g) * D + e];
      const int h = kvh * gq + g;
      p.part_o[(((int64_t)b * p.num_heads + h) * p.nc + chunk) * D + e] = s;
    }
    if (tid < gq) {
      const int h = kvh * gq + tid;
      float* dst = p.part_ml + (((int64_t)b * p.num_heads + h) * p.nc + chunk) * 2;
      dst[0] = ml[tid * 2 + 0];
      dst[1] = ml[tid * 2 + 1];
    }
    if (!loads_ok && tid == 0) atomicExch(p.err, 1);  // a tile never arrived: results are invalid
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
  // weights of every chunk: warp g owns q head g.  wts [gq][nc] lives in the K|V tile area.
  float* wts = smem;
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
  // About 3.5 CTAs per SM over the whole grid; the chunk is a power of two in [32, 128] and
  // large enough for the merge weights [gq][nc] to fit in the K|V tile area.
  const int64_t cols = (int64_t)batch * num_kv_heads;
  const int64_t want_nc = (7ll * sm_count() / 2 + cols - 1) / cols;
  int tc = 128;
  while (tc > 32 && (max_seq_len + tc - 1) / tc < want_nc) tc >>= 1;
  const int64_t cap = max_seq_len < kSeqCap ? max_seq_len : kSeqCap;
  while (tc < 256 && (int64_t)gq * ((cap + tc - 1) / tc) > (int64_t)2 * tc * head_dim) tc <<= 1;
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

  const int D = a.head_dim;
  if (L.tc < 32 || L.tc > 256 || (L.tc & (L.tc - 1)) || (int64_t)gq * L.nc > (int64_t)2 * L.tc * D)
    return fail(TB_ERR_ARG, "attention: chunk %d is not a power of two in [32, 256] or too small for %d chunks", L.tc, L.nc);
  const size_t smem = sizeof(float) * attn_smem_floats(D, L.tc, gq);
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
