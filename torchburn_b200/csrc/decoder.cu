// The decoder handle: RustQwenDecoder / WgpuQwenDecoder (src/llm/decoder.rs:111-171,
// src/wgpu/decode.rs:297-334) on one B200, or on one rank of a tensor-parallel group.
//
// One step = embedding gather, then per layer five kernels
//   [RMSNorm + QKV GEMV] -> [RoPE + KV append + split-K attention + merge]
//   -> [O GEMV + residual] -> [RMSNorm + gate/up GEMV + SwiGLU] -> [down GEMV + residual]
// and [RMSNorm + lm_head GEMV]; the same order as step_internal
// (src/llm/decoder.rs:1051-1374).  The kernels are chained with programmatic
// dependent launch, so each kernel's weight stream starts while its predecessor
// drains, and the whole step is replayed from a CUDA graph (the reference's wgpu
// path records one command stream per token for the same reason,
// src/wgpu/decode.rs:6-7).  Token ids and offsets live in device memory, so one
// graph serves every position.
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <new>
#include <vector>

#include "tb_common.cuh"
#include "tp.cuh"

using namespace tb;

namespace {

struct LayerDev {
  float* input_norm_w = nullptr;
  uint8_t* qkv_w = nullptr;
  float* qkv_s = nullptr;
  uint8_t* o_w = nullptr;
  float* o_s = nullptr;
  float* post_norm_w = nullptr;
  uint8_t* gate_w = nullptr;
  float* gate_s = nullptr;
  uint8_t* up_w = nullptr;
  float* up_s = nullptr;
  uint8_t* down_w = nullptr;
  float* down_s = nullptr;
  float* qkv_b = nullptr;
};

constexpr int kMaxBatch = 64;

}  // namespace

struct tb_decoder {
  tb_model_config cfg;
  // full and per-rank dimensions
  int64_t V = 0, H = 0, I = 0, S = 0;
  int L = 0, nh = 0, nkv = 0, hd = 0, G = 0, B = 1;
  int tp = 1, rank = 0;
  int nh_l = 0, nkv_l = 0;
  int64_t I_l = 0, V_l = 0, q_dim_l = 0, tq_l = 0;
  int device = 0;

  float* embed = nullptr;
  std::vector<LayerDev> layers;
  float* final_norm_w = nullptr;
  uint8_t* lm_w = nullptr;
  float* lm_s = nullptr;
  float *cos_t = nullptr, *sin_t = nullptr;
  float *k_cache = nullptr, *v_cache = nullptr;  // [L][B][Hkv_l][S][d]
  float *x = nullptr, *qkv = nullptr, *attn = nullptr, *h = nullptr, *logits = nullptr;
  // Split RMSNorm (batch 1, one GPU): the residual-stream producers also write x times the next
  // norm's weights and the sums of squares of x per 8 elements; the consumers start from those.
  float *xn = nullptr, *ss8 = nullptr;
  bool split_norm = false;
  // The whole batch-1 step as one persistent kernel (w4_step.cu): phase list, barrier words,
  // attention partials and a host-mapped word the kernel raises when a bounded wait ran out.
  bool fused_step = false;
  bool logits_shared = false;   // tensor parallel: d->logits points into the peer-mapped block
  StepPhase* d_phases = nullptr;
  unsigned* d_step_sync = nullptr;
  float *step_part_o = nullptr, *step_part_ml = nullptr;
  int* h_step_fault = nullptr;
  StepProgram prog;
  float* partial = nullptr;  // tensor parallel: this rank's partial sums [B, H]
  float* logits_l = nullptr; // tensor parallel: this rank's logit slice [B, V_l]
  int32_t *d_tokens = nullptr, *d_offsets = nullptr, *d_eff = nullptr;
  int32_t *d_hist = nullptr, *d_hist_pos = nullptr;
  int64_t hist_cap = 0;
  int32_t* h_io = nullptr;  // pinned: tokens | offsets
  int32_t* h_feed = nullptr; // pinned: per-step (token, offset) pairs for prefill
  int64_t feed_cap = 0;
  void* attn_scratch = nullptr;
  void* argmax_scratch = nullptr;
  void* xq_scratch = nullptr;  // digit form of the activations for batch > 1
  // layer-0 stage snapshots (TB_DECODER_NO_GRAPH only)
  float *dbg_embed = nullptr, *dbg_normed = nullptr, *dbg_qkv = nullptr, *dbg_attn = nullptr,
        *dbg_x_attn = nullptr, *dbg_h = nullptr, *dbg_x_out = nullptr;

  cudaStream_t stream = nullptr;
  cudaGraphExec_t graphs[kMaxBatch + 1] = {};
  cudaGraphExec_t graphs_greedy[kMaxBatch + 1] = {};
  cudaGraphExec_t graphs_verify[kMaxBatch + 1] = {};   // the rows of the batch are positions of sequence 0
  bool verify_shared = false;                           // set around a multi-position verify step
  bool use_graph = true;
  bool pdl = true;
  // Kernels launched with programmatic dependent launch (bit 0 qkv, 1 attention, 2 o_proj,
  // 3 gate/up, 4 down, 5 lm_head; bit 6: every projection of a batched step - measured 3% (batch 8)
  // to 9% (batch 32) slower than plain stream order, so off).  Measured on B200: the attention kernel gains from starting
  // its K/V tile copies early; the persistent GEMV kernels run slower when they are made
  // resident before their predecessor has finished, so they keep plain stream order.
  int pdl_mask = 2;
  int64_t kv_used = 0;
  int last_batch = 1;
  bool device_lost = false;
  int launches_per_step = 0;
  TpState* tpst = nullptr;
  std::vector<float> host_logits;  // sampling on the host
};

namespace {

#define DEC_CUDA(dec, expr)                                                                     \
  do {                                                                                          \
    cudaError_t _e = (expr);                                                                    \
    if (_e != cudaSuccess) {                                                                    \
      if (_e != cudaErrorMemoryAllocation && _e != cudaErrorInvalidValue) (dec)->device_lost = true; \
      return fail(_e == cudaErrorMemoryAllocation ? TB_ERR_OOM : TB_ERR_CUDA, "%s failed: %s",  \
                  #expr, cudaGetErrorString(_e));                                               \
    }                                                                                           \
  } while (0)

tb_status check_alive(const tb_decoder* d, const char* what) {
  if (!d) return fail(TB_ERR_ARG, "%s: null decoder", what);
  if (d->device_lost) return fail(TB_ERR_DEVICE_LOST, "%s: device lost; create a new decoder", what);
  return TB_OK;
}

template <typename T>
tb_status dalloc(T** p, size_t count) {
  *p = nullptr;
  if (count == 0) return TB_OK;
  cudaError_t e = cudaMalloc((void**)p, count * sizeof(T));
  if (e != cudaSuccess) return fail(TB_ERR_OOM, "Out of memory allocating %zu MB on the device (%s)",
                                    count * sizeof(T) / (1024 * 1024), cudaGetErrorString(e));
  return TB_OK;
}

size_t kv_layer_stride(const tb_decoder* d) { return (size_t)d->B * d->nkv_l * d->S * d->hd; }

// Enqueues one step for `b` sequences on d->stream (direct launches; also what
// a graph capture records).  debug: copy layer-0 intermediates.
tb_status enqueue_step(tb_decoder* d, int b, bool debug, cudaEvent_t before_lm_head = nullptr) {
  cudaStream_t st = d->stream;
  const bool pdl = d->pdl;
  const int pm = d->pdl_mask;
  int launches = 0;
  if (d->fused_step && b == 1 && !debug && before_lm_head == nullptr) {
    // embedding (+ the first norm's weights and sums of squares), then every layer and lm_head in one kernel
    TB_TRY(launch_step_embed(d->embed, d->d_tokens, d->d_offsets, d->layers[0].input_norm_w, d->x, d->xn, d->ss8,
                             d->d_eff, d->V, d->H, d->S, st));
    TB_TRY(launch_w4_step(d->prog, st));
    d->launches_per_step = 2;
    return TB_OK;
  }
  TB_TRY(launch_embed_gather(d->embed, d->d_tokens, d->d_offsets, d->x, d->d_eff, b, d->V, d->H, d->S,
                             false, st));
  ++launches;
  auto snap = [&](float* dst, const float* src, size_t n) -> tb_status {
    if (!debug) return TB_OK;
    TB_CUDA_TRY(cudaMemcpyAsync(dst, src, n * sizeof(float), cudaMemcpyDeviceToDevice, st));
    return TB_OK;
  };
  TB_TRY(snap(d->dbg_embed, d->x, d->H));
  const bool sn = d->split_norm && b == 1 && !debug && (d->tp == 1 || tp_low_latency(d->tpst, b, d->H));
  for (int l = 0; l < d->L; ++l) {
    const LayerDev& W = d->layers[l];
    const bool dbg = debug && l == 0;
    {  // A + B: RMSNorm fused into the QKV projection
      GemvArgs a;
      a.x = d->x; a.w = W.qkv_w; a.scales = W.qkv_s; a.bias = W.qkv_b; a.out = d->qkv;
      a.norm_w = W.input_norm_w; a.eps = d->cfg.rms_norm_eps;
      a.x_normed_out = dbg ? d->dbg_normed : nullptr;
      if (sn && l > 0) { a.x = d->xn; a.x_ss8 = d->ss8; a.norm_w = nullptr; }
      a.m = b; a.n = d->tq_l; a.k = d->H; a.g = d->G; a.pdl = pdl && !debug && ((pm & 1) || (b > 1 && (pm & 64)));
      a.xq_scratch = d->xq_scratch;
      TB_TRY(launch_w4_gemv(a, st));
      launches += w4_gemv_launches(a);
    }
    {  // C + D + E
      AttnArgs a;
      a.qkv = d->qkv;
      a.k_cache = d->k_cache + (size_t)l * kv_layer_stride(d);
      a.v_cache = d->v_cache + (size_t)l * kv_layer_stride(d);
      a.cos_t = d->cos_t; a.sin_t = d->sin_t; a.offsets = d->d_eff; a.out = d->attn;
      a.scratch = d->attn_scratch; a.q_rot_out = dbg ? d->dbg_qkv : nullptr;
      a.batch = b; a.num_heads = d->nh_l; a.num_kv_heads = d->nkv_l; a.head_dim = d->hd;
      a.max_seq_len = d->S; a.pdl = pdl && !debug && (pm & 2);
      if (d->verify_shared && b > 1) {
        // several positions of sequence 0: every row's k and v go into the cache first; the attention kernel
        // then only reads it (and must not start reading before that kernel has finished: no early launch)
        a.shared_cache = true;
        a.pdl = false;
        TB_TRY(launch_rope_append_rows(a, st));
        ++launches;
      }
      // The kernel strides sequences by [Hkv, S, d]; with batch > 1 that is the layout of
      // one layer's block [B][Hkv][S][d].
      TB_TRY(launch_attention_decode(a, st));
      ++launches;
    }
    if (dbg) TB_TRY(snap(d->dbg_attn, d->attn, d->q_dim_l));
    {  // F + G
      GemvArgs a;
      a.x = d->attn; a.w = W.o_w; a.scales = W.o_s; a.m = b; a.n = d->H; a.k = d->q_dim_l; a.g = d->G;
      a.pdl = pdl && !debug && ((pm & 4) || (b > 1 && (pm & 64)));
      if (d->tp == 1) { a.out = d->x; a.resid = d->x; }
      else { a.out = tp_partial_buffer(d->tpst, d->partial); }
      if (sn && d->tp == 1) { a.out_scaled = d->xn; a.out_scale_w = W.post_norm_w; a.out_ss8 = d->ss8; }
      a.xq_scratch = d->xq_scratch;
      TB_TRY(launch_w4_gemv(a, st));
      launches += w4_gemv_launches(a);
      if (d->tp > 1) {
        TB_TRY(tp_allreduce_residual(d->tpst, a.out, d->x, b, d->H, st, &launches, sn ? W.post_norm_w : nullptr,
                                     sn ? d->xn : nullptr, sn ? d->ss8 : nullptr));
      }
    }
    if (dbg) TB_TRY(snap(d->dbg_x_attn, d->x, d->H));
    {  // H + I: RMSNorm fused into the gate/up projection with the SwiGLU epilogue
      GemvArgs a;
      a.x = d->x; a.w = W.gate_w; a.scales = W.gate_s; a.w2 = W.up_w; a.scales2 = W.up_s; a.out = d->h;
      a.norm_w = W.post_norm_w; a.eps = d->cfg.rms_norm_eps;
      if (sn) { a.x = d->xn; a.x_ss8 = d->ss8; a.norm_w = nullptr; }
      a.m = b; a.n = d->I_l; a.k = d->H; a.g = d->G; a.pdl = pdl && !debug && ((pm & 8) || (b > 1 && (pm & 64)));
      a.xq_scratch = d->xq_scratch;
      TB_TRY(launch_w4_gemv(a, st));
      launches += w4_gemv_launches(a);
    }
    if (dbg) TB_TRY(snap(d->dbg_h, d->h, d->I_l));
    {  // I' + J
      GemvArgs a;
      a.x = d->h; a.w = W.down_w; a.scales = W.down_s; a.m = b; a.n = d->H; a.k = d->I_l; a.g = d->G;
      a.pdl = pdl && !debug && ((pm & 16) || (b > 1 && (pm & 64)));
      if (d->tp == 1) { a.out = d->x; a.resid = d->x; }
      else { a.out = tp_partial_buffer(d->tpst, d->partial); }
      const float* next_norm_w = l + 1 < d->L ? d->layers[l + 1].input_norm_w : d->final_norm_w;
      if (sn && d->tp == 1) { a.out_scaled = d->xn; a.out_ss8 = d->ss8; a.out_scale_w = next_norm_w; }
      a.xq_scratch = d->xq_scratch;
      TB_TRY(launch_w4_gemv(a, st));
      launches += w4_gemv_launches(a);
      if (d->tp > 1) {
        TB_TRY(tp_allreduce_residual(d->tpst, a.out, d->x, b, d->H, st, &launches, sn ? next_norm_w : nullptr,
                                     sn ? d->xn : nullptr, sn ? d->ss8 : nullptr));
      }
    }
    if (dbg) TB_TRY(snap(d->dbg_x_out, d->x, d->H));
  }
  if (before_lm_head) TB_CUDA_TRY(cudaEventRecord(before_lm_head, st));
  {  // 3 + 4: final RMSNorm fused into lm_head
    GemvArgs a;
    a.x = d->x; a.w = d->lm_w; a.scales = d->lm_s;
    a.norm_w = d->final_norm_w; a.eps = d->cfg.rms_norm_eps;
    if (sn) { a.x = d->xn; a.x_ss8 = d->ss8; a.norm_w = nullptr; }
    a.m = b; a.n = d->V_l; a.k = d->H; a.g = d->G; a.pdl = pdl && !debug && ((pm & 32) || (b > 1 && (pm & 64)));
    a.out = d->tp == 1 ? d->logits : d->logits_l;
    a.xq_scratch = d->xq_scratch;
    TB_TRY(launch_w4_gemv(a, st));
    launches += w4_gemv_launches(a);
    if (d->tp > 1) { TB_TRY(tp_allgather_logits(d->tpst, d->logits_l, d->logits, b, d->V_l, st, &launches)); }
  }
  d->launches_per_step = launches;
  return TB_OK;
}

tb_status build_graph(tb_decoder* d, int b, bool greedy, cudaGraphExec_t* out) {
  *out = nullptr;
  cudaGraph_t graph = nullptr;
  DEC_CUDA(d, cudaStreamBeginCapture(d->stream, cudaStreamCaptureModeThreadLocal));
  tb_status s = enqueue_step(d, b, false);
  if (s == TB_OK && greedy) s = launch_argmax(d->logits, d->V, b, d->d_tokens, d->d_offsets, d->d_hist, d->d_hist_pos, d->argmax_scratch, d->stream);
  cudaError_t e = cudaStreamEndCapture(d->stream, &graph);
  if (s != TB_OK) {
    if (graph) cudaGraphDestroy(graph);
    return s;
  }
  if (e != cudaSuccess) return fail(TB_ERR_CUDA, "graph capture failed: %s", cudaGetErrorString(e));
  e = cudaGraphInstantiate(out, graph, 0);
  cudaGraphDestroy(graph);
  if (e != cudaSuccess) {
    *out = nullptr;
    return fail(TB_ERR_CUDA, "graph instantiate failed: %s", cudaGetErrorString(e));
  }
  return TB_OK;
}

// Runs one step for b sequences whose tokens/offsets are already in d_tokens/d_offsets.
tb_status run_step(tb_decoder* d, int b, bool greedy) {
  if (d->use_graph) {
    cudaGraphExec_t* slot = d->verify_shared ? &d->graphs_verify[b] : (greedy ? &d->graphs_greedy[b] : &d->graphs[b]);
    if (!*slot) {
      tb_status s = build_graph(d, b, greedy, slot);
      if (s != TB_OK) {
        // A capture problem is not a device problem: fall back to direct launches.
        cudaGetLastError();
        d->use_graph = false;
      }
    }
    if (*slot) {
      DEC_CUDA(d, cudaGraphLaunch(*slot, d->stream));
      return TB_OK;
    }
  }
  TB_TRY(enqueue_step(d, b, !d->use_graph && (d->cfg.flags & TB_DECODER_NO_GRAPH)));
  if (greedy) TB_TRY(launch_argmax(d->logits, d->V, b, d->d_tokens, d->d_offsets, d->d_hist, d->d_hist_pos, d->argmax_scratch, d->stream));
  return TB_OK;
}

tb_status fault_word(tb_decoder* d, int** dev_ptr);

// Lays out the batch-1 step for the persistent kernel when every projection fits its rules
// (otherwise the decoder keeps the chain of single kernels).
tb_status build_step_program(tb_decoder* d) {
  d->fused_step = false;
  if (d->cfg.flags & (TB_DECODER_NO_FUSED_STEP | TB_DECODER_NO_GRAPH)) return TB_OK;
  if (d->tp == 1 && !(d->cfg.flags & TB_DECODER_FUSED_STEP)) return TB_OK;   // one GPU: the chain of kernels is faster (measured)
  StepTp tpa;
  if (d->tp > 1 && !tp_step_areas(d->tpst, &tpa)) return TB_OK;   // no peer memory: the chain of kernels with NCCL
  if (d->d_phases) return TB_OK;
  if (d->hd != 64 && d->hd != 128) return TB_OK;
  const int G = d->G;
  if (d->H % 32 != 0 || !w4_step_supports(d->tq_l, d->H, G, 1) || !w4_step_supports(d->H, d->q_dim_l, G, 1) ||
      !w4_step_supports(d->I_l, d->H, G, 2) || !w4_step_supports(d->H, d->I_l, G, 1) || !w4_step_supports(d->V_l, d->H, G, 1))
    return TB_OK;
  const int grid = w4_step_grid();
  const int nc = grid > 0 ? w4_step_attn_split(grid, d->nkv_l) : 0;
  if (grid <= 0 || nc <= 0) return TB_OK;

  std::vector<StepPhase> ph;
  int rot = 0, n_exch = 0;
  const bool tpm = d->tp > 1;
  // tensor parallel: the sum over the ranks of a row-parallel projection's rows, with the residual
  auto exchange = [&](const float* next_norm_w) {
    StepPhase q;
    q.kind = 3; q.n = (int)d->H; q.xi = n_exch++;
    q.resid = d->x; q.out = d->x; q.out_scaled = d->xn; q.out_scale_w = next_norm_w; q.out_ss8 = d->ss8;
    return q;
  };
  auto gemv = [&](int64_t n, int64_t k, int nw) {
    StepPhase q;
    q.kind = 0; q.n = (int)n; q.k = (int)k; q.ng = (int)(k / G); q.gshift = G == 32 ? 0 : (G == 64 ? 1 : 2);
    q.nw = nw; q.rs = w4_step_rows_per_stage(k, G, nw); q.rot = rot; q.eps = d->cfg.rms_norm_eps;
    rot = (rot + (int)(((n + 7) / 8) % grid)) % grid;
    return q;
  };
  for (int l = 0; l < d->L; ++l) {
    const LayerDev& W = d->layers[l];
    {  // A + B: QKV on the pre-weighted x
      StepPhase q = gemv(d->tq_l, d->H, 1);
      q.w[0] = W.qkv_w; q.sc[0] = W.qkv_s; q.bias[0] = W.qkv_b; q.x = d->xn; q.x_ss8 = d->ss8; q.out = d->qkv;
      ph.push_back(q);
    }
    {  // C + D + E: RoPE, append, split-K attention; then the merge of the partials
      StepPhase q;
      q.kind = 1;
      q.k_cache = d->k_cache + (size_t)l * kv_layer_stride(d);
      q.v_cache = d->v_cache + (size_t)l * kv_layer_stride(d);
      ph.push_back(q);
      StepPhase m;
      m.kind = 2;
      ph.push_back(m);
    }
    {  // F + G
      StepPhase q = gemv(d->H, d->q_dim_l, 1);
      q.w[0] = W.o_w; q.sc[0] = W.o_s; q.x = d->attn;
      if (!tpm) {
        q.resid = d->x; q.out = d->x; q.out_scaled = d->xn; q.out_scale_w = W.post_norm_w; q.out_ss8 = d->ss8;
        ph.push_back(q);
      } else {
        q.tp_mode = 1; q.xi = n_exch;
        ph.push_back(q);
        ph.push_back(exchange(W.post_norm_w));
      }
    }
    {  // H + I
      StepPhase q = gemv(d->I_l, d->H, 2);
      q.w[0] = W.gate_w; q.sc[0] = W.gate_s; q.w[1] = W.up_w; q.sc[1] = W.up_s; q.x = d->xn; q.x_ss8 = d->ss8; q.out = d->h;
      ph.push_back(q);
    }
    {  // I' + J
      StepPhase q = gemv(d->H, d->I_l, 1);
      q.w[0] = W.down_w; q.sc[0] = W.down_s; q.x = d->h;
      const float* next_norm_w = l + 1 < d->L ? d->layers[l + 1].input_norm_w : d->final_norm_w;
      if (!tpm) {
        q.resid = d->x; q.out = d->x; q.out_scaled = d->xn; q.out_ss8 = d->ss8; q.out_scale_w = next_norm_w;
        ph.push_back(q);
      } else {
        q.tp_mode = 1; q.xi = n_exch;
        ph.push_back(q);
        ph.push_back(exchange(next_norm_w));
      }
    }
  }
  {  // 3 + 4: lm_head on the pre-weighted x
    StepPhase q = gemv(d->V_l, d->H, 1);
    q.w[0] = d->lm_w; q.sc[0] = d->lm_s; q.x = d->xn; q.x_ss8 = d->ss8; q.out = d->logits;
    if (tpm) { q.tp_mode = 2; q.xi = (int)(d->rank * d->V_l); }   // this rank's slice into every rank's logits
    ph.push_back(q);
  }
  TB_TRY(dalloc(&d->d_phases, ph.size()));
  TB_CUDA_TRY(cudaMemcpy(d->d_phases, ph.data(), ph.size() * sizeof(StepPhase), cudaMemcpyHostToDevice));
  TB_TRY(dalloc(&d->d_step_sync, (size_t)8));
  TB_CUDA_TRY(cudaMemset(d->d_step_sync, 0, 8 * sizeof(unsigned)));
  TB_TRY(dalloc(&d->step_part_o, (size_t)d->nh_l * nc * d->hd));
  TB_TRY(dalloc(&d->step_part_ml, (size_t)d->nh_l * nc * 2));
  int* dev_fault = nullptr;
  TB_TRY(fault_word(d, &dev_fault));
  StepProgram& g = d->prog;
  g.phases = d->d_phases; g.nphases = (int)ph.size(); g.grid = grid; g.sync = d->d_step_sync;
  g.host_fault = dev_fault;
  g.qkv = d->qkv; g.attn = d->attn; g.cos_t = d->cos_t; g.sin_t = d->sin_t; g.offsets = d->d_eff;
  g.part_o = d->step_part_o; g.part_ml = d->step_part_ml;
  g.num_heads = d->nh_l; g.num_kv_heads = d->nkv_l; g.head_dim = d->hd; g.nc = nc; g.max_seq_len = d->S;
  if (tpm) { g.tp = tpa; g.n_exchanges = n_exch; }
  d->fused_step = true;
  return TB_OK;
}

// The host-mapped fault word of a decoder (allocated on first use); returns its device pointer.
tb_status fault_word(tb_decoder* d, int** dev_ptr) {
  if (!d->h_step_fault) {
    TB_CUDA_TRY(cudaHostAlloc((void**)&d->h_step_fault, sizeof(int), cudaHostAllocMapped));
    *d->h_step_fault = 0;
  }
  TB_CUDA_TRY(cudaHostGetDevicePointer((void**)dev_ptr, d->h_step_fault, 0));
  return TB_OK;
}

// A bounded device-side wait ran out during the last step: the results are invalid and the
// decoder is unusable from here on (the kernel ended; the context is intact).
tb_status check_step_fault(tb_decoder* d) {
  if (d->h_step_fault && *reinterpret_cast<volatile int*>(d->h_step_fault)) {
    d->device_lost = true;
    return fail(TB_ERR_TIMEOUT, "a bounded device-side wait of the decode step ran out; the step's results are invalid");
  }
  return TB_OK;
}

void note_kv(tb_decoder* d, int64_t token, int64_t offset) {
  if (token >= 0 && token < d->V && offset >= 0 && offset < d->S && offset + 1 > d->kv_used)
    d->kv_used = offset + 1;  // src/llm/decoder.rs:1092
}

int32_t clamp_i32(int64_t v) { return v < -1 ? -1 : (v > 0x7ffffff0 ? 0x7ffffff0 : (int32_t)v); }

tb_status feed_and_step(tb_decoder* d, const int64_t* tokens, const int64_t* offsets, int b) {
  for (int i = 0; i < b; ++i) {
    d->h_io[i] = clamp_i32(tokens[i]);
    d->h_io[kMaxBatch + i] = clamp_i32(offsets[i]);
    note_kv(d, tokens[i], offsets[i]);
  }
  DEC_CUDA(d, cudaMemcpyAsync(d->d_tokens, d->h_io, sizeof(int32_t) * b, cudaMemcpyHostToDevice, d->stream));
  DEC_CUDA(d, cudaMemcpyAsync(d->d_offsets, d->h_io + kMaxBatch, sizeof(int32_t) * b, cudaMemcpyHostToDevice, d->stream));
  d->last_batch = b;
  return run_step(d, b, false);
}

// n consecutive positions of sequence 0, max_batch of them per step: the rows of a step are positions of the
// ONE sequence (batched products, attention rows sharing sequence 0's cache, causal inside the block).  All
// tokens and offsets are staged in pinned memory first, every step copying from its own part, so that the host
// never rewrites words an earlier, still queued copy has yet to read.  rows_host (optional) receives the
// logits of every position.  Afterwards the decoder's own logits are those of the last position.
tb_status run_positions(tb_decoder* d, const int64_t* tokens, int64_t n, int64_t start_offset, float* rows_host) {
  if (n > d->feed_cap) {
    cudaFreeHost(d->h_feed);
    d->h_feed = nullptr;
    d->feed_cap = 0;
    DEC_CUDA(d, cudaMallocHost((void**)&d->h_feed, sizeof(int32_t) * 2 * n));
    d->feed_cap = n;
  }
  for (int64_t i = 0; i < n; ++i) {
    d->h_feed[i] = clamp_i32(tokens[i]);
    d->h_feed[n + i] = clamp_i32(start_offset + i);
    note_kv(d, tokens[i], start_offset + i);
  }
  int last_m = 1;
  for (int64_t i = 0; i < n;) {
    const int m = (int)(n - i < d->B ? n - i : d->B);
    DEC_CUDA(d, cudaMemcpyAsync(d->d_tokens, d->h_feed + i, sizeof(int32_t) * m, cudaMemcpyHostToDevice, d->stream));
    DEC_CUDA(d, cudaMemcpyAsync(d->d_offsets, d->h_feed + n + i, sizeof(int32_t) * m, cudaMemcpyHostToDevice, d->stream));
    d->last_batch = m;
    d->verify_shared = m > 1;
    const tb_status s = run_step(d, m, false);
    d->verify_shared = false;
    TB_TRY(s);
    if (rows_host)
      DEC_CUDA(d, cudaMemcpyAsync(rows_host + i * d->V, d->logits, sizeof(float) * (size_t)m * d->V, cudaMemcpyDeviceToHost, d->stream));
    last_m = m;
    i += m;
  }
  if (last_m > 1)
    DEC_CUDA(d, cudaMemcpyAsync(d->logits, d->logits + (size_t)(last_m - 1) * d->V, sizeof(float) * d->V, cudaMemcpyDeviceToDevice, d->stream));
  d->last_batch = 1;
  DEC_CUDA(d, cudaStreamSynchronize(d->stream));
  return check_step_fault(d);
}

}  // namespace

extern "C" {

tb_status tb_decoder_create(tb_decoder** out, const tb_model_config* cfg,
                            const float* embed_tokens, const tb_layer_weights* layers,
                            const float* final_norm_w, const uint8_t* lm_head_w,
                            const float* lm_head_s, tb_space ws) {
  if (!out) return fail(TB_ERR_ARG, "tb_decoder_create: null out");
  *out = nullptr;
  if (!cfg || !embed_tokens || !layers || !final_norm_w || !lm_head_w || !lm_head_s)
    return fail(TB_ERR_ARG, "tb_decoder_create: null argument");
  const tb_model_config& c = *cfg;
  // src/llm/decoder.rs:214-233
  if (c.hidden_size <= 0 || c.hidden_size % 4 != 0)
    return fail(TB_ERR_ARG, "hidden_size (%lld) must be divisible by 4 (SIMD alignment)", (long long)c.hidden_size);
  if (c.group_size != 32 && c.group_size != 64 && c.group_size != 128)
    return fail(TB_ERR_UNSUPPORTED, "TB_UNSUPPORTED: group_size %d (supported: 32, 64, 128)", c.group_size);
  if (c.hidden_size % c.group_size != 0)
    return fail(TB_ERR_ARG, "hidden_size (%lld) must be divisible by group_size (%d)", (long long)c.hidden_size, c.group_size);
  if (c.head_dim <= 0 || c.head_dim % 2 != 0)
    return fail(TB_ERR_ARG, "head_dim (%d) must be even for RoPE half_dim computation", c.head_dim);
  if (c.num_kv_heads <= 0 || c.num_heads <= 0 || c.num_heads % c.num_kv_heads != 0)
    return fail(TB_ERR_ARG, "num_heads (%d) must be divisible by num_kv_heads (%d) for GQA", c.num_heads, c.num_kv_heads);
  if (c.head_dim != 32 && c.head_dim != 64 && c.head_dim != 128)
    return fail(TB_ERR_UNSUPPORTED, "TB_UNSUPPORTED: head_dim %d (supported: 32, 64, 128)", c.head_dim);
  if (c.num_heads / c.num_kv_heads > 8)
    return fail(TB_ERR_UNSUPPORTED, "TB_UNSUPPORTED: more than 8 q heads per kv head");
  if (c.vocab_size <= 0 || c.intermediate_size <= 0 || c.num_layers <= 0 || c.max_seq_len <= 0)
    return fail(TB_ERR_ARG, "tb_decoder_create: non-positive dimension");
  if (c.max_seq_len > 32768)
    return fail(TB_ERR_UNSUPPORTED, "TB_UNSUPPORTED: max_seq_len %lld (attention covers at most 32768 positions)", (long long)c.max_seq_len);
  const int B = c.max_batch <= 0 ? 1 : c.max_batch;
  if (B > kMaxBatch) return fail(TB_ERR_UNSUPPORTED, "TB_UNSUPPORTED: max_batch %d (max %d)", B, kMaxBatch);
  const int tp = c.tp_size <= 0 ? 1 : c.tp_size;
  if (c.tp_rank < 0 || c.tp_rank >= tp) return fail(TB_ERR_ARG, "tp_rank %d outside [0, %d)", c.tp_rank, tp);
  const int64_t q_dim = (int64_t)c.num_heads * c.head_dim;
  if (tp > 1) {
    if (c.num_kv_heads % tp || c.num_heads % tp || c.intermediate_size % ((int64_t)tp * c.group_size) ||
        q_dim % ((int64_t)tp * c.group_size) || c.vocab_size % tp)
      return fail(TB_ERR_ARG, "tensor parallel size %d does not divide the heads / intermediate / vocab into whole groups", tp);
  }
  if (q_dim % c.group_size != 0 || c.intermediate_size % c.group_size != 0)
    return fail(TB_ERR_ARG, "num_heads*head_dim and intermediate_size must be divisible by group_size (%d)", c.group_size);

  tb_decoder* d = new (std::nothrow) tb_decoder();
  if (!d) return fail(TB_ERR_OOM, "tb_decoder_create: host allocation failed");
  d->cfg = c;
  d->V = c.vocab_size; d->H = c.hidden_size; d->I = c.intermediate_size; d->S = c.max_seq_len;
  d->L = c.num_layers; d->nh = c.num_heads; d->nkv = c.num_kv_heads; d->hd = c.head_dim; d->G = c.group_size;
  d->B = B; d->tp = tp; d->rank = c.tp_rank;
  d->nh_l = d->nh / tp; d->nkv_l = d->nkv / tp; d->I_l = d->I / tp; d->V_l = d->V / tp;
  d->q_dim_l = (int64_t)d->nh_l * d->hd;
  d->tq_l = d->q_dim_l + 2ll * d->nkv_l * d->hd;
  d->use_graph = !(c.flags & TB_DECODER_NO_GRAPH);
  d->pdl = !(c.flags & TB_DECODER_NO_PDL);
  {
    // Split RMSNorm needs the persistent M = 1 kernel for every projection of a layer.
    auto ok_k = [&](int64_t k) { return k % 32 == 0 && k >= 2048 && k <= 15360 && ((k / d->G) * 4) % 16 == 0; };
    // one GPU: producers are the O / down kernels (all three K must qualify); tensor parallel: the
    // producer is the low-latency exchange kernel, only the consumers (K = H) must qualify
    d->split_norm = tp == 1 ? (ok_k(d->H) && ok_k(d->q_dim_l) && ok_k(d->I_l)) : ok_k(d->H);
  }
  cudaGetDevice(&d->device);

  tb_status s = TB_OK;
  auto fin = [&](tb_status st) -> tb_status {
    tb_decoder_destroy(d);
    return st;
  };
#define CR(expr) do { s = (expr); if (s != TB_OK) return fin(s); } while (0)
#define CRC(expr) do { cudaError_t _e = (expr); if (_e != cudaSuccess) return fin(fail(_e == cudaErrorMemoryAllocation ? TB_ERR_OOM : TB_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(_e))); } while (0)

  CRC(cudaStreamCreateWithFlags(&d->stream, cudaStreamNonBlocking));
  const int64_t H = d->H, G = d->G;
  CR(upload((void**)&d->embed, embed_tokens, sizeof(float) * d->V * H, ws));
  CR(upload((void**)&d->final_norm_w, final_norm_w, sizeof(float) * H, ws));
  CR(upload((void**)&d->lm_w, lm_head_w, (size_t)d->V_l * (H / 2), ws));
  CR(upload((void**)&d->lm_s, lm_head_s, sizeof(float) * d->V_l * (H / G), ws));
  d->layers.resize(d->L);
  for (int l = 0; l < d->L; ++l) {
    const tb_layer_weights& w = layers[l];
    LayerDev& o = d->layers[l];
    if (!w.input_norm_w || !w.qkv_w || !w.qkv_s || !w.o_w || !w.o_s || !w.post_norm_w || !w.gate_w ||
        !w.gate_s || !w.up_w || !w.up_s || !w.down_w || !w.down_s)
      return fin(fail(TB_ERR_ARG, "Each layer requires 12 tensors: input_norm, qkv_w, qkv_s, o_w, o_s, post_norm, gate_w, gate_s, up_w, up_s, down_w, down_s (layer %d)", l));
    CR(upload((void**)&o.input_norm_w, w.input_norm_w, sizeof(float) * H, ws));
    CR(upload((void**)&o.qkv_w, w.qkv_w, (size_t)d->tq_l * (H / 2), ws));
    CR(upload((void**)&o.qkv_s, w.qkv_s, sizeof(float) * d->tq_l * (H / G), ws));
    CR(upload((void**)&o.o_w, w.o_w, (size_t)H * (d->q_dim_l / 2), ws));
    CR(upload((void**)&o.o_s, w.o_s, sizeof(float) * H * (d->q_dim_l / G), ws));
    CR(upload((void**)&o.post_norm_w, w.post_norm_w, sizeof(float) * H, ws));
    CR(upload((void**)&o.gate_w, w.gate_w, (size_t)d->I_l * (H / 2), ws));
    CR(upload((void**)&o.gate_s, w.gate_s, sizeof(float) * d->I_l * (H / G), ws));
    CR(upload((void**)&o.up_w, w.up_w, (size_t)d->I_l * (H / 2), ws));
    CR(upload((void**)&o.up_s, w.up_s, sizeof(float) * d->I_l * (H / G), ws));
    CR(upload((void**)&o.down_w, w.down_w, (size_t)H * (d->I_l / 2), ws));
    CR(upload((void**)&o.down_s, w.down_s, sizeof(float) * H * (d->I_l / G), ws));
    if (w.qkv_b) CR(upload((void**)&o.qkv_b, w.qkv_b, sizeof(float) * d->tq_l, ws));
  }
  {  // RoPE tables in float64, src/llm/decoder.rs:336-350
    const int hd = d->hd, half = hd / 2;
    std::vector<float> ct((size_t)d->S * hd), sn((size_t)d->S * hd);
    std::vector<double> freq(half);
    for (int i = 0; i < half; ++i) freq[i] = 1.0 / std::pow(c.rope_theta, (2.0 * (double)i) / (double)hd);
    for (int64_t pos = 0; pos < d->S; ++pos)
      for (int i = 0; i < half; ++i) {
        const double val = (double)pos * freq[i];
        const float cv = (float)std::cos(val), sv = (float)std::sin(val);
        ct[pos * hd + i] = cv; ct[pos * hd + i + half] = cv;
        sn[pos * hd + i] = sv; sn[pos * hd + i + half] = sv;
      }
    CR(upload((void**)&d->cos_t, ct.data(), sizeof(float) * ct.size(), TB_HOST));
    CR(upload((void**)&d->sin_t, sn.data(), sizeof(float) * sn.size(), TB_HOST));
  }
  const size_t kv_elems = (size_t)d->L * kv_layer_stride(d);
  CR(dalloc(&d->k_cache, kv_elems));
  CR(dalloc(&d->v_cache, kv_elems));
  CRC(cudaMemset(d->k_cache, 0, kv_elems * sizeof(float)));
  CRC(cudaMemset(d->v_cache, 0, kv_elems * sizeof(float)));
  CR(dalloc(&d->x, (size_t)B * H));
  CR(dalloc(&d->xn, (size_t)H));
  CR(dalloc(&d->ss8, (size_t)(H / 8 + 4)));
  CR(dalloc(&d->qkv, (size_t)B * d->tq_l));
  CR(dalloc(&d->attn, (size_t)B * d->q_dim_l));
  CR(dalloc(&d->h, (size_t)B * d->I_l));
  CR(dalloc(&d->logits, (size_t)B * d->V));
  CRC(cudaMemset(d->logits, 0, (size_t)B * d->V * sizeof(float)));
  if (tp > 1) {
    CR(dalloc(&d->partial, (size_t)B * H));
    CR(dalloc(&d->logits_l, (size_t)B * d->V_l));
  }
  CR(dalloc(&d->d_tokens, (size_t)kMaxBatch));
  CR(dalloc(&d->d_offsets, (size_t)kMaxBatch));
  CR(dalloc(&d->d_eff, (size_t)kMaxBatch));
  CR(dalloc(&d->d_hist_pos, (size_t)1));
  CRC(cudaMemset(d->d_hist_pos, 0, sizeof(int32_t)));
  CRC(cudaMallocHost((void**)&d->h_io, sizeof(int32_t) * 2 * kMaxBatch));
  const size_t sb = attention_scratch_bytes(B, d->nh_l, d->nkv_l, d->hd, d->S);
  CRC(cudaMalloc(&d->attn_scratch, sb));
  CRC(cudaMemset(d->attn_scratch, 0, sb));
  if (B > 1) {
    int64_t kmax = d->H > d->I_l ? d->H : d->I_l;
    if (d->q_dim_l > kmax) kmax = d->q_dim_l;
    CRC(cudaMalloc(&d->xq_scratch, w4_mma_scratch_bytes(B, kmax)));
    CRC(cudaMemset(d->xq_scratch, 0, 4096));  // the tickets of the K split start at zero
  }
  CRC(cudaMalloc(&d->argmax_scratch, 16 * kMaxBatch));
  CRC(cudaMemset(d->argmax_scratch, 0, 16 * kMaxBatch));
  CR(build_step_program(d));
  if (c.flags & TB_DECODER_NO_GRAPH) {
    CR(dalloc(&d->dbg_embed, (size_t)H)); CR(dalloc(&d->dbg_normed, (size_t)B * H));
    CR(dalloc(&d->dbg_qkv, (size_t)B * d->tq_l)); CR(dalloc(&d->dbg_attn, (size_t)d->q_dim_l));
    CR(dalloc(&d->dbg_x_attn, (size_t)H)); CR(dalloc(&d->dbg_h, (size_t)d->I_l));
    CR(dalloc(&d->dbg_x_out, (size_t)H));
  }
  // Warm-up with an out-of-range token: every kernel runs once (function attributes get
  // set outside of any graph capture), nothing is written to the KV cache, logits stay 0.
  if (tp == 1) {
    int64_t tok = -1, off = 0;
    const bool g = d->use_graph;
    d->use_graph = false;
    const int flags = d->cfg.flags;
    d->cfg.flags &= ~TB_DECODER_NO_GRAPH;
    s = feed_and_step(d, &tok, &off, 1);
    d->cfg.flags = flags;
    d->use_graph = g;
    if (s != TB_OK) return fin(s);
    CRC(cudaStreamSynchronize(d->stream));
  }
#undef CR
#undef CRC
  *out = d;
  return TB_OK;
}

void tb_decoder_destroy(tb_decoder* d) {
  if (!d) return;
  if (d->stream) cudaStreamSynchronize(d->stream);
  for (int i = 0; i <= kMaxBatch; ++i) {
    if (d->graphs[i]) cudaGraphExecDestroy(d->graphs[i]);
    if (d->graphs_greedy[i]) cudaGraphExecDestroy(d->graphs_greedy[i]);
    if (d->graphs_verify[i]) cudaGraphExecDestroy(d->graphs_verify[i]);
  }
  if (d->tpst) tp_destroy(d->tpst);
  cudaFree(d->embed); cudaFree(d->final_norm_w); cudaFree(d->lm_w); cudaFree(d->lm_s);
  for (LayerDev& o : d->layers) {
    cudaFree(o.input_norm_w); cudaFree(o.qkv_w); cudaFree(o.qkv_s); cudaFree(o.o_w); cudaFree(o.o_s);
    cudaFree(o.post_norm_w); cudaFree(o.gate_w); cudaFree(o.gate_s); cudaFree(o.up_w); cudaFree(o.up_s);
    cudaFree(o.down_w); cudaFree(o.down_s); cudaFree(o.qkv_b);
  }
  cudaFree(d->cos_t); cudaFree(d->sin_t); cudaFree(d->k_cache); cudaFree(d->v_cache);
  cudaFree(d->xn); cudaFree(d->ss8);
  cudaFree(d->d_phases); cudaFree(d->d_step_sync); cudaFree(d->step_part_o); cudaFree(d->step_part_ml);
  if (d->h_step_fault) cudaFreeHost(d->h_step_fault);
  cudaFree(d->x); cudaFree(d->qkv); cudaFree(d->attn); cudaFree(d->h);
  if (!d->logits_shared) cudaFree(d->logits);
  cudaFree(d->partial); cudaFree(d->logits_l);
  cudaFree(d->d_tokens); cudaFree(d->d_offsets); cudaFree(d->d_eff); cudaFree(d->d_hist); cudaFree(d->d_hist_pos);
  cudaFreeHost(d->h_io); cudaFreeHost(d->h_feed);
  cudaFree(d->attn_scratch);
  cudaFree(d->argmax_scratch);
  cudaFree(d->xq_scratch);
  cudaFree(d->dbg_embed); cudaFree(d->dbg_normed); cudaFree(d->dbg_qkv); cudaFree(d->dbg_attn);
  cudaFree(d->dbg_x_attn); cudaFree(d->dbg_h); cudaFree(d->dbg_x_out);
  if (d->stream) cudaStreamDestroy(d->stream);
  delete d;
}

tb_status tb_decoder_step_batch(tb_decoder* d, const int64_t* token_ids, const int64_t* offsets,
                                int32_t batch, float* logits_host) {
  TB_TRY(check_alive(d, "tb_decoder_step_batch"));
  if (!token_ids || !offsets) return fail(TB_ERR_ARG, "tb_decoder_step_batch: null tokens/offsets");
  if (batch < 1 || batch > d->B) return fail(TB_ERR_ARG, "tb_decoder_step_batch: batch %d outside [1, max_batch=%d]", batch, d->B);
  TB_TRY(feed_and_step(d, token_ids, offsets, batch));
  if (logits_host)
    DEC_CUDA(d, cudaMemcpyAsync(logits_host, d->logits, sizeof(float) * batch * d->V, cudaMemcpyDeviceToHost, d->stream));
  DEC_CUDA(d, cudaStreamSynchronize(d->stream));
  return check_step_fault(d);
}

tb_status tb_decoder_step(tb_decoder* d, int64_t token_id, int64_t offset, float* logits_host) {
  return tb_decoder_step_batch(d, &token_id, &offset, 1, logits_host);
}

tb_status tb_decoder_prefill_tokens(tb_decoder* d, const int64_t* tokens, int64_t n,
                                    int64_t start_offset, int64_t* end_offset) {
  TB_TRY(check_alive(d, "tb_decoder_prefill_tokens"));
  if (n == 0) {  // src/llm/decoder.rs:432-434
    if (end_offset) *end_offset = start_offset;
    return TB_OK;
  }
  if (!tokens || n < 0 || start_offset < 0) return fail(TB_ERR_ARG, "tb_decoder_prefill_tokens: bad arguments");
  if (start_offset + n > d->S)
    return fail(TB_ERR_ARG, "prefill %lld tokens at offset %lld exceeds max_seq_len %lld", (long long)n, (long long)start_offset, (long long)d->S);
  if (d->B > 1 && n > 1) {
    // A decoder built for several rows takes max_batch positions of the prompt per step, like
    // tb_decoder_verify_tokens: one pass over the weights for every max_batch tokens instead of one per token
    // (the reference steps token by token, src/llm/decoder.rs:436-445; the cache rows and the last logits are
    // the same up to the summation order of the batched products).
    TB_TRY(run_positions(d, tokens, n, start_offset, nullptr));
    if (end_offset) *end_offset = start_offset + n;
    return TB_OK;
  }
  if (n > d->feed_cap) {
    cudaFreeHost(d->h_feed);
    d->h_feed = nullptr;
    d->feed_cap = 0;
    DEC_CUDA(d, cudaMallocHost((void**)&d->h_feed, sizeof(int32_t) * 2 * n));
    d->feed_cap = n;
  }
  for (int64_t i = 0; i < n; ++i) {
    d->h_feed[2 * i] = clamp_i32(tokens[i]);
    d->h_feed[2 * i + 1] = clamp_i32(start_offset + i);
    note_kv(d, tokens[i], start_offset + i);
  }
  d->last_batch = 1;
  for (int64_t i = 0; i < n; ++i) {
    DEC_CUDA(d, cudaMemcpyAsync(d->d_tokens, d->h_feed + 2 * i, sizeof(int32_t), cudaMemcpyHostToDevice, d->stream));
    DEC_CUDA(d, cudaMemcpyAsync(d->d_offsets, d->h_feed + 2 * i + 1, sizeof(int32_t), cudaMemcpyHostToDevice, d->stream));
    TB_TRY(run_step(d, 1, false));
  }
  DEC_CUDA(d, cudaStreamSynchronize(d->stream));
  if (end_offset) *end_offset = start_offset + n;
  return check_step_fault(d);
}

tb_status tb_decoder_prefill(tb_decoder* d, const int64_t* tokens, int64_t n, float* logits_host) {
  TB_TRY(check_alive(d, "tb_decoder_prefill"));
  if (n <= 0 || !tokens) return fail(TB_ERR_ARG, "empty prefill");
  if (n > d->S) return fail(TB_ERR_ARG, "prefill exceeds max_seq_len");
  TB_TRY(tb_decoder_prefill_tokens(d, tokens, n, 0, nullptr));
  if (logits_host) return tb_decoder_get_logits(d, logits_host);
  return TB_OK;
}

tb_status tb_decoder_verify_tokens(tb_decoder* d, int64_t start_offset, const int64_t* tokens,
                                   int64_t n, float* logits_host) {
  TB_TRY(check_alive(d, "tb_decoder_verify_tokens"));
  if (n == 0) return TB_OK;
  if (!tokens || !logits_host || n < 0 || start_offset < 0) return fail(TB_ERR_ARG, "tb_decoder_verify_tokens: bad arguments");
  if (start_offset + n > d->S) return fail(TB_ERR_ARG, "verify exceeds max_seq_len");
  // Up to max_batch positions per step: the rows of the batch are consecutive positions of sequence 0, so the
  // projections run as one batched product per matrix and the attention rows share sequence 0's cache
  // (causal inside the block: row r attends to [0, start + r]).  A decoder built for one row steps one
  // position at a time, like src/llm/decoder.rs:575-579.
  return run_positions(d, tokens, n, start_offset, logits_host);
}

tb_status tb_decoder_speculative_accept(tb_decoder* d, int64_t offset, const int64_t* draft_tokens, int64_t k,
                                        const float* draft_probs, float temperature, float top_p,
                                        uint64_t* rng_state, int64_t* accepted, int64_t* bonus) {
  TB_TRY(check_alive(d, "tb_decoder_speculative_accept"));
  if (!accepted || !bonus || !rng_state || k < 0 || offset < 0 || (k > 0 && (!draft_tokens || !draft_probs)))
    return fail(TB_ERR_ARG, "tb_decoder_speculative_accept: bad arguments");
  if (k == 0) {  // src/llm/decoder.rs:594-596
    *accepted = 0;
    *bonus = d->V - 1;
    return TB_OK;
  }
  std::vector<float> rows;
  try {
    rows.resize((size_t)k * (size_t)d->V);
  } catch (...) {
    return fail(TB_ERR_OOM, "tb_decoder_speculative_accept: host allocation failed");
  }
  TB_TRY(tb_decoder_verify_tokens(d, offset, draft_tokens, k, rows.data()));
  return tb_speculative_accept_rows(rows.data(), d->V, draft_tokens, k, draft_probs, temperature, top_p, rng_state,
                                    accepted, bonus);
}

tb_status tb_decoder_reset_kv_cache(tb_decoder* d) {
  TB_TRY(check_alive(d, "tb_decoder_reset_kv_cache"));
  const int64_t used = d->kv_used < d->S ? d->kv_used : d->S;
  if (used == 0) return TB_OK;  // src/llm/decoder.rs:452-455
  const size_t pitch = (size_t)d->S * d->hd * sizeof(float);
  const size_t width = (size_t)used * d->hd * sizeof(float);
  const size_t rows = (size_t)d->L * d->B * d->nkv_l;
  DEC_CUDA(d, cudaMemset2DAsync(d->k_cache, pitch, 0, width, rows, d->stream));
  DEC_CUDA(d, cudaMemset2DAsync(d->v_cache, pitch, 0, width, rows, d->stream));
  DEC_CUDA(d, cudaStreamSynchronize(d->stream));
  d->kv_used = 0;
  return TB_OK;
}

tb_status tb_decoder_copy_kv_cache_from(tb_decoder* d, const float* const* k, const float* const* v,
                                        int32_t num_given, int64_t seq_len, int64_t src_max_len,
                                        int32_t seq, tb_space space) {
  TB_TRY(check_alive(d, "tb_decoder_copy_kv_cache_from"));
  if (!k || !v || num_given < 0 || seq < 0 || seq >= d->B) return fail(TB_ERR_ARG, "tb_decoder_copy_kv_cache_from: bad arguments");
  if (seq_len < 0 || seq_len > d->S || seq_len > src_max_len) return fail(TB_ERR_ARG, "KV cache copy out of bounds");
  const int nl = num_given < d->L ? num_given : d->L;  // src/llm/decoder.rs:486
  const size_t spitch = (size_t)src_max_len * d->hd * sizeof(float);
  const size_t dpitch = (size_t)d->S * d->hd * sizeof(float);
  const size_t width = (size_t)seq_len * d->hd * sizeof(float);
  const cudaMemcpyKind kind = space == TB_HOST ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToDevice;
  if (seq_len > 0)
    for (int l = 0; l < nl; ++l) {
      if (!k[l] || !v[l]) return fail(TB_ERR_ARG, "tb_decoder_copy_kv_cache_from: null layer tensor");
      const size_t base = (size_t)l * kv_layer_stride(d) + (size_t)seq * d->nkv_l * d->S * d->hd;
      DEC_CUDA(d, cudaMemcpy2DAsync(d->k_cache + base, dpitch, k[l], spitch, width, d->nkv_l, kind, d->stream));
      DEC_CUDA(d, cudaMemcpy2DAsync(d->v_cache + base, dpitch, v[l], spitch, width, d->nkv_l, kind, d->stream));
    }
  DEC_CUDA(d, cudaStreamSynchronize(d->stream));
  if (seq_len > d->kv_used) d->kv_used = seq_len;  // src/llm/decoder.rs:521
  return TB_OK;
}

tb_status tb_decoder_read_kv_cache(tb_decoder* d, int32_t layer, int32_t seq, float* k_host, float* v_host) {
  TB_TRY(check_alive(d, "tb_decoder_read_kv_cache"));
  if (layer < 0 || layer >= d->L || seq < 0 || seq >= d->B || !k_host || !v_host) return fail(TB_ERR_ARG, "tb_decoder_read_kv_cache: bad arguments");
  const size_t n = (size_t)d->nkv_l * d->S * d->hd;
  const size_t base = (size_t)layer * kv_layer_stride(d) + (size_t)seq * n;
  DEC_CUDA(d, cudaMemcpyAsync(k_host, d->k_cache + base, n * sizeof(float), cudaMemcpyDeviceToHost, d->stream));
  DEC_CUDA(d, cudaMemcpyAsync(v_host, d->v_cache + base, n * sizeof(float), cudaMemcpyDeviceToHost, d->stream));
  DEC_CUDA(d, cudaStreamSynchronize(d->stream));
  return TB_OK;
}

int64_t tb_decoder_kv_len(const tb_decoder* d) { return d ? d->kv_used : 0; }

tb_status tb_decoder_get_logits(tb_decoder* d, float* logits_host) {
  TB_TRY(check_alive(d, "tb_decoder_get_logits"));
  if (!logits_host) return fail(TB_ERR_ARG, "tb_decoder_get_logits: null buffer");
  DEC_CUDA(d, cudaMemcpyAsync(logits_host, d->logits, sizeof(float) * d->last_batch * d->V, cudaMemcpyDeviceToHost, d->stream));
  DEC_CUDA(d, cudaStreamSynchronize(d->stream));
  return TB_OK;
}

const float* tb_decoder_logits_device(const tb_decoder* d) { return d ? d->logits : nullptr; }

tb_status tb_decoder_generate_greedy(tb_decoder* d, int64_t first_token, int64_t start_offset,
                                     int64_t n_new, int64_t* out_tokens) {
  TB_TRY(check_alive(d, "tb_decoder_generate_greedy"));
  if (n_new == 0) return TB_OK;
  if (!out_tokens || n_new < 0 || start_offset < 0) return fail(TB_ERR_ARG, "tb_decoder_generate_greedy: bad arguments");
  if (start_offset + n_new > d->S) return fail(TB_ERR_ARG, "generate exceeds max_seq_len");
  if (n_new > d->hist_cap) {
    // First use: room for the longest possible run (max_seq_len tokens), so that the graphs, which
    // hold this pointer, are never rebuilt in the middle of a generation.
    cudaFree(d->d_hist);
    d->d_hist = nullptr;
    d->hist_cap = 0;
    const int64_t cap = n_new > d->S ? n_new : d->S;
    TB_TRY(dalloc(&d->d_hist, (size_t)cap));
    d->hist_cap = cap;
    // the graph holds the history pointer: rebuild
    for (int i = 0; i <= kMaxBatch; ++i)
      if (d->graphs_greedy[i]) { cudaGraphExecDestroy(d->graphs_greedy[i]); d->graphs_greedy[i] = nullptr; }
  }
  d->h_io[0] = clamp_i32(first_token);
  d->h_io[kMaxBatch] = clamp_i32(start_offset);
  DEC_CUDA(d, cudaMemcpyAsync(d->d_tokens, d->h_io, sizeof(int32_t), cudaMemcpyHostToDevice, d->stream));
  DEC_CUDA(d, cudaMemcpyAsync(d->d_offsets, d->h_io + kMaxBatch, sizeof(int32_t), cudaMemcpyHostToDevice, d->stream));
  DEC_CUDA(d, cudaMemsetAsync(d->d_hist_pos, 0, sizeof(int32_t), d->stream));
  d->last_batch = 1;
  for (int64_t i = 0; i < n_new; ++i) TB_TRY(run_step(d, 1, true));
  std::vector<int32_t> hist((size_t)n_new);
  DEC_CUDA(d, cudaMemcpyAsync(hist.data(), d->d_hist, sizeof(int32_t) * n_new, cudaMemcpyDeviceToHost, d->stream));
  DEC_CUDA(d, cudaStreamSynchronize(d->stream));
  TB_TRY(check_step_fault(d));
  int64_t tok = first_token;
  for (int64_t i = 0; i < n_new; ++i) {
    note_kv(d, tok, start_offset + i);
    out_tokens[i] = hist[i];
    tok = hist[i];
  }
  return TB_OK;
}

tb_status tb_decoder_decode_greedy(tb_decoder* d, int64_t token_id, int64_t offset, int64_t* next_token) {
  if (!next_token) return fail(TB_ERR_ARG, "tb_decoder_decode_greedy: null out");
  if (d && (offset < 0 || offset >= d->S || token_id < 0 || token_id >= d->V)) {
    // zero logits -> argmax 0 (src/llm/decoder.rs:1066-1078, 895-906)
    TB_TRY(tb_decoder_step(d, token_id, offset, nullptr));
    *next_token = 0;
    return TB_OK;
  }
  return tb_decoder_generate_greedy(d, token_id, offset, 1, next_token);
}

namespace {
float next_uniform(uint64_t* state) {
  uint64_t x = *state ? *state : 0x9E3779B97F4A7C15ull;
  x ^= x << 13; x ^= x >> 7; x ^= x << 17;
  *state = x;
  return (float)((x >> 40) & 0xFFFFFF) / 16777216.0f;  // 24 random bits in [0, 1)
}
}  // namespace

tb_status tb_decoder_decode_and_sample(tb_decoder* d, int64_t token_id, int64_t offset, float temperature,
                                       int64_t top_k, float repetition_penalty, const int64_t* recent,
                                       int64_t n_recent, float top_p, uint64_t* rng_state, int64_t* next_token) {
  TB_TRY(check_alive(d, "tb_decoder_decode_and_sample"));
  if (!next_token) return fail(TB_ERR_ARG, "tb_decoder_decode_and_sample: null out");
  const bool greedy = !std::isfinite(temperature) || temperature <= 0.0f || top_k == 1;
  const bool penalised = repetition_penalty > 1.0f && n_recent > 0;
  if (greedy && !penalised) return tb_decoder_decode_greedy(d, token_id, offset, next_token);
  if (d->host_logits.size() < (size_t)d->V) d->host_logits.resize((size_t)d->V);
  TB_TRY(tb_decoder_step(d, token_id, offset, d->host_logits.data()));
  TB_TRY(tb_apply_repetition_penalty(d->host_logits.data(), d->V, recent, n_recent, repetition_penalty));
  uint64_t local = 0x2545F4914F6CDD1Dull;
  const float u = next_uniform(rng_state ? rng_state : &local);
  return tb_sample_logits(d->host_logits.data(), d->V, temperature, top_k, top_p, u, next_token);
}

tb_status tb_decoder_generate_loop(tb_decoder* d, int64_t first_token, int64_t seq_len, int64_t max_new_tokens,
                                   float temperature, int64_t top_k, float repetition_penalty, float top_p,
                                   int64_t eos_token_id, const int64_t* recent_seed, int64_t n_recent_seed,
                                   uint64_t* rng_state, int64_t* out_tokens, int64_t* n_out, int64_t* end_offset) {
  TB_TRY(check_alive(d, "tb_decoder_generate_loop"));
  if (!out_tokens || !n_out || max_new_tokens < 0 || seq_len < 0) return fail(TB_ERR_ARG, "tb_decoder_generate_loop: bad arguments");
  int64_t recent[64];
  int64_t nrec = 0;
  for (int64_t i = 0; i < n_recent_seed; ++i) nrec = tb_push_recent_window(recent, nrec, recent_seed[i]);
  int64_t next = first_token, generated = 0;
  uint64_t local = 0x2545F4914F6CDD1Dull;
  while (generated < max_new_tokens) {  // decoder.rs:811-829
    if (eos_token_id >= 0 && next == eos_token_id) break;
    out_tokens[generated++] = next;
    nrec = tb_push_recent_window(recent, nrec, next);
    const int64_t offset = seq_len + generated - 1;
    TB_TRY(tb_decoder_decode_and_sample(d, next, offset, temperature, top_k, repetition_penalty, recent, nrec, top_p,
                                        rng_state ? rng_state : &local, &next));
  }
  *n_out = generated;
  if (end_offset) *end_offset = seq_len + generated;
  return TB_OK;
}

tb_status tb_decoder_debug_stage(tb_decoder* d, const char* name, float* out_host, int64_t cap, int64_t* n) {
  TB_TRY(check_alive(d, "tb_decoder_debug_stage"));
  if (!name || !n) return fail(TB_ERR_ARG, "tb_decoder_debug_stage: null argument");
  if (!(d->cfg.flags & TB_DECODER_NO_GRAPH))
    return fail(TB_ERR_UNSUPPORTED, "debug stages are recorded only by a decoder created with TB_DECODER_NO_GRAPH");
  const float* src = nullptr;
  int64_t cnt = 0;
  if (!strcmp(name, "embed")) { src = d->dbg_embed; cnt = d->H; }
  else if (!strcmp(name, "normed")) { src = d->dbg_normed; cnt = d->H; }
  else if (!strcmp(name, "qkv")) { src = d->dbg_qkv; cnt = d->tq_l; }
  else if (!strcmp(name, "attn")) { src = d->dbg_attn; cnt = d->q_dim_l; }
  else if (!strcmp(name, "x_attn")) { src = d->dbg_x_attn; cnt = d->H; }
  else if (!strcmp(name, "h")) { src = d->dbg_h; cnt = d->I_l; }
  else if (!strcmp(name, "x_out")) { src = d->dbg_x_out; cnt = d->H; }
  else return fail(TB_ERR_ARG, "unknown stage '%s'", name);
  *n = cnt;
  if (out_host && cap > 0) {
    const int64_t m = cap < cnt ? cap : cnt;
    DEC_CUDA(d, cudaMemcpyAsync(out_host, src, sizeof(float) * m, cudaMemcpyDeviceToHost, d->stream));
    DEC_CUDA(d, cudaStreamSynchronize(d->stream));
  }
  return TB_OK;
}

tb_status tb_decoder_step_timed(tb_decoder* d, int64_t token_id, int64_t offset, float* logits_host, float ms_out[3]) {
  TB_TRY(check_alive(d, "tb_decoder_step_timed"));
  if (!ms_out) return fail(TB_ERR_ARG, "tb_decoder_step_timed: null ms_out");
  cudaEvent_t ev[4];
  for (auto& e : ev) DEC_CUDA(d, cudaEventCreate(&e));
  d->h_io[0] = clamp_i32(token_id);
  d->h_io[kMaxBatch] = clamp_i32(offset);
  note_kv(d, token_id, offset);
  d->last_batch = 1;
  DEC_CUDA(d, cudaMemcpyAsync(d->d_tokens, d->h_io, sizeof(int32_t), cudaMemcpyHostToDevice, d->stream));
  DEC_CUDA(d, cudaMemcpyAsync(d->d_offsets, d->h_io + kMaxBatch, sizeof(int32_t), cudaMemcpyHostToDevice, d->stream));
  DEC_CUDA(d, cudaEventRecord(ev[0], d->stream));
  // direct launches (no graph) so that an event can sit in front of lm_head
  tb_status s = enqueue_step(d, 1, false, ev[1]);
  if (s == TB_OK) {
    DEC_CUDA(d, cudaEventRecord(ev[2], d->stream));
    if (logits_host)
      DEC_CUDA(d, cudaMemcpyAsync(logits_host, d->logits, sizeof(float) * d->V, cudaMemcpyDeviceToHost, d->stream));
    DEC_CUDA(d, cudaEventRecord(ev[3], d->stream));
    DEC_CUDA(d, cudaStreamSynchronize(d->stream));
    cudaEventElapsedTime(&ms_out[0], ev[0], ev[1]);
    cudaEventElapsedTime(&ms_out[1], ev[1], ev[2]);
    cudaEventElapsedTime(&ms_out[2], ev[2], ev[3]);
  }
  for (auto& e : ev) cudaEventDestroy(e);
  return s;
}

tb_status tb_decoder_tp_init(tb_decoder* d, const uint8_t id[128], tb_allgather_fn allgather, void* user) {
  TB_TRY(check_alive(d, "tb_decoder_tp_init"));
  if (!id) return fail(TB_ERR_ARG, "tb_decoder_tp_init: null id");
  if (d->tp < 2) return fail(TB_ERR_ARG, "tb_decoder_tp_init: the decoder was created with tp_size 1");
  if (d->tpst) return fail(TB_ERR_ARG, "tb_decoder_tp_init: already initialised");
  TB_TRY(tp_create(&d->tpst, d->rank, d->tp, id, (size_t)d->B * d->H, allgather, user,
                   (d->cfg.flags & TB_DECODER_NCCL_ONLY) != 0, (size_t)d->H, (size_t)d->B * d->V));
  if (float* shared_logits = tp_step_logits(d->tpst)) {
    // the gathered logits live in the block every rank has mapped: the step kernel of each rank
    // stores its vocabulary slice straight into every rank's copy
    cudaFree(d->logits);
    d->logits = shared_logits;
    d->logits_shared = true;
  }
  {  // a wait of an exchange kernel that runs out is reported like one of the step kernel: TB_ERR_TIMEOUT
    int* dev_fault = nullptr;
    TB_TRY(fault_word(d, &dev_fault));
    tp_set_host_fault(d->tpst, dev_fault);
  }
  TB_TRY(build_step_program(d));
  // warm-up with an out-of-range token (collective: every rank runs it)
  int64_t tok = -1, off = 0;
  const bool g = d->use_graph;
  d->use_graph = false;
  tb_status s = feed_and_step(d, &tok, &off, 1);
  d->use_graph = g;
  if (s != TB_OK) return s;
  DEC_CUDA(d, cudaStreamSynchronize(d->stream));
  return TB_OK;
}

int32_t tb_decoder_is_device_lost(const tb_decoder* d) { return d && d->device_lost ? 1 : 0; }
void tb_decoder_mark_device_lost(tb_decoder* d) { if (d) d->device_lost = true; }
int32_t tb_decoder_launches_per_step(const tb_decoder* d) { return d ? d->launches_per_step : 0; }
void* tb_decoder_stream(const tb_decoder* d) { return d ? (void*)d->stream : nullptr; }

}  // extern "C"
