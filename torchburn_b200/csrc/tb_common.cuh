// Shared host/device helpers of the torchburn_b200 library.
#pragma once

#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/torchburn_b200.h"

namespace tb {

// Thread-local last-error message behind tb_last_error_string().
void set_error(const char* fmt, ...);
tb_status fail(tb_status code, const char* fmt, ...);

#define TB_CUDA_TRY(expr)                                                                  \
  do {                                                                                     \
    cudaError_t _e = (expr);                                                               \
    if (_e != cudaSuccess) {                                                               \
      return ::tb::fail(_e == cudaErrorMemoryAllocation ? TB_ERR_OOM : TB_ERR_CUDA,        \
                        "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__,  \
                        __LINE__);                                                         \
    }                                                                                      \
  } while (0)

#define TB_TRY(expr)                   \
  do {                                 \
    tb_status _s = (expr);             \
    if (_s != TB_OK) return _s;        \
  } while (0)

inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }

// Number of SMs of the current device (cached per device).
int sm_count();
// Copies `bytes` from host or device memory into a fresh device allocation.
tb_status upload(void** dst, const void* src, size_t bytes, tb_space space);

// ---- per-CTA timestamps of the hot kernels (off unless a buffer was registered) -------------
// The role of the reference's timestamp queries (src/wgpu/profiler.rs).  Every launch of an
// instrumented kernel gets the next block of kTlBlock 64-bit words of the registered device
// buffer: words 0-7 = {kind, grid size, 0...}, then 8 event slots for each of the first
// kTlCtas CTAs, holding %globaltimer values in ns.
constexpr int kTlCtas = 512;
constexpr int kTlBlock = (1 + kTlCtas) * 8;
unsigned long long* timeline_next_block();   // null when no buffer is registered or it is full
void timeline_register(void* device_buffer, int64_t bytes);
int timeline_blocks_used();
#ifdef __CUDACC__
__device__ __forceinline__ void tl_mark(unsigned long long* tl, int cta, int ev) {
  if (tl != nullptr && cta < kTlCtas) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    tl[(1 + cta) * 8 + ev] = t;
  }
}
__device__ __forceinline__ void tl_header(unsigned long long* tl, int kind, int grid) {
  if (tl != nullptr) {
    tl[0] = (unsigned long long)kind;
    tl[1] = (unsigned long long)grid;
  }
}
#endif

// ---- argument blocks of the kernel launchers (all pointers DEVICE) ----------

// One grouped-INT4 projection y = W x (+ epilogue).  See w4_gemv.cu.
struct GemvArgs {
  const float* x = nullptr;        // [m, k]
  const uint8_t* w = nullptr;      // [n, k/2]
  const float* scales = nullptr;   // [n, k/g]
  const float* bias = nullptr;     // [n] or null
  const uint8_t* w2 = nullptr;     // SwiGLU: the "up" matrix (w is "gate")
  const float* scales2 = nullptr;
  const float* bias2 = nullptr;
  const float* norm_w = nullptr;   // fused RMSNorm of x before the product: [k] or null
  float eps = 0.f;
  const float* resid = nullptr;    // out = resid + y when not null: [m, n]
  float* out = nullptr;            // [m, n]
  float* x_normed_out = nullptr;   // optional copy of the normalised x (debug): [m, k]
  // Split RMSNorm (M = 1, persistent kernel only).  A producer launch may also write
  // out_scaled = out * out_scale_w (the next norm's weights) and out_ss8[i] = sum of out^2 over
  // rows 8i..8i+7.  A consumer launch whose x is such a pre-weighted vector passes x_ss8 (and eps,
  // no norm_w): its row sums are divided by sqrt(sum(x_ss8)/k + eps).  This halves the bytes every
  // CTA pulls from L2 before its first product and takes the norm's barrier off that path.
  const float* x_ss8 = nullptr;
  float* out_scaled = nullptr;
  const float* out_scale_w = nullptr;
  float* out_ss8 = nullptr;
  int m = 1;
  int64_t n = 0, k = 0;
  int g = 32;
  bool pdl = false;                // launch with programmatic stream serialization
  void* xq_scratch = nullptr;      // m > 1: room for the digit form of x (w4_mma_scratch_bytes);
                                   // null = allocate on the stream for the duration of the call
};

tb_status launch_w4_gemv(const GemvArgs& a, cudaStream_t stream);
// Kernels that call starts (1, or 2 with the activation pre-pass of the tensor-core kernels).
int w4_gemv_launches(const GemvArgs& a);
// Frees the per-stream workspaces that calls with several activation rows and no workspace of their own keep.
void release_workspaces();
// Tuning hook: xmode 0 = fp32 products (M = 1 only), 1 = integer products; rows_per_warp /
// warps force the launch shape of the M = 1 kernels (0 = automatic).
void set_gemv_tuning(int xmode, int rows_per_warp, int warps);

// Tensor-core kernel for 2 <= M (w4_mma.cu).
size_t w4_mma_scratch_bytes(int m, int64_t k);
tb_status launch_w4_mma(const GemvArgs& a, void* scratch, cudaStream_t stream);
// tcgen05 kernel for 16 < M (w4_tc5.cu); its operand images live behind the first 4096 bytes of the same scratch.
size_t w4_tc5_scratch_bytes(int m, int64_t k);
bool w4_tc5_supported(const GemvArgs& a);
tb_status launch_w4_tc5(const GemvArgs& a, void* scratch, cudaStream_t stream);
void set_tc5_enabled(int on);
int tc5_fault_flag();

// Persistent TMA-ring kernel for M = 1 (w4_stream.cu).
bool w4_stream_supported(const GemvArgs& a);
tb_status launch_w4_stream(const GemvArgs& a, cudaStream_t stream);
void set_stream_tuning(int enabled, int ctas_per_sm, int ring_kb, int epl, int groups);
int stream_fault_flag();

struct AttnArgs {
  const float* qkv = nullptr;   // [b, (Hq+2Hkv)*d], before RoPE
  float* k_cache = nullptr;     // [b, Hkv, max_seq, d]
  float* v_cache = nullptr;
  const float* cos_t = nullptr; // [max_seq, d] (or [b, d] when per_call_tables)
  const float* sin_t = nullptr;
  const int32_t* offsets = nullptr;  // [b]
  float* out = nullptr;         // [b, Hq*d]
  void* scratch = nullptr;
  float* q_rot_out = nullptr;   // optional: rotated q|k|v copy (debug) [b, (Hq+2Hkv)*d]
  int batch = 1, num_heads = 0, num_kv_heads = 0, head_dim = 0;
  int64_t max_seq_len = 0;
  bool per_call_tables = false; // cos/sin hold one row per sequence instead of a table
  bool shared_cache = false;    // the rows are positions of ONE sequence (sequence 0's cache); launch_rope_append_rows goes first
  bool pdl = false;
};
size_t attention_scratch_bytes(int batch, int num_heads, int num_kv_heads, int head_dim,
                               int64_t max_seq_len);
// Byte offset of the ticket counters inside the scratch block (they must be zero before the
// first launch).
size_t attention_counters_offset(int batch, int num_heads, int num_kv_heads, int head_dim,
                                 int64_t max_seq_len, size_t* counter_bytes);
// Tuning hook: force the positions per attention CTA (0 = automatic).
void set_attention_chunk_override(int tc);
// Tuning hook: resident CTAs per SM the grid is sized for and ring depth (0 = automatic).
void set_attention_tuning(int ctas_per_sm, int stages);
// 1 once a bounded wait of the attention kernel ran out (results of that launch are invalid).
int attention_fault_flag();
tb_status launch_attention_decode(const AttnArgs& a, cudaStream_t stream);
tb_status launch_rope_append_rows(const AttnArgs& a, cudaStream_t stream);
// The library's built-in scratch block for tb_attention_decode_static (attention.cu).
size_t static_attention_scratch_capacity();
tb_status static_attention_scratch(void** ptr);

// ---- the whole decode step as one persistent kernel (w4_step.cu) ------------------------------
// A step is a list of phases that every CTA of one cooperative grid walks in order, with a
// grid-wide barrier after each: projections (kind 0), the split-K attention over one layer's
// cache (kind 1), the merge of its partials (kind 2) and, tensor parallel, the sum of the ranks'
// partial rows with the residual (kind 3; n rows, exchange number xi, no barrier in front of it).
struct StepPhase {
  int kind = 0;
  int n = 0;            // projection: output rows (row pairs for the SwiGLU form)
  int k = 0;            // projection: input features
  int ng = 0;           // scales per row
  int gshift = 0;       // log2(group_size / 32)
  int rs = 8;           // rows per ring stage and matrix (1, 2, 4 or 8)
  int nw = 1;           // 2 = gate/up pair with the SwiGLU epilogue
  int rot = 0;          // rotation of the balanced split of the 8-row rounds over the CTAs
  float eps = 0.f;
  int tp_mode = 0;      // tensor parallel: 1 = push the rows to every rank's receive area (exchange number xi),
                        // 2 = store them into every rank's logits at column offset xi
  int xi = 0;
  int pad = 0;
  const uint8_t* w[2] = {nullptr, nullptr};
  const float* sc[2] = {nullptr, nullptr};
  const float* bias[2] = {nullptr, nullptr};
  const float* x = nullptr;          // [k]
  const float* x_ss8 = nullptr;      // x is pre-weighted by the norm; sums of squares per 8 elements (null: no norm)
  const float* resid = nullptr;      // out = resid + y
  float* out = nullptr;
  float* out_scaled = nullptr;       // optional out * out_scale_w (the next norm's weights)
  const float* out_scale_w = nullptr;
  float* out_ss8 = nullptr;          // optional sums of squares of out per 8 rows
  float* k_cache = nullptr;          // attention: this layer's [Hkv, max_seq_len, d]
  float* v_cache = nullptr;
  const void* reserved = nullptr;
};
constexpr int kStepPhaseWords = 11;
static_assert(sizeof(StepPhase) == 16 * kStepPhaseWords, "StepPhase is copied as 16-byte words");

// Tensor-parallel side of the step kernel: pointers into every rank's shared block (peer memory).
struct StepTp {
  int rank = 0, size = 1, hidden = 0;
  uint2* recv[8] = {};          // [2][size][hidden] {partial, exchange number}: rank r's receive area
  float* logits[8] = {};        // rank r's copy of the gathered logits
  uint32_t* flags[8] = {};      // rank r's words [size]: source s stores the exchange number at [s]
  uint32_t* epoch = nullptr;    // this rank: exchanges completed by earlier launches
  int* err = nullptr;
};

struct StepProgram {
  const StepPhase* phases = nullptr;   // device array
  int nphases = 0;
  int grid = 0;                        // CTAs the program was laid out for (rot fields, attention split)
  unsigned* sync = nullptr;            // device, 16-byte aligned: [0..3] barrier arrivals, [4] exit tickets; zero before the first launch
  int* host_fault = nullptr;           // optional host-mapped word, set to 1 when a bounded wait ran out
  const float* qkv = nullptr;          // [(Hq + 2 Hkv) * d] of the current token, before RoPE
  float* attn = nullptr;               // [Hq * d]
  const float* cos_t = nullptr;
  const float* sin_t = nullptr;
  const int32_t* offsets = nullptr;    // [1] effective offset (-1: nothing to attend to)
  float* part_o = nullptr;             // [Hq, nc, d]
  float* part_ml = nullptr;            // [Hq, nc, 2]
  int num_heads = 0, num_kv_heads = 0, head_dim = 0;
  int nc = 0;                          // CTAs per kv head in the attention phases
  int64_t max_seq_len = 0;
  StepTp tp;                           // size 1: one GPU
  int n_exchanges = 0;                 // in-kernel exchanges per launch (tensor parallel)
};
// CTAs of the step kernel on the current device (0 when it cannot run there).
int w4_step_grid();
// Shape rules of one projection phase.
bool w4_step_supports(int64_t n, int64_t k, int g, int nw);
int w4_step_rows_per_stage(int64_t k, int g, int nw);
// Attention split: CTAs per kv head and bytes of the two partial arrays.
int w4_step_attn_split(int grid, int num_kv_heads);
tb_status launch_w4_step(const StepProgram& prog, cudaStream_t stream);
tb_status launch_w4_step_gemv(const GemvArgs& a, cudaStream_t stream);
// x = table[token] (zeros and offset -1 when token or offset is out of range), xn = x * norm_w,
// ss8[i] = sum of x^2 over elements 8i..8i+7: what the first phase of a step starts from.
tb_status launch_step_embed(const float* table, const int32_t* tokens, const int32_t* offsets, const float* norm_w,
                            float* x, float* xn, float* ss8, int32_t* eff_offsets, int64_t vocab, int64_t hidden,
                            int64_t max_seq_len, cudaStream_t stream);
int step_fault_flag();
// Test hook: cycles a device-side wait of the step kernel may take before it gives up (0 = default).
void set_step_wait_limit(long long cycles);
void set_step_debug(int flags);
tb_status step_wait_probe(long long limit_cycles);

tb_status launch_rms_norm(const float* x, const float* w, float* out, int64_t m, int64_t n,
                          float eps, cudaStream_t stream);
// x[b] = table[tokens[b]] and eff_offsets[b] = offsets[b] when token and offset are in range,
// else x[b] = 0 and eff_offsets[b] = -1 (src/llm/decoder.rs:1066-1092).
tb_status launch_embed_gather(const float* table, const int32_t* tokens, const int32_t* offsets,
                              float* x, int32_t* eff_offsets, int batch, int64_t vocab,
                              int64_t hidden, int64_t max_seq_len, bool pdl, cudaStream_t stream);
tb_status launch_quantize_int4(const float* w, int64_t n, int64_t k, int g, uint8_t* packed,
                               float* scales, cudaStream_t stream);
// out_tokens[b] = first index of the maximum of logits[b] (src/llm/decoder.rs:895-906); when
// next_offsets is not null, next_offsets[b] += 1 (feeds the next step of a generate loop).
// When hist is not null, sequence 0's token is appended at hist[(*hist_pos)++].
tb_status launch_argmax(const float* logits, int64_t vocab, int batch, int32_t* out_tokens,
                        int32_t* next_offsets, int32_t* hist, int32_t* hist_pos, void* scratch,
                        cudaStream_t stream);
// `scratch`: batch * 12 bytes (8-byte aligned), zero before the first launch; left zero.

}  // namespace tb
