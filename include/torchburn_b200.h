/*
 * torchburn_b200 - C ABI of the B200 (sm_100a) implementation of torchburn's
 * quantized decode hot path: the grouped INT4 W4A32 linear and the LLM decoder
 * step built around it.
 *
 * Every entry point is plain C: pointers, sizes, an opaque handle, an integer
 * status.  No C++ exception crosses this boundary.  Each declaration names the
 * interface of the reference (kuntal-devrat/torchburn, paths relative to its
 * source tree) that it stands in for.
 *
 * Memory spaces.  Weights are handed over once (host or device memory, stated
 * by a tb_space argument) and copied into device memory owned by the handle,
 * like RustQwenDecoder::new copies every weight into its own Vec
 * (src/llm/decoder.rs:235-332).  Activations and results are host or device
 * pointers as stated per call.  `stream` arguments are a cudaStream_t passed as
 * void* (NULL = the legacy default stream).
 *
 * Threading.  Stateless functions and tb_linear handles may be used from
 * several host threads on distinct streams.  A tb_decoder is not re-entrant
 * (the reference's decoder methods take &mut self).
 *
 * Errors.  Functions return TB_OK or a negative-free small status code;
 * tb_last_error_string() gives the message of the calling thread's last
 * failure.  There is no CPU fallback: without a usable CUDA device every
 * compute entry point fails with TB_ERR_CUDA.
 */
#ifndef TORCHBURN_B200_H
#define TORCHBURN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* The library is built with hidden visibility; only this ABI is exported. */
#if defined(__GNUC__)
#pragma GCC visibility push(default)
#endif

typedef int32_t tb_status;
enum {
  TB_OK = 0,
  TB_ERR_ARG = 1,         /* NULL pointer / bad enum: PyValueError in the reference */
  TB_ERR_SHAPE = 2,       /* "TB_UNSUPPORTED:" shape errors, src/quantization/packed_v2.rs:566-596 */
  TB_ERR_DTYPE = 3,       /* kept for ABI completeness; this ABI is typed */
  TB_ERR_OOM = 4,         /* PyMemoryError, src/llm/decoder.rs:239-246 */
  TB_ERR_CUDA = 5,        /* any CUDA runtime failure */
  TB_ERR_NCCL = 6,
  TB_ERR_TIMEOUT = 7,     /* a bounded device-side wait ran out */
  TB_ERR_DEVICE_LOST = 8, /* sticky, src/wgpu/decode.rs:692-716 */
  TB_ERR_UNSUPPORTED = 9
};

typedef enum tb_space { TB_HOST = 0, TB_DEVICE = 1 } tb_space;

#define TB_ABI_VERSION 1

int32_t tb_abi_version(void);
/* Message of the calling thread's most recent failure ("" if none). */
const char* tb_last_error_string(void);
/* One-line JSON description of the current CUDA device (name, SM count, ...).
 * Stands in for cpu_features_report, src/ffi/debug_ffi.rs:12-22. */
tb_status tb_device_report(char* buf, size_t cap);

/* ------------------------------------------------------------------------
 * Raw kernel surface on DEVICE pointers: the counterpart of the pointer-level
 * functions re-exported for benches and parity tests, src/kernels/mod.rs:16-25.
 * All tensors are contiguous and row-major.
 * ---------------------------------------------------------------------- */

/* out[j] = sum_g scales[j,g] * sum_{i in g} x[i] * code(w[j,i]) + bias[j].
 * x [k] f32, w [n, k/2] u8 (element i of a row in byte i/2, low nibble for
 * even i, code = nibble - 8), scales [n, k/group_size] f32, bias [n] or NULL.
 * Replaces gemv_w4a32_grouped, src/quantization/gemv.rs:1514-1684.
 * group_size must be 32 or 64 and divide k (the reference's SIMD tiers make the
 * same assumption, gemv.rs:1579-1600). */
tb_status tb_gemv_w4a32_grouped(const float* x, const uint8_t* w, const float* scales,
                                const float* bias, float* out, int64_t n, int64_t k,
                                int32_t group_size, void* stream);

/* x [m,k] -> out [m,n]; same arithmetic per row of x.
 * Replaces gemm_w4a32_grouped, src/quantization/gemv.rs:1690-1725. */
tb_status tb_gemm_w4a32_grouped(const float* x, const uint8_t* w, const float* scales,
                                const float* bias, float* out, int64_t m, int64_t n, int64_t k,
                                int32_t group_size, void* stream);

/* h[r,j] = silu(gate_j(x_r)) * up_j(x_r), silu(g) = g / (1 + exp(-g)).
 * Replaces the SwiGLU neuron loop, src/llm/decoder.rs:1280-1328 and
 * src/quantization/gemv/swiglu.rs:205-289. gate_b/up_b may be NULL. */
tb_status tb_swiglu_gemv_w4a32(const float* x, const uint8_t* gate_w, const float* gate_s,
                               const float* gate_b, const uint8_t* up_w, const float* up_s,
                               const float* up_b, float* h, int64_t m, int64_t n, int64_t k,
                               int32_t group_size, void* stream);

/* out[r,i] = x[r,i] * (1/sqrt(mean(x[r]^2) + eps)) * w[i], rows = m.
 * Replaces fast_rms_norm, src/quantization/fused_ops.rs:1066-1117. */
tb_status tb_fast_rms_norm(const float* x, const float* w, float* out, int64_t m, int64_t n,
                           float eps, void* stream);

/* Per (row, group): scale = max(absmax/7, 1e-8); code = clamp(rint(w/scale), -8, 7);
 * byte j = (code[2j]+8) | (code[2j+1]+8) << 4.  All pointers DEVICE.
 * Replaces quantize_weight_int4_grouped, python/torchburn/quantization.py:53-118
 * (bit-exact, including round-half-to-even and fp32 division). */
tb_status tb_quantize_weight_int4_grouped(const float* w, int64_t n, int64_t k,
                                          int32_t group_size, uint8_t* packed, float* scales,
                                          void* stream);

/* GQA decode attention for one new position per sequence.
 * qkv [b, (Hq+2Hkv)*d] f32 = [q | k | v] of the new token BEFORE RoPE.  The
 * call rotates q and k (rotate-half, tables cos/sin [max_seq_len, d]), writes
 * k,v into the caches at [seq, kv_h, offset, :] and computes, per q head h
 * (kv_h = h / (Hq/Hkv)), softmax((q.k_t)/sqrt(d)) over t in [0, offset] times V.
 * k_cache, v_cache: [b, Hkv, max_seq_len, d] f32.  offsets [b] int32 DEVICE.
 * out [b, Hq*d].  max_seq_len above 32768 is refused with TB_ERR_UNSUPPORTED (the reference
 * attends to at most 32768 positions, src/llm/decoder.rs:1180).  `scratch` is device memory of
 * tb_attention_scratch_bytes(),
 * zero-filled once before its first use (the kernel leaves its counters zero).
 * Replaces steps C-E of step_internal, src/llm/decoder.rs:1127-1213
 * (src/shaders/rope_append.wgsl + attn_decode.wgsl on the wgpu path). */
size_t tb_attention_scratch_bytes(int32_t batch, int32_t num_heads, int32_t num_kv_heads,
                                  int32_t head_dim, int64_t max_seq_len);
tb_status tb_attention_decode(const float* qkv, float* k_cache, float* v_cache,
                              const float* cos_table, const float* sin_table,
                              const int32_t* offsets, float* out, void* scratch, int32_t batch,
                              int32_t num_heads, int32_t num_kv_heads, int32_t head_dim,
                              int64_t max_seq_len, void* stream);

/* tb_attention_decode for callers that cannot allocate device memory.  (No counterpart in
 * the reference: its attention runs on the host and needs no scratch.)
 *
 * Who needs it: a server that hands out all of its device memory at start-up and has nothing
 * left to cudaMalloc from; code that may run while some thread of the process is capturing a
 * CUDA graph, where an allocation would invalidate the capture; a latency-critical loop that
 * cannot afford the device-wide stall of an allocation.  For them the split-K partials and
 * ticket counters live in a block of tb_attention_static_scratch_bytes() (8 MiB) that is part
 * of the library's device image - every GPU that loads the library carries it until the
 * process exits.  The caller still passes all inputs and outputs; arguments and results are
 * those of tb_attention_decode.
 *
 * Limit: shapes with tb_attention_scratch_bytes(...) above that size fail with
 * TB_ERR_UNSUPPORTED (use tb_attention_decode with your own scratch).  The call allocates
 * nothing: no cudaMalloc / cudaFree, only a memset of its counters and the kernel launch.
 * The first call on each device looks up the block's device address; make that first call
 * before any stream capture begins.  All calls on a device share the one block, which keeps
 * the previous call's contents: the entry point clears what must start at zero itself, but
 * two calls that overlap on the GPU (different streams) race on it - serialise them. */
size_t tb_attention_static_scratch_bytes(void);
tb_status tb_attention_decode_static(const float* qkv, float* k_cache, float* v_cache,
                                     const float* cos_table, const float* sin_table,
                                     const int32_t* offsets, float* out, int32_t batch,
                                     int32_t num_heads, int32_t num_kv_heads, int32_t head_dim,
                                     int64_t max_seq_len, void* stream);

/* Profiling hook in the role of the reference's timestamp queries (src/wgpu/profiler.rs:1-120).
 * After a device buffer is registered, every launch of the streaming GEMV and of the attention
 * kernel - launches recorded into a CUDA graph included, so register before the first step of a
 * decoder - takes the next block of 4104 64-bit words: words 0-1 = {kind (1 GEMV, 2 attention),
 * grid size}, then for each of the first 512 CTAs eight %globaltimer values in ns: 0 entry,
 * 1 past the grid dependency wait, 2 activations ready, 3 first stage arrived, 4 last stage
 * consumed, 5 exit, 6 first copy requested, 7 last copy requested.  NULL switches it off.
 * tb_debug_timeline_blocks returns how many blocks were handed out. */
void tb_debug_timeline(void* device_buffer, int64_t bytes);
int32_t tb_debug_timeline_blocks(void);
/* Test hook of the persistent step kernel: bit 0 = the projections consume their weight stream
 * without multiplying (measures the stream alone; results are meaningless).  Process-wide. */
void tb_debug_step_flags(int32_t flags);
/* Failure detection without a fault (the role of the reference's device-lost handling,
 * src/wgpu/decode.rs:1140-1145): launches one warp that waits, with the given limit in clock
 * cycles, on an mbarrier nobody completes and on a grid barrier that is one arrival short.  Both
 * waits must give up and raise the fault word.  Returns TB_ERR_TIMEOUT when they did (the word is
 * cleared again), TB_ERR_CUDA on any other outcome.  Nothing hangs, traps or faults. */
tb_status tb_debug_wait_probe(int64_t limit_cycles);
/* The limit, in clock cycles, of every bounded wait of the persistent step kernel and of the tensor-parallel
 * exchange kernels' waits for their peers (0 = the defaults of about two and ten seconds).  Failure-detection tests shorten it so that a peer that never arrives is reported
 * (TB_ERR_TIMEOUT, decoder marked lost) within a second.  Process-wide. */
void tb_debug_step_wait_limit(int64_t cycles);
/* One projection through the persistent step kernel's code path (a program of one phase):
 * out = W x + bias, or silu(W x) * (W2 x) when w2/scales2 are not NULL.  All pointers DEVICE.
 * For parity tests and profiling of that path at any shape; tb_gemv_w4a32_grouped is the
 * product entry point.  TB_ERR_UNSUPPORTED for shapes the step kernel does not take. */
tb_status tb_debug_step_gemv(const float* x, const uint8_t* w, const float* scales, const float* bias,
                             const uint8_t* w2, const float* scales2, float* out, int64_t n, int64_t k,
                             int32_t group_size, void* stream);

/* Tuning hook: positions of the KV sequence handled per attention CTA (a power
 * of two in [64, 512]; 0 = choose from the shape).  Process-wide; plays the role
 * of TORCHBURN_ROWS_PER_WG, src/wgpu/backend.rs:428-437. */
void tb_set_attention_chunk(int32_t positions);
/* Tuning hook: how many resident CTAs per SM the attention grid is sized for (the current
 * sequence length is divided evenly among them) and the depth of each CTA's ring of
 * shared-memory stages (at most 8).  0 = automatic for either.  Process-wide. */
void tb_set_attention_tuning(int32_t ctas_per_sm, int32_t ring_stages);
/* Tuning hook for the M = 1 GEMV kernels.  product_mode 1 (default): activations are
 * rounded per 32-element block to 24-bit fixed point and multiplied with integer dot
 * products (2 <= M <= 16 with integer mma.sync; 16 < M on tcgen05 with exact bf16 codes and the
 * activations as three bf16 pieces); 0: fp32 products for M = 1; 2: integer products on
 * CUDA cores for every M (no tensor cores); 3: like 1 but the integer mma.sync kernel for every
 * M >= 2 (no tcgen05).  rows_per_warp in {0,1,2,4} and warps in {0,4,8} force
 * the launch shape (0 = choose from the matrix size).  Process-wide. */
void tb_set_gemv_tuning(int32_t product_mode, int32_t rows_per_warp, int32_t warps);
/* Tuning hook for the persistent M = 1 kernel (one long-lived CTA per SM fed by a ring of
 * bulk asynchronous copies): enabled 0 routes every product to the per-row-tile kernels;
 * ctas_per_sm in {1, 2, ...}; ring_kb = shared-memory ring size per CTA (0 = default);
 * elements_per_lane in {0, 16, 32} and groups in {0..4} force the split of K over lanes and
 * the number of tiles a CTA works on at once (0 = choose from the shape). */
void tb_set_stream_tuning(int32_t enabled, int32_t ctas_per_sm, int32_t ring_kb,
                          int32_t elements_per_lane, int32_t groups);
/* The stateless products (tb_gemm_w4a32_grouped, tb_swiglu_gemv_w4a32, tb_linear_forward, ...) with two or more
 * activation rows need a workspace (digit form of x, partial sums of a K split).  The library keeps one block
 * per (device, stream), allocated at the first such call on the stream outside a graph capture and grown on
 * demand - the reference allocates its outputs per call too (src/quantization/packed_v2.rs:598-606).  This frees
 * all of them (after a device synchronize); later calls allocate again. */
void tb_release_workspaces(void);
/* 1 after a bounded device-side wait ran out in any kernel of this library on the current
 * device (the results of that launch are invalid), 0 otherwise, -1 if the flag could not
 * be read.  Device-side waits never spin without a limit. */
int32_t tb_device_fault_flag(void);

/* ------------------------------------------------------------------------
 * QuantizedLinear (python/torchburn/quantization.py:756-869) as a handle.
 * ---------------------------------------------------------------------- */
typedef struct tb_linear tb_linear;

/* qweight [out_features, in_features/2] u8, scales [out_features,
 * in_features/group_size] f32, bias [out_features] or NULL; copied to device.
 * Shape rules of w4a32_grouped_linear, src/quantization/packed_v2.rs:573-596. */
tb_status tb_linear_create(tb_linear** out, const uint8_t* qweight, const float* scales,
                           const float* bias, int64_t out_features, int64_t in_features,
                           int32_t group_size, tb_space weight_space);
void tb_linear_destroy(tb_linear* lin);

/* The interleaved "v2" weight layout (src/quantization/packed_v2.rs:26-143,
 * python/torchburn/quantization.py:121-170): group size 64 only; each group of a row is one
 * 34-byte block = 32 bytes of packed nibbles + the scale as IEEE binary16, little-endian; a row
 * is (in_features / 64) blocks.  All of these are host functions.
 *   tb_f32_to_f16 / tb_f16_to_f32   f32_to_f16 (round to nearest even) and f16_to_f32 (:30-112)
 *   tb_pack_v1_to_v2                pack_rows_w4a32_group64_v1_to_v2 (:114-143)
 *   tb_unpack_v2_to_v1              the inverse; the fp32 scales are the binary16 values
 *   tb_linear_create_v2             a tb_linear from v2 blocks (host or device), the role of
 *                                   w4a32_grouped_linear_v2 (quantization.py:172-190): unpacked
 *                                   once, then the same kernels run with the binary16 scales.
 * in_features not divisible by 64 -> TB_ERR_SHAPE ("TB_UNSUPPORTED:", as packed_v2.rs:566-596). */
uint16_t tb_f32_to_f16(float value);
float tb_f16_to_f32(uint16_t bits);
tb_status tb_pack_v1_to_v2(const uint8_t* qweight, const float* scales, int64_t out_features,
                           int64_t in_features, uint8_t* blocks);
tb_status tb_unpack_v2_to_v1(const uint8_t* blocks, int64_t out_features, int64_t in_features,
                             uint8_t* qweight, float* scales);
tb_status tb_linear_create_v2(tb_linear** out, const uint8_t* blocks, const float* bias,
                              int64_t out_features, int64_t in_features, tb_space weight_space);
/* QuantizedLinear.forward -> w4a32_grouped_linear (quantization.py:826-866,
 * src/ffi/quantization_ffi.rs:56-85): x [m, in_features] -> out [m, out_features].
 * io_space says where x and out live; host buffers are staged through pinned
 * memory owned by the handle and the call returns after the result is in `out`. */
tb_status tb_linear_forward(tb_linear* lin, const float* x, int64_t m, float* out,
                            tb_space io_space, void* stream);
/* Device views of the handle's operands (for the raw kernel surface). */
tb_status tb_linear_device_ptrs(const tb_linear* lin, const uint8_t** qweight,
                                const float** scales, const float** bias);

/* fused_swiglu_mlp / fused_swiglu_mlp_batched: out = down(silu(gate(x)) * up(x)),
 * x [m, hidden] -> out [m, hidden].  src/ffi/quantization_ffi.rs:203-218, 517-532;
 * src/quantization/fused_ops.rs:138-424, 1267-1319. */
tb_status tb_fused_swiglu_mlp(tb_linear* gate, tb_linear* up, tb_linear* down, const float* x,
                              int64_t m, float* out, tb_space io_space, void* stream);

/* fused_attention_step_w4a32 (src/ffi/quantization_ffi.rs:344-363,
 * src/quantization/fused_ops.rs:891-1062): QKV GEMV -> RoPE with the given
 * cos/sin (length head_dim, for this position) -> write K,V into the caller's
 * caches [1, Hkv, max_seq_len, d] (DEVICE, mutated) -> attention -> O GEMV.
 * x [hidden], cos/sin and out [hidden] in io_space. */
tb_status tb_fused_attention_step(tb_linear* qkv, tb_linear* o, const float* x, float* k_cache,
                                  float* v_cache, const float* cos_p, const float* sin_p,
                                  int64_t offset, int32_t num_heads, int32_t num_kv_heads,
                                  int32_t head_dim, int64_t max_seq_len, float* out,
                                  tb_space io_space, void* stream);

/* fused_transformer_layer_step_w4a32 (src/ffi/quantization_ffi.rs:406-438,
 * src/quantization/fused_transformer.rs:16-376): one decoder layer for one token, IN PLACE on x:
 *   x += O(attention(rope(QKV(rms_norm(x, input_norm_w))))); x += down(silu(gate(n)) * up(n)),
 *   n = rms_norm(x, post_norm_w).
 * The 17 weight / bias tensors of the reference's positional arguments travel in one struct, all
 * DEVICE pointers in the layouts of tb_gemv_w4a32_grouped; the four biases after qkv_b may be NULL
 * like the reference's Option arguments.  k_cache / v_cache: [1, Hkv, max_seq_len, d] f32, DEVICE,
 * mutated at `offset` (the reference writes through its const capsules, fused_transformer.rs:172-187).
 * cos_p / sin_p: the rotation of THIS position, length head_dim.  x [hidden], cos_p and sin_p live
 * in io_space.  hidden_size and intermediate_size are explicit (the reference reads them from the
 * tensor shapes).  Errors: TB_ERR_ARG for null tensors or an offset outside the cache,
 * TB_ERR_SHAPE with the "TB_UNSUPPORTED:" marker for shapes the linears refuse. */
typedef struct tb_layer_step_weights {
  const float* input_norm_w;
  const uint8_t* qkv_w;
  const float* qkv_s;
  const float* qkv_b;
  const uint8_t* o_w;
  const float* o_s;
  const float* o_b;
  const float* post_norm_w;
  const uint8_t* gate_w;
  const float* gate_s;
  const float* gate_b;
  const uint8_t* up_w;
  const float* up_s;
  const float* up_b;
  const uint8_t* down_w;
  const float* down_s;
  const float* down_b;
} tb_layer_step_weights;
tb_status tb_fused_transformer_layer_step(float* x, const tb_layer_step_weights* w, float* k_cache, float* v_cache,
                                          const float* cos_p, const float* sin_p, int64_t offset,
                                          int64_t hidden_size, int64_t intermediate_size, int32_t num_heads,
                                          int32_t num_kv_heads, int32_t head_dim, int64_t max_seq_len,
                                          int32_t group_size, float eps, tb_space io_space, void* stream);

/* ------------------------------------------------------------------------
 * Decoder: RustQwenDecoder / WgpuQwenDecoder (src/llm/decoder.rs:111-171,
 * src/wgpu/decode.rs:297-334) as a handle.
 * ---------------------------------------------------------------------- */

/* Constructor arguments, src/llm/decoder.rs:176-210 (defaults there:
 * group_size 64, rms_norm_eps 1e-6, max_seq_len 2048, rope_theta 1e6).
 * max_batch > 1 and tp_size > 1 have no counterpart in the reference. */
typedef struct tb_model_config {
  int64_t vocab_size;
  int64_t hidden_size;
  int64_t intermediate_size;
  int32_t num_layers;
  int32_t num_heads;
  int32_t num_kv_heads;
  int32_t head_dim;
  int32_t group_size;
  float rms_norm_eps;
  int64_t max_seq_len;
  double rope_theta;
  int32_t max_batch; /* independent sequences decoded together; 0 means 1 */
  int32_t tp_size;   /* tensor-parallel ranks; 0 means 1 */
  int32_t tp_rank;
  int32_t flags;     /* TB_DECODER_* */
} tb_model_config;

enum {
  TB_DECODER_NO_GRAPH = 1,   /* launch kernels directly instead of replaying a CUDA graph */
  TB_DECODER_NCCL_ONLY = 2,  /* tensor parallel: use ncclAllReduce, not the fused peer-memory kernel */
  TB_DECODER_NO_PDL = 4,     /* chain the kernels with plain stream order instead of programmatic dependent launch */
  TB_DECODER_NO_FUSED_STEP = 8, /* batch-1 steps as a chain of single kernels, never the one persistent step kernel */
  TB_DECODER_FUSED_STEP = 16    /* batch-1 steps as the one persistent step kernel also on one GPU.  With neither flag the
                                   faster form is taken: the step kernel with tensor parallelism (the exchange lives inside
                                   it), the chain of kernels on one GPU (measured 8% faster there) */
};

/* Per-layer weights in the capsule order of create_rust_qwen_decoder,
 * python/torchburn/quantization.py:603-621.  With tp_size > 1 these are the
 * rank's shards (see tb_shard_*). */
typedef struct tb_layer_weights {
  const float* input_norm_w;
  const uint8_t* qkv_w;
  const float* qkv_s;
  const uint8_t* o_w;
  const float* o_s;
  const float* post_norm_w;
  const uint8_t* gate_w;
  const float* gate_s;
  const uint8_t* up_w;
  const float* up_s;
  const uint8_t* down_w;
  const float* down_s;
  const float* qkv_b; /* NULL when the architecture has no qkv bias */
} tb_layer_weights;

typedef struct tb_decoder tb_decoder;

/* RustQwenDecoder::new, src/llm/decoder.rs:175-424: validates the dimensions
 * (:214-233 -> TB_ERR_ARG), copies all weights to the device, builds the RoPE
 * tables in float64 (:336-350), allocates zeroed KV caches [Hkv, max_seq_len, d]
 * per layer and sequence (:353-359) and all scratch. */
tb_status tb_decoder_create(tb_decoder** out, const tb_model_config* cfg,
                            const float* embed_tokens, const tb_layer_weights* layers,
                            const float* final_norm_w, const uint8_t* lm_head_w,
                            const float* lm_head_s, tb_space weight_space);
void tb_decoder_destroy(tb_decoder* dec);

/* step(token_id, offset) -> logits, src/llm/decoder.rs:538-541 / decode_step
 * :729-750.  logits_host [vocab] may be NULL (logits stay on the device; read
 * them with tb_decoder_get_logits).  An out-of-range token or offset yields
 * all-zero logits and TB_OK (decoder.rs:1066-1078). */
tb_status tb_decoder_step(tb_decoder* dec, int64_t token_id, int64_t offset, float* logits_host);
/* `batch` independent sequences advance one token each (sequence b uses KV
 * slot b).  logits_host [batch, vocab] or NULL.  The reference batches by
 * running one decoder object per sequence (python/torchburn/llm/speculative.py:293-379). */
tb_status tb_decoder_step_batch(tb_decoder* dec, const int64_t* token_ids, const int64_t* offsets,
                                int32_t batch, float* logits_host);
/* prefill_tokens, src/llm/decoder.rs:431-447: the prompt's positions in order;
 * *end_offset = start_offset + n; TB_ERR_ARG when it would pass max_seq_len.
 * A decoder built for one row steps token by token like the reference; one
 * built with max_batch > 1 takes max_batch positions of sequence 0 per
 * batched step (one pass over the weights for all of them). */
tb_status tb_decoder_prefill_tokens(tb_decoder* dec, const int64_t* tokens, int64_t n,
                                    int64_t start_offset, int64_t* end_offset);
/* prefill, src/llm/decoder.rs:545-558: tokens at offsets 0..n-1, last logits out. */
tb_status tb_decoder_prefill(tb_decoder* dec, const int64_t* tokens, int64_t n, float* logits_host);
/* verify_tokens, src/llm/decoder.rs:565-582: logits_host [n, vocab]. */
tb_status tb_decoder_verify_tokens(tb_decoder* dec, int64_t start_offset, const int64_t* tokens,
                                   int64_t n, float* logits_host);
/* reset_kv_cache, src/llm/decoder.rs:449-477 (clears the written prefix). */
tb_status tb_decoder_reset_kv_cache(tb_decoder* dec);
/* copy_kv_cache_from_tensors, src/llm/decoder.rs:479-523: per layer l <
 * num_given, k[l]/v[l] are [Hkv, src_max_len, d] f32 in `space`; the first
 * seq_len positions of every head are copied into sequence slot `seq`. */
tb_status tb_decoder_copy_kv_cache_from(tb_decoder* dec, const float* const* k,
                                        const float* const* v, int32_t num_given, int64_t seq_len,
                                        int64_t src_max_len, int32_t seq, tb_space space);
/* Reads back layer `layer`'s caches of sequence `seq`: [Hkv, max_seq_len, d] each. */
tb_status tb_decoder_read_kv_cache(tb_decoder* dec, int32_t layer, int32_t seq, float* k_host,
                                   float* v_host);
/* kv_len, src/llm/decoder.rs:527. */
int64_t tb_decoder_kv_len(const tb_decoder* dec);
/* get_logits, src/llm/decoder.rs:532: logits of the last step, [batch, vocab]. */
tb_status tb_decoder_get_logits(tb_decoder* dec, float* logits_host);
/* Device pointer of the logits buffer [max_batch, vocab] (valid until destroy). */
const float* tb_decoder_logits_device(const tb_decoder* dec);
/* decode_and_sample with greedy settings (temperature <= 0 or top_k == 1),
 * src/llm/decoder.rs:753-789, 895-906: argmax on the device, 8 bytes read back. */
tb_status tb_decoder_decode_greedy(tb_decoder* dec, int64_t token_id, int64_t offset,
                                   int64_t* next_token);
/* generate_loop with greedy settings, src/llm/decoder.rs:791-832: feeds each
 * argmax back as the next token without leaving the device; out_tokens [n_new]. */
tb_status tb_decoder_generate_greedy(tb_decoder* dec, int64_t first_token, int64_t start_offset,
                                     int64_t n_new, int64_t* out_tokens);
/* Host-side sampling, src/llm/decoder.rs:878-1020.  tb_apply_repetition_penalty: each distinct
 * in-vocabulary token of `recent` once, positive logits divided by the penalty, negative ones
 * multiplied (no-op for penalty <= 1).  tb_sample_logits: greedy when temperature <= 0, not
 * finite, or top_k == 1; otherwise softmax((top-k logits - max) / temperature), optional
 * nucleus cut (an item is dropped once the mass before it exceeds top_p), then the first
 * candidate whose running mass reaches uniform01 * kept mass.  The reference draws uniform01
 * from its thread RNG; here the caller passes it.  tb_push_recent_window keeps the last 64
 * tokens (`recent` must have room for 64); returns the new length. */
tb_status tb_apply_repetition_penalty(float* logits, int64_t vocab, const int64_t* recent,
                                      int64_t n_recent, float penalty);
tb_status tb_sample_logits(const float* logits, int64_t vocab, float temperature, int64_t top_k,
                           float top_p, float uniform01, int64_t* token);
int64_t tb_push_recent_window(int64_t* recent, int64_t n_recent, int64_t token);
/* decode_and_sample, src/llm/decoder.rs:753-777 / decode_and_sample_inner :835-852: one step,
 * logits to the host, penalty, sampling.  Greedy settings without a penalty stay on the device
 * (8 bytes read back).  `rng_state` (non-zero) is advanced by a xorshift64 step per draw. */
tb_status tb_decoder_decode_and_sample(tb_decoder* dec, int64_t token_id, int64_t offset,
                                       float temperature, int64_t top_k, float repetition_penalty,
                                       const int64_t* recent, int64_t n_recent, float top_p,
                                       uint64_t* rng_state, int64_t* next_token);
/* generate_loop, src/llm/decoder.rs:791-832: stops at eos_token_id (negative = none) or after
 * max_new_tokens; recent_seed (may be NULL) seeds the 64-token penalty window.  out_tokens
 * [max_new_tokens]; *n_out tokens written; *end_offset = seq_len + *n_out. */
tb_status tb_decoder_generate_loop(tb_decoder* dec, int64_t first_token, int64_t seq_len,
                                   int64_t max_new_tokens, float temperature, int64_t top_k,
                                   float repetition_penalty, float top_p, int64_t eos_token_id,
                                   const int64_t* recent_seed, int64_t n_recent_seed,
                                   uint64_t* rng_state, int64_t* out_tokens, int64_t* n_out,
                                   int64_t* end_offset);
/* speculative_accept, src/llm/decoder.rs:583-727.  _rows is the acceptance rule alone (host):
 * target_logits [k, vocab] are the target model's logits at the k verified positions,
 * draft_probs [k, vocab] the draft model's probabilities, draft_tokens [k] the proposals.
 * Leviathan acceptance with probability min(1, p_target / p_draft); on the first rejection the
 * bonus token is drawn from max(0, p_target - p_draft); when all are accepted it is drawn from
 * the last row with the top-p cut.  *rng_state is a splitmix64 state owned by the caller (the
 * reference seeds its own from the clock).  k = 0 gives (0, vocab - 1).  The decoder form first
 * runs the k draft tokens at offset, offset+1, ... (the KV cache advances as in the reference). */
tb_status tb_speculative_accept_rows(const float* target_logits, int64_t vocab,
                                     const int64_t* draft_tokens, int64_t k,
                                     const float* draft_probs, float temperature, float top_p,
                                     uint64_t* rng_state, int64_t* accepted, int64_t* bonus);
tb_status tb_decoder_speculative_accept(tb_decoder* dec, int64_t offset, const int64_t* draft_tokens,
                                        int64_t k, const float* draft_probs, float temperature,
                                        float top_p, uint64_t* rng_state, int64_t* accepted,
                                        int64_t* bonus);
/* Layer-0 intermediates of the last step by name, like debug_step_stages,
 * src/wgpu/profiler.rs:75: "embed", "normed", "qkv", "attn", "x_attn", "h",
 * "x_out".  Only recorded when the decoder was created with TB_DECODER_NO_GRAPH.
 * Writes up to cap floats (sequence 0); *n = element count of the stage. */
tb_status tb_decoder_debug_stage(tb_decoder* dec, const char* name, float* out_host, int64_t cap,
                                 int64_t* n);
/* profile_step_breakdown, src/wgpu/profiler.rs:14-73: CUDA-event milliseconds of
 * one step split into (layers, lm_head, readback). */
tb_status tb_decoder_step_timed(tb_decoder* dec, int64_t token_id, int64_t offset,
                                float* logits_host, float ms_out[3]);
/* is_device_lost / mark_device_lost, src/wgpu/decode.rs:692-699. */
int32_t tb_decoder_is_device_lost(const tb_decoder* dec);
void tb_decoder_mark_device_lost(tb_decoder* dec);
/* Number of kernels one step launches (for accounting). */
int32_t tb_decoder_launches_per_step(const tb_decoder* dec);
/* The decoder's CUDA stream (cudaStream_t as void*). */
void* tb_decoder_stream(const tb_decoder* dec);

/* ------------------------------------------------------------------------
 * Tensor parallelism over one NVLink/NVSwitch box.  No counterpart in the
 * reference (it has no multi-device code); the layout is Megatron style:
 * QKV and gate/up split by output rows (whole heads per rank), o_proj and down
 * split by input columns, one all-reduce of [batch, hidden] after each.
 * ---------------------------------------------------------------------- */

/* Host-side shard helpers (pure byte slicing; no GPU needed).
 * Rows [row0, row0+rows) of a packed matrix / its scales. */
tb_status tb_shard_rows(const uint8_t* packed, const float* scales, int64_t n, int64_t k,
                        int32_t group_size, int64_t row0, int64_t rows, uint8_t* packed_out,
                        float* scales_out);
/* Input columns [col0, col0+cols) of every row; col0 and cols must be
 * multiples of group_size. */
tb_status tb_shard_cols(const uint8_t* packed, const float* scales, int64_t n, int64_t k,
                        int32_t group_size, int64_t col0, int64_t cols, uint8_t* packed_out,
                        float* scales_out);
/* Rank `rank` of `size`'s slice of a fused [q;k;v] projection (whole heads):
 * output rows [q heads of the rank | k heads | v heads].  bias/bias_out may be NULL. */
tb_status tb_shard_qkv(const uint8_t* packed, const float* scales, const float* bias,
                       int64_t hidden, int32_t num_heads, int32_t num_kv_heads, int32_t head_dim,
                       int32_t group_size, int32_t rank, int32_t size, uint8_t* packed_out,
                       float* scales_out, float* bias_out);

/* 128-byte NCCL unique id for tb_decoder_tp_init (rank 0 makes it, the caller
 * distributes it by any means). */
tb_status tb_tp_unique_id(uint8_t id[128]);
/* Joins the decoder (created with tp_size > 1) to its communicator.  Collective:
 * every rank calls it.  peer_exchange, when not NULL, is a callback the library
 * uses to all-gather `bytes` bytes per rank among the ranks (the caller's own
 * transport, e.g. torch.distributed); it enables the fused peer-memory
 * all-reduce.  Without it every all-reduce is ncclAllReduce. */
typedef int32_t (*tb_allgather_fn)(void* user, const void* send, void* recv, size_t bytes);
tb_status tb_decoder_tp_init(tb_decoder* dec, const uint8_t id[128], tb_allgather_fn allgather,
                             void* user);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif

#ifdef __cplusplus
}
#endif
#endif /* TORCHBURN_B200_H */
