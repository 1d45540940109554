/*
 * CPU oracle for the quantized decode hot path of kuntal-devrat/torchburn.
 *
 * TEST INFRASTRUCTURE ONLY.  This is a C restatement of the reference's CPU
 * algorithm (the reference is Rust + Python and cannot be compiled where this
 * library is built).  It is the checker the CUDA path is compared against and
 * the CPU baseline that is timed beside it.  Nothing in the product library
 * links, loads or calls it.
 *
 * Every function cites the reference file:line it follows (paths are relative
 * to the torchburn source tree).
 *
 * Pinning: the quantizer and the decoder step are checked against outputs of
 * the reference's own Python code (python/torchburn/quantization.py and
 * python/torchburn/llm/model.py), stored under tests/golden/, and against the
 * closed-form known-answer cases of the reference's Rust parity tests.
 */
#ifndef TB_ORACLE_H
#define TB_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* SIMD tier selection (mirrors src/dispatch.rs CpuTier, minus the lossy W4A8
 * VNNI tier which is deliberately not restated as the oracle). */
enum { TBO_TIER_AUTO = 0, TBO_TIER_SCALAR = 1, TBO_TIER_AVX2 = 2, TBO_TIER_AVX512 = 3 };

/* Force a tier (test hook, like dispatch.rs force_tier). Returns the tier that
 * will actually run (a tier the host lacks degrades to the best supported). */
int tbo_force_tier(int tier);
int tbo_best_tier(void);
void tbo_set_threads(int n);
int tbo_get_threads(void);

/* python/torchburn/quantization.py:80-96 (production quantizer). */
int tbo_quantize_int4_grouped(const float* w, int64_t n, int64_t k, int group_size,
                              uint8_t* packed, float* scales);
/* tests/test_parity.py:51-64 (reference dequantisation). */
void tbo_dequant_int4_grouped(const uint8_t* packed, const float* scales, int64_t n, int64_t k,
                              int group_size, float* w_out);
/* Integer codes only: q[j,i] in [-8,7]. src/quantization/gemv.rs:1486-1502. */
void tbo_unpack_codes(const uint8_t* packed, int64_t n, int64_t k, int8_t* codes);

/* src/quantization/gemv.rs:1514-1684. bias may be NULL. */
void tbo_gemv_w4a32_grouped(const float* x, const uint8_t* w, const float* scales,
                            const float* bias, float* out, int64_t n, int64_t k, int group_size);
/* src/quantization/gemv.rs:1690-1725. */
void tbo_gemm_w4a32_grouped(const float* x, const uint8_t* w, const float* scales,
                            const float* bias, float* out, int64_t m, int64_t n, int64_t k,
                            int group_size);
/* float64 dequant-dot of the same operands: an "exact" yardstick used to show
 * that two fp32 implementations differ only by rounding. */
void tbo_gemm_w4a32_f64(const float* x, const uint8_t* w, const float* scales, const float* bias,
                        double* out, int64_t m, int64_t n, int64_t k, int group_size);

/* src/quantization/fused_ops.rs:1066-1117. */
void tbo_rms_norm(const float* x, const float* w, float* out, int64_t n, float eps);
/* src/llm/decoder.rs:336-350: tables [max_seq_len, head_dim]. */
void tbo_rope_tables(int64_t max_seq_len, int head_dim, double theta, float* cos_t, float* sin_t);
/* src/llm/decoder.rs:28-68. */
void tbo_rope_apply_head(float* head, const float* cos_p, const float* sin_p, int half_dim);
/* src/llm/decoder.rs:1157-1213: q [Hq,d]; caches [Hkv,max_seq_len,d]; out [Hq,d]. */
void tbo_attention_decode(const float* q, const float* k_cache, const float* v_cache, float* out,
                          int num_heads, int num_kv_heads, int head_dim, int64_t max_seq_len,
                          int64_t seq_len);
/* src/llm/decoder.rs:1280-1328 + src/quantization/gemv/swiglu.rs:205-289. */
void tbo_swiglu_gemv(const float* x, const uint8_t* gw, const float* gs, const float* gb,
                     const uint8_t* uw, const float* us, const float* ub, float* h, int64_t n,
                     int64_t k, int group_size);

/* src/quantization/fused_ops.rs:138-424 (T=1) and :1267-1319 (batched). */
void tbo_fused_swiglu_mlp(const float* x, int64_t m, const uint8_t* gw, const float* gs,
                          const float* gb, const uint8_t* uw, const float* us, const float* ub,
                          const uint8_t* dw, const float* ds, const float* db, float* out,
                          int64_t hidden, int64_t inter, int group_size);

/* Per-layer weights, in the order of python/torchburn/quantization.py:603-621. */
typedef struct tbo_layer_weights {
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
} tbo_layer_weights;

/* Constructor arguments of RustQwenDecoder, src/llm/decoder.rs:176-210. */
typedef struct tbo_model_config {
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
} tbo_model_config;

typedef struct tbo_decoder tbo_decoder;

/* src/llm/decoder.rs:175-424. Weights are BORROWED (not copied): the caller
 * keeps them alive. Returns NULL on invalid dimensions (decoder.rs:214-233). */
tbo_decoder* tbo_decoder_create(const tbo_model_config* cfg, const float* embed_tokens,
                                const tbo_layer_weights* layers, const float* final_norm_w,
                                const uint8_t* lm_head_w, const float* lm_head_s);
void tbo_decoder_destroy(tbo_decoder* d);
/* src/llm/decoder.rs:1051-1374. */
void tbo_decoder_step(tbo_decoder* d, int64_t token_id, int64_t offset);
/* src/llm/decoder.rs:431-447; returns new offset or -1 (exceeds max_seq_len). */
int64_t tbo_decoder_prefill_tokens(tbo_decoder* d, const int64_t* tokens, int64_t n,
                                   int64_t start_offset);
/* src/llm/decoder.rs:449-477. */
void tbo_decoder_reset_kv_cache(tbo_decoder* d);
int64_t tbo_decoder_kv_len(const tbo_decoder* d);
const float* tbo_decoder_logits(const tbo_decoder* d);
float* tbo_decoder_k_cache(tbo_decoder* d, int layer);
float* tbo_decoder_v_cache(tbo_decoder* d, int layer);
void tbo_decoder_set_kv_len(tbo_decoder* d, int64_t n);
/* Layer-0 intermediates of the last step, by name ("embed", "normed", "qkv",
 * "attn", "x_attn", "h", "x_out"), for stage-by-stage comparison.  Returns the
 * element count or -1 for an unknown name. */
int64_t tbo_decoder_debug_stage(const tbo_decoder* d, const char* name, const float** data);

/* src/llm/decoder.rs:878-1020 greedy branch: argmax (first maximum wins). */
int64_t tbo_argmax(const float* logits, int64_t n);

/* src/llm/decoder.rs:878-899 and :908-1020 (the random draw is the argument u). */
void tbo_apply_repetition_penalty(float* logits, int64_t vocab, const int64_t* recent, int64_t n_recent,
                                  float penalty);
int64_t tbo_sample_logits(const float* logits, int64_t vocab, float temperature, int64_t top_k, float top_p,
                          float u);

/* src/llm/decoder.rs:583-727 after the verify loop: acceptance over given target logits [k, v];
 * *rng is the splitmix64 state (the reference seeds it from the clock). */
int64_t tbo_speculative_accept_rows(const float* target_logits, int64_t v, const int64_t* draft_tokens, int64_t k,
                                    const float* draft_probs, float temperature, float top_p, uint64_t* rng,
                                    int64_t* bonus);

/* v2 layout, src/quantization/packed_v2.rs:26-203. */
uint16_t tbo_f32_to_f16(float v);
float tbo_f16_to_f32(uint16_t bits);
void tbo_pack_v1_to_v2(const uint8_t* w_packed, const float* scales, int64_t n, int64_t k, uint8_t* out);
void tbo_gemv_w4a32_v2(const float* x, const uint8_t* blocks, const float* bias, float* out, int64_t n, int64_t k);

#ifdef __cplusplus
}
#endif
#endif
