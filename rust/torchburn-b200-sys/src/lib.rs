// UNCOMPILED IN THIS TREE: there is no Rust toolchain where this library is built; the file is kept in
// step with include/torchburn_b200.h by a test that parses both (tests/test_abi_cpu.py).
//
//! Raw FFI declarations of libtorchburn_b200.so, the B200 (sm_100a) implementation of torchburn's
//! quantized decode hot path.  One declaration per symbol of `include/torchburn_b200.h`, in the
//! header's order; the header documents each entry point and names the interface of the reference
//! it replaces:
//!
//! * `tb_gemv_w4a32_grouped` / `tb_gemm_w4a32_grouped` / `tb_fast_rms_norm` stand in for the raw
//!   pointer kernels re-exported from `src/kernels/mod.rs:16-25`;
//! * `tb_linear_*`, `tb_fused_swiglu_mlp`, `tb_fused_attention_step`,
//!   `tb_fused_transformer_layer_step` for the PyO3 functions of
//!   `src/ffi/quantization_ffi.rs:56-65, 203-218, 344-363, 406-438, 517-532`;
//! * `tb_decoder_*` for `RustQwenDecoder` (`src/llm/decoder.rs:176-210, 431-832`).
//!
//! A safe wrapper crate (`torchburn-b200`) would own the handles (`Drop` calling the `_destroy`
//! functions), turn `tb_status` into `Result` with `tb_last_error_string()` as the message, and
//! implement the decoder protocol of `python/torchburn/llm/speculative.py:13-16` on top.
#![allow(non_camel_case_types)]

use std::os::raw::{c_char, c_void};

pub type tb_status = i32;
pub const TB_OK: tb_status = 0;
pub const TB_ERR_ARG: tb_status = 1;
pub const TB_ERR_SHAPE: tb_status = 2;
pub const TB_ERR_DTYPE: tb_status = 3;
pub const TB_ERR_OOM: tb_status = 4;
pub const TB_ERR_CUDA: tb_status = 5;
pub const TB_ERR_NCCL: tb_status = 6;
pub const TB_ERR_TIMEOUT: tb_status = 7;
pub const TB_ERR_DEVICE_LOST: tb_status = 8;
pub const TB_ERR_UNSUPPORTED: tb_status = 9;

pub const TB_ABI_VERSION: i32 = 1;

#[repr(C)]
#[derive(Clone, Copy, Debug, PartialEq, Eq)]
pub enum tb_space {
    TB_HOST = 0,
    TB_DEVICE = 1,
}

pub const TB_DECODER_NO_GRAPH: i32 = 1;
pub const TB_DECODER_NCCL_ONLY: i32 = 2;
pub const TB_DECODER_NO_PDL: i32 = 4;
pub const TB_DECODER_NO_FUSED_STEP: i32 = 8;
pub const TB_DECODER_FUSED_STEP: i32 = 16;

/// Opaque handle of a quantized linear layer (QuantizedLinear).
#[repr(C)]
pub struct tb_linear {
    _private: [u8; 0],
}

/// Opaque handle of a decoder (RustQwenDecoder / WgpuQwenDecoder).
#[repr(C)]
pub struct tb_decoder {
    _private: [u8; 0],
}

/// Constructor arguments of the decoder, `src/llm/decoder.rs:176-210`.
#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct tb_model_config {
    pub vocab_size: i64,
    pub hidden_size: i64,
    pub intermediate_size: i64,
    pub num_layers: i32,
    pub num_heads: i32,
    pub num_kv_heads: i32,
    pub head_dim: i32,
    pub group_size: i32,
    pub rms_norm_eps: f32,
    pub max_seq_len: i64,
    pub rope_theta: f64,
    pub max_batch: i32,
    pub tp_size: i32,
    pub tp_rank: i32,
    pub flags: i32,
}

/// Per-layer weights in the capsule order of `create_rust_qwen_decoder`.
#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct tb_layer_weights {
    pub input_norm_w: *const f32,
    pub qkv_w: *const u8,
    pub qkv_s: *const f32,
    pub o_w: *const u8,
    pub o_s: *const f32,
    pub post_norm_w: *const f32,
    pub gate_w: *const u8,
    pub gate_s: *const f32,
    pub up_w: *const u8,
    pub up_s: *const f32,
    pub down_w: *const u8,
    pub down_s: *const f32,
    pub qkv_b: *const f32,
}

/// The 17 weight / bias tensors of `fused_transformer_layer_step_w4a32`.
#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct tb_layer_step_weights {
    pub input_norm_w: *const f32,
    pub qkv_w: *const u8,
    pub qkv_s: *const f32,
    pub qkv_b: *const f32,
    pub o_w: *const u8,
    pub o_s: *const f32,
    pub o_b: *const f32,
    pub post_norm_w: *const f32,
    pub gate_w: *const u8,
    pub gate_s: *const f32,
    pub gate_b: *const f32,
    pub up_w: *const u8,
    pub up_s: *const f32,
    pub up_b: *const f32,
    pub down_w: *const u8,
    pub down_s: *const f32,
    pub down_b: *const f32,
}

/// All-gather of `bytes` bytes per rank supplied by the caller (tb_decoder_tp_init).
pub type tb_allgather_fn =
    Option<unsafe extern "C" fn(user: *mut c_void, send: *const c_void, recv: *mut c_void, bytes: usize) -> i32>;

#[link(name = "torchburn_b200")]
extern "C" {
    pub fn tb_abi_version() -> i32;
    pub fn tb_last_error_string() -> *const c_char;
    pub fn tb_device_report(buf: *mut c_char, cap: usize) -> tb_status;
    pub fn tb_gemv_w4a32_grouped(x: *const f32, w: *const u8, scales: *const f32, bias: *const f32, out: *mut f32, n: i64, k: i64, group_size: i32, stream: *mut c_void) -> tb_status;
    pub fn tb_gemm_w4a32_grouped(x: *const f32, w: *const u8, scales: *const f32, bias: *const f32, out: *mut f32, m: i64, n: i64, k: i64, group_size: i32, stream: *mut c_void) -> tb_status;
    pub fn tb_swiglu_gemv_w4a32(x: *const f32, gate_w: *const u8, gate_s: *const f32, gate_b: *const f32, up_w: *const u8, up_s: *const f32, up_b: *const f32, h: *mut f32, m: i64, n: i64, k: i64, group_size: i32, stream: *mut c_void) -> tb_status;
    pub fn tb_fast_rms_norm(x: *const f32, w: *const f32, out: *mut f32, m: i64, n: i64, eps: f32, stream: *mut c_void) -> tb_status;
    pub fn tb_quantize_weight_int4_grouped(w: *const f32, n: i64, k: i64, group_size: i32, packed: *mut u8, scales: *mut f32, stream: *mut c_void) -> tb_status;
    pub fn tb_attention_scratch_bytes(batch: i32, num_heads: i32, num_kv_heads: i32, head_dim: i32, max_seq_len: i64) -> usize;
    pub fn tb_attention_decode(qkv: *const f32, k_cache: *mut f32, v_cache: *mut f32, cos_table: *const f32, sin_table: *const f32, offsets: *const i32, out: *mut f32, scratch: *mut c_void, batch: i32, num_heads: i32, num_kv_heads: i32, head_dim: i32, max_seq_len: i64, stream: *mut c_void) -> tb_status;
    pub fn tb_attention_static_scratch_bytes() -> usize;
    pub fn tb_attention_decode_static(qkv: *const f32, k_cache: *mut f32, v_cache: *mut f32, cos_table: *const f32, sin_table: *const f32, offsets: *const i32, out: *mut f32, batch: i32, num_heads: i32, num_kv_heads: i32, head_dim: i32, max_seq_len: i64, stream: *mut c_void) -> tb_status;
    pub fn tb_debug_timeline(device_buffer: *mut c_void, bytes: i64);
    pub fn tb_debug_timeline_blocks() -> i32;
    pub fn tb_debug_step_flags(flags: i32);
    pub fn tb_debug_wait_probe(limit_cycles: i64) -> tb_status;
    pub fn tb_debug_step_wait_limit(cycles: i64);
    pub fn tb_debug_step_gemv(x: *const f32, w: *const u8, scales: *const f32, bias: *const f32, w2: *const u8, scales2: *const f32, out: *mut f32, n: i64, k: i64, group_size: i32, stream: *mut c_void) -> tb_status;
    pub fn tb_set_attention_chunk(positions: i32);
    pub fn tb_set_attention_tuning(ctas_per_sm: i32, ring_stages: i32);
    pub fn tb_set_gemv_tuning(product_mode: i32, rows_per_warp: i32, warps: i32);
    pub fn tb_set_stream_tuning(enabled: i32, ctas_per_sm: i32, ring_kb: i32, elements_per_lane: i32, groups: i32);
    pub fn tb_release_workspaces();
    pub fn tb_device_fault_flag() -> i32;
    pub fn tb_linear_create(out: *mut *mut tb_linear, qweight: *const u8, scales: *const f32, bias: *const f32, out_features: i64, in_features: i64, group_size: i32, weight_space: tb_space) -> tb_status;
    pub fn tb_linear_destroy(lin: *mut tb_linear);
    pub fn tb_f32_to_f16(value: f32) -> u16;
    pub fn tb_f16_to_f32(bits: u16) -> f32;
    pub fn tb_pack_v1_to_v2(qweight: *const u8, scales: *const f32, out_features: i64, in_features: i64, blocks: *mut u8) -> tb_status;
    pub fn tb_unpack_v2_to_v1(blocks: *const u8, out_features: i64, in_features: i64, qweight: *mut u8, scales: *mut f32) -> tb_status;
    pub fn tb_linear_create_v2(out: *mut *mut tb_linear, blocks: *const u8, bias: *const f32, out_features: i64, in_features: i64, weight_space: tb_space) -> tb_status;
    pub fn tb_linear_forward(lin: *mut tb_linear, x: *const f32, m: i64, out: *mut f32, io_space: tb_space, stream: *mut c_void) -> tb_status;
    pub fn tb_linear_device_ptrs(lin: *const tb_linear, qweight: *mut *const u8, scales: *mut *const f32, bias: *mut *const f32) -> tb_status;
    pub fn tb_fused_swiglu_mlp(gate: *mut tb_linear, up: *mut tb_linear, down: *mut tb_linear, x: *const f32, m: i64, out: *mut f32, io_space: tb_space, stream: *mut c_void) -> tb_status;
    pub fn tb_fused_attention_step(qkv: *mut tb_linear, o: *mut tb_linear, x: *const f32, k_cache: *mut f32, v_cache: *mut f32, cos_p: *const f32, sin_p: *const f32, offset: i64, num_heads: i32, num_kv_heads: i32, head_dim: i32, max_seq_len: i64, out: *mut f32, io_space: tb_space, stream: *mut c_void) -> tb_status;
    pub fn tb_fused_transformer_layer_step(x: *mut f32, w: *const tb_layer_step_weights, k_cache: *mut f32, v_cache: *mut f32, cos_p: *const f32, sin_p: *const f32, offset: i64, hidden_size: i64, intermediate_size: i64, num_heads: i32, num_kv_heads: i32, head_dim: i32, max_seq_len: i64, group_size: i32, eps: f32, io_space: tb_space, stream: *mut c_void) -> tb_status;
    pub fn tb_decoder_create(out: *mut *mut tb_decoder, cfg: *const tb_model_config, embed_tokens: *const f32, layers: *const tb_layer_weights, final_norm_w: *const f32, lm_head_w: *const u8, lm_head_s: *const f32, weight_space: tb_space) -> tb_status;
    pub fn tb_decoder_destroy(dec: *mut tb_decoder);
    pub fn tb_decoder_step(dec: *mut tb_decoder, token_id: i64, offset: i64, logits_host: *mut f32) -> tb_status;
    pub fn tb_decoder_step_batch(dec: *mut tb_decoder, token_ids: *const i64, offsets: *const i64, batch: i32, logits_host: *mut f32) -> tb_status;
    pub fn tb_decoder_prefill_tokens(dec: *mut tb_decoder, tokens: *const i64, n: i64, start_offset: i64, end_offset: *mut i64) -> tb_status;
    pub fn tb_decoder_prefill(dec: *mut tb_decoder, tokens: *const i64, n: i64, logits_host: *mut f32) -> tb_status;
    pub fn tb_decoder_verify_tokens(dec: *mut tb_decoder, start_offset: i64, tokens: *const i64, n: i64, logits_host: *mut f32) -> tb_status;
    pub fn tb_decoder_reset_kv_cache(dec: *mut tb_decoder) -> tb_status;
    pub fn tb_decoder_copy_kv_cache_from(dec: *mut tb_decoder, k: *const *const f32, v: *const *const f32, num_given: i32, seq_len: i64, src_max_len: i64, seq: i32, space: tb_space) -> tb_status;
    pub fn tb_decoder_read_kv_cache(dec: *mut tb_decoder, layer: i32, seq: i32, k_host: *mut f32, v_host: *mut f32) -> tb_status;
    pub fn tb_decoder_kv_len(dec: *const tb_decoder) -> i64;
    pub fn tb_decoder_get_logits(dec: *mut tb_decoder, logits_host: *mut f32) -> tb_status;
    pub fn tb_decoder_logits_device(dec: *const tb_decoder) -> *const f32;
    pub fn tb_decoder_decode_greedy(dec: *mut tb_decoder, token_id: i64, offset: i64, next_token: *mut i64) -> tb_status;
    pub fn tb_decoder_generate_greedy(dec: *mut tb_decoder, first_token: i64, start_offset: i64, n_new: i64, out_tokens: *mut i64) -> tb_status;
    pub fn tb_apply_repetition_penalty(logits: *mut f32, vocab: i64, recent: *const i64, n_recent: i64, penalty: f32) -> tb_status;
    pub fn tb_sample_logits(logits: *const f32, vocab: i64, temperature: f32, top_k: i64, top_p: f32, uniform01: f32, token: *mut i64) -> tb_status;
    pub fn tb_push_recent_window(recent: *mut i64, n_recent: i64, token: i64) -> i64;
    pub fn tb_decoder_decode_and_sample(dec: *mut tb_decoder, token_id: i64, offset: i64, temperature: f32, top_k: i64, repetition_penalty: f32, recent: *const i64, n_recent: i64, top_p: f32, rng_state: *mut u64, next_token: *mut i64) -> tb_status;
    pub fn tb_decoder_generate_loop(dec: *mut tb_decoder, first_token: i64, seq_len: i64, max_new_tokens: i64, temperature: f32, top_k: i64, repetition_penalty: f32, top_p: f32, eos_token_id: i64, recent_seed: *const i64, n_recent_seed: i64, rng_state: *mut u64, out_tokens: *mut i64, n_out: *mut i64, end_offset: *mut i64) -> tb_status;
    pub fn tb_speculative_accept_rows(target_logits: *const f32, vocab: i64, draft_tokens: *const i64, k: i64, draft_probs: *const f32, temperature: f32, top_p: f32, rng_state: *mut u64, accepted: *mut i64, bonus: *mut i64) -> tb_status;
    pub fn tb_decoder_speculative_accept(dec: *mut tb_decoder, offset: i64, draft_tokens: *const i64, k: i64, draft_probs: *const f32, temperature: f32, top_p: f32, rng_state: *mut u64, accepted: *mut i64, bonus: *mut i64) -> tb_status;
    pub fn tb_decoder_debug_stage(dec: *mut tb_decoder, name: *const c_char, out_host: *mut f32, cap: i64, n: *mut i64) -> tb_status;
    pub fn tb_decoder_step_timed(dec: *mut tb_decoder, token_id: i64, offset: i64, logits_host: *mut f32, ms_out: *mut f32) -> tb_status;
    pub fn tb_decoder_is_device_lost(dec: *const tb_decoder) -> i32;
    pub fn tb_decoder_mark_device_lost(dec: *mut tb_decoder);
    pub fn tb_decoder_launches_per_step(dec: *const tb_decoder) -> i32;
    pub fn tb_decoder_stream(dec: *const tb_decoder) -> *mut c_void;
    pub fn tb_shard_rows(packed: *const u8, scales: *const f32, n: i64, k: i64, group_size: i32, row0: i64, rows: i64, packed_out: *mut u8, scales_out: *mut f32) -> tb_status;
    pub fn tb_shard_cols(packed: *const u8, scales: *const f32, n: i64, k: i64, group_size: i32, col0: i64, cols: i64, packed_out: *mut u8, scales_out: *mut f32) -> tb_status;
    pub fn tb_shard_qkv(packed: *const u8, scales: *const f32, bias: *const f32, hidden: i64, num_heads: i32, num_kv_heads: i32, head_dim: i32, group_size: i32, rank: i32, size: i32, packed_out: *mut u8, scales_out: *mut f32, bias_out: *mut f32) -> tb_status;
    pub fn tb_tp_unique_id(id: *mut u8) -> tb_status;
    pub fn tb_decoder_tp_init(dec: *mut tb_decoder, id: *const u8, allgather: tb_allgather_fn, user: *mut c_void) -> tb_status;
}
