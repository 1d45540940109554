"""ctypes binding of libtorchburn_b200.so (the C ABI of include/torchburn_b200.h)."""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# TORCHBURN_B200_LIB points at a library built elsewhere (default: the in-tree build).
LIB_PATH = os.environ.get("TORCHBURN_B200_LIB") or os.path.join(_HERE, "lib", "libtorchburn_b200.so")

TB_OK = 0
TB_HOST, TB_DEVICE = 0, 1
TB_DECODER_NO_GRAPH, TB_DECODER_NCCL_ONLY, TB_DECODER_NO_PDL, TB_DECODER_NO_FUSED_STEP, TB_DECODER_FUSED_STEP = 1, 2, 4, 8, 16
STATUS_NAMES = {1: "TB_ERR_ARG", 2: "TB_ERR_SHAPE", 3: "TB_ERR_DTYPE", 4: "TB_ERR_OOM", 5: "TB_ERR_CUDA",
                6: "TB_ERR_NCCL", 7: "TB_ERR_TIMEOUT", 8: "TB_ERR_DEVICE_LOST", 9: "TB_ERR_UNSUPPORTED"}


class TorchBurnB200Error(RuntimeError):
    """A C-ABI call failed; ``status`` is the tb_status code."""

    def __init__(self, status: int, message: str):
        super().__init__(f"{STATUS_NAMES.get(status, status)}: {message}")
        self.status = status


class ModelConfig(C.Structure):
    _fields_ = [
        ("vocab_size", C.c_int64), ("hidden_size", C.c_int64), ("intermediate_size", C.c_int64),
        ("num_layers", C.c_int32), ("num_heads", C.c_int32), ("num_kv_heads", C.c_int32),
        ("head_dim", C.c_int32), ("group_size", C.c_int32), ("rms_norm_eps", C.c_float),
        ("max_seq_len", C.c_int64), ("rope_theta", C.c_double), ("max_batch", C.c_int32),
        ("tp_size", C.c_int32), ("tp_rank", C.c_int32), ("flags", C.c_int32),
    ]


class LayerWeights(C.Structure):
    _fields_ = [(k, C.c_void_p) for k in (
        "input_norm_w", "qkv_w", "qkv_s", "o_w", "o_s", "post_norm_w", "gate_w", "gate_s", "up_w",
        "up_s", "down_w", "down_s", "qkv_b")]


class LayerStepWeights(C.Structure):
    _fields_ = [(k, C.c_void_p) for k in (
        "input_norm_w", "qkv_w", "qkv_s", "qkv_b", "o_w", "o_s", "o_b", "post_norm_w", "gate_w", "gate_s", "gate_b",
        "up_w", "up_s", "up_b", "down_w", "down_s", "down_b")]


ALLGATHER_FN = C.CFUNCTYPE(C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t)

_p, _i64, _i32, _f32, _sz = C.c_void_p, C.c_int64, C.c_int32, C.c_float, C.c_size_t
_PP = C.POINTER(C.c_void_p)

# name -> (restype, argtypes); every symbol the header declares
SIGNATURES = {
    "tb_abi_version": (_i32, []),
    "tb_last_error_string": (C.c_char_p, []),
    "tb_device_report": (_i32, [C.c_char_p, _sz]),
    "tb_gemv_w4a32_grouped": (_i32, [_p, _p, _p, _p, _p, _i64, _i64, _i32, _p]),
    "tb_gemm_w4a32_grouped": (_i32, [_p, _p, _p, _p, _p, _i64, _i64, _i64, _i32, _p]),
    "tb_swiglu_gemv_w4a32": (_i32, [_p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i32, _p]),
    "tb_fast_rms_norm": (_i32, [_p, _p, _p, _i64, _i64, _f32, _p]),
    "tb_quantize_weight_int4_grouped": (_i32, [_p, _i64, _i64, _i32, _p, _p, _p]),
    "tb_attention_scratch_bytes": (_sz, [_i32, _i32, _i32, _i32, _i64]),
    "tb_attention_decode": (_i32, [_p, _p, _p, _p, _p, _p, _p, _p, _i32, _i32, _i32, _i32, _i64, _p]),
    "tb_attention_static_scratch_bytes": (_sz, []),
    "tb_attention_decode_static": (_i32, [_p, _p, _p, _p, _p, _p, _p, _i32, _i32, _i32, _i32, _i64, _p]),
    "tb_debug_timeline": (None, [_p, _i64]),
    "tb_debug_timeline_blocks": (_i32, []),
    "tb_debug_step_flags": (None, [_i32]),
    "tb_debug_wait_probe": (_i32, [_i64]),
    "tb_debug_step_wait_limit": (None, [_i64]),
    "tb_debug_step_gemv": (_i32, [_p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i32, _p]),
    "tb_set_attention_chunk": (None, [_i32]),
    "tb_set_attention_tuning": (None, [_i32, _i32]),
    "tb_set_gemv_tuning": (None, [_i32, _i32, _i32]),
    "tb_set_stream_tuning": (None, [_i32, _i32, _i32, _i32, _i32]),
    "tb_release_workspaces": (None, []),
    "tb_device_fault_flag": (_i32, []),
    "tb_linear_create": (_i32, [_PP, _p, _p, _p, _i64, _i64, _i32, _i32]),
    "tb_f32_to_f16": (C.c_uint16, [_f32]),
    "tb_f16_to_f32": (_f32, [C.c_uint16]),
    "tb_pack_v1_to_v2": (_i32, [_p, _p, _i64, _i64, _p]),
    "tb_unpack_v2_to_v1": (_i32, [_p, _i64, _i64, _p, _p]),
    "tb_linear_create_v2": (_i32, [_PP, _p, _p, _i64, _i64, _i32]),
    "tb_linear_destroy": (None, [_p]),
    "tb_linear_forward": (_i32, [_p, _p, _i64, _p, _i32, _p]),
    "tb_linear_device_ptrs": (_i32, [_p, _PP, _PP, _PP]),
    "tb_fused_swiglu_mlp": (_i32, [_p, _p, _p, _p, _i64, _p, _i32, _p]),
    "tb_fused_attention_step": (_i32, [_p, _p, _p, _p, _p, _p, _p, _i64, _i32, _i32, _i32, _i64, _p, _i32, _p]),
    "tb_fused_transformer_layer_step": (_i32, [_p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i32, _i32, _i32, _i64, _i32, _f32, _i32, _p]),
    "tb_decoder_create": (_i32, [_PP, C.POINTER(ModelConfig), _p, _p, _p, _p, _p, _i32]),
    "tb_decoder_destroy": (None, [_p]),
    "tb_decoder_step": (_i32, [_p, _i64, _i64, _p]),
    "tb_decoder_step_batch": (_i32, [_p, _p, _p, _i32, _p]),
    "tb_decoder_prefill_tokens": (_i32, [_p, _p, _i64, _i64, C.POINTER(_i64)]),
    "tb_decoder_prefill": (_i32, [_p, _p, _i64, _p]),
    "tb_decoder_verify_tokens": (_i32, [_p, _i64, _p, _i64, _p]),
    "tb_decoder_reset_kv_cache": (_i32, [_p]),
    "tb_decoder_copy_kv_cache_from": (_i32, [_p, _p, _p, _i32, _i64, _i64, _i32, _i32]),
    "tb_decoder_read_kv_cache": (_i32, [_p, _i32, _i32, _p, _p]),
    "tb_decoder_kv_len": (_i64, [_p]),
    "tb_decoder_get_logits": (_i32, [_p, _p]),
    "tb_decoder_logits_device": (_p, [_p]),
    "tb_decoder_decode_greedy": (_i32, [_p, _i64, _i64, C.POINTER(_i64)]),
    "tb_decoder_generate_greedy": (_i32, [_p, _i64, _i64, _i64, _p]),
    "tb_apply_repetition_penalty": (_i32, [_p, _i64, _p, _i64, _f32]),
    "tb_sample_logits": (_i32, [_p, _i64, _f32, _i64, _f32, _f32, C.POINTER(_i64)]),
    "tb_push_recent_window": (_i64, [_p, _i64, _i64]),
    "tb_decoder_decode_and_sample": (_i32, [_p, _i64, _i64, _f32, _i64, _f32, _p, _i64, _f32, C.POINTER(C.c_uint64), C.POINTER(_i64)]),
    "tb_speculative_accept_rows": (_i32, [_p, _i64, _p, _i64, _p, _f32, _f32, _p, _p, _p]),
    "tb_decoder_speculative_accept": (_i32, [_p, _i64, _p, _i64, _p, _f32, _f32, _p, _p, _p]),
    "tb_decoder_generate_loop": (_i32, [_p, _i64, _i64, _i64, _f32, _i64, _f32, _f32, _i64, _p, _i64, C.POINTER(C.c_uint64), _p, C.POINTER(_i64), C.POINTER(_i64)]),
    "tb_decoder_debug_stage": (_i32, [_p, C.c_char_p, _p, _i64, C.POINTER(_i64)]),
    "tb_decoder_step_timed": (_i32, [_p, _i64, _i64, _p, C.POINTER(_f32 * 3)]),
    "tb_decoder_is_device_lost": (_i32, [_p]),
    "tb_decoder_mark_device_lost": (None, [_p]),
    "tb_decoder_launches_per_step": (_i32, [_p]),
    "tb_decoder_stream": (_p, [_p]),
    "tb_shard_rows": (_i32, [_p, _p, _i64, _i64, _i32, _i64, _i64, _p, _p]),
    "tb_shard_cols": (_i32, [_p, _p, _i64, _i64, _i32, _i64, _i64, _p, _p]),
    "tb_shard_qkv": (_i32, [_p, _p, _p, _i64, _i32, _i32, _i32, _i32, _i32, _i32, _p, _p, _p]),
    "tb_tp_unique_id": (_i32, [_p]),
    "tb_decoder_tp_init": (_i32, [_p, _p, ALLGATHER_FN, _p]),
}

_lib = None


def lib():
    """The loaded library.  Raises if it has not been built - there is no fallback."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m torchburn_b200.build` "
                "(needs nvcc; there is no CPU fallback)")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def last_error() -> str:
    return lib().tb_last_error_string().decode("utf-8", "replace")


def check(status: int) -> None:
    if status != TB_OK:
        msg = last_error()
        # Same exception classes the reference raises (src/llm/decoder.rs:214-246, 435-442)
        if status == 1:
            raise ValueError(msg)
        if status == 4:
            raise MemoryError(msg)
        raise TorchBurnB200Error(status, msg)


def abi_version() -> int:
    return int(lib().tb_abi_version())


def device_report() -> dict:
    import json

    buf = C.create_string_buffer(1024)
    check(lib().tb_device_report(buf, 1024))
    return json.loads(buf.value.decode())
