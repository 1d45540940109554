"""Host-side mirror of the reference's decoder object (RustQwenDecoder,
src/llm/decoder.rs:111-171, and its factory create_rust_qwen_decoder,
python/torchburn/quantization.py:575-647) over tb_decoder_* of the C ABI."""
from __future__ import annotations

import ctypes as C
from typing import Any, List, Optional, Sequence

import numpy as np

from . import _lib
from ._lib import TB_DEVICE, TB_HOST, LayerWeights, ModelConfig, check, lib

_LAYER_ORDER = ["input_norm_w", "qkv_w", "qkv_s", "o_w", "o_s", "post_norm_w", "gate_w", "gate_s",
                "up_w", "up_s", "down_w", "down_s", "qkv_b"]
_U8 = {"qkv_w", "o_w", "gate_w", "up_w", "down_w"}


def _is_torch(a) -> bool:
    return type(a).__module__.startswith("torch")


class _Operands:
    """Keeps weight arrays alive and yields raw pointers; all in one memory space."""

    def __init__(self):
        self.keep: List[Any] = []
        self.space: Optional[int] = None

    def ptr(self, a, dtype) -> Optional[int]:
        if a is None:
            return None
        if _is_torch(a):
            import torch

            t = a.detach().contiguous().to(torch.uint8 if dtype == np.uint8 else torch.float32)
            space = TB_DEVICE if t.device.type == "cuda" else TB_HOST
            p = t.data_ptr()
        else:
            t = np.ascontiguousarray(a, dtype=dtype)
            space = TB_HOST
            p = t.ctypes.data
        if self.space is None:
            self.space = space
        elif self.space != space:
            raise ValueError("decoder weights must all live in the same memory space (all host or all CUDA)")
        self.keep.append(t)
        return p


class B200QwenDecoder:
    """The reference's decoder class on a B200.

    Constructor arguments follow RustQwenDecoder::new (src/llm/decoder.rs:176-210):
    ``layers_data`` is a list of per-layer sequences in the order
    [input_norm, qkv_w, qkv_s, o_w, o_s, post_norm, gate_w, gate_s, up_w, up_s,
    down_w, down_s, (qkv_b)] (numpy arrays or torch tensors; dicts keyed by those
    names are accepted too).  ``max_batch``, ``tp_size``/``tp_rank``, ``debug`` and
    ``fused_step`` (True: batch-1 steps as the one persistent step kernel; False: as a chain of single
    kernels; None: the faster of the two - the step kernel with tensor parallelism, the chain on one
    GPU) have no counterpart in the reference.
    """

    def __init__(self, embed_tokens, layers_data: Sequence, final_norm_w, lm_head_w, lm_head_s,
                 num_layers: int, hidden_size: int, intermediate_size: int, num_heads: int,
                 num_kv_heads: int, head_dim: int, group_size: int = 64, rms_norm_eps: float = 1e-6,
                 max_seq_len: int = 2048, rope_theta: float = 1000000.0, max_batch: int = 1,
                 tp_size: int = 1, tp_rank: int = 0, debug: bool = False, vocab_size: Optional[int] = None,
                 nccl_only: bool = False, pdl: bool = True, fused_step: Optional[bool] = None):
        self._h = None
        ops = _Operands()
        emb_p = ops.ptr(embed_tokens, np.float32)
        self.vocab_size = int(vocab_size if vocab_size is not None else embed_tokens.shape[0])
        arr = (LayerWeights * num_layers)()
        if len(layers_data) != num_layers:
            raise ValueError(f"layers_data has {len(layers_data)} entries, num_layers is {num_layers}")
        for i, ld in enumerate(layers_data):
            if isinstance(ld, dict):
                items = [ld.get(k) for k in _LAYER_ORDER]
            else:
                items = list(ld) + [None] * (13 - len(ld))
                if len(ld) < 12:
                    raise _lib.TorchBurnB200Error(2, "Each layer requires 12 capsules: input_norm, qkv_w, qkv_s, o_w, o_s, post_norm, gate_w, gate_s, up_w, up_s, down_w, down_s")
            for key, item in zip(_LAYER_ORDER, items):
                setattr(arr[i], key, ops.ptr(item, np.uint8 if key in _U8 else np.float32))
        fn_p = ops.ptr(final_norm_w, np.float32)
        lw_p = ops.ptr(lm_head_w, np.uint8)
        ls_p = ops.ptr(lm_head_s, np.float32)
        flags = ((_lib.TB_DECODER_NO_GRAPH if debug else 0) | (_lib.TB_DECODER_NCCL_ONLY if nccl_only else 0)
                 | (0 if pdl else _lib.TB_DECODER_NO_PDL) | (0 if fused_step is None else (_lib.TB_DECODER_FUSED_STEP if fused_step else _lib.TB_DECODER_NO_FUSED_STEP)))
        cfg = ModelConfig(vocab_size=self.vocab_size, hidden_size=hidden_size, intermediate_size=intermediate_size,
                          num_layers=num_layers, num_heads=num_heads, num_kv_heads=num_kv_heads, head_dim=head_dim,
                          group_size=group_size, rms_norm_eps=rms_norm_eps, max_seq_len=max_seq_len,
                          rope_theta=rope_theta, max_batch=max_batch, tp_size=tp_size, tp_rank=tp_rank, flags=flags)
        self.cfg = cfg
        h = C.c_void_p()
        check(lib().tb_decoder_create(C.byref(h), C.byref(cfg), emb_p, C.cast(arr, C.c_void_p), fn_p, lw_p, ls_p,
                                      ops.space if ops.space is not None else TB_HOST))
        self._h = h
        self.max_batch = max_batch
        self.max_seq_len = max_seq_len
        self._logits = np.empty((max_batch, self.vocab_size), np.float32)
        self._rng = C.c_uint64(0x9E3779B97F4A7C15)
        del ops  # the library copied everything to the device

    def __del__(self):
        self.close()

    def close(self) -> None:
        if getattr(self, "_h", None):
            lib().tb_decoder_destroy(self._h)
            self._h = None

    # ---- methods of RustQwenDecoder (src/llm/decoder.rs:431-565, 729-832) ----
    def prefill_tokens(self, tokens: Sequence[int], start_offset: int = 0) -> int:
        t = np.ascontiguousarray(tokens, dtype=np.int64)
        end = C.c_int64()
        check(lib().tb_decoder_prefill_tokens(self._h, t.ctypes.data, t.size, start_offset, C.byref(end)))
        return int(end.value)

    def reset_kv_cache(self) -> None:
        check(lib().tb_decoder_reset_kv_cache(self._h))

    def copy_kv_cache_from_tensors(self, k_tensors: Sequence, v_tensors: Sequence, seq_len: int, seq: int = 0) -> None:
        ops = _Operands()
        n = min(len(k_tensors), len(v_tensors))
        kp = (C.c_void_p * n)(*[ops.ptr(k, np.float32) for k in k_tensors[:n]])
        vp = (C.c_void_p * n)(*[ops.ptr(v, np.float32) for v in v_tensors[:n]])
        src_max = int(k_tensors[0].shape[-2]) if n and len(k_tensors[0].shape) >= 2 else seq_len
        check(lib().tb_decoder_copy_kv_cache_from(self._h, C.cast(kp, C.c_void_p), C.cast(vp, C.c_void_p), n,
                                                  seq_len, src_max, seq, ops.space if ops.space is not None else TB_HOST))

    def kv_len(self) -> int:
        return int(lib().tb_decoder_kv_len(self._h))

    def get_logits(self) -> np.ndarray:
        check(lib().tb_decoder_get_logits(self._h, self._logits.ctypes.data))
        return self._logits[0].copy()

    def step(self, token_id: int, offset: int) -> np.ndarray:
        check(lib().tb_decoder_step(self._h, int(token_id), int(offset), self._logits.ctypes.data))
        return self._logits[0].copy()

    def decode_step(self, token_id: int, offset: int) -> np.ndarray:
        """decode_step (src/llm/decoder.rs:729-750): logits of shape [1, vocab]."""
        return self.step(token_id, offset)[None, :]

    def step_batch(self, token_ids: Sequence[int], offsets: Sequence[int]) -> np.ndarray:
        t = np.ascontiguousarray(token_ids, dtype=np.int64)
        o = np.ascontiguousarray(offsets, dtype=np.int64)
        if t.size != o.size:
            raise ValueError("token_ids and offsets differ in length")
        check(lib().tb_decoder_step_batch(self._h, t.ctypes.data, o.ctypes.data, t.size, self._logits.ctypes.data))
        return self._logits[: t.size].copy()

    def prefill(self, tokens: Sequence[int]) -> np.ndarray:
        t = np.ascontiguousarray(tokens, dtype=np.int64)
        if t.size == 0:
            raise ValueError("empty prefill")
        check(lib().tb_decoder_prefill(self._h, t.ctypes.data, t.size, self._logits.ctypes.data))
        return self._logits[0].copy()

    def verify_tokens(self, start_offset: int, tokens: Sequence[int]) -> np.ndarray:
        t = np.ascontiguousarray(tokens, dtype=np.int64)
        out = np.empty((t.size, self.vocab_size), np.float32)
        check(lib().tb_decoder_verify_tokens(self._h, start_offset, t.ctypes.data, t.size, out.ctypes.data))
        return out

    def decode_and_sample(self, token_id: int, offset: int, temperature: float = 0.7, top_k: int = 40,
                          repetition_penalty: float = 1.0, recent_tokens: Optional[Sequence[int]] = None,
                          top_p: float = 1.0) -> int:
        """decode_and_sample (src/llm/decoder.rs:753-777): one step, repetition penalty, sampling.
        Greedy settings without a penalty keep the argmax on the device."""
        rec = np.ascontiguousarray(recent_tokens if recent_tokens is not None else [], dtype=np.int64)
        nxt = C.c_int64()
        check(lib().tb_decoder_decode_and_sample(self._h, int(token_id), int(offset), temperature, top_k,
                                                 repetition_penalty, rec.ctypes.data, rec.size, top_p,
                                                 C.byref(self._rng), C.byref(nxt)))
        return int(nxt.value)

    def generate_loop(self, first_token: int, seq_len: int, max_new_tokens: int, temperature: float = 0.7,
                      top_k: int = 40, repetition_penalty: float = 1.0, top_p: float = 1.0,
                      eos_token_id: Optional[int] = None, recent_seed: Optional[Sequence[int]] = None):
        """generate_loop (src/llm/decoder.rs:791-832): returns (tokens, final KV position)."""
        out = np.empty(max(max_new_tokens, 1), np.int64)
        seed = np.ascontiguousarray(recent_seed if recent_seed is not None else [], dtype=np.int64)
        n, end = C.c_int64(), C.c_int64()
        check(lib().tb_decoder_generate_loop(self._h, int(first_token), int(seq_len), int(max_new_tokens), temperature,
                                             top_k, repetition_penalty, top_p, -1 if eos_token_id is None else int(eos_token_id),
                                             seed.ctypes.data, seed.size, C.byref(self._rng), out.ctypes.data,
                                             C.byref(n), C.byref(end)))
        return [int(t) for t in out[: n.value]], int(end.value)

    def speculative_accept(self, offset: int, draft_tokens: Sequence[int], draft_probs, temperature: float = 1.0,
                           top_p: float = 1.0):
        """speculative_accept (src/llm/decoder.rs:587-727): verifies the draft tokens at offset,
        offset+1, ... with this (target) decoder and applies Leviathan acceptance against
        draft_probs [K, V]; returns (accepted_count, bonus_token)."""
        toks = np.ascontiguousarray(draft_tokens, dtype=np.int64)
        probs = np.ascontiguousarray(draft_probs, dtype=np.float32).reshape(-1)
        if toks.size and probs.size != toks.size * self.vocab_size:
            raise ValueError("draft_probs must be K x V row-major")  # decoder.rs:598-602
        acc, bonus = C.c_int64(), C.c_int64()
        check(lib().tb_decoder_speculative_accept(self._h, int(offset), toks.ctypes.data, toks.size, probs.ctypes.data,
                                                  temperature, top_p, C.byref(self._rng), C.byref(acc), C.byref(bonus)))
        return int(acc.value), int(bonus.value)

    def seed(self, value: int) -> None:
        """Seeds the sampling RNG (the reference uses an unseeded thread RNG)."""
        self._rng = C.c_uint64(value or 1)

    # ---- extras -------------------------------------------------------------
    def read_kv_cache(self, layer: int, seq: int = 0):
        shape = (self.cfg.num_kv_heads // max(self.cfg.tp_size, 1), self.max_seq_len, self.cfg.head_dim)
        k = np.empty(shape, np.float32)
        v = np.empty(shape, np.float32)
        check(lib().tb_decoder_read_kv_cache(self._h, layer, seq, k.ctypes.data, v.ctypes.data))
        return k, v

    def debug_stage(self, name: str) -> np.ndarray:
        n = C.c_int64()
        check(lib().tb_decoder_debug_stage(self._h, name.encode(), None, 0, C.byref(n)))
        out = np.empty(n.value, np.float32)
        check(lib().tb_decoder_debug_stage(self._h, name.encode(), out.ctypes.data, n.value, C.byref(n)))
        return out

    def step_timed(self, token_id: int, offset: int):
        ms = (C.c_float * 3)()
        check(lib().tb_decoder_step_timed(self._h, int(token_id), int(offset), self._logits.ctypes.data, C.byref(ms)))
        return tuple(float(v) for v in ms)

    def is_device_lost(self) -> bool:
        return bool(lib().tb_decoder_is_device_lost(self._h))

    def mark_device_lost(self) -> None:
        lib().tb_decoder_mark_device_lost(self._h)

    def launches_per_step(self) -> int:
        return int(lib().tb_decoder_launches_per_step(self._h))

    @property
    def handle(self):
        return self._h


def create_b200_qwen_decoder(model: Any, max_seq_len: int = 4096, group_size: Optional[int] = None,
                             **kwargs) -> B200QwenDecoder:
    """create_rust_qwen_decoder (python/torchburn/quantization.py:575-647) for the B200 decoder.

    ``model`` is a quantized model laid out like the reference's UniversalTransformer:
    ``embed_tokens``, ``layers[i].input_layernorm / self_attn.qkv_proj / self_attn.o_proj /
    post_attention_layernorm / mlp.{gate,up,down}_proj``, ``norm``, ``lm_head`` (modules with
    ``qweight`` / ``scales`` / optional ``bias``) and ``config``.  The reference passes a
    hard-coded group size of 64 here (:637); this factory reads it from the modules."""
    layers = []
    for layer in model.layers:
        att, mlp = layer.self_attn, layer.mlp
        caps = [layer.input_layernorm.weight, att.qkv_proj.qweight, att.qkv_proj.scales, att.o_proj.qweight,
                att.o_proj.scales, layer.post_attention_layernorm.weight, mlp.gate_proj.qweight,
                mlp.gate_proj.scales, mlp.up_proj.qweight, mlp.up_proj.scales, mlp.down_proj.qweight,
                mlp.down_proj.scales]
        if getattr(att.qkv_proj, "bias", None) is not None:
            caps.append(att.qkv_proj.bias)
        layers.append(caps)
    cfg = model.config
    g = group_size if group_size is not None else getattr(model.lm_head, "group_size", 64)
    return B200QwenDecoder(
        model.embed_tokens.weight, layers, model.norm.weight, model.lm_head.qweight, model.lm_head.scales,
        len(model.layers), cfg.hidden_size, cfg.intermediate_size, cfg.num_attention_heads,
        cfg.num_key_value_heads, cfg.head_dim, g, cfg.rms_norm_eps, max_seq_len, cfg.rope_theta, **kwargs)
