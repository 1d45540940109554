"""ctypes binding of the CPU oracle (oracle/tb_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by ``__graft_entry__.smoke()`` and
by ``bench.py``'s CPU-baseline / reference legs as the checker.  The product
package never imports it.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from typing import Dict, List, Optional, Sequence

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "build", "libtb_oracle.so")

TIER_AUTO, TIER_SCALAR, TIER_AVX2, TIER_AVX512 = 0, 1, 2, 3
TIER_NAMES = {1: "scalar", 2: "avx2", 3: "avx512"}


def build(force: bool = False) -> str:
    """Compile the oracle with gcc (a few seconds); returns the library path."""
    src = os.path.join(_HERE, "tb_oracle.c")
    hdr = os.path.join(_HERE, "tb_oracle.h")
    if (
        not force
        and os.path.exists(_LIB_PATH)
        and os.path.getmtime(_LIB_PATH) >= max(os.path.getmtime(src), os.path.getmtime(hdr))
    ):
        return _LIB_PATH
    subprocess.run(["make", "-C", _HERE, "-B"], check=True, capture_output=True)
    return _LIB_PATH


class LayerWeights(C.Structure):
    _fields_ = [
        ("input_norm_w", C.c_void_p), ("qkv_w", C.c_void_p), ("qkv_s", C.c_void_p),
        ("o_w", C.c_void_p), ("o_s", C.c_void_p), ("post_norm_w", C.c_void_p),
        ("gate_w", C.c_void_p), ("gate_s", C.c_void_p), ("up_w", C.c_void_p),
        ("up_s", C.c_void_p), ("down_w", C.c_void_p), ("down_s", C.c_void_p),
        ("qkv_b", C.c_void_p),
    ]


class ModelConfig(C.Structure):
    _fields_ = [
        ("vocab_size", C.c_int64), ("hidden_size", C.c_int64), ("intermediate_size", C.c_int64),
        ("num_layers", C.c_int32), ("num_heads", C.c_int32), ("num_kv_heads", C.c_int32),
        ("head_dim", C.c_int32), ("group_size", C.c_int32), ("rms_norm_eps", C.c_float),
        ("max_seq_len", C.c_int64), ("rope_theta", C.c_double),
    ]


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_LIB_PATH)
        p, i64, i32, f32, f64 = C.c_void_p, C.c_int64, C.c_int, C.c_float, C.c_double
        L.tbo_force_tier.argtypes = [i32]; L.tbo_force_tier.restype = i32
        L.tbo_best_tier.restype = i32
        L.tbo_set_threads.argtypes = [i32]
        L.tbo_get_threads.restype = i32
        L.tbo_quantize_int4_grouped.argtypes = [p, i64, i64, i32, p, p]
        L.tbo_quantize_int4_grouped.restype = i32
        L.tbo_dequant_int4_grouped.argtypes = [p, p, i64, i64, i32, p]
        L.tbo_unpack_codes.argtypes = [p, i64, i64, p]
        L.tbo_gemv_w4a32_grouped.argtypes = [p, p, p, p, p, i64, i64, i32]
        L.tbo_gemm_w4a32_grouped.argtypes = [p, p, p, p, p, i64, i64, i64, i32]
        L.tbo_gemm_w4a32_f64.argtypes = [p, p, p, p, p, i64, i64, i64, i32]
        L.tbo_rms_norm.argtypes = [p, p, p, i64, f32]
        L.tbo_rope_tables.argtypes = [i64, i32, f64, p, p]
        L.tbo_rope_apply_head.argtypes = [p, p, p, i32]
        L.tbo_attention_decode.argtypes = [p, p, p, p, i32, i32, i32, i64, i64]
        L.tbo_swiglu_gemv.argtypes = [p, p, p, p, p, p, p, p, i64, i64, i32]
        L.tbo_fused_swiglu_mlp.argtypes = [p, i64, p, p, p, p, p, p, p, p, p, p, i64, i64, i32]
        L.tbo_decoder_create.argtypes = [p, p, p, p, p, p]; L.tbo_decoder_create.restype = p
        L.tbo_decoder_destroy.argtypes = [p]
        L.tbo_decoder_step.argtypes = [p, i64, i64]
        L.tbo_decoder_prefill_tokens.argtypes = [p, p, i64, i64]
        L.tbo_decoder_prefill_tokens.restype = i64
        L.tbo_decoder_reset_kv_cache.argtypes = [p]
        L.tbo_decoder_kv_len.argtypes = [p]; L.tbo_decoder_kv_len.restype = i64
        L.tbo_decoder_logits.argtypes = [p]; L.tbo_decoder_logits.restype = p
        L.tbo_decoder_k_cache.argtypes = [p, i32]; L.tbo_decoder_k_cache.restype = p
        L.tbo_decoder_v_cache.argtypes = [p, i32]; L.tbo_decoder_v_cache.restype = p
        L.tbo_decoder_set_kv_len.argtypes = [p, i64]
        L.tbo_decoder_debug_stage.argtypes = [p, C.c_char_p, C.POINTER(p)]
        L.tbo_decoder_debug_stage.restype = i64
        L.tbo_argmax.argtypes = [p, i64]; L.tbo_argmax.restype = i64
        L.tbo_speculative_accept_rows.argtypes = [p, i64, p, i64, p, f32, f32, p, p]; L.tbo_speculative_accept_rows.restype = i64
        L.tbo_f32_to_f16.argtypes = [f32]; L.tbo_f32_to_f16.restype = C.c_uint16
        L.tbo_f16_to_f32.argtypes = [C.c_uint16]; L.tbo_f16_to_f32.restype = f32
        L.tbo_pack_v1_to_v2.argtypes = [p, p, i64, i64, p]
        L.tbo_gemv_w4a32_v2.argtypes = [p, p, p, p, i64, i64]
        L.tbo_apply_repetition_penalty.argtypes = [p, i64, p, i64, f32]
        L.tbo_sample_logits.argtypes = [p, i64, f32, i64, f32, f32]; L.tbo_sample_logits.restype = i64
        _lib = L
    return _lib


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _u8(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.uint8)


def _ptr(a: Optional[np.ndarray]):
    return None if a is None else a.ctypes.data


def force_tier(tier: int) -> int:
    return lib().tbo_force_tier(tier)


def best_tier() -> int:
    return lib().tbo_best_tier()


def set_threads(n: int) -> None:
    lib().tbo_set_threads(n)


def get_threads() -> int:
    return lib().tbo_get_threads()


def quantize_int4_grouped(w: np.ndarray, group_size: int):
    w = _f32(w)
    n, k = w.shape
    if k % group_size != 0:
        raise ValueError(f"Weight dimension K={k} must be divisible by group_size={group_size}.")
    packed = np.empty((n, (k + 1) // 2), np.uint8)
    scales = np.empty((n, k // group_size), np.float32)
    rc = lib().tbo_quantize_int4_grouped(_ptr(w), n, k, group_size, _ptr(packed), _ptr(scales))
    assert rc == 0
    return packed, scales


def dequant_int4_grouped(packed, scales, group_size: int) -> np.ndarray:
    packed, scales = _u8(packed), _f32(scales)
    n, k = packed.shape[0], packed.shape[1] * 2
    out = np.empty((n, k), np.float32)
    lib().tbo_dequant_int4_grouped(_ptr(packed), _ptr(scales), n, k, group_size, _ptr(out))
    return out


def unpack_codes(packed) -> np.ndarray:
    packed = _u8(packed)
    n, k = packed.shape[0], packed.shape[1] * 2
    out = np.empty((n, k), np.int8)
    lib().tbo_unpack_codes(_ptr(packed), n, k, _ptr(out))
    return out


def gemm_w4a32_grouped(x, packed, scales, bias, group_size: int) -> np.ndarray:
    x, packed, scales = _f32(x), _u8(packed), _f32(scales)
    x2 = x.reshape(-1, x.shape[-1])
    m, k = x2.shape
    n = packed.shape[0]
    b = None if bias is None else _f32(bias)
    out = np.empty((m, n), np.float32)
    lib().tbo_gemm_w4a32_grouped(_ptr(x2), _ptr(packed), _ptr(scales), _ptr(b), _ptr(out), m, n, k, group_size)
    return out.reshape(x.shape[:-1] + (n,))


def gemm_w4a32_f64(x, packed, scales, bias, group_size: int) -> np.ndarray:
    x, packed, scales = _f32(x), _u8(packed), _f32(scales)
    x2 = x.reshape(-1, x.shape[-1])
    m, k = x2.shape
    n = packed.shape[0]
    b = None if bias is None else _f32(bias)
    out = np.empty((m, n), np.float64)
    lib().tbo_gemm_w4a32_f64(_ptr(x2), _ptr(packed), _ptr(scales), _ptr(b), _ptr(out), m, n, k, group_size)
    return out.reshape(x.shape[:-1] + (n,))


def rms_norm(x, w, eps: float) -> np.ndarray:
    x, w = _f32(x), _f32(w)
    out = np.empty_like(x)
    lib().tbo_rms_norm(_ptr(x), _ptr(w), _ptr(out), x.size, eps)
    return out


def rope_tables(max_seq_len: int, head_dim: int, theta: float):
    c = np.empty((max_seq_len, head_dim), np.float32)
    s = np.empty((max_seq_len, head_dim), np.float32)
    lib().tbo_rope_tables(max_seq_len, head_dim, theta, _ptr(c), _ptr(s))
    return c, s


def rope_apply_head(head, cos_p, sin_p) -> np.ndarray:
    h = _f32(head).copy()
    cp, sp = _f32(cos_p), _f32(sin_p)
    lib().tbo_rope_apply_head(_ptr(h), _ptr(cp), _ptr(sp), h.size // 2)
    return h


def attention_decode(q, k_cache, v_cache, seq_len: int) -> np.ndarray:
    q, k_cache, v_cache = _f32(q), _f32(k_cache), _f32(v_cache)
    nh, hd = q.shape
    nkv, max_seq, _ = k_cache.shape
    out = np.empty((nh, hd), np.float32)
    lib().tbo_attention_decode(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), nh, nkv, hd, max_seq, seq_len)
    return out


def swiglu_gemv(x, gw, gs, gb, uw, us, ub, group_size: int) -> np.ndarray:
    x, gw, gs, uw, us = _f32(x), _u8(gw), _f32(gs), _u8(uw), _f32(us)
    gb = None if gb is None else _f32(gb)
    ub = None if ub is None else _f32(ub)
    n, k = gw.shape[0], x.size
    h = np.empty(n, np.float32)
    lib().tbo_swiglu_gemv(_ptr(x), _ptr(gw), _ptr(gs), _ptr(gb), _ptr(uw), _ptr(us), _ptr(ub), _ptr(h), n, k, group_size)
    return h


def fused_swiglu_mlp(x, gw, gs, gb, uw, us, ub, dw, ds, db, group_size: int) -> np.ndarray:
    x = _f32(x)
    x2 = x.reshape(-1, x.shape[-1])
    m, hidden = x2.shape
    gw, gs, uw, us, dw, ds = _u8(gw), _f32(gs), _u8(uw), _f32(us), _u8(dw), _f32(ds)
    gb = None if gb is None else _f32(gb)
    ub = None if ub is None else _f32(ub)
    db = None if db is None else _f32(db)
    inter = gw.shape[0]
    out = np.empty((m, dw.shape[0]), np.float32)
    lib().tbo_fused_swiglu_mlp(_ptr(x2), m, _ptr(gw), _ptr(gs), _ptr(gb), _ptr(uw), _ptr(us), _ptr(ub),
                               _ptr(dw), _ptr(ds), _ptr(db), _ptr(out), hidden, inter, group_size)
    return out.reshape(x.shape[:-1] + (dw.shape[0],))


def argmax(logits) -> int:
    l = _f32(logits)
    return int(lib().tbo_argmax(_ptr(l), l.size))


def apply_repetition_penalty(logits, recent, penalty: float) -> np.ndarray:
    l = _f32(logits).copy()
    r = np.ascontiguousarray(recent, dtype=np.int64)
    lib().tbo_apply_repetition_penalty(_ptr(l), l.size, _ptr(r), r.size, penalty)
    return l


def sample_logits(logits, temperature: float, top_k: int, top_p: float, u: float) -> int:
    l = _f32(logits)
    return int(lib().tbo_sample_logits(_ptr(l), l.size, temperature, top_k, top_p, u))


def speculative_accept_rows(target_logits, draft_tokens, draft_probs, temperature: float, top_p: float, seed: int):
    """Returns (accepted, bonus, new_rng_state)."""
    tl = _f32(target_logits)
    dp = _f32(draft_probs)
    toks = np.ascontiguousarray(draft_tokens, dtype=np.int64)
    v = tl.shape[-1] if tl.ndim > 1 else tl.size
    rng = C.c_uint64(seed)
    bonus = C.c_int64()
    acc = lib().tbo_speculative_accept_rows(_ptr(tl), v, _ptr(toks), toks.size, _ptr(dp), temperature, top_p,
                                            C.byref(rng), C.byref(bonus))
    return int(acc), int(bonus.value), int(rng.value)


def f32_to_f16(v: float) -> int:
    return int(lib().tbo_f32_to_f16(v))


def f16_to_f32(bits: int) -> float:
    return float(lib().tbo_f16_to_f32(bits))


def pack_v1_to_v2(packed, scales) -> np.ndarray:
    pk = np.ascontiguousarray(packed, dtype=np.uint8)
    sc = _f32(scales)
    n, k = pk.shape[0], pk.shape[1] * 2
    out = np.empty((n, (k // 64) * 34), np.uint8)
    lib().tbo_pack_v1_to_v2(_ptr(pk), _ptr(sc), n, k, _ptr(out))
    return out


def gemv_w4a32_v2(x, blocks, bias=None) -> np.ndarray:
    xv = _f32(x).reshape(-1)
    b = np.ascontiguousarray(blocks, dtype=np.uint8)
    n, k = b.shape[0], (b.shape[1] // 34) * 64
    out = np.empty(n, np.float32)
    bb = _f32(bias) if bias is not None else None
    lib().tbo_gemv_w4a32_v2(_ptr(xv), _ptr(b), _ptr(bb), _ptr(out), n, k)
    return out


LAYER_KEYS = ["input_norm_w", "qkv_w", "qkv_s", "o_w", "o_s", "post_norm_w", "gate_w", "gate_s",
              "up_w", "up_s", "down_w", "down_s", "qkv_b"]


class OracleDecoder:
    """CPU decoder with the method set of the reference's RustQwenDecoder
    (src/llm/decoder.rs:431-565)."""

    def __init__(self, cfg: Dict, embed_tokens, layers: Sequence[Dict], final_norm_w, lm_head_w, lm_head_s):
        self._keep: List[np.ndarray] = []

        def keep(a, dt):
            a = np.ascontiguousarray(a, dtype=dt)
            self._keep.append(a)
            return a

        self.cfg = dict(cfg)
        embed = keep(embed_tokens, np.float32)
        c = ModelConfig(
            vocab_size=embed.shape[0], hidden_size=cfg["hidden_size"],
            intermediate_size=cfg["intermediate_size"], num_layers=len(layers),
            num_heads=cfg["num_heads"], num_kv_heads=cfg["num_kv_heads"], head_dim=cfg["head_dim"],
            group_size=cfg.get("group_size", 64), rms_norm_eps=cfg.get("rms_norm_eps", 1e-6),
            max_seq_len=cfg.get("max_seq_len", 2048), rope_theta=cfg.get("rope_theta", 1e6),
        )
        arr = (LayerWeights * len(layers))()
        for i, lw in enumerate(layers):
            for key in LAYER_KEYS:
                v = lw.get(key)
                if v is None:
                    setattr(arr[i], key, None)
                else:
                    dt = np.uint8 if key.endswith("_w") and "norm" not in key else np.float32
                    setattr(arr[i], key, keep(v, dt).ctypes.data)
        fn = keep(final_norm_w, np.float32)
        lw_, ls_ = keep(lm_head_w, np.uint8), keep(lm_head_s, np.float32)
        self.vocab_size = int(embed.shape[0])
        self._h = lib().tbo_decoder_create(C.byref(c), _ptr(embed), C.cast(arr, C.c_void_p), _ptr(fn), _ptr(lw_), _ptr(ls_))
        if not self._h:
            raise ValueError("invalid decoder dimensions")
        self._c = c

    def __del__(self):
        if getattr(self, "_h", None):
            lib().tbo_decoder_destroy(self._h)
            self._h = None

    def step(self, token_id: int, offset: int) -> np.ndarray:
        lib().tbo_decoder_step(self._h, token_id, offset)
        return self.get_logits()

    def prefill_tokens(self, tokens: Sequence[int], start_offset: int = 0) -> int:
        t = np.ascontiguousarray(tokens, dtype=np.int64)
        r = lib().tbo_decoder_prefill_tokens(self._h, _ptr(t), t.size, start_offset)
        if r < 0:
            raise ValueError(f"prefill {t.size} tokens at offset {start_offset} exceeds max_seq_len {self._c.max_seq_len}")
        return int(r)

    def reset_kv_cache(self) -> None:
        lib().tbo_decoder_reset_kv_cache(self._h)

    def kv_len(self) -> int:
        return int(lib().tbo_decoder_kv_len(self._h))

    def set_kv_len(self, n: int) -> None:
        lib().tbo_decoder_set_kv_len(self._h, n)

    def get_logits(self) -> np.ndarray:
        p = lib().tbo_decoder_logits(self._h)
        return np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_float)), (self.vocab_size,)).copy()

    def kv_cache(self, layer: int):
        """Views (not copies) of the layer's K and V caches [Hkv, max_seq_len, d]."""
        shape = (self._c.num_kv_heads, self._c.max_seq_len, self._c.head_dim)
        k = np.ctypeslib.as_array(C.cast(lib().tbo_decoder_k_cache(self._h, layer), C.POINTER(C.c_float)), shape)
        v = np.ctypeslib.as_array(C.cast(lib().tbo_decoder_v_cache(self._h, layer), C.POINTER(C.c_float)), shape)
        return k, v

    def debug_stage(self, name: str) -> np.ndarray:
        p = C.c_void_p()
        n = lib().tbo_decoder_debug_stage(self._h, name.encode(), C.byref(p))
        if n < 0:
            raise KeyError(name)
        return np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_float)), (n,)).copy()
