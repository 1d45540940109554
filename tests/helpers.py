"""Shared test helpers: the reference's error metric, closed-form input
generators restated from the reference's Rust parity tests, golden loaders."""
from __future__ import annotations

import os

import numpy as np

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def max_rel_err(actual, expected) -> float:
    """max|a-e| / max(max|e|, 1e-6): the reference's robust metric
    (tests/parity/int4.rs:131-141, tests/test_parity.py:104)."""
    a = np.asarray(actual, dtype=np.float64)
    e = np.asarray(expected, dtype=np.float64)
    return float(np.abs(a - e).max() / max(np.abs(e).max(), 1e-6))


def rust_test_quantize_grouped(w: np.ndarray, k: int, group_size: int):
    """The TEST-SIDE quantizer of tests/parity/int4.rs:12-38 (scale 1.0 for an
    all-zero group, multiply by the reciprocal, round half away from zero)."""
    w = np.asarray(w, dtype=np.float32).reshape(-1, k)
    n = w.shape[0]
    ng = k // group_size
    grp = w.reshape(n, ng, group_size)
    max_abs = np.abs(grp).max(axis=2)
    scales = np.where(max_abs > 1e-8, max_abs / np.float32(7.0), np.float32(1.0)).astype(np.float32)
    inv = (np.float32(1.0) / scales).astype(np.float32)
    v = (grp * inv[:, :, None]).astype(np.float32)
    r = np.sign(v) * np.floor(np.abs(v) + np.float32(0.5))  # f32::round
    q = np.clip(r, -8, 7).astype(np.int8).reshape(n, k)
    u = (q + 8).astype(np.uint8)
    packed = (u[:, 0::2] | (u[:, 1::2] << 4)).astype(np.uint8)
    return packed, scales


def load_decoder_golden(name: str):
    z = np.load(os.path.join(GOLDEN, name))
    c = z["cfg"]
    cfg = dict(vocab_size=int(c[0]), hidden_size=int(c[1]), intermediate_size=int(c[2]),
               num_layers=int(c[3]), num_heads=int(c[4]), num_kv_heads=int(c[5]), head_dim=int(c[6]),
               group_size=int(c[7]), max_seq_len=int(c[8]),
               rms_norm_eps=float(z["cfg_f"][0]), rope_theta=float(z["cfg_f"][1]))
    layers = []
    for i in range(cfg["num_layers"]):
        lw = {}
        for key in ["input_norm_w", "qkv_w", "qkv_s", "o_w", "o_s", "post_norm_w", "gate_w", "gate_s",
                    "up_w", "up_s", "down_w", "down_s"]:
            lw[key] = z[f"l{i}_{key}"]
        lw["qkv_b"] = z[f"l{i}_qkv_b"] if f"l{i}_qkv_b" in z.files else None
        layers.append(lw)
    return cfg, z["embed_tokens"], layers, z["final_norm_w"], z["lm_head_w"], z["lm_head_s"], z


def synth_model(cfg: dict, seed: int, quantize, std: float = 0.02, qkv_bias: bool = False):
    """Random-init weights of a decoder (std 0.02 like model.py:509-515), quantized
    with `quantize(w, group_size) -> (packed, scales)`."""
    rng = np.random.default_rng(seed)
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    hd, nh, nkv, G = cfg["head_dim"], cfg["num_heads"], cfg["num_kv_heads"], cfg["group_size"]
    tq = (nh + 2 * nkv) * hd

    def qlin(n, k):
        return quantize((rng.standard_normal((n, k)) * std).astype(np.float32), G)

    layers = []
    for _ in range(cfg["num_layers"]):
        lw = {"input_norm_w": (1 + 0.1 * rng.standard_normal(H)).astype(np.float32),
              "post_norm_w": (1 + 0.1 * rng.standard_normal(H)).astype(np.float32)}
        lw["qkv_w"], lw["qkv_s"] = qlin(tq, H)
        lw["o_w"], lw["o_s"] = qlin(H, nh * hd)
        lw["gate_w"], lw["gate_s"] = qlin(I, H)
        lw["up_w"], lw["up_s"] = qlin(I, H)
        lw["down_w"], lw["down_s"] = qlin(H, I)
        lw["qkv_b"] = (0.05 * rng.standard_normal(tq)).astype(np.float32) if qkv_bias else None
        layers.append(lw)
    embed = (rng.standard_normal((V, H)) * std).astype(np.float32)
    final_norm = (1 + 0.1 * rng.standard_normal(H)).astype(np.float32)
    lm_w, lm_s = quantize(embed, G) if cfg.get("tied", True) else qlin(V, H)
    return embed, layers, final_norm, lm_w, lm_s
