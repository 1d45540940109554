"""Host-side tensor-parallel helpers shared by the CPU (gloo) and GPU (nccl) tests:
sharding through the library's tb_shard_* entry points and a step-by-step sharded
decoder built from oracle pieces with a pluggable all-reduce."""
from __future__ import annotations

import numpy as np


def shard_model(tb, cfg, layers, lm_w, lm_s, rank, size):
    """Returns (layers_r, lm_w_r, lm_s_r): rank's shards, made by tb_shard_rows/cols/qkv."""
    L = tb.lib()
    H, I, V, G = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"], cfg["group_size"]
    nh, nkv, hd = cfg["num_heads"], cfg["num_kv_heads"], cfg["head_dim"]
    q_dim = nh * hd
    tq_l = (nh + 2 * nkv) * hd // size

    def rows(p, s, n, k, r0, cnt):
        po = np.empty((cnt, k // 2), np.uint8); so = np.empty((cnt, k // G), np.float32)
        assert L.tb_shard_rows(p.ctypes.data, s.ctypes.data, n, k, G, r0, cnt, po.ctypes.data, so.ctypes.data) == 0, tb.last_error()
        return po, so

    def cols(p, s, n, k, c0, cnt):
        po = np.empty((n, cnt // 2), np.uint8); so = np.empty((n, cnt // G), np.float32)
        assert L.tb_shard_cols(p.ctypes.data, s.ctypes.data, n, k, G, c0, cnt, po.ctypes.data, so.ctypes.data) == 0, tb.last_error()
        return po, so

    out = []
    for lw in layers:
        c = {k: np.ascontiguousarray(v) if v is not None else None for k, v in lw.items()}
        r = {"input_norm_w": c["input_norm_w"], "post_norm_w": c["post_norm_w"]}
        po = np.empty((tq_l, H // 2), np.uint8); so = np.empty((tq_l, H // G), np.float32)
        bo = np.empty(tq_l, np.float32) if c.get("qkv_b") is not None else None
        assert L.tb_shard_qkv(c["qkv_w"].ctypes.data, c["qkv_s"].ctypes.data,
                              c["qkv_b"].ctypes.data if bo is not None else None, H, nh, nkv, hd, G, rank, size,
                              po.ctypes.data, so.ctypes.data, bo.ctypes.data if bo is not None else None) == 0, tb.last_error()
        r["qkv_w"], r["qkv_s"], r["qkv_b"] = po, so, bo
        r["o_w"], r["o_s"] = cols(c["o_w"], c["o_s"], H, q_dim, rank * (q_dim // size), q_dim // size)
        r["gate_w"], r["gate_s"] = rows(c["gate_w"], c["gate_s"], I, H, rank * (I // size), I // size)
        r["up_w"], r["up_s"] = rows(c["up_w"], c["up_s"], I, H, rank * (I // size), I // size)
        r["down_w"], r["down_s"] = cols(c["down_w"], c["down_s"], H, I, rank * (I // size), I // size)
        out.append(r)
    lw_r, ls_r = rows(np.ascontiguousarray(lm_w), np.ascontiguousarray(lm_s), V, H, rank * (V // size), V // size)
    return out, lw_r, ls_r


class ShardedOracleDecoder:
    """One tensor-parallel rank of the decoder step, from oracle pieces.  `allreduce(vec)`
    sums a float32 vector over the ranks; `allgather(vec)` concatenates in rank order."""

    def __init__(self, oracle, cfg, embed, layers_r, fnorm, lm_w_r, lm_s_r, size, allreduce, allgather):
        self.o, self.cfg, self.embed, self.layers, self.fnorm = oracle, cfg, embed, layers_r, fnorm
        self.lm_w, self.lm_s, self.size, self.allreduce, self.allgather = lm_w_r, lm_s_r, size, allreduce, allgather
        self.nh_l, self.nkv_l, self.hd = cfg["num_heads"] // size, cfg["num_kv_heads"] // size, cfg["head_dim"]
        S = cfg["max_seq_len"]
        self.cos, self.sin = oracle.rope_tables(S, self.hd, cfg["rope_theta"])
        self.k = [np.zeros((self.nkv_l, S, self.hd), np.float32) for _ in layers_r]
        self.v = [np.zeros((self.nkv_l, S, self.hd), np.float32) for _ in layers_r]

    def step(self, tok, off):
        o, c, G = self.o, self.cfg, self.cfg["group_size"]
        x = self.embed[tok].copy()
        qd, kd = self.nh_l * self.hd, self.nkv_l * self.hd
        for l, W in enumerate(self.layers):
            n = o.rms_norm(x, W["input_norm_w"], c["rms_norm_eps"])
            qkv = o.gemm_w4a32_grouped(n, W["qkv_w"], W["qkv_s"], W["qkv_b"], G)
            q = qkv[:qd].reshape(self.nh_l, self.hd).copy()
            k = qkv[qd:qd + kd].reshape(self.nkv_l, self.hd).copy()
            v = qkv[qd + kd:].reshape(self.nkv_l, self.hd)
            for h in range(self.nh_l): q[h] = o.rope_apply_head(q[h], self.cos[off], self.sin[off])
            for h in range(self.nkv_l): k[h] = o.rope_apply_head(k[h], self.cos[off], self.sin[off])
            self.k[l][:, off], self.v[l][:, off] = k, v
            attn = o.attention_decode(q, self.k[l], self.v[l], off + 1).reshape(-1)
            x = x + self.allreduce(o.gemm_w4a32_grouped(attn, W["o_w"], W["o_s"], None, G))  # row-parallel o_proj
            n = o.rms_norm(x, W["post_norm_w"], c["rms_norm_eps"])
            h = o.swiglu_gemv(n, W["gate_w"], W["gate_s"], None, W["up_w"], W["up_s"], None, G)
            x = x + self.allreduce(o.gemm_w4a32_grouped(h, W["down_w"], W["down_s"], None, G))  # row-parallel down
        n = o.rms_norm(x, self.fnorm, c["rms_norm_eps"])
        return self.allgather(o.gemm_w4a32_grouped(n, self.lm_w, self.lm_s, None, G))
