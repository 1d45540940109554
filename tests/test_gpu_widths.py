"""GPU parity at the widths the benchmarks run: Llama-3-8B true width (hidden 4096,
intermediate 14336, 32 q / 8 kv heads of 128) at reduced depth with the context near 4096, the
Llama-3-70B shapes as their tensor-parallel-8 shards, the full Llama MLP matrices at M = 16 and
64, and the persistent step kernel's projection path at those shapes.  Everything against the
CPU oracle, through the C ABI; tolerances as everywhere: 1e-4 per stage, 1e-3 on logits, cache
rows bit-exact."""
import ctypes as C

import numpy as np
import pytest

from helpers import max_rel_err

pytestmark = pytest.mark.gpu

STAGE_TOL = 1e-4
LOGIT_TOL = 1e-3


@pytest.fixture(scope="module")
def torch():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("no CUDA device: GPU tests need a B200")
    return torch


@pytest.fixture(scope="module")
def tb(torch):
    import torchburn_b200 as tb

    return tb


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _quantized(torch, tb, n, k, g, seed, std=0.02):
    """Random N(0, std) weights quantized on the GPU (bit-exact with the oracle's quantizer, which
    other tests establish); returns host arrays."""
    gen = torch.Generator("cuda").manual_seed(seed)
    w = torch.randn(n, k, device="cuda", generator=gen) * std
    p, s = tb.quantize_weight_int4_grouped(w, group_size=g)
    return p.cpu().numpy(), s.cpu().numpy()


def _llama_width_model(torch, tb, cfg, seed):
    H, I, V, G = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"], cfg["group_size"]
    nh, nkv, hd = cfg["num_heads"], cfg["num_kv_heads"], cfg["head_dim"]
    rng = np.random.default_rng(seed)
    layers = []
    for l in range(cfg["num_layers"]):
        lw = {"input_norm_w": (1 + 0.1 * rng.standard_normal(H)).astype(np.float32),
              "post_norm_w": (1 + 0.1 * rng.standard_normal(H)).astype(np.float32), "qkv_b": None}
        lw["qkv_w"], lw["qkv_s"] = _quantized(torch, tb, (nh + 2 * nkv) * hd, H, G, seed * 100 + l * 5)
        lw["o_w"], lw["o_s"] = _quantized(torch, tb, H, nh * hd, G, seed * 100 + l * 5 + 1)
        lw["gate_w"], lw["gate_s"] = _quantized(torch, tb, I, H, G, seed * 100 + l * 5 + 2)
        lw["up_w"], lw["up_s"] = _quantized(torch, tb, I, H, G, seed * 100 + l * 5 + 3)
        lw["down_w"], lw["down_s"] = _quantized(torch, tb, H, I, G, seed * 100 + l * 5 + 4)
        layers.append(lw)
    embed = (rng.standard_normal((V, H)) * 0.02).astype(np.float32)
    fnorm = (1 + 0.1 * rng.standard_normal(H)).astype(np.float32)
    lm_w, lm_s = _quantized(torch, tb, V, H, G, seed * 100 + 99)
    return embed, layers, fnorm, lm_w, lm_s


def _make(tb, cfg, embed, layers, fnorm, lm_w, lm_s, **kw):
    lay = [[lw[k] for k in ["input_norm_w", "qkv_w", "qkv_s", "o_w", "o_s", "post_norm_w", "gate_w", "gate_s",
                            "up_w", "up_s", "down_w", "down_s"]] for lw in layers]
    return tb.B200QwenDecoder(embed, lay, fnorm, lm_w, lm_s, cfg["num_layers"], cfg["hidden_size"],
                              cfg["intermediate_size"], cfg["num_heads"], cfg["num_kv_heads"], cfg["head_dim"],
                              cfg["group_size"], cfg["rms_norm_eps"], cfg["max_seq_len"], cfg["rope_theta"], **kw)


def _prefill_both(dec, refs, cfg, ctx, seed, seqs):
    """The same seeded K/V prefix in the CUDA decoder (copy_kv_cache_from_tensors) and the oracle decoders."""
    rng = np.random.default_rng(seed)
    nkv, hd, L = cfg["num_kv_heads"], cfg["head_dim"], cfg["num_layers"]
    base_k = [(rng.standard_normal((nkv, ctx, hd)) * 0.5).astype(np.float32) for _ in range(L)]
    base_v = [rng.standard_normal((nkv, ctx, hd)).astype(np.float32) for _ in range(L)]
    for b in range(seqs):
        ks = [np.roll(k, b, axis=1) for k in base_k]   # every sequence its own prefix, cheaply
        vs = [np.roll(v, b, axis=1) for v in base_v]
        dec.copy_kv_cache_from_tensors(ks, vs, ctx, seq=b)
        for l in range(L):
            ek, ev = refs[b].kv_cache(l)
            ek[:, :ctx], ev[:, :ctx] = ks[l], vs[l]
        refs[b].set_kv_len(ctx)


LLAMA8B_L2 = dict(vocab_size=8192, hidden_size=4096, intermediate_size=14336, num_layers=2, num_heads=32,
                  num_kv_heads=8, head_dim=128, group_size=32, max_seq_len=4160, rms_norm_eps=1e-6, rope_theta=5e5)


@pytest.mark.parametrize("fused", [True, False])
def test_llama8b_width_depth2_batch1_context_4090(torch, tb, oracle, fused):
    """Workload configuration 4 at true width, two layers, the context pre-filled to 4090 positions:
    six batch-1 steps through the CUDA-graph path - the persistent step kernel (fused) and the
    chain of single kernels with the split RMSNorm - logits, new cache rows, and the layer-0 stages
    of a debug decoder."""
    cfg = dict(LLAMA8B_L2)
    embed, layers, fnorm, lm_w, lm_s = _llama_width_model(torch, tb, cfg, 31)
    ref = oracle.OracleDecoder(cfg, embed, layers, fnorm, lm_w, lm_s)
    dec = _make(tb, cfg, embed, layers, fnorm, lm_w, lm_s, fused_step=fused)
    ctx = 4090
    _prefill_both(dec, [ref], cfg, ctx, 5, 1)
    dbg = None
    if fused:
        dbg = _make(tb, cfg, embed, layers, fnorm, lm_w, lm_s, debug=True)
        _prefill_both(dbg, [oracle.OracleDecoder(cfg, embed, layers, fnorm, lm_w, lm_s)], cfg, ctx, 5, 1)
    toks = np.random.default_rng(1).integers(0, cfg["vocab_size"], 6)
    for i, t in enumerate(toks):
        want = ref.step(int(t), ctx + i)
        got = dec.step(int(t), ctx + i)
        assert max_rel_err(got, want) < LOGIT_TOL, i
        if dbg is not None:
            got_dbg = dbg.step(int(t), ctx + i)
            assert max_rel_err(got_dbg, want) < LOGIT_TOL, i
            if i in (0, 5):
                for name in ("normed", "qkv", "attn", "x_attn", "h", "x_out"):
                    assert max_rel_err(dbg.debug_stage(name), ref.debug_stage(name)) < STAGE_TOL, (i, name)
    assert oracle.argmax(dec.get_logits()) == oracle.argmax(ref.get_logits())
    for l in range(cfg["num_layers"]):
        gk, gv = dec.read_kv_cache(l)
        ek, ev = ref.kv_cache(l)
        # the prefix is untouched (bit for bit); the six new rows match the oracle's
        assert np.array_equal(gk[:, :ctx], ek[:, :ctx]) and np.array_equal(gv[:, :ctx], ev[:, :ctx])
        assert max_rel_err(gk[:, ctx:ctx + 6], ek[:, ctx:ctx + 6]) < STAGE_TOL
        assert max_rel_err(gv[:, ctx:ctx + 6], ev[:, ctx:ctx + 6]) < STAGE_TOL
        assert not gk[:, ctx + 6:].any() and not gv[:, ctx + 6:].any()
    assert tb.lib().tb_device_fault_flag() == 0


@pytest.mark.parametrize("ranks", [4, 8])
def test_llama8b_one_rank_of_tp_shapes_in_the_step_kernel(torch, tb, oracle, ranks):
    """The phase shapes one rank of a tensor-parallel Llama-3-8B decoder runs in the persistent step
    kernel, on ONE GPU (the exchange aside, which the multi-GPU tests cover): heads, kv heads, the
    intermediate width and the vocabulary divided by the number of ranks - 8 ranks: one kv head
    (64 attention splits), o_proj K = 512 (one warp covers K), down K = 1792, 16032 logits.  A model of
    exactly those widths against the oracle at a context of 4090."""
    cfg = dict(LLAMA8B_L2, num_heads=32 // ranks, num_kv_heads=8 // ranks, intermediate_size=14336 // ranks,
               vocab_size=128256 // ranks if ranks == 8 else 8192)
    embed, layers, fnorm, lm_w, lm_s = _llama_width_model(torch, tb, cfg, 70 + ranks)
    ref = oracle.OracleDecoder(cfg, embed, layers, fnorm, lm_w, lm_s)
    dec = _make(tb, cfg, embed, layers, fnorm, lm_w, lm_s, fused_step=True)
    ctx = 4090
    _prefill_both(dec, [ref], cfg, ctx, 9, 1)
    toks = np.random.default_rng(ranks).integers(0, cfg["vocab_size"], 4)
    for i, t in enumerate(toks):
        assert max_rel_err(dec.step(int(t), ctx + i), ref.step(int(t), ctx + i)) < LOGIT_TOL, i
    assert dec.launches_per_step() == 2   # the embedding kernel + the persistent step kernel
    assert tb.lib().tb_device_fault_flag() == 0


@pytest.mark.parametrize("batch,steps", [(2, 2), (3, 1), (4, 2), (8, 2), (32, 1)])
def test_llama8b_width_depth2_batched_steps(torch, tb, oracle, batch, steps):
    """The same model at batch 2, 3, 4 (the persistent streaming kernel with the digits of every row in
    registers; the K = 14336 projection takes it up to 2 rows), 8 and 32 (step_batch: tensor-core rows kernels
    at true width), the attention kernel over `batch` sequences near context 4096."""
    cfg = dict(LLAMA8B_L2)
    embed, layers, fnorm, lm_w, lm_s = _llama_width_model(torch, tb, cfg, 31)
    refs = [oracle.OracleDecoder(cfg, embed, layers, fnorm, lm_w, lm_s) for _ in range(batch)]
    dec = _make(tb, cfg, embed, layers, fnorm, lm_w, lm_s, max_batch=batch)
    ctx = 4090
    _prefill_both(dec, refs, cfg, ctx, 6, batch)
    rng = np.random.default_rng(2)
    for i in range(steps):
        toks = rng.integers(0, cfg["vocab_size"], batch)
        got = dec.step_batch(toks, [ctx + i] * batch)
        for b in range(batch):
            want = refs[b].step(int(toks[b]), ctx + i)
            assert max_rel_err(got[b], want) < LOGIT_TOL, (i, b)
    gk, gv = dec.read_kv_cache(1, seq=batch - 1)
    ek, ev = refs[batch - 1].kv_cache(1)
    assert max_rel_err(gk[:, ctx:ctx + steps], ek[:, ctx:ctx + steps]) < STAGE_TOL
    assert max_rel_err(gv[:, ctx:ctx + steps], ev[:, ctx:ctx + steps]) < STAGE_TOL
    assert tb.lib().tb_device_fault_flag() == 0


def test_llama70b_layer_as_tp8_shards(torch, tb, oracle):
    """Workload configuration 5 (hidden 8192, intermediate 28672, 64 q / 8 kv heads) as its eight
    tensor-parallel shards on one GPU: tb_shard_* cuts one layer's matrices, every shard runs through
    the CUDA linears (o_proj K = 1024, down K = 3584, gate/up N = 3584 per shard), the partial sums
    are added on the host in rank order and compared with the unsharded oracle; plus the attention
    of the full head layout and of one kv head per call at context 8192."""
    H, I, nh, nkv, hd, G, tp = 8192, 28672, 64, 8, 128, 32, 8
    rng = np.random.default_rng(70)
    L = tb.lib()

    def shard_cols(p, s, n, k, r):
        po, so = np.empty((n, k // tp // 2), np.uint8), np.empty((n, k // tp // G), np.float32)
        assert L.tb_shard_cols(p.ctypes.data, s.ctypes.data, n, k, G, r * (k // tp), k // tp, po.ctypes.data, so.ctypes.data) == 0
        return po, so

    def shard_rows(p, s, n, k, r):
        po, so = np.empty((n // tp, k // 2), np.uint8), np.empty((n // tp, k // G), np.float32)
        assert L.tb_shard_rows(p.ctypes.data, s.ctypes.data, n, k, G, r * (n // tp), n // tp, po.ctypes.data, so.ctypes.data) == 0
        return po, so

    def linear(x, p, s):
        return tb.w4a32_grouped_linear(dev(torch, x), dev(torch, p), dev(torch, s), None, G).cpu().numpy()

    # o_proj: row-parallel, K = 8192 split in 8 slices of 1024
    ow, os_ = _quantized(torch, tb, H, nh * hd, G, 701)
    attn = rng.standard_normal((1, nh * hd)).astype(np.float32)
    want = np.asarray(oracle.gemm_w4a32_grouped(attn, ow, os_, None, G)).reshape(1, -1)
    got = np.zeros_like(want)
    for r in range(tp):
        p, s = shard_cols(ow, os_, H, nh * hd, r)
        got = got + linear(attn[:, r * 1024:(r + 1) * 1024], p, s)
    assert max_rel_err(got, want) < STAGE_TOL
    # gate/up: column-parallel (N = 28672 in 8 slices of 3584), down: row-parallel (K slices of 3584)
    gw, gs = _quantized(torch, tb, I, H, G, 702)
    uw, us = _quantized(torch, tb, I, H, G, 703)
    dw, ds = _quantized(torch, tb, H, I, G, 704)
    x = rng.standard_normal((1, H)).astype(np.float32)
    h_want = np.asarray(oracle.swiglu_gemv(x, gw, gs, None, uw, us, None, G)).reshape(1, -1)
    out_want = np.asarray(oracle.gemm_w4a32_grouped(h_want, dw, ds, None, G)).reshape(1, -1)
    out_got = np.zeros_like(out_want)
    for r in range(tp):
        gp, gsc = shard_rows(gw, gs, I, H, r)
        up, usc = shard_rows(uw, us, I, H, r)
        h_r = torch.empty(1, I // tp, device="cuda")
        d_x, d_gp, d_gs, d_up, d_us = dev(torch, x), dev(torch, gp), dev(torch, gsc), dev(torch, up), dev(torch, usc)
        assert L.tb_swiglu_gemv_w4a32(d_x.data_ptr(), d_gp.data_ptr(), d_gs.data_ptr(), None, d_up.data_ptr(), d_us.data_ptr(),
                                      None, h_r.data_ptr(), 1, I // tp, H, G, None) == 0, tb.last_error()
        h_r = h_r.cpu().numpy()
        assert max_rel_err(h_r, h_want[:, r * (I // tp):(r + 1) * (I // tp)]) < STAGE_TOL, r
        dp, dsc = shard_cols(dw, ds, H, I, r)
        out_got = out_got + linear(h_r, dp, dsc)
    assert max_rel_err(out_got, out_want) < STAGE_TOL
    # attention: the full head layout, and one kv head per call (the TP = 8 slice), context 8192
    for heads, kvh in ((nh, nkv), (nh // tp, 1)):
        S, off = 8192, 8191
        qkv = rng.standard_normal((1, (heads + 2 * kvh) * hd)).astype(np.float32)
        kc = (rng.standard_normal((1, kvh, S, hd)) * 0.5).astype(np.float32)
        vc = rng.standard_normal((1, kvh, S, hd)).astype(np.float32)
        cos_t, sin_t = oracle.rope_tables(S, hd, 5e5)
        scratch = torch.zeros(L.tb_attention_scratch_bytes(1, heads, kvh, hd, S), dtype=torch.uint8, device="cuda")
        d_k, d_v = dev(torch, kc), dev(torch, vc)
        out = torch.empty(1, heads * hd, device="cuda")
        assert L.tb_attention_decode(dev(torch, qkv).data_ptr(), d_k.data_ptr(), d_v.data_ptr(), dev(torch, cos_t).data_ptr(),
                                     dev(torch, sin_t).data_ptr(), dev(torch, np.asarray([off], np.int32)).data_ptr(),
                                     out.data_ptr(), scratch.data_ptr(), 1, heads, kvh, hd, S, None) == 0, tb.last_error()
        q = qkv[0, :heads * hd].reshape(heads, hd).copy()
        k = qkv[0, heads * hd:(heads + kvh) * hd].reshape(kvh, hd).copy()
        v = qkv[0, (heads + kvh) * hd:].reshape(kvh, hd)
        for hh in range(heads):
            q[hh] = oracle.rope_apply_head(q[hh], cos_t[off], sin_t[off])
        for hh in range(kvh):
            k[hh] = oracle.rope_apply_head(k[hh], cos_t[off], sin_t[off])
        ek, ev = kc[0].copy(), vc[0].copy()
        ek[:, off], ev[:, off] = k, v
        assert max_rel_err(out.cpu().numpy().reshape(heads, hd), oracle.attention_decode(q, ek, ev, off + 1)) < STAGE_TOL
    assert L.tb_device_fault_flag() == 0


@pytest.mark.parametrize("k,n", [(4096, 14336), (14336, 4096)])
def test_config2_full_matrices_all_rows(torch, tb, oracle, k, n):
    """Workload configuration 2 at full size: every output row of both Llama MLP shapes at
    M = 1, 4, 16 and 64 against the oracle (not a sample of rows)."""
    p, s = _quantized(torch, tb, n, k, 32, k)
    d_p, d_s = dev(torch, p), dev(torch, s)
    rng = np.random.default_rng(n)
    for m in (1, 4, 16, 64):
        x = rng.standard_normal((m, k)).astype(np.float32)
        got = tb.w4a32_grouped_linear(dev(torch, x), d_p, d_s, None, 32).cpu().numpy()
        assert got.shape == (m, n)
        assert max_rel_err(got, oracle.gemm_w4a32_grouped(x, p, s, None, 32)) < STAGE_TOL, m
    assert tb.lib().tb_device_fault_flag() == 0


@pytest.mark.parametrize("n,k,g,pair", [
    (6144, 4096, 32, False), (4096, 4096, 32, False), (14336, 4096, 32, True), (4096, 14336, 32, False),
    (1152, 896, 32, False), (4864, 896, 32, True), (896, 4864, 32, False), (4096, 4096, 64, False),
    (10240 // 8, 8192, 32, False), (8192, 1024, 32, False), (3584, 8192, 32, True), (8192, 3584, 32, False),
    (1001, 2048, 128, False),
])
def test_step_kernel_projection_path_matches_oracle(torch, tb, oracle, n, k, g, pair):
    """The projection phase of the persistent step kernel, run as a one-phase program, at the
    shapes of configurations 3, 4 and 5 (full and as tensor-parallel-8 shards), with all-positive
    activations in one case (the -8 offset of the codes is taken in the integer domain)."""
    L = tb.lib()
    rng = np.random.default_rng(n + k)
    p, s = _quantized(torch, tb, n, k, g, n * 7 + k)
    p2 = s2 = None
    if pair:
        p2, s2 = _quantized(torch, tb, n, k, g, n * 7 + k + 1)
    for positive in (False, True):
        x = rng.standard_normal((1, k)).astype(np.float32)
        if positive:
            x = np.abs(x) + 0.5
        d_x, d_p, d_s = dev(torch, x), dev(torch, p), dev(torch, s)
        d_p2 = dev(torch, p2) if pair else None
        d_s2 = dev(torch, s2) if pair else None
        out = torch.full((1, n), float("nan"), device="cuda")
        rc = L.tb_debug_step_gemv(d_x.data_ptr(), d_p.data_ptr(), d_s.data_ptr(), None, d_p2.data_ptr() if pair else None,
                                  d_s2.data_ptr() if pair else None, out.data_ptr(), n, k, g, None)
        assert rc == 0, tb.last_error()
        torch.cuda.synchronize()
        got = out.cpu().numpy()
        if pair:
            want = np.asarray(oracle.swiglu_gemv(x, p, s, None, p2, s2, None, g)).reshape(1, -1)
            assert max_rel_err(got, want) < STAGE_TOL, positive
        else:
            want = oracle.gemm_w4a32_grouped(x, p, s, None, g)
            assert max_rel_err(got, want) < STAGE_TOL, positive
            # no further from a float64 evaluation than 4x the reference's own fp32 kernel is
            exact = oracle.gemm_w4a32_f64(x, p, s, None, g)
            assert max_rel_err(got, exact) <= 4 * max(max_rel_err(want, exact), 1e-7), positive
    assert L.tb_device_fault_flag() == 0


@pytest.mark.parametrize("H,I,nh,nkv,hd,g,host_io", [(896, 4864, 14, 2, 64, 32, True), (2048, 4096, 16, 4, 128, 64, False)])
def test_fused_transformer_layer_step_in_place(torch, tb, oracle, H, I, nh, nkv, hd, g, host_io):
    """fused_transformer_layer_step_w4a32 (src/quantization/fused_transformer.rs:16-376): one layer in
    place on x, every optional bias present, against the same ten steps composed from oracle pieces;
    the caches change in the one slot [kv_h, offset, :] only."""
    rng = np.random.default_rng(H + I)
    S, off = 96, 57
    tq = (nh + 2 * nkv) * hd
    W = {}
    for name, (n, k) in {"qkv": (tq, H), "o": (H, nh * hd), "gate": (I, H), "up": (I, H), "down": (H, I)}.items():
        W[name + "_w"], W[name + "_s"] = _quantized(torch, tb, n, k, g, H + n + k)
        W[name + "_b"] = (0.05 * rng.standard_normal(n)).astype(np.float32)
    W["input_norm_w"] = (1 + 0.1 * rng.standard_normal(H)).astype(np.float32)
    W["post_norm_w"] = (1 + 0.1 * rng.standard_normal(H)).astype(np.float32)
    x0 = rng.standard_normal(H).astype(np.float32)
    kc = (rng.standard_normal((1, nkv, S, hd)) * 0.5).astype(np.float32)
    vc = rng.standard_normal((1, nkv, S, hd)).astype(np.float32)
    cos_t, sin_t = oracle.rope_tables(S, hd, 1e6)
    eps = 1e-6
    # the oracle's ten steps
    n1 = oracle.rms_norm(x0, W["input_norm_w"], eps)
    qkv = np.asarray(oracle.gemm_w4a32_grouped(n1, W["qkv_w"], W["qkv_s"], W["qkv_b"], g)).reshape(-1)
    q = qkv[:nh * hd].reshape(nh, hd).copy()
    k = qkv[nh * hd:(nh + nkv) * hd].reshape(nkv, hd).copy()
    v = qkv[(nh + nkv) * hd:].reshape(nkv, hd)
    for h in range(nh):
        q[h] = oracle.rope_apply_head(q[h], cos_t[off], sin_t[off])
    for h in range(nkv):
        k[h] = oracle.rope_apply_head(k[h], cos_t[off], sin_t[off])
    ek, ev = kc[0].copy(), vc[0].copy()
    ek[:, off], ev[:, off] = k, v
    attn = oracle.attention_decode(q, ek, ev, off + 1).reshape(-1)
    x1 = x0 + np.asarray(oracle.gemm_w4a32_grouped(attn, W["o_w"], W["o_s"], W["o_b"], g)).reshape(-1)
    n2 = oracle.rms_norm(x1, W["post_norm_w"], eps)
    hmid = np.asarray(oracle.swiglu_gemv(n2, W["gate_w"], W["gate_s"], W["gate_b"], W["up_w"], W["up_s"], W["up_b"], g)).reshape(-1)
    want = x1 + np.asarray(oracle.gemm_w4a32_grouped(hmid, W["down_w"], W["down_s"], W["down_b"], g)).reshape(-1)
    # the library, in place
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    d_k, d_v = t(kc), t(vc)
    x = torch.from_numpy(x0.copy()) if host_io else t(x0)
    tb.fused_transformer_layer_step(x, t(W["input_norm_w"]), t(W["qkv_w"]), t(W["qkv_s"]), t(W["qkv_b"]), t(W["o_w"]), t(W["o_s"]),
                                    t(W["o_b"]), t(W["post_norm_w"]), t(W["gate_w"]), t(W["gate_s"]), t(W["gate_b"]), t(W["up_w"]),
                                    t(W["up_s"]), t(W["up_b"]), t(W["down_w"]), t(W["down_s"]), t(W["down_b"]), d_k, d_v,
                                    torch.from_numpy(cos_t[off]), torch.from_numpy(sin_t[off]), off, nh, nkv, hd, g, eps)
    assert max_rel_err(x.cpu().numpy(), want) < STAGE_TOL
    gk, gv = d_k.cpu().numpy()[0], d_v.cpu().numpy()[0]
    assert max_rel_err(gk[:, off], k) < 1e-6 and max_rel_err(gv[:, off], v) < 1e-6
    mask = np.ones(S, bool); mask[off] = False
    assert np.array_equal(gk[:, mask], kc[0][:, mask]) and np.array_equal(gv[:, mask], vc[0][:, mask])
    # errors of the reference's entry point: an offset outside the cache
    with pytest.raises(ValueError):
        tb.fused_transformer_layer_step(x, t(W["input_norm_w"]), t(W["qkv_w"]), t(W["qkv_s"]), None, t(W["o_w"]), t(W["o_s"]), None,
                                        t(W["post_norm_w"]), t(W["gate_w"]), t(W["gate_s"]), None, t(W["up_w"]), t(W["up_s"]), None,
                                        t(W["down_w"]), t(W["down_s"]), None, d_k, d_v, torch.from_numpy(cos_t[off]),
                                        torch.from_numpy(sin_t[off]), S, nh, nkv, hd, g, eps)


def test_fp32_product_mode_is_selectable_and_matches_oracle(torch, tb, oracle):
    """tb_set_gemv_tuning(0, ...): the M = 1 kernels multiply in fp32 (the reference's own W4A32
    arithmetic) instead of block fixed point; same tolerance, tighter distance from float64."""
    L = tb.lib()
    rng = np.random.default_rng(12)
    n, k, g = 4096, 4096, 32
    p, s = _quantized(torch, tb, n, k, g, 1212)
    x = rng.standard_normal((1, k)).astype(np.float32)
    want = oracle.gemm_w4a32_grouped(x, p, s, None, g)
    exact = oracle.gemm_w4a32_f64(x, p, s, None, g)
    try:
        L.tb_set_gemv_tuning(0, 0, 0)
        got = tb.w4a32_grouped_linear(dev(torch, x), dev(torch, p), dev(torch, s), None, g).cpu().numpy()
    finally:
        L.tb_set_gemv_tuning(1, 0, 0)
    assert max_rel_err(got, want) < STAGE_TOL
    assert max_rel_err(got, exact) <= 4 * max(max_rel_err(want, exact), 1e-7)
    got_int = tb.w4a32_grouped_linear(dev(torch, x), dev(torch, p), dev(torch, s), None, g).cpu().numpy()
    assert max_rel_err(got_int, want) < STAGE_TOL


@pytest.mark.parametrize("n,k,g,m,bias,pair", [
    (640, 1024, 32, 24, True, False),      # K split over several CTAs (atomic partial sums), bias
    (300, 512, 64, 19, False, False),      # rows past n inside the only tile, padded activation rows
    (1001, 2048, 128, 33, True, False),    # a group spans two 64-element stages
    (4096, 4096, 32, 64, False, False),    # o_proj of configuration 4
    (512, 14336, 32, 100, False, False),   # two passes (64 + 36 rows), K = 14336
    (777, 1024, 32, 17, False, True),      # SwiGLU pair, ragged n
    (4864, 896, 32, 48, True, True),       # Qwen gate/up with bias
    (14336, 4096, 32, 64, False, True),    # Llama gate/up at M = 64
    (256, 128, 32, 20, True, False),       # K = 128: two stages only, fewer than the ring and the prefetch depth
    (200, 256, 128, 65, False, True),      # pair with 128-element groups, a second pass of one row
    (1536, 1024, 64, 40, True, True),      # pair with 64-element groups
    (96, 8192, 64, 31, False, False),      # one ragged tile, K split 64 ways at most
])
def test_tcgen05_batched_product_matches_oracle(torch, tb, oracle, n, k, g, m, bias, pair):
    """More than 16 activation rows take the tcgen05 kernel (bf16 codes from tensor memory, three
    bf16 pieces of every activation, the scale applied per group outside the tensor core).  It
    must stay as close to the float64 result as the reference's own fp32 kernel, and agree with
    the integer mma.sync kernel it replaces (tb_set_gemv_tuning(3, ..) keeps that one selectable)."""
    L = tb.lib()
    rng = np.random.default_rng(n * 3 + k + m)
    p, s = _quantized(torch, tb, n, k, g, n + k + m, std=0.05)
    x = rng.standard_normal((m, k)).astype(np.float32)
    b = rng.standard_normal(n).astype(np.float32) if bias else None
    d = lambda a: dev(torch, a) if a is not None else None
    if pair:
        p2, s2 = _quantized(torch, tb, n, k, g, n + k + m + 1, std=0.05)
        b2 = rng.standard_normal(n).astype(np.float32) if bias else None
        t = [d(a) for a in (x, p, s, b, p2, s2, b2)]
        ptr = lambda a: a.data_ptr() if a is not None else None

        def run():
            h = torch.full((m, n), float("nan"), device="cuda")
            assert L.tb_swiglu_gemv_w4a32(ptr(t[0]), ptr(t[1]), ptr(t[2]), ptr(t[3]), ptr(t[4]), ptr(t[5]), ptr(t[6]),
                                          h.data_ptr(), m, n, k, g, None) == 0, tb.last_error()
            torch.cuda.synchronize()
            return h.cpu().numpy()
        want = np.stack([oracle.swiglu_gemv(x[i], p, s, b, p2, s2, b2, g) for i in range(m)])
    else:
        def run():
            return tb.w4a32_grouped_linear(d(x), d(p), d(s), d(b), g).cpu().numpy()
        want = oracle.gemm_w4a32_grouped(x, p, s, b, g).reshape(m, n)
    got = run()
    assert got.shape == (m, n)
    assert max_rel_err(got, want) < STAGE_TOL
    try:
        L.tb_set_gemv_tuning(3, 0, 0)
        old = run()
    finally:
        L.tb_set_gemv_tuning(1, 0, 0)
    assert max_rel_err(old, want) < STAGE_TOL
    assert max_rel_err(got, old) < 1e-5
    if not pair:
        exact = oracle.gemm_w4a32_f64(x, p, s, b, g)
        assert max_rel_err(got, exact) <= max(4 * max_rel_err(want, exact), 2e-6)
    assert L.tb_device_fault_flag() == 0


@pytest.mark.parametrize("n,k,g,m,bias,pair", [
    (4096, 4096, 32, 2, True, False),      # o_proj shape
    (6144, 4096, 32, 2, False, False),     # QKV shape
    (14336, 4096, 32, 2, True, True),      # gate/up pair
    (4096, 14336, 32, 2, False, False),    # the K = 14336 projection: 14 consumer warps
    (1001, 2048, 64, 2, True, False),      # ragged last round, 64-element groups
    (520, 7168, 128, 2, False, True),      # 128-element groups, pair
    (96, 8192, 32, 2, True, True),         # fewer rounds than CTAs
    (4096, 4096, 32, 3, True, False),      # three and four rows of a narrow matrix: the CUDA-core kernel
    (6144, 4096, 32, 4, False, False),
])
def test_two_rows_take_the_persistent_kernel_and_match_oracle(torch, tb, oracle, n, k, g, m, bias, pair):
    """Two activation rows take a variant of the persistent streaming kernel of the M = 1 path: a lane keeps
    the digits of its block of K for both rows and multiplies each weight word with both (one pass over the
    weights).  Against the oracle, against the kernel that runs with the streaming kernel switched off, and
    against the float64 bound of the single-row kernel.  Three and four rows of a narrow matrix run on the
    CUDA-core kernel (same checks; the switch changes nothing for them)."""
    L = tb.lib()
    rng = np.random.default_rng(n + 7 * k + m)
    p, s = _quantized(torch, tb, n, k, g, n + k + m, std=0.05)
    x = rng.standard_normal((m, k)).astype(np.float32)
    b = rng.standard_normal(n).astype(np.float32) if bias else None
    d = lambda a: dev(torch, a) if a is not None else None
    if pair:
        p2, s2 = _quantized(torch, tb, n, k, g, n + k + m + 1, std=0.05)
        b2 = rng.standard_normal(n).astype(np.float32) if bias else None
        t = [d(a) for a in (x, p, s, b, p2, s2, b2)]
        ptr = lambda a: a.data_ptr() if a is not None else None

        def run():
            h = torch.full((m, n), float("nan"), device="cuda")
            assert L.tb_swiglu_gemv_w4a32(ptr(t[0]), ptr(t[1]), ptr(t[2]), ptr(t[3]), ptr(t[4]), ptr(t[5]), ptr(t[6]),
                                          h.data_ptr(), m, n, k, g, None) == 0, tb.last_error()
            torch.cuda.synchronize()
            return h.cpu().numpy()
        want = np.stack([oracle.swiglu_gemv(x[i], p, s, b, p2, s2, b2, g) for i in range(m)])
    else:
        def run():
            return tb.w4a32_grouped_linear(d(x), d(p), d(s), d(b), g).cpu().numpy()
        want = oracle.gemm_w4a32_grouped(x, p, s, b, g).reshape(m, n)
    got = run()
    assert got.shape == (m, n)
    assert max_rel_err(got, want) < STAGE_TOL
    try:
        L.tb_set_stream_tuning(0, 0, 0, 0, 0)
        old = run()
    finally:
        L.tb_set_stream_tuning(1, 0, 0, 0, 0)
    assert max_rel_err(old, want) < STAGE_TOL
    assert max_rel_err(got, old) < 1e-5
    if not pair:
        exact = oracle.gemm_w4a32_f64(x, p, s, b, g)
        assert max_rel_err(got, exact) <= max(4 * max_rel_err(want, exact), 2e-6)
    assert L.tb_device_fault_flag() == 0


def test_products_with_several_rows_keep_a_workspace_per_stream(torch, tb, oracle):
    """Stateless products with two or more rows keep their workspace per (device, stream): a second call reuses
    it, a wider K grows it, another stream gets its own, tb_release_workspaces frees them and the next call
    allocates again.  Results stay those of the oracle throughout, also when calls are captured into a graph."""
    L = tb.lib()
    rng = np.random.default_rng(5)
    g = 32
    cases = []
    for n, k, m in ((256, 1024, 8), (192, 4096, 12), (256, 1024, 40)):
        p, s = _quantized(torch, tb, n, k, g, n + k + m, std=0.05)
        x = rng.standard_normal((m, k)).astype(np.float32)
        cases.append((dev(torch, x), dev(torch, p), dev(torch, s), oracle.gemm_w4a32_grouped(x, p, s, None, g).reshape(m, n), m, n, k))

    def check(stream=None):
        for x, p, s, want, m, n, k in cases:
            y = torch.full((m, n), float("nan"), device="cuda")
            st = stream.cuda_stream if stream is not None else None
            assert L.tb_gemm_w4a32_grouped(x.data_ptr(), p.data_ptr(), s.data_ptr(), None, y.data_ptr(), m, n, k, g, st) == 0, tb.last_error()
            (stream.synchronize() if stream is not None else torch.cuda.synchronize())
            assert max_rel_err(y.cpu().numpy(), want) < STAGE_TOL

    check()
    check()
    side = torch.cuda.Stream()
    check(side)
    # captured: the block of the stream exists already, so the graph holds kernels only
    x, p, s, want, m, n, k = cases[1]
    y = torch.zeros((m, n), device="cuda")
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        assert L.tb_gemm_w4a32_grouped(x.data_ptr(), p.data_ptr(), s.data_ptr(), None, y.data_ptr(), m, n, k, g,
                                       torch.cuda.current_stream().cuda_stream) == 0, tb.last_error()
    graph.replay()
    torch.cuda.synchronize()
    assert max_rel_err(y.cpu().numpy(), want) < STAGE_TOL
    del graph
    L.tb_release_workspaces()
    check()
    check(side)
    L.tb_release_workspaces()
    assert L.tb_device_fault_flag() == 0


def test_bounded_device_wait_runs_out_and_reports_timeout(torch, tb):
    """Failure detection without a fault: a wait of the step kernel on a barrier that nothing
    completes, with a limit of a millisecond.  The kernel must return, raise the fault word and
    the entry point must report TB_ERR_TIMEOUT; the context stays usable."""
    L = tb.lib()
    assert L.tb_device_fault_flag() == 0
    rc = L.tb_debug_wait_probe(2_000_000)   # cycles: about a millisecond
    assert rc == 7, (rc, tb.last_error())   # TB_ERR_TIMEOUT
    assert "wait" in tb.last_error()
    assert L.tb_device_fault_flag() == 0    # the probe clears the word it raised
    # the device still works
    x = torch.ones(4, device="cuda")
    assert float((x * 2).sum().item()) == 8.0
