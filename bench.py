"""Headline benchmark: INT4 decode tokens/s of a Llama-3-8B-shaped model on B200(s).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--impl reference]

N=1 workload: the headline configuration "Llama-3-8B-architecture INT4 decode" - hidden 4096,
32 layers, 32 q / 8 kv heads, head_dim 128, intermediate 14336, vocab 128256,
group 32, random init (std 0.02), fp32 KV cache pre-filled to a context of 4096,
batch 1.  For N>1 (launched by torchrun, one rank per GPU) the same model is sharded
tensor-parallel over the N GPUs ("strong" scaling: the work per token is fixed).

One step = one decode step (all layers + lm_head) for `batch` sequences.
 * value        : tokens/s with everything resident in HBM, K steps enqueued back to
                  back (the device-side greedy generate loop), CUDA events on the
                  decoder's stream, max over ranks.
 * e2e          : the same metric through tb_decoder_step with HOST buffers: every
                  step copies the token id in (pinned) and the [vocab] fp32 logits out.
 * roofline     : the dominant kernel (fused RMSNorm + gate/up GEMV + SwiGLU), timed
                  alone over the 32 layers' distinct weights (2.3 GB, far above L2).
 * cpu_baseline : the CPU oracle's SIMD path on this box's host cores (thread count set
                  explicitly): full steps, every layer + lm_head, bounded by the step count.
`--impl reference` prints the CPU arm alone in the same JSON shape.

Synthetic data throughout (no checkpoints or datasets are involved): weights
N(0, 0.02) quantized with the reference's quantizer arithmetic, token ids uniform,
KV pre-filled with seeded N(0,1) values.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np

LLAMA8B = dict(vocab_size=128256, hidden_size=4096, intermediate_size=14336, num_layers=32, num_heads=32,
               num_kv_heads=8, head_dim=128, group_size=32, rms_norm_eps=1e-6, rope_theta=500000.0)
LLAMA70B = dict(vocab_size=128256, hidden_size=8192, intermediate_size=28672, num_layers=80, num_heads=64,
                num_kv_heads=8, head_dim=128, group_size=32, rms_norm_eps=1e-6, rope_theta=500000.0)
QWEN05B = dict(vocab_size=151936, hidden_size=896, intermediate_size=4864, num_layers=24, num_heads=14,
               num_kv_heads=2, head_dim=64, group_size=32, rms_norm_eps=1e-6, rope_theta=1000000.0)
CONTEXT = 4096
_RESULT_LINE = []   # the one JSON line of this process (rank 0), printed at the very end
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from an ncu
# capture of that kernel at this shape (None until a capture exists for the kernel).
DOMINANT_KERNEL_DRAM_TRAFFIC = 73_476_096 + 1_689_088


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


def weight_bytes(n, k, g):
    return n * k // 2 + n * (k // g) * 4


def step_weight_bytes(c, tp=1):
    H, I, V, G = c["hidden_size"], c["intermediate_size"], c["vocab_size"], c["group_size"]
    q_dim = c["num_heads"] * c["head_dim"]
    tq = q_dim + 2 * c["num_kv_heads"] * c["head_dim"]
    per_layer = weight_bytes(tq, H, G) + weight_bytes(H, q_dim, G) + 2 * weight_bytes(I, H, G) + weight_bytes(H, I, G) + 2 * H * 4
    return c["num_layers"] * per_layer + weight_bytes(V, H, G) + H * 4


def kv_bytes_per_seq(c, ctx):
    return c["num_layers"] * 2 * c["num_kv_heads"] * ctx * c["head_dim"] * 4


class ClockSampler:
    """Samples SM clock and throttle reasons during the timed region (read-only NVML)."""

    REASONS = {0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x10: "sync_boost",
               0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown",
               0x100: "display_clock_setting"}

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._t = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nv = None

    def _run(self):
        while not self._stop.is_set():
            try:
                self.samples.append(int(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM)))
                mask = int(self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.05)

    def __enter__(self):
        if self.nv is not None:
            self._t = threading.Thread(target=self._run, daemon=True)
            self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._t is not None:
            self._t.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["unavailable"]}
        return {"sm_mhz": float(np.median(self.samples)), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ----------------------------------------------------------------- CPU arm
def host_cpu():
    """(usable hardware threads of this process, CPU model name)."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    model = "unknown"
    try:
        for line in open("/proc/cpuinfo"):
            if line.startswith("model name"):
                model = line.split(":", 1)[1].strip()
                break
    except OSError:
        pass
    return n, model


def cpu_full_step(c, ctx, steps, warmup, seed=0):
    """Times FULL decode steps (every layer + lm_head, fp32 KV cache at `ctx`) of the CPU oracle -
    the reference's SIMD path restated in C - on all host threads this process may use.  The
    thread count is set explicitly (launchers such as torchrun export OMP_NUM_THREADS=1).
    Weights are random packed nibbles with scales of the magnitude the quantizer produces for
    N(0, 0.02) weights; timing does not depend on their values."""
    from oracle import oracle as o

    threads, cpu_model = host_cpu()
    o.set_threads(threads)
    rng = np.random.default_rng(seed)
    H, I, G, V = c["hidden_size"], c["intermediate_size"], c["group_size"], c["vocab_size"]
    nh, nkv, hd, L = c["num_heads"], c["num_kv_heads"], c["head_dim"], c["num_layers"]
    cfg = dict(c, max_seq_len=ctx + 8)

    def rlin(n, k):
        w = np.frombuffer(rng.bytes(n * (k // 2)), dtype=np.uint8).reshape(n, k // 2)
        s = (rng.random((n, k // G), dtype=np.float32) * np.float32(0.004) + np.float32(0.006))
        return w, s

    layers = []
    for _ in range(L):
        lw = {"input_norm_w": np.ones(H, np.float32), "post_norm_w": np.ones(H, np.float32), "qkv_b": None}
        lw["qkv_w"], lw["qkv_s"] = rlin((nh + 2 * nkv) * hd, H)
        lw["o_w"], lw["o_s"] = rlin(H, nh * hd)
        lw["gate_w"], lw["gate_s"] = rlin(I, H)
        lw["up_w"], lw["up_s"] = rlin(I, H)
        lw["down_w"], lw["down_s"] = rlin(H, I)
        layers.append(lw)
    embed = rng.standard_normal((V, H), dtype=np.float32) * np.float32(0.02)
    lm_w, lm_s = rlin(V, H)
    dec = o.OracleDecoder(cfg, embed, layers, np.ones(H, np.float32), lm_w, lm_s)
    for l in range(L):  # context pre-filled with seeded values
        k, v = dec.kv_cache(l)
        k[:, :ctx] = rng.standard_normal((nkv, ctx, hd), dtype=np.float32) * np.float32(0.5)
        v[:, :ctx] = rng.standard_normal((nkv, ctx, hd), dtype=np.float32)
    dec.set_kv_len(ctx)
    for i in range(warmup):
        dec.step(3 + i, ctx)
    times = []
    for i in range(steps):
        t0 = time.perf_counter()
        dec.step(5 + i, ctx)
        times.append(time.perf_counter() - t0)
    total = float(np.sum(times))
    return {
        "value": steps / total, "unit": "tokens/s", "cores": threads, "kind": "port",
        "tier": o.TIER_NAMES.get(o.best_tier(), "?"), "cpu_model": cpu_model,
        "sample": (f"full step: all {L} layers + lm_head with a {ctx}-token fp32 KV cache, {steps} timed steps after "
                   f"{warmup} warm-up steps (median {np.median(times) * 1e3:.1f} ms, best {np.min(times) * 1e3:.1f} ms per step)"),
        "ms_per_step": total / steps * 1e3, "ms_per_step_best": float(np.min(times)) * 1e3,
    }


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    c = dict(LLAMA8B)
    t0 = time.perf_counter()
    steps, warmup = max(1, min(args.steps, 64)), max(1, min(args.warmup, 8))
    r = cpu_full_step(c, CONTEXT, steps, warmup)
    line = {
        "impl": "reference", "metric": "decode_tokens_per_s", "value": r["value"],
        "unit": "tokens/s", "n_gpus": args.gpus, "steps": steps, "warmup": warmup,
        "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": workload_config(c, 1, args.gpus),
        "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample", "tier", "cpu_model")},
        "e2e": {"value": r["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "wall_s": time.perf_counter() - t0,
        "note": "CPU restatement of the reference's SIMD path (the Rust reference cannot be built here); batch 1; "
                "the same host cores at every --gpus value",
    }
    _RESULT_LINE.append(json.dumps(line))


def workload_config(c, batch, n_gpus):
    return {
        "workload": f"{ {4096: 'llama-3-8b', 8192: 'llama-3-70b'}.get(c['hidden_size'], 'qwen2.5-0.5b')}-shaped INT4 (group {c['group_size']}) W4A32 decode, batch {batch}, fp32 KV at context {CONTEXT}",
        "hidden": c["hidden_size"], "layers": c["num_layers"], "heads": f"{c['num_heads']}q/{c['num_kv_heads']}kv",
        "head_dim": c["head_dim"], "intermediate": c["intermediate_size"], "vocab": c["vocab_size"],
        "batch": batch, "context": CONTEXT, "parallelism": f"tp{n_gpus}",
        "l2": "per-step working set (4.7 GB weights + 1.07 GB KV per sequence) exceeds the 126 MB L2; no flush needed",
    }


# ----------------------------------------------------------------- GPU arm
def build_model(torch, tb, c, device, tp, rank, seed=1234, direct_shards=False):
    """Random-init Llama-shaped weights generated and quantized on the GPU; under
    tensor parallelism every rank generates the same full matrix and keeps its shard.
    direct_shards (throughput-only runs of models too large for that): every rank generates
    matrices of its shard's shape; the ranks' shards are then not slices of one model."""
    if direct_shards:
        return build_model_direct(torch, tb, c, device, tp, rank, seed)
    gen = torch.Generator(device).manual_seed(seed)
    H, I, V, G = c["hidden_size"], c["intermediate_size"], c["vocab_size"], c["group_size"]
    nh, nkv, hd = c["num_heads"], c["num_kv_heads"], c["head_dim"]
    q_dim, kv_dim = nh * hd, nkv * hd

    def qlin(n, k):
        w = torch.randn(n, k, device=device, generator=gen) * 0.02
        return tb.quantize_weight_int4_grouped(w, group_size=G)

    def rows(p, s, r0, n):
        return p[r0:r0 + n].contiguous(), s[r0:r0 + n].contiguous()

    def cols(p, s, c0, n):
        return p[:, c0 // 2:(c0 + n) // 2].contiguous(), s[:, c0 // G:(c0 + n) // G].contiguous()

    layers = []
    for _ in range(c["num_layers"]):
        qkv_p, qkv_s = qlin(q_dim + 2 * kv_dim, H)
        o_p, o_s = qlin(H, q_dim)
        g_p, g_s = qlin(I, H)
        u_p, u_s = qlin(I, H)
        d_p, d_s = qlin(H, I)
        if tp > 1:
            ql, kl, il = q_dim // tp, kv_dim // tp, I // tp
            idx = torch.cat([torch.arange(rank * ql, (rank + 1) * ql), q_dim + torch.arange(rank * kl, (rank + 1) * kl),
                             q_dim + kv_dim + torch.arange(rank * kl, (rank + 1) * kl)]).to(device)
            qkv_p, qkv_s = qkv_p[idx].contiguous(), qkv_s[idx].contiguous()
            o_p, o_s = cols(o_p, o_s, rank * ql, ql)
            g_p, g_s = rows(g_p, g_s, rank * il, il)
            u_p, u_s = rows(u_p, u_s, rank * il, il)
            d_p, d_s = cols(d_p, d_s, rank * il, il)
        ones = torch.ones(H, device=device)
        layers.append([ones, qkv_p, qkv_s, o_p, o_s, ones, g_p, g_s, u_p, u_s, d_p, d_s])
    embed = torch.randn(V, H, device=device, generator=gen) * 0.02
    lm_p, lm_s = qlin(V, H)
    if tp > 1:
        lm_p, lm_s = rows(lm_p, lm_s, rank * (V // tp), V // tp)
    return embed, layers, torch.ones(H, device=device), lm_p, lm_s


def build_model_direct(torch, tb, c, device, tp, rank, seed):
    gen = torch.Generator(device).manual_seed(seed + rank)
    H, I, V, G = c["hidden_size"], c["intermediate_size"], c["vocab_size"], c["group_size"]
    q_dim, kv_dim = c["num_heads"] * c["head_dim"], c["num_kv_heads"] * c["head_dim"]

    def qlin(n, k):
        w = torch.randn(n, k, device=device, generator=gen) * 0.02
        return tb.quantize_weight_int4_grouped(w, group_size=G)

    ones = torch.ones(H, device=device)
    layers = []
    for _ in range(c["num_layers"]):
        layers.append([ones, *qlin((q_dim + 2 * kv_dim) // tp, H), *qlin(H, q_dim // tp), ones, *qlin(I // tp, H), *qlin(I // tp, H),
                       *qlin(H, I // tp)])
    embed = torch.randn(V, H, device=device, generator=torch.Generator(device).manual_seed(seed)) * 0.02
    lm_p, lm_s = qlin(V // tp, H)
    return embed, layers, ones, lm_p, lm_s


def prefill_kv(torch, dec, c, device, ctx, batch, tp, rank, seed=99):
    gen = torch.Generator(device).manual_seed(seed)
    nkv_l = c["num_kv_heads"] // tp
    for b in range(batch):
        ks, vs = [], []
        for _ in range(c["num_layers"]):
            k = torch.randn(c["num_kv_heads"], ctx, c["head_dim"], device=device, generator=gen) * 0.5
            v = torch.randn(c["num_kv_heads"], ctx, c["head_dim"], device=device, generator=gen)
            ks.append(k[rank * nkv_l:(rank + 1) * nkv_l].contiguous())
            vs.append(v[rank * nkv_l:(rank + 1) * nkv_l].contiguous())
        dec.copy_kv_cache_from_tensors(ks, vs, ctx, seq=b)


def make_decoder(tb, c, model, max_seq, batch, tp, rank, args, **kw):
    embed, layers, fnorm, lm_p, lm_s = model
    return tb.B200QwenDecoder(embed, layers, fnorm, lm_p, lm_s, c["num_layers"], c["hidden_size"],
                              c["intermediate_size"], c["num_heads"], c["num_kv_heads"], c["head_dim"], c["group_size"],
                              c["rms_norm_eps"], max_seq, c["rope_theta"], max_batch=batch, tp_size=tp, tp_rank=rank,
                              vocab_size=c["vocab_size"], nccl_only=args.nccl_only, pdl=not args.no_pdl, debug=args.no_graph,
                              fused_step=(False if args.chain else (True if args.step_kernel else None)), **kw)


def timed_steps(torch, dist, tb, dec, device, tp, batch, ctx, steps, warmup, repeats):
    """`repeats` timed regions of exactly `steps` decode steps each (CUDA events on the decoder's
    stream, a barrier and a device synchronisation on both sides, max over ranks); returns the
    list of milliseconds per region."""
    L = tb.lib()
    stream = torch.cuda.ExternalStream(L.tb_decoder_stream(dec.handle), device=device)
    out_tokens = np.empty(max(steps, warmup), np.int64)

    def barrier():
        if tp > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    def generate(first, start, n):
        if batch == 1:
            tb._lib.check(L.tb_decoder_generate_greedy(dec.handle, first, start, n, out_tokens.ctypes.data))
        else:
            toks = np.full(batch, first, np.int64)
            for i in range(n):
                offs = np.full(batch, start + i, np.int64)
                tb._lib.check(L.tb_decoder_step_batch(dec.handle, toks.ctypes.data, offs.ctypes.data, batch, None))

    generate(11, ctx, warmup)
    barrier()
    out = []
    for r in range(repeats):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        generate(12 + r, ctx + warmup, steps)
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        if tp > 1:
            t = torch.tensor([ms], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        out.append(ms)
    return out


def tp_correctness_check(torch, dist, tb, c, device, tp, rank, args):
    """Outside every timed region: a two-layer model of the benchmark's true widths, sharded over the
    `tp` ranks, against the same model unsharded on rank 0's GPU - the logits of three steps."""
    small = dict(c, num_layers=2, vocab_size=8192)
    full = build_model(torch, tb, small, device, 1, 0, seed=4321)
    shard = build_model(torch, tb, small, device, tp, rank, seed=4321)
    dec = make_decoder(tb, small, shard, 64, 1, tp, rank, args)
    from torchburn_b200.tp import init_tensor_parallel

    init_tensor_parallel(dec, dist, device)
    ref = make_decoder(tb, small, full, 64, 1, 1, 0, args) if rank == 0 else None
    worst = 0.0
    for off, tok in enumerate((17, 4000, 911)):
        got = dec.step(tok, off)
        if rank == 0:
            want = ref.step(tok, off)
            worst = max(worst, float(np.abs(got - want).max() / max(np.abs(want).max(), 1e-6)))
    fault = int(tb.lib().tb_device_fault_flag())
    dist.barrier()
    dec.close()
    if ref is not None:
        ref.close()
    return {"max_rel_err": worst, "ranks": tp, "fault_flag": fault,
            "what": "2 layers at the benchmark's widths, vocabulary 8192: sharded decoder against the unsharded one on rank 0, logits of 3 steps"}


def _graph_time(torch, device, one_pass, launches_per_pass, passes=10):
    """Captures one pass of raw C-ABI launches into a CUDA graph (so that the host's call
    overhead does not pace the device) and times `passes` replays with CUDA events."""
    side = torch.cuda.Stream(device)
    with torch.cuda.stream(side):
        for _ in range(3):
            one_pass()
    torch.cuda.synchronize(device)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        one_pass()
    st = torch.cuda.current_stream(device)
    for _ in range(3):
        graph.replay()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(device)
    e0.record(st)
    for _ in range(passes):
        graph.replay()
    e1.record(st)
    torch.cuda.synchronize(device)
    return e0.elapsed_time(e1) * 1e-3 / (passes * launches_per_pass)


def _graph_time_streams(torch, device, launch, n_launches, n_streams=4, passes=10):
    """The same, with the launches spread round-robin over `n_streams` streams that fork from and join the
    captured stream: the graph's kernel nodes have no edges between streams, so independent launches overlap
    (launch gap, prologue and tail of one under the streaming of another).  A throughput, not a latency."""
    main = torch.cuda.Stream(device)
    subs = [torch.cuda.Stream(device) for _ in range(n_streams)]

    def one_pass():
        cur = torch.cuda.current_stream(device)
        for sub in subs:
            sub.wait_stream(cur)
        for i in range(n_launches):
            launch(i, subs[i % n_streams].cuda_stream, i % n_streams)
        for sub in subs:
            cur.wait_stream(sub)

    with torch.cuda.stream(main):
        for _ in range(3):
            one_pass()
    torch.cuda.synchronize(device)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=main):
        one_pass()
    st = torch.cuda.current_stream(device)
    for _ in range(3):
        graph.replay()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(device)
    e0.record(st)
    for _ in range(passes):
        graph.replay()
    e1.record(st)
    torch.cuda.synchronize(device)
    return e0.elapsed_time(e1) * 1e-3 / (passes * n_launches)


def time_dominant_kernel(torch, tb, c, layers, device, tp):
    """gate/up GEMV + SwiGLU alone, over all layers' distinct weights (2.3 GB at tp=1, far above
    L2), CUDA events on the launch stream."""
    H, G = c["hidden_size"], c["group_size"]
    I_l = c["intermediate_size"] // tp
    x = torch.randn(1, H, device=device)
    h = torch.empty(1, I_l, device=device)
    L = tb.lib()

    def one_pass():
        st = torch.cuda.current_stream(device).cuda_stream
        for lw in layers:
            rc = L.tb_swiglu_gemv_w4a32(x.data_ptr(), lw[6].data_ptr(), lw[7].data_ptr(), None, lw[8].data_ptr(),
                                        lw[9].data_ptr(), None, h.data_ptr(), 1, I_l, H, G, st)
            assert rc == 0, tb.last_error()

    sec = _graph_time(torch, device, one_pass, len(layers))
    alg = 2 * weight_bytes(I_l, H, G) + H * 4 + I_l * 4
    return alg, sec, len(layers)


def time_c2_gemm(torch, tb, c, layers, device):
    """workload configuration 2: the batched grouped INT4 product at the Llama-3-8B MLP shapes,
    M in {1, 4, 16, 64}; (K=4096, N=14336) runs over the layers' distinct gate matrices and
    (K=14336, N=4096) over their down matrices (1.17 GB each, far above L2)."""
    H, I, G = c["hidden_size"], c["intermediate_size"], c["group_size"]
    L = tb.lib()
    out = []
    for name, n, k, wi, si in (("gate/up shape K=4096 N=14336", I, H, 6, 7), ("down shape K=14336 N=4096", H, I, 10, 11)):
        for m in (1, 4, 16, 64):
            x = torch.randn(m, k, device=device)
            y = torch.empty(m, n, device=device)

            def one_pass():
                st = torch.cuda.current_stream(device).cuda_stream
                for lw in layers:
                    rc = L.tb_gemm_w4a32_grouped(x.data_ptr(), lw[wi].data_ptr(), lw[si].data_ptr(), None, y.data_ptr(), m, n, k, G, st)
                    assert rc == 0, tb.last_error()

            sec = _graph_time(torch, device, one_pass, len(layers), passes=5)
            alg = weight_bytes(n, k, G) + m * k * 4 + m * n * 4
            out.append({"shape": name, "m": m, "us_per_launch": sec * 1e6, "achieved_gbs": alg / sec / 1e9,
                        "tflops": 2.0 * m * n * k / sec / 1e12, "launches_per_call": 1 if m == 1 else 2})
    return out


def time_c1_gemv(torch, tb, device, copies=64):
    """workload configuration 1: a single 4096x4096 group-32 GEMV, rotating over `copies` distinct
    weight copies (672 MB, > 5x L2) so every launch streams from HBM."""
    n = k = 4096
    g = 32
    gen = torch.Generator(device).manual_seed(7)
    ws = []
    for _ in range(copies):
        w = torch.randn(n, k, device=device, generator=gen) * 0.02
        ws.append(tb.quantize_weight_int4_grouped(w, group_size=g))
    x = torch.randn(1, k, device=device, generator=gen)
    out = torch.empty(1, n, device=device)
    L = tb.lib()

    def one_pass():
        st = torch.cuda.current_stream(device).cuda_stream
        for p, s in ws:
            rc = L.tb_gemv_w4a32_grouped(x.data_ptr(), p.data_ptr(), s.data_ptr(), None, out.data_ptr(), n, k, g, st)
            assert rc == 0, tb.last_error()

    sec = _graph_time(torch, device, one_pass, copies)
    outs = torch.empty(4, n, device=device)

    def launch(i, stream, slot):
        p, s = ws[i]
        rc = L.tb_gemv_w4a32_grouped(x.data_ptr(), p.data_ptr(), s.data_ptr(), None, outs[slot].data_ptr(), n, k, g, stream)
        assert rc == 0, tb.last_error()

    sec4 = _graph_time_streams(torch, device, launch, copies, 4)
    alg = weight_bytes(n, k, g) + k * 4 + n * 4
    return alg, sec, sec4


def run_gpu(args):
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    tp = world
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if tp > 1:
        dist.init_process_group("nccl", device_id=device)
    import torchburn_b200 as tb

    global CONTEXT
    c = dict(LLAMA8B)
    direct = False
    if args.model == "qwen05b":  # workload configuration 3 (single GPU, context 1024); not the headline workload
        c, CONTEXT = dict(QWEN05B), 1024
    elif args.model == "llama70b":  # workload configuration 5: tensor parallel 8, batch 16, context 8192; throughput only
        c, CONTEXT, direct = dict(LLAMA70B), 8192, True
    B, K, W = args.batch, args.steps, max(args.warmup, 3)
    R = 1 if args.quick else max(1, args.repeats)
    max_seq = CONTEXT + 64 * ((K + W + 63) // 64) + 64
    model = build_model(torch, tb, c, device, tp, rank, direct_shards=direct)
    layers = model[1]
    dec = make_decoder(tb, c, model, max_seq, B, tp, rank, args)
    if tp > 1:
        from torchburn_b200.tp import init_tensor_parallel

        init_tensor_parallel(dec, dist, device)
    prefill_kv(torch, dec, c, device, CONTEXT, B, tp, rank)
    stream = torch.cuda.ExternalStream(lib_stream(tb, dec), device=device)
    L = tb.lib()

    def barrier():
        if tp > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    # ---- device-resident: greedy generate loop, K steps enqueued back to back, R regions ----
    with ClockSampler(local) as clocks:
        regions = timed_steps(torch, dist, tb, dec, device, tp, B, CONTEXT, K, W, R)
    ms = float(np.median(regions))
    ms_per_step = ms / K
    value = B * 1e3 / ms_per_step

    # ---- end to end through the C ABI with host buffers ----
    logits_host = torch.empty(B, c["vocab_size"], dtype=torch.float32).pin_memory()
    toks = np.full(B, 5, np.int64)
    offs = np.full(B, CONTEXT, np.int64)

    def e2e_step(i):
        offs[:] = CONTEXT + (i % 32)
        tb._lib.check(L.tb_decoder_step_batch(dec.handle, toks.ctypes.data, offs.ctypes.data, B, logits_host.data_ptr()))
        toks[:] = int(logits_host[0, :1024].argmax())  # the host consumes the result

    for i in range(W):
        e2e_step(i)
    barrier()
    e2e_regions, wall_regions = [], []
    for _ in range(R):
        e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e2.record(stream)
        for i in range(K):
            e2e_step(i)
        e3.record(stream)
        barrier()
        wall_regions.append((time.perf_counter() - t0) * 1e3)
        e2e_ms = max(e2.elapsed_time(e3), 0.0)
        if tp > 1:
            t = torch.tensor([e2e_ms], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_ms = float(t.item())
        e2e_regions.append(e2e_ms)
    e2e_ms, wall_ms = float(np.median(e2e_regions)), float(np.median(wall_regions))
    e2e_value = B * 1e3 / (e2e_ms / K)
    launches_per_step = dec.launches_per_step()

    def finish():
        if tp > 1:
            dist.barrier()
            dist.destroy_process_group()

    if args.quick:
        dec.close()
        if rank == 0:
            _RESULT_LINE.append(json.dumps({"value": value, "ms_per_step": ms_per_step, "e2e": e2e_value, "n_gpus": tp, "batch": B, "model": args.model,
                              "launches_per_step": launches_per_step,
                              "weights_only_frac_of_measured": step_weight_bytes(c) / tp / (ms_per_step * 1e-3) / 1e9 / measured_peak()[0],
                              "weights_plus_kv_frac_of_measured": (step_weight_bytes(c) + B * kv_bytes_per_seq(c, CONTEXT)) / tp / (ms_per_step * 1e-3) / 1e9 / measured_peak()[0]}))
        finish()
        return

    # ---- outside the headline region (every rank takes part where the model is sharded) ----
    # the other form of the batch-1 step (persistent step kernel <-> chain of single kernels), same workload
    other_form = None
    if B == 1 and tp == 1 and not args.quick and not args.no_graph:
        import argparse as _ap

        is_step_kernel = dec.launches_per_step() == 2
        alt_args = _ap.Namespace(**dict(vars(args), chain=is_step_kernel, step_kernel=not is_step_kernel))
        alt = make_decoder(tb, c, model, max_seq, B, tp, rank, alt_args)
        prefill_kv(torch, alt, c, device, CONTEXT, B, tp, rank)
        alt_ms = float(np.median(timed_steps(torch, dist, tb, alt, device, tp, B, CONTEXT, K, W, 3))) / K
        other_form = {"form": "chain of single kernels (--chain)" if is_step_kernel else "persistent step kernel (--step-kernel)",
                      "tokens_per_s": B * 1e3 / alt_ms, "ms_per_step": alt_ms, "launches_per_step": alt.launches_per_step()}
        alt.close()
    # correctness of the sharded path at this N
    tp_check = tp_correctness_check(torch, dist, tb, c, device, tp, rank, args) if tp > 1 else None
    # the other batch sizes of the workload configuration (8 and 32), and the small batches 2 and 4: tokens/s
    batch_sweep = None
    verify = None
    prefill = None
    if args.model == "llama8b" and B == 1 and args.batch_sweep:
        dec.close()
        dec = None
        big = make_decoder(tb, c, model, CONTEXT + 192, 32, tp, rank, args)
        if tp > 1:
            init_tensor_parallel(big, dist, device)
        prefill_kv(torch, big, c, device, CONTEXT, 32, tp, rank)
        batch_sweep = {"1": {"tokens_per_s": value, "ms_per_step": ms_per_step}}
        for bb in (2, 4, 8, 32):
            r_ms = timed_steps(torch, dist, tb, big, device, tp, bb, CONTEXT, 8, 3, 3)
            m = float(np.median(r_ms)) / 8
            batch_sweep[str(bb)] = {"tokens_per_s": bb * 1e3 / m, "ms_per_step": m,
                                    "weights_plus_kv_frac": (step_weight_bytes(c) + bb * kv_bytes_per_seq(c, CONTEXT)) / tp / (m * 1e-3) / 1e9 / measured_peak()[0]}
        # speculative verify (src/llm/decoder.rs:565-581): K + 1 = 5 positions of one sequence as ONE batched step
        # against 5 single-position steps, through the host API (token ids in, 5 rows of logits out)
        if tp == 1:
            vt = [11, 22, 33, 44, 55]

            def wall(fn, reps=5):
                fn()
                torch.cuda.synchronize(device)
                best = None
                for _ in range(reps):
                    t0 = time.perf_counter()
                    fn()
                    dt = (time.perf_counter() - t0) * 1e3
                    best = dt if best is None else min(best, dt)
                return best

            ms_b = wall(lambda: big.verify_tokens(CONTEXT, vt))
            ms_s = wall(lambda: [big.step(t, CONTEXT + i) for i, t in enumerate(vt)])
            verify = {"positions": len(vt), "ms_one_batched_step": ms_b, "ms_single_steps": ms_s,
                      "note": "best of 5 wall-clock calls of verify_tokens / of 5 step() calls, context 4096"}
            # prompt processing (src/llm/decoder.rs:431-447): 128 prompt positions ending at the context length,
            # 32 per batched step on this decoder against one step per token
            pt = [int(t) for t in np.random.default_rng(5).integers(0, c["vocab_size"], 128)]
            ms_pb = wall(lambda: big.prefill_tokens(pt, CONTEXT - 128), reps=3)
            ms_ps = wall(lambda: [big.step(t, CONTEXT - 128 + i) for i, t in enumerate(pt)], reps=2)
            prefill = {"tokens": len(pt), "ms_batched": ms_pb, "ms_token_by_token": ms_ps, "tokens_per_s_batched": len(pt) * 1e3 / ms_pb,
                       "note": "wall clock, positions 3968..4095 of one sequence; decoder built for 32 rows"}
        big.close()
    if rank != 0:
        if dec is not None:
            dec.close()
        finish()
        return

    # ---- rank 0: roofline of the dominant kernel, config-1 GEMV, config 2, config 3, CPU baseline ----
    peak, peak_kind = measured_peak()
    alg, sec, _ = time_dominant_kernel(torch, tb, c, layers, device, tp)
    achieved = alg / sec / 1e9
    roofline = {"bound": "hbm", "kernel": "w4_stream_kernel<EPI=SwiGLU> (gate/up GEMV + SwiGLU, 2 x [14336 x 4096] INT4 g32)", "achieved": achieved,
                "peak": peak, "peak_kind": f"of {peak_kind}", "unit": "GB/s", "frac": achieved / peak,
                "frac_of_nominal_8TBs": achieved / NOMINAL_HBM_GBS, "traffic": DOMINANT_KERNEL_DRAM_TRAFFIC,
                "algorithmic_bytes_per_launch": alg, "us_per_launch": sec * 1e6,
                "traffic_note": "dram bytes read+written per launch from the ncu capture of the same kernel and shape (tp=1)"}
    if tp > 1:
        roofline["traffic"] = None
    c1_alg, c1_sec, c1_sec4 = time_c1_gemv(torch, tb, device)
    wb = step_weight_bytes(c) / tp
    kvb = kv_bytes_per_seq(c, CONTEXT) / tp
    step_s = ms_per_step * 1e-3
    line = {
        "metric": "decode_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": tp, "steps": K, "warmup": W,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": workload_config(c, B, tp),
        "repeats": {"regions": R, "steps_per_region": K, "ms_per_step_median": ms_per_step, "ms_per_step_min": min(regions) / K,
                    "ms_per_step_max": max(regions) / K},
        "roofline": roofline,
        "step_roofline": {
            "weight_bytes_per_step_per_gpu": wb, "kv_bytes_per_step_per_gpu": kvb * B,
            "weights_only_frac": wb / step_s / 1e9 / peak, "weights_plus_kv_frac": (wb + kvb * B) / step_s / 1e9 / peak,
            "peak_kind": f"of {peak_kind}", "launches_per_step": launches_per_step},
        "step_form": "persistent step kernel" if launches_per_step == 2 else "chain of single kernels", "other_step_form": other_form,
        "verify_tokens": verify, "prefill_tokens": prefill,
        "gemv_config1": {"shape": "4096x4096 group 32, M=1", "algorithmic_bytes": c1_alg, "us_per_launch": c1_sec * 1e6,
                         "achieved_gbs": c1_alg / c1_sec / 1e9, "frac_of_measured": c1_alg / c1_sec / 1e9 / peak,
                         "frac_of_nominal_8TBs": c1_alg / c1_sec / 1e9 / NOMINAL_HBM_GBS,
                         "note": "64 rotating weight copies (672 MB), one CUDA graph of 64 launches replayed",
                         "independent_launches_4_streams": {"us_per_launch": c1_sec4 * 1e6, "achieved_gbs": c1_alg / c1_sec4 / 1e9,
                                                            "frac_of_measured": c1_alg / c1_sec4 / 1e9 / peak,
                                                            "note": "the same 64 launches as graph nodes on 4 forked streams: independent GEMVs overlap; a throughput, not the latency of one call"}},
        "gemm_config2": (time_c2_gemm(torch, tb, c, layers, device) if tp == 1 else None),
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": 16 * B, "d2h_bytes_per_step": 4 * B * c["vocab_size"],
                "ms_per_step": e2e_ms / K, "wall_ms_per_step": wall_ms / K, "regions": R},
        "gpu_launches": (launches_per_step + 1) * K,
        "clocks": clocks.summary(),
    }
    if tp_check is not None:
        line["tp_check"] = tp_check
    if batch_sweep is not None:
        line["batch_sweep"] = batch_sweep
    if dec is not None:
        dec.close()
    del model, layers
    torch.cuda.empty_cache()
    if tp == 1 and args.model == "llama8b" and args.config3:
        line["qwen05b_config3"] = time_config3(torch, tb, device, args)
    if args.cpu_baseline:
        line["cpu_baseline"] = {k: v for k, v in cpu_full_step(c, CONTEXT, 8, 2).items() if not k.startswith("ms_per_step")}
    _RESULT_LINE.append(json.dumps(line))
    finish()


def time_config3(torch, tb, device, args):
    """Workload configuration 3: Qwen2.5-0.5B-shaped decode, batch 1, fp32 KV pre-filled to 1024."""
    c, ctx = dict(QWEN05B), 1024
    model = build_model(torch, tb, c, device, 1, 0, seed=77)
    dec = make_decoder(tb, c, model, ctx + 256, 1, 1, 0, args)
    prefill_kv(torch, dec, c, device, ctx, 1, 1, 0)
    r_ms = timed_steps(torch, None, tb, dec, device, 1, 1, ctx, 64, 8, 3)
    m = float(np.median(r_ms)) / 64
    peak, kind = measured_peak()
    wb = step_weight_bytes(c)
    out = {"workload": "qwen2.5-0.5b-shaped INT4 (group 32) decode, batch 1, fp32 KV at context 1024",
           "tokens_per_s": 1e3 / m, "ms_per_step": m, "launches_per_step": dec.launches_per_step(),
           "weights_only_frac": wb / (m * 1e-3) / 1e9 / peak, "peak_kind": f"of {kind}",
           "weight_streaming_roofline_tokens_per_s": peak * 1e9 / wb}
    dec.close()
    return out


def lib_stream(tb, dec):
    return tb.lib().tb_decoder_stream(dec.handle)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--model", default="llama8b", choices=["llama8b", "qwen05b", "llama70b"],
                    help="qwen05b: workload configuration 3; llama70b: configuration 5 (8 GPUs, --batch 16); both with --quick")
    ap.add_argument("--repeats", type=int, default=5, help="timed regions of --steps steps each; the median is reported")
    ap.add_argument("--no-batch-sweep", dest="batch_sweep", action="store_false", help="skip the batch 2 / 4 / 8 / 32 measurements")
    ap.add_argument("--no-config3", dest="config3", action="store_false", help="skip the Qwen2.5-0.5B-shaped measurement")
    ap.add_argument("--nccl-only", action="store_true", help="tensor parallel: plain ncclAllReduce instead of the fused kernel")
    ap.add_argument("--no-cpu-baseline", dest="cpu_baseline", action="store_false")
    ap.add_argument("--no-pdl", action="store_true", help="plain stream order between kernels (A/B of programmatic dependent launch)")
    ap.add_argument("--no-graph", action="store_true", help="direct launches instead of CUDA-graph replay")
    ap.add_argument("--chain", action="store_true", help="batch-1 steps as a chain of single kernels (the default on one GPU)")
    ap.add_argument("--step-kernel", dest="step_kernel", action="store_true", help="batch-1 steps as the one persistent step kernel (the default with tensor parallelism)")
    ap.add_argument("--quick", action="store_true", help="skip the kernel-alone and CPU measurements")
    args = ap.parse_args()
    # Exactly ONE line reaches stdout: the JSON.  Whatever libraries print there meanwhile (NCCL's version
    # banner, for one) goes to stderr: file descriptor 1 points at stderr until the end.
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    try:
        if args.impl == "reference":
            run_reference(args)
        else:
            run_gpu(args)
    finally:
        sys.stdout.flush()
        os.dup2(real_stdout, 1)
        os.close(real_stdout)
    if _RESULT_LINE:
        print(_RESULT_LINE[-1], flush=True)


if __name__ == "__main__":
    main()
