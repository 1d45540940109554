"""Tensor-parallel decoder on 2, 4 and 8 GPUs (each case is skipped on a box with fewer GPUs): one
process per GPU, NCCL for the plumbing.  Every form of the exchange must reproduce the oracle:
the persistent step kernel with the exchange inside it (batch 1), the chain of kernels with the
low-latency push exchange, the pull-form exchange (large partials), and plain ncclAllReduce.
The model has 8 kv heads, so 8 ranks hold one kv head each and the o_proj slice is 128 wide."""
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _rank_main(rank, world, port, q, variant):
    sys.path.insert(0, HERE)
    sys.path.insert(0, os.path.dirname(HERE))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import torch
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import torchburn_b200 as tb
        from helpers import max_rel_err, synth_model
        from oracle import oracle as o
        from torchburn_b200.tp import init_tensor_parallel
        from tp_helpers import shard_model

        nccl_only = variant == "nccl"
        cfg = dict(vocab_size=1024, hidden_size=1024, intermediate_size=2048, num_layers=3, num_heads=16,
                   num_kv_heads=8, head_dim=64, group_size=32, max_seq_len=64, rms_norm_eps=1e-6, rope_theta=5e5)
        B = 3
        if variant in ("wide", "pull", "widechain"):
            # hidden 2048: the projections that consume the residual stream take the persistent kernel of the
            # chain and the low-latency exchange also writes their pre-weighted input and its sums of squares;
            # "pull": 9 sequences x 2048 floats exceed the low-latency exchange, the pull form takes over
            cfg.update(vocab_size=512, hidden_size=2048, intermediate_size=4096, num_layers=2, num_heads=16,
                       num_kv_heads=8, head_dim=128, tied=False)
            B = 9 if variant == "pull" else 3
        embed, layers, fnorm, lm_w, lm_s = synth_model(cfg, 3, o.quantize_int4_grouped, qkv_bias=True)
        layers_r, lw_r, ls_r = shard_model(tb, cfg, layers, lm_w, lm_s, rank, world)
        order = ["input_norm_w", "qkv_w", "qkv_s", "o_w", "o_s", "post_norm_w", "gate_w", "gate_s", "up_w", "up_s",
                 "down_w", "down_s", "qkv_b"]
        dec = tb.B200QwenDecoder(embed, [[lw[k] for k in order] for lw in layers_r], fnorm, lw_r, ls_r,
                                 cfg["num_layers"], cfg["hidden_size"], cfg["intermediate_size"], cfg["num_heads"],
                                 cfg["num_kv_heads"], cfg["head_dim"], cfg["group_size"], cfg["rms_norm_eps"],
                                 cfg["max_seq_len"], cfg["rope_theta"], max_batch=B, tp_size=world, tp_rank=rank,
                                 vocab_size=cfg["vocab_size"], nccl_only=nccl_only, fused_step=variant not in ("chain", "widechain"))
        init_tensor_parallel(dec, dist, torch.device("cuda", rank), fused=not nccl_only)
        launches = None
        ref = o.OracleDecoder(cfg, embed, layers, fnorm, lm_w, lm_s)
        worst = 0.0
        toks = [3, 500, 17, 17, 255, 9, 1000 % cfg["vocab_size"], 1]
        for off, tok in enumerate(toks):
            worst = max(worst, max_rel_err(dec.step(tok, off), ref.step(tok, off)))
            launches = dec.launches_per_step()
        # greedy decode on the device (the step kernel + argmax, no host round trip between steps)
        nxt = dec.decode_and_sample(5, len(toks), temperature=0.0)
        greedy_ok = nxt == o.argmax(ref.step(5, len(toks)))
        # batched step: B sequences at once against B oracles (the chain of kernels with an exchange kernel)
        refs = [o.OracleDecoder(cfg, embed, layers, fnorm, lm_w, lm_s) for _ in range(B)]
        dec.reset_kv_cache()
        for off in range(3):
            tk = [(7 * off + 11 * b + 1) % cfg["vocab_size"] for b in range(B)]
            got = dec.step_batch(tk, [off] * B)
            for b in range(B):
                worst = max(worst, max_rel_err(got[b], refs[b].step(tk[b], off)))
        # prompt processing and verify on the sharded decoder: B positions of sequence 0 per batched step
        # (attention rows share the rank's part of sequence 0's cache), the last slab ragged
        ref2 = o.OracleDecoder(cfg, embed, layers, fnorm, lm_w, lm_s)
        V = cfg["vocab_size"]
        dec.reset_kv_cache()
        ptoks = [(13 * i + 5) % V for i in range(2 * B + 1)]
        assert dec.prefill_tokens(ptoks, 0) == len(ptoks)
        want = [ref2.step(t, i) for i, t in enumerate(ptoks)]
        worst = max(worst, max_rel_err(dec.get_logits().reshape(-1)[:V], want[-1]))
        vt = [(29 * i + 2) % V for i in range(B + 1)]
        rows = dec.verify_tokens(len(ptoks), vt)
        for i, t in enumerate(vt):
            worst = max(worst, max_rel_err(rows[i], ref2.step(t, len(ptoks) + i)))
        fault = tb.lib().tb_device_fault_flag()
        q.put((rank, worst, fault, launches, greedy_ok))
        dec.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,variant", [(2, "step"), (2, "chain"), (2, "nccl"), (2, "wide"), (2, "widechain"), (2, "pull"),
                                           (4, "step"), (4, "chain"), (8, "step"), (8, "chain")])
def test_tp_decoder_matches_oracle(world, variant):
    import torch

    if not torch.cuda.is_available():
        pytest.fail("no CUDA device")
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29900 + (os.getpid() % 40) + 50 * ["step", "chain", "nccl", "wide", "pull", "widechain"].index(variant) + world
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, q, variant)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=420) for _ in procs]
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    for rank, worst, fault, launches, greedy_ok in results:
        assert worst < 1e-3, (rank, worst)
        assert fault == 0
        assert greedy_ok
        if variant == "step":
            assert launches == 2, launches   # the embedding kernel + the one persistent step kernel
        elif variant in ("chain", "widechain"):
            assert launches > 2


def _rank_peer_missing(rank, world, port, q, fused):
    sys.path.insert(0, HERE)
    sys.path.insert(0, os.path.dirname(HERE))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import time

    import torch
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import torchburn_b200 as tb
        from helpers import synth_model
        from oracle import oracle as o
        from torchburn_b200.tp import init_tensor_parallel
        from tp_helpers import shard_model

        cfg = dict(vocab_size=1024, hidden_size=1024, intermediate_size=2048, num_layers=2, num_heads=16,
                   num_kv_heads=8, head_dim=64, group_size=32, max_seq_len=64, rms_norm_eps=1e-6, rope_theta=5e5)
        embed, layers, fnorm, lm_w, lm_s = synth_model(cfg, 3, o.quantize_int4_grouped, qkv_bias=True)
        layers_r, lw_r, ls_r = shard_model(tb, cfg, layers, lm_w, lm_s, rank, world)
        order = ["input_norm_w", "qkv_w", "qkv_s", "o_w", "o_s", "post_norm_w", "gate_w", "gate_s", "up_w", "up_s",
                 "down_w", "down_s", "qkv_b"]
        dec = tb.B200QwenDecoder(embed, [[lw[k] for k in order] for lw in layers_r], fnorm, lw_r, ls_r,
                                 cfg["num_layers"], cfg["hidden_size"], cfg["intermediate_size"], cfg["num_heads"],
                                 cfg["num_kv_heads"], cfg["head_dim"], cfg["group_size"], cfg["rms_norm_eps"],
                                 cfg["max_seq_len"], cfg["rope_theta"], tp_size=world, tp_rank=rank,
                                 vocab_size=cfg["vocab_size"], fused_step=fused)
        init_tensor_parallel(dec, dist, torch.device("cuda", rank))
        dec.step(3, 0)                      # a normal step of both ranks
        dist.barrier()
        status, lost, seconds = None, None, None
        if rank == 0:
            tb.lib().tb_debug_step_wait_limit(1_500_000_000)   # under a second at 1.9 GHz
            t0 = time.perf_counter()
            try:
                dec.step(5, 1)              # rank 1 never runs this step: its partial rows never arrive
                status = 0
            except tb.TorchBurnB200Error as e:
                status = e.status
            seconds = time.perf_counter() - t0
            lost = dec.is_device_lost()
            try:
                dec.step(6, 2)              # a lost decoder refuses further work
                after = 0
            except tb.TorchBurnB200Error as e:
                after = e.status
            q.put((rank, status, lost, seconds, after))
        else:
            time.sleep(8)                   # stays away from the step; launches nothing meanwhile
            q.put((rank, None, dec.is_device_lost(), None, None))
        dist.barrier()                      # both ranks are alive: no kernel of either is waiting for the other
        dec.close()
    finally:
        dist.destroy_process_group()


def test_tp_peer_that_never_arrives_is_reported_as_timeout(fused=True):
    """Failure detection without a fault: rank 1 stays away from a step (on the host, between steps, with
    nothing in flight); the bounded waits of rank 0's step kernel run out, the kernel ends, the call
    returns TB_ERR_TIMEOUT within seconds and the decoder is marked lost.  Plain peer stores and
    loads only (no multimem), NVLS off in NCCL.  (Only the persistent step kernel is tested this way:
    the chain of kernels gathers the logits with ncclAllGather, whose wait for a missing peer is NCCL's
    own and is not bounded by this library.)"""
    import torch

    if not torch.cuda.is_available():
        pytest.fail("no CUDA device")
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29960 + (os.getpid() % 15) + (20 if fused else 0)
    procs = [ctx.Process(target=_rank_peer_missing, args=(r, 2, port, q, fused)) for r in range(2)]
    for p in procs:
        p.start()
    results = dict((r[0], r) for r in (q.get(timeout=300) for _ in procs))
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    _, status, lost, seconds, after = results[0]
    assert status == 7, status              # TB_ERR_TIMEOUT
    assert lost
    assert seconds < 10
    assert after == 8                       # TB_ERR_DEVICE_LOST
    assert not results[1][2]                # the rank that stayed away is unaffected
