"""Tensor-parallel host logic on CPU: two gloo ranks shard a model with the library's
tb_shard_* helpers, run the sharded step (oracle arithmetic, gloo all-reduce after o_proj
and down, gloo all-gather of the logits) and must reproduce the unsharded oracle."""
import os
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def _rank_main(rank, world, port, q):
    sys.path.insert(0, HERE)
    sys.path.insert(0, os.path.dirname(HERE))
    import torch
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import torchburn_b200 as tb
        from helpers import max_rel_err, synth_model
        from oracle import oracle as o
        from tp_helpers import ShardedOracleDecoder, shard_model

        o.set_threads(2)
        cfg = dict(vocab_size=512, hidden_size=256, intermediate_size=512, num_layers=2, num_heads=8,
                   num_kv_heads=4, head_dim=32, group_size=32, max_seq_len=32, rms_norm_eps=1e-6, rope_theta=5e5)
        embed, layers, fnorm, lm_w, lm_s = synth_model(cfg, 3, o.quantize_int4_grouped, qkv_bias=True)
        layers_r, lw_r, ls_r = shard_model(tb, cfg, layers, lm_w, lm_s, rank, world)

        def allreduce(v):
            t = torch.from_numpy(np.ascontiguousarray(v, dtype=np.float32))
            dist.all_reduce(t)
            return t.numpy()

        def allgather(v):
            t = torch.from_numpy(np.ascontiguousarray(v, dtype=np.float32))
            outs = [torch.empty_like(t) for _ in range(world)]
            dist.all_gather(outs, t)
            return torch.cat(outs).numpy()

        dec = ShardedOracleDecoder(o, cfg, embed, layers_r, fnorm, lw_r, ls_r, world, allreduce, allgather)
        ref = o.OracleDecoder(cfg, embed, layers, fnorm, lm_w, lm_s)
        worst = 0.0
        for off, tok in enumerate([3, 500, 17, 17, 255, 9]):
            worst = max(worst, max_rel_err(dec.step(tok, off), ref.step(tok, off)))
        # KV shards are the rank's kv heads of the unsharded cache
        k_ref, v_ref = ref.kv_cache(1)
        nkv_l = cfg["num_kv_heads"] // world
        kv_ok = (max_rel_err(dec.k[1], k_ref[rank * nkv_l:(rank + 1) * nkv_l]) < 1e-5 and
                 max_rel_err(dec.v[1], v_ref[rank * nkv_l:(rank + 1) * nkv_l]) < 1e-5)
        q.put((rank, worst, kv_ok))
    finally:
        dist.destroy_process_group()


def test_two_rank_sharded_step_matches_unsharded_oracle():
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 400)
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    for rank, worst, kv_ok in results:
        assert worst < 1e-5, (rank, worst)  # only the fp32 summation order differs
        assert kv_ok
