"""tb_attention_decode_static: attention for callers that cannot allocate device memory
(all memory pre-assigned, a graph capture in progress, no room for an allocation stall).
It must give what tb_attention_decode gives with caller-provided scratch - on two calls in a
row, the second with another shape, because both share one built-in block that still holds
the first call's leftovers.  Collected last on purpose (file name)."""
import numpy as np
import pytest

from helpers import max_rel_err

pytestmark = pytest.mark.gpu
TOL = 1e-4  # the per-stage tolerance of the other GPU tests


def _case(torch, tb, oracle, nh, nkv, hd, max_seq, offsets, seed):
    rng = np.random.default_rng(seed)
    b = len(offsets)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    qkv = dev(rng.standard_normal((b, (nh + 2 * nkv) * hd)).astype(np.float32))
    kc = (rng.standard_normal((b, nkv, max_seq, hd)) * 0.5).astype(np.float32)
    vc = rng.standard_normal((b, nkv, max_seq, hd)).astype(np.float32)
    cos_t, sin_t = oracle.rope_tables(max_seq, hd, 1e6)
    d_cos, d_sin = dev(cos_t), dev(sin_t)
    d_off = dev(np.asarray(offsets, np.int32))
    L = tb.lib()
    # existing entry point, scratch from the caller
    k1, v1 = dev(kc), dev(vc)
    scratch = torch.zeros(L.tb_attention_scratch_bytes(b, nh, nkv, hd, max_seq), dtype=torch.uint8, device="cuda")
    want = torch.empty(b, nh * hd, device="cuda")
    assert L.tb_attention_decode(qkv.data_ptr(), k1.data_ptr(), v1.data_ptr(), d_cos.data_ptr(), d_sin.data_ptr(),
                                 d_off.data_ptr(), want.data_ptr(), scratch.data_ptr(), b, nh, nkv, hd, max_seq, None) == 0
    # new entry point: same inputs and outputs, no scratch argument
    k2, v2 = dev(kc), dev(vc)
    got = torch.full((b, nh * hd), float("nan"), device="cuda")
    rc = L.tb_attention_decode_static(qkv.data_ptr(), k2.data_ptr(), v2.data_ptr(), d_cos.data_ptr(), d_sin.data_ptr(),
                                      d_off.data_ptr(), got.data_ptr(), b, nh, nkv, hd, max_seq, None)
    assert rc == 0, tb.last_error()
    torch.cuda.synchronize()
    assert max_rel_err(got.cpu().numpy(), want.cpu().numpy()) < TOL
    assert torch.equal(k1, k2) and torch.equal(v1, v2)  # same cache append
    # ... and directly against the CPU oracle: rotate q and k, append, attend to [0, offset]
    g, gk, gv = got.cpu().numpy(), k2.cpu().numpy(), v2.cpu().numpy()
    qkv_h = qkv.cpu().numpy()
    for s_, off in enumerate(offsets):
        q = qkv_h[s_, :nh * hd].reshape(nh, hd).copy()
        k = qkv_h[s_, nh * hd:(nh + nkv) * hd].reshape(nkv, hd).copy()
        v = qkv_h[s_, (nh + nkv) * hd:].reshape(nkv, hd)
        for h in range(nh):
            q[h] = oracle.rope_apply_head(q[h], cos_t[off], sin_t[off])
        for h in range(nkv):
            k[h] = oracle.rope_apply_head(k[h], cos_t[off], sin_t[off])
        ek, ev = kc[s_].copy(), vc[s_].copy()
        ek[:, off], ev[:, off] = k, v
        assert np.array_equal(gk[s_], ek) and np.array_equal(gv[s_], ev)
        assert max_rel_err(g[s_].reshape(nh, hd), oracle.attention_decode(q, ek, ev, off + 1)) < TOL
    assert L.tb_device_fault_flag() == 0  # no bounded wait of the kernel ran out


def test_static_scratch_attention_matches_regular_entry_point(oracle):
    import torch

    if not torch.cuda.is_available():
        pytest.fail("no CUDA device")
    import torchburn_b200 as tb

    L = tb.lib()
    assert L.tb_attention_static_scratch_bytes() == 8 << 20
    _case(torch, tb, oracle, 32, 8, 128, 2048, [2047], seed=1)        # first call on this device (set-up)
    _case(torch, tb, oracle, 14, 2, 64, 1024, [5, 1023, 300], seed=2)  # second call, other shape, reused block
    _case(torch, tb, oracle, 32, 8, 128, 2048, [100], seed=3)
    # a shape beyond the built-in block is refused with a clear message, nothing is launched
    assert L.tb_attention_scratch_bytes(16, 64, 8, 128, 32768) > L.tb_attention_static_scratch_bytes()
    rc = L.tb_attention_decode_static(None, None, None, None, None, None, None, 16, 64, 8, 128, 32768, None)
    assert rc == 9 and "built-in block" in tb.last_error()
