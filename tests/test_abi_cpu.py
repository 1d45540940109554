"""CPU-side checks of the product library: it builds, loads, exports every
symbol the header declares, validates arguments without a GPU, and its host-only
shard helpers slice bytes correctly."""
import ctypes as C
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def tb():
    from torchburn_b200 import build as tb_build

    tb_build.build()
    import torchburn_b200 as tb

    tb.lib()
    return tb


def test_header_symbols_all_exported(tb):
    hdr = open(os.path.join(ROOT, "include", "torchburn_b200.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    declared = set(re.findall(r"\b(tb_[a-z0-9_]+)\s*\(", hdr)) - {"tb_allgather_fn"}
    assert len(declared) >= 40
    from torchburn_b200 import _lib

    missing = [s for s in sorted(declared) if not hasattr(tb.lib(), s)]
    assert not missing, f"not exported: {missing}"
    assert declared == set(_lib.SIGNATURES), "ctypes table and header disagree"
    assert tb.abi_version() == 1


def test_rust_sys_crate_declares_exactly_the_header(tb):
    """rust/torchburn-b200-sys/src/lib.rs (sources only: no Rust toolchain here) must declare every
    function of the header, no other, with the same number of arguments, and the same struct fields."""
    hdr = open(os.path.join(ROOT, "include", "torchburn_b200.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    rs = open(os.path.join(ROOT, "rust", "torchburn-b200-sys", "src", "lib.rs")).read()
    rs_code = re.sub(r"//.*", "", rs)

    def argc(args):
        args = " ".join(args.split())
        return 0 if args in ("", "void") else args.count(",") + 1

    c_fns = {name: argc(args) for name, args in re.findall(r"\b(tb_[a-z0-9_]+)\s*\(([^;{]*?)\)\s*;", hdr, flags=re.S)
             if name != "tb_allgather_fn"}
    r_fns = {name: argc(args) for name, args in re.findall(r"pub fn (tb_[a-z0-9_]+)\(([^;]*?)\)(?:\s*->\s*[^;]+)?;", rs_code, flags=re.S)}
    assert set(c_fns) == set(r_fns), (sorted(set(c_fns) - set(r_fns)), sorted(set(r_fns) - set(c_fns)))
    assert c_fns == r_fns, {k: (c_fns[k], r_fns[k]) for k in c_fns if c_fns[k] != r_fns[k]}
    # struct fields, in order
    for name in ("tb_model_config", "tb_layer_weights", "tb_layer_step_weights"):
        c_body = re.search(r"typedef struct %s \{(.*?)\} %s;" % (name, name), hdr, flags=re.S).group(1)
        c_fields = re.findall(r"(\w+)\s*;", c_body)
        r_body = re.search(r"pub struct %s \{(.*?)\n\}" % name, rs_code, flags=re.S).group(1)
        r_fields = re.findall(r"pub (\w+)\s*:", r_body)
        assert c_fields == r_fields, name
    # status codes
    for code, val in re.findall(r"\b(TB_(?:OK|ERR_\w+))\s*=\s*(\d+)", hdr):
        assert re.search(r"pub const %s: tb_status = %s;" % (code, val), rs_code), code
    assert rs.startswith("// UNCOMPILED")


def test_no_oracle_in_product():
    # the product package must not import, load or link the oracle
    for dirpath, _, files in os.walk(os.path.join(ROOT, "torchburn_b200")):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".cpp", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "tb_oracle" not in text and "from oracle" not in text and "import oracle" not in text, f


def test_argument_errors_without_gpu(tb):
    L = tb.lib()
    assert L.tb_gemv_w4a32_grouped(None, None, None, None, None, 4, 64, 32, None) == 1  # TB_ERR_ARG
    assert "null" in tb.last_error()
    buf = (C.c_float * 64)()
    wb = (C.c_uint8 * 128)()
    assert L.tb_gemv_w4a32_grouped(buf, wb, buf, None, buf, 4, 64, 48, None) == 2  # bad group size
    assert "TB_UNSUPPORTED" in tb.last_error()
    assert L.tb_gemv_w4a32_grouped(buf, wb, buf, None, buf, 4, 80, 32, None) == 2  # k % g != 0
    h = C.c_void_p()
    assert L.tb_linear_create(C.byref(h), wb, buf, None, 0, 64, 32, 0) == 2
    assert L.tb_decoder_create(C.byref(h), None, None, None, None, None, None, 0) == 1
    assert L.tb_decoder_kv_len(None) == 0
    assert L.tb_decoder_is_device_lost(None) == 0


def test_decoder_create_validates_dimensions(tb):
    # src/llm/decoder.rs:214-233 -> ValueError before anything touches the device
    from torchburn_b200 import B200QwenDecoder

    z = np.zeros((8, 8), np.float32)
    lay = [[z] * 12]
    with pytest.raises(ValueError, match="divisible by 4"):
        B200QwenDecoder(z, lay, z, z, z, 1, 66, 64, 2, 2, 32, 32)
    with pytest.raises(ValueError, match="divisible by group_size"):
        B200QwenDecoder(z, lay, z, z, z, 1, 96, 64, 2, 2, 32, 64)
    with pytest.raises(ValueError, match="must be even"):
        B200QwenDecoder(z, lay, z, z, z, 1, 64, 64, 2, 2, 31, 32)
    with pytest.raises(ValueError, match="divisible by num_kv_heads"):
        B200QwenDecoder(z, lay, z, z, z, 1, 64, 64, 3, 2, 32, 32)


def test_shard_helpers_roundtrip(tb):
    L = tb.lib()
    rng = np.random.default_rng(0)
    n, k, g = 48, 256, 32
    packed = rng.integers(0, 256, (n, k // 2), dtype=np.uint8)
    scales = rng.random((n, k // g), dtype=np.float32)
    # rows: concatenating the shards gives the original back
    parts_p, parts_s = [], []
    for r in range(4):
        po = np.empty((n // 4, k // 2), np.uint8)
        so = np.empty((n // 4, k // g), np.float32)
        assert L.tb_shard_rows(packed.ctypes.data, scales.ctypes.data, n, k, g, r * (n // 4), n // 4, po.ctypes.data, so.ctypes.data) == 0
        parts_p.append(po); parts_s.append(so)
    assert np.array_equal(np.concatenate(parts_p), packed) and np.array_equal(np.concatenate(parts_s), scales)
    # cols
    parts_p, parts_s = [], []
    for r in range(4):
        po = np.empty((n, k // 8), np.uint8)
        so = np.empty((n, k // g // 4), np.float32)
        assert L.tb_shard_cols(packed.ctypes.data, scales.ctypes.data, n, k, g, r * (k // 4), k // 4, po.ctypes.data, so.ctypes.data) == 0
        parts_p.append(po); parts_s.append(so)
    assert np.array_equal(np.concatenate(parts_p, axis=1), packed) and np.array_equal(np.concatenate(parts_s, axis=1), scales)
    po = np.empty((n, 8), np.uint8); so = np.empty((n, 1), np.float32)
    assert L.tb_shard_cols(packed.ctypes.data, scales.ctypes.data, n, k, g, 16, 16, po.ctypes.data, so.ctypes.data) == 2
    # qkv: whole heads per rank, [q | k | v] order kept
    nh, nkv, hd, H = 8, 4, 4, 64
    rows = (nh + 2 * nkv) * hd
    qp = rng.integers(0, 256, (rows, H // 2), dtype=np.uint8)
    qs = rng.random((rows, H // g), dtype=np.float32)
    qb = rng.random(rows, dtype=np.float32)
    for rank in range(2):
        lr = rows // 2
        po = np.empty((lr, H // 2), np.uint8); so = np.empty((lr, H // g), np.float32); bo = np.empty(lr, np.float32)
        assert L.tb_shard_qkv(qp.ctypes.data, qs.ctypes.data, qb.ctypes.data, H, nh, nkv, hd, g, rank, 2, po.ctypes.data, so.ctypes.data, bo.ctypes.data) == 0
        ql, kl = nh * hd // 2, nkv * hd // 2
        idx = np.concatenate([np.arange(rank * ql, (rank + 1) * ql), nh * hd + np.arange(rank * kl, (rank + 1) * kl),
                              (nh + nkv) * hd + np.arange(rank * kl, (rank + 1) * kl)])
        assert np.array_equal(po, qp[idx]) and np.array_equal(so, qs[idx]) and np.array_equal(bo, qb[idx])
