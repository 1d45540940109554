"""Host-side mirror of python/torchburn/quantization.py for the INT4 W4A32 path.

Same names, arguments, shapes and error behaviour; the arithmetic runs in the
sm_100a kernels of libtorchburn_b200.so.  torch is used only to hold device
memory and to hand over pointers and the current stream.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import numpy as np
import torch
import torch.nn as nn

from . import _lib
from ._lib import TB_DEVICE, TB_HOST, check, lib


def _stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _require_cuda() -> torch.device:
    if not torch.cuda.is_available():
        raise _lib.TorchBurnB200Error(5, "no CUDA device: torchburn_b200 has no CPU fallback")
    return torch.device("cuda", torch.cuda.current_device())


def quantize_weight_int4_grouped(
    weight: torch.Tensor, group_size: int = 64, chunk_size: int = 1024
) -> Tuple[torch.Tensor, torch.Tensor]:
    """quantize_weight_int4_grouped of python/torchburn/quantization.py:53-118 on the GPU.

    Returns (packed [N, K/2] uint8, scales [N, K/group_size] float32) on the
    device of ``weight``; bit-identical to the reference's torch-CPU arithmetic
    (fp32 division, round half to even).  ``chunk_size`` is accepted for
    signature compatibility (the reference chunks rows only to bound host RAM).
    """
    if weight.ndim != 2:
        raise ValueError(
            f"Expected 2D weight matrix for quantize_weight_int4_grouped, got {weight.ndim}D tensor of shape {tuple(weight.shape)}")
    N, K = weight.shape
    if K % group_size != 0:
        raise ValueError(
            f"Weight dimension K={K} must be divisible by group_size={group_size}. "
            f"Consider padding the weight tensor along dim 1 to a multiple of {group_size}.")
    orig_device = weight.device
    dev = orig_device if orig_device.type == "cuda" else _require_cuda()
    w = weight.detach().to(device=dev, dtype=torch.float32).contiguous()
    packed = torch.empty((N, (K + 1) // 2), dtype=torch.uint8, device=dev)
    scales = torch.empty((N, K // group_size), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        check(lib().tb_quantize_weight_int4_grouped(w.data_ptr(), N, K, group_size, packed.data_ptr(),
                                                    scales.data_ptr(), _stream_ptr(dev)))
    return packed.to(orig_device), scales.to(orig_device)


def _flattened_rows(shape) -> int:
    n = 1
    for d in shape[:-1]:
        n *= int(d)
    return n


def w4a32_grouped_linear(
    x: torch.Tensor, w_packed: torch.Tensor, scales: torch.Tensor,
    bias: Optional[torch.Tensor] = None, group_size: int = 64,
) -> torch.Tensor:
    """w4a32_grouped_linear of python/torchburn/quantization.py:245-269.

    x (..., K) -> (..., N).  Tensors may live on the CPU (they are staged to
    the GPU for the call, as the reference copies nothing and computes on the
    host) or on a CUDA device (no copies; runs on torch's current stream).
    """
    x_orig_shape = x.shape
    K = x_orig_shape[-1]
    on_cpu = x.device.type != "cuda"
    dev = _require_cuda() if on_cpu else x.device
    x_2d = x.reshape(-1, K).contiguous().float().to(dev)
    w = w_packed.contiguous().to(dev)
    s = scales.contiguous().float().to(dev)
    b = bias.contiguous().float().to(dev) if bias is not None else None
    if w.dtype != torch.uint8 or w.ndim != 2:
        raise _lib.TorchBurnB200Error(3, "TB_UNSUPPORTED: w4a32_grouped_linear: w_packed must be a 2D uint8 tensor")
    N = w.shape[0]
    if w.shape[1] != (K + 1) // 2:
        raise _lib.TorchBurnB200Error(2, f"TB_UNSUPPORTED: w4a32_grouped_linear: packed weight shape {tuple(w.shape)} does not match K={K}")
    ng = (K + group_size - 1) // group_size
    if tuple(s.shape) != (N, ng):
        raise _lib.TorchBurnB200Error(2, f"TB_UNSUPPORTED: w4a32_grouped_linear: scales shape {tuple(s.shape)} != ({N}, {ng})")
    if b is not None and b.numel() != N:
        raise _lib.TorchBurnB200Error(2, f"TB_UNSUPPORTED: w4a32_grouped_linear: bias has {b.numel()} elements, expected {N}")
    M = x_2d.shape[0]
    out = torch.empty((M, N), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        check(lib().tb_gemm_w4a32_grouped(x_2d.data_ptr(), w.data_ptr(), s.data_ptr(),
                                          b.data_ptr() if b is not None else None, out.data_ptr(),
                                          M, N, K, group_size, _stream_ptr(dev)))
    out = out.reshape(list(x_orig_shape[:-1]) + [N])
    return out.cpu() if on_cpu else out


# ---- the interleaved "v2" layout (34-byte blocks, binary16 scales, group 64) -----------------
def _v2_unpack(blocked: torch.Tensor):
    """blocked (N, G*34) uint8 -> (packed (N, G*32) uint8, scales (N, G) float32) through the C ABI."""
    if blocked.dtype != torch.uint8 or blocked.ndim != 2 or blocked.shape[1] % 34 != 0:
        raise _lib.TorchBurnB200Error(2, "TB_UNSUPPORTED: v2 weights must be a (N, groups*34) uint8 tensor")
    b = np.ascontiguousarray(blocked.detach().cpu().numpy())
    n, ng = b.shape[0], b.shape[1] // 34
    packed = np.empty((n, ng * 32), np.uint8)
    scales = np.empty((n, ng), np.float32)
    check(lib().tb_unpack_v2_to_v1(b.ctypes.data, n, ng * 64, packed.ctypes.data, scales.ctypes.data))
    return torch.from_numpy(packed), torch.from_numpy(scales)


def quantize_weight_int4_grouped_v2(weight: torch.Tensor, group_size: int = 64, chunk_size: int = 1024) -> torch.Tensor:
    """quantize_weight_int4_grouped_v2 of python/torchburn/quantization.py:121-151: the same codes
    and scales as the v1 quantizer, stored as one 34-byte block per 64-element group."""
    if group_size != 64:
        raise ValueError("the v2 layout is defined for group_size 64")
    N, K = weight.shape
    if K % group_size != 0:
        raise ValueError(f"K={K} must be divisible by group_size={group_size}")
    packed, scales = quantize_weight_int4_grouped(weight, group_size=group_size, chunk_size=chunk_size)
    p = np.ascontiguousarray(packed.cpu().numpy())
    sc = np.ascontiguousarray(scales.cpu().numpy(), dtype=np.float32)
    out = np.empty((N, (K // 64) * 34), np.uint8)
    check(lib().tb_pack_v1_to_v2(p.ctypes.data, sc.ctypes.data, N, K, out.ctypes.data))
    return torch.from_numpy(out)


def dequantize_int4_grouped_v2(blocked: torch.Tensor, group_size: int = 64) -> torch.Tensor:
    """dequantize_int4_grouped_v2 of python/torchburn/quantization.py:154-169: the f32 matrix (N, K)."""
    packed, scales = _v2_unpack(blocked)
    lo = (packed & 0x0F).to(torch.int8)
    hi = ((packed >> 4) & 0x0F).to(torch.int8)
    q = torch.stack([lo, hi], dim=2).reshape(packed.shape[0], -1) - 8
    return q.float() * scales.repeat_interleave(64, dim=1)


def w4a32_grouped_linear_v2(x: torch.Tensor, blocked: torch.Tensor, bias: Optional[torch.Tensor] = None,
                            group_size: int = 64) -> torch.Tensor:
    """w4a32_grouped_linear_v2 of python/torchburn/quantization.py:172-190: x (..., K) @ dequant(blocked)^T
    + bias.  The blocks are unpacked (binary16 scales widened to fp32) and the v1 kernels run."""
    if group_size != 64:
        raise ValueError("the v2 layout is defined for group_size 64")
    packed, scales = _v2_unpack(blocked)
    return w4a32_grouped_linear(x, packed, scales, bias, group_size=64)


class QuantizedLinear(nn.Module):
    """Drop-in for the reference's QuantizedLinear (python/torchburn/quantization.py:756-869), bits=4.

    Same constructor, buffers (``qweight`` [N, K/2] uint8, ``scales`` [N, K/G]
    float32), ``bias`` parameter and ``from_float``.  ``bits=8`` (per-channel
    int8) is outside the INT4 decode path and raises.
    """

    qweight: torch.Tensor
    scales: torch.Tensor
    bias: Optional[torch.Tensor]

    def __init__(self, in_features: int, out_features: int, bias: bool = False, bits: int = 4,
                 group_size: int = 64, backend: str = "b200"):
        super().__init__()
        if bits == 8:
            raise NotImplementedError("torchburn_b200 covers the INT4 (bits=4) decode path only")
        if bits != 4:
            raise ValueError(f"Supported quantization bits are 8 and 4, got {bits}")
        self.in_features = in_features
        self.out_features = out_features
        self.bits = bits
        self.group_size = group_size
        self.backend = backend
        self.register_buffer("qweight", torch.zeros((out_features, (in_features + 1) // 2), dtype=torch.uint8))
        num_groups = (in_features + group_size - 1) // group_size
        self.register_buffer("scales", torch.ones((out_features, num_groups), dtype=torch.float32))
        if bias:
            self.bias = nn.Parameter(torch.zeros(out_features, dtype=torch.float32))
        else:
            self.register_parameter("bias", None)

    @classmethod
    def from_float(cls, linear: nn.Linear, bits: int = 4, group_size: int = 64, backend: str = "b200") -> "QuantizedLinear":
        has_bias = linear.bias is not None
        ql = cls(linear.in_features, linear.out_features, bias=has_bias, bits=bits, group_size=group_size, backend=backend)
        with torch.no_grad():
            qw, sc = quantize_weight_int4_grouped(linear.weight, group_size=group_size)
            ql.qweight.copy_(qw)
            ql.scales.copy_(sc)
            if has_bias:
                ql.bias.copy_(linear.bias.float())
        return ql.to(linear.weight.device)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return w4a32_grouped_linear(x, self.qweight, self.scales, self.bias, group_size=self.group_size)

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}, "
                f"bits={self.bits}, group_size={self.group_size}, backend={self.backend}")


class _LinearHandle:
    """tb_linear over a module's (or raw tensors') weights; uploads once."""

    def __init__(self, qweight, scales, bias, group_size):
        qweight = qweight.contiguous()
        scales = scales.contiguous().float()
        bias = bias.detach().contiguous().float() if bias is not None else None
        n, k = qweight.shape[0], qweight.shape[1] * 2
        space = TB_DEVICE if qweight.device.type == "cuda" else TB_HOST
        if space == TB_DEVICE:
            scales = scales.to(qweight.device)
            bias = bias.to(qweight.device) if bias is not None else None
        h = C.c_void_p()
        check(lib().tb_linear_create(C.byref(h), qweight.data_ptr(), scales.data_ptr(),
                                     bias.data_ptr() if bias is not None else None, n, k, group_size, space))
        self.h = h
        self.n, self.k = n, k

    def __del__(self):
        if getattr(self, "h", None):
            lib().tb_linear_destroy(self.h)
            self.h = None


def _handle_of(m) -> _LinearHandle:
    key = (m.qweight.data_ptr(), m.qweight._version, m.scales.data_ptr(), m.scales._version)
    cached = getattr(m, "_tb_handle", None)
    if cached is None or cached[0] != key:
        cached = (key, _LinearHandle(m.qweight, m.scales, m.bias, m.group_size))
        object.__setattr__(m, "_tb_handle", cached)
    return cached[1]


def _io(x: torch.Tensor):
    xf = x.contiguous().float()
    if xf.device.type == "cuda":
        return xf, TB_DEVICE, xf.device
    return xf, TB_HOST, _require_cuda()


def fused_swiglu_mlp(x: torch.Tensor, gate_proj, up_proj, down_proj) -> torch.Tensor:
    """fused_swiglu_mlp of python/torchburn/quantization.py:299-405: down(silu(gate(x)) * up(x))
    for modules carrying qweight/scales/bias/group_size; x (..., hidden) -> (..., hidden_out)."""
    xf, space, dev = _io(x)
    hidden = xf.shape[-1]
    m = _flattened_rows(xf.shape)
    g, u, d = _handle_of(gate_proj), _handle_of(up_proj), _handle_of(down_proj)
    out = torch.empty(list(xf.shape[:-1]) + [d.n], dtype=torch.float32, device=xf.device)
    with torch.cuda.device(dev):
        check(lib().tb_fused_swiglu_mlp(g.h, u.h, d.h, xf.data_ptr(), m, out.data_ptr(), space, _stream_ptr(dev)))
    assert hidden == g.k
    return out


def fused_swiglu_mlp_batched(x, gate_proj, up_proj, down_proj) -> torch.Tensor:
    """fused_swiglu_mlp_batched (src/quantization/fused_ops.rs:1267-1319): same call for m > 1."""
    return fused_swiglu_mlp(x, gate_proj, up_proj, down_proj)


def fused_attention_step(x, qkv_proj, o_proj, k_cache, v_cache, cos, sin, offset: int, num_heads: int,
                         num_kv_heads: int, head_dim: int) -> torch.Tensor:
    """fused_attention_step of python/torchburn/quantization.py:408-485.

    x (1, 1, hidden); k_cache / v_cache [1, Hkv, max_seq_len, d] CUDA tensors,
    updated in place at ``offset``; cos / sin hold this position's row
    (any shape with head_dim trailing elements).  Returns (1, 1, hidden).
    """
    if k_cache.device.type != "cuda" or v_cache.device.type != "cuda":
        raise _lib.TorchBurnB200Error(1, "fused_attention_step: the KV caches must be CUDA tensors (they are updated in place)")
    if not (k_cache.is_contiguous() and v_cache.is_contiguous()) or k_cache.dtype != torch.float32:
        raise _lib.TorchBurnB200Error(3, "TB_UNSUPPORTED: fused_attention_step: KV caches must be contiguous float32")
    dev = k_cache.device
    max_seq_len = k_cache.shape[2]
    on_cuda = x.device.type == "cuda"
    xf = x.reshape(-1).contiguous().float()
    cs = cos.reshape(-1)[-head_dim:].contiguous().float().to(xf.device)
    sn = sin.reshape(-1)[-head_dim:].contiguous().float().to(xf.device)
    q, o = _handle_of(qkv_proj), _handle_of(o_proj)
    out = torch.empty(o.n, dtype=torch.float32, device=xf.device)
    with torch.cuda.device(dev):
        check(lib().tb_fused_attention_step(q.h, o.h, xf.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                                            cs.data_ptr(), sn.data_ptr(), int(offset), num_heads, num_kv_heads,
                                            head_dim, max_seq_len, out.data_ptr(),
                                            TB_DEVICE if on_cuda else TB_HOST, _stream_ptr(dev)))
    return out.reshape(1, 1, -1)


def fused_transformer_layer_step(x, input_norm_w, qkv_w, qkv_s, qkv_b, o_w, o_s, o_b, post_norm_w, gate_w, gate_s, gate_b,
                                 up_w, up_s, up_b, down_w, down_s, down_b, k_cache, v_cache, cos, sin, offset: int,
                                 num_heads: int, num_kv_heads: int, head_dim: int, group_size: int, eps: float = 1e-6) -> None:
    """fused_transformer_layer_step_w4a32 (src/ffi/quantization_ffi.rs:406-438): one decoder layer
    for one token IN PLACE on ``x`` (a contiguous float32 tensor whose last dimension is the hidden
    size, on the host or on the GPU); same positional arguments as the reference.  Weights and the
    KV caches [1, Hkv, max_seq_len, d] are CUDA tensors; the caches are updated at ``offset``."""
    if k_cache.device.type != "cuda" or v_cache.device.type != "cuda":
        raise _lib.TorchBurnB200Error(1, "fused_transformer_layer_step: the KV caches must be CUDA tensors (they are updated in place)")
    if not (x.is_contiguous() and x.dtype == torch.float32):
        raise _lib.TorchBurnB200Error(3, "TB_UNSUPPORTED: fused_transformer_layer_step: x must be contiguous float32 (it is updated in place)")
    dev = k_cache.device
    w = _lib.LayerStepWeights()
    keep = []
    for name, t, dt in (("input_norm_w", input_norm_w, torch.float32), ("qkv_w", qkv_w, torch.uint8), ("qkv_s", qkv_s, torch.float32),
                        ("qkv_b", qkv_b, torch.float32), ("o_w", o_w, torch.uint8), ("o_s", o_s, torch.float32), ("o_b", o_b, torch.float32),
                        ("post_norm_w", post_norm_w, torch.float32), ("gate_w", gate_w, torch.uint8), ("gate_s", gate_s, torch.float32),
                        ("gate_b", gate_b, torch.float32), ("up_w", up_w, torch.uint8), ("up_s", up_s, torch.float32),
                        ("up_b", up_b, torch.float32), ("down_w", down_w, torch.uint8), ("down_s", down_s, torch.float32),
                        ("down_b", down_b, torch.float32)):
        if t is None:
            setattr(w, name, None)
            continue
        td = t.detach().to(device=dev, dtype=dt).contiguous()
        keep.append(td)
        setattr(w, name, td.data_ptr())
    hidden, inter = x.shape[-1], gate_w.shape[0]
    on_cuda = x.device.type == "cuda"
    cs = cos.reshape(-1)[-head_dim:].contiguous().float().to(x.device)
    sn = sin.reshape(-1)[-head_dim:].contiguous().float().to(x.device)
    with torch.cuda.device(dev):
        check(lib().tb_fused_transformer_layer_step(x.data_ptr(), C.byref(w), k_cache.data_ptr(), v_cache.data_ptr(), cs.data_ptr(),
                                                    sn.data_ptr(), int(offset), hidden, inter, num_heads, num_kv_heads, head_dim,
                                                    k_cache.shape[2], group_size, float(eps), TB_DEVICE if on_cuda else TB_HOST,
                                                    _stream_ptr(dev)))
