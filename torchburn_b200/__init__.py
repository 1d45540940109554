"""torchburn_b200 - the quantized decode hot path of torchburn on NVIDIA B200.

Host-side mirror of the reference's Python surface for this path
(python/torchburn/quantization.py): ``quantize_weight_int4_grouped``,
``w4a32_grouped_linear``, ``QuantizedLinear``, the fused MLP / attention steps and
the decoder object, all executing hand-written sm_100a CUDA kernels through the
C ABI in ``include/torchburn_b200.h``.  There is no CPU fallback: importing the
package without the built library raises.
"""
from ._lib import TorchBurnB200Error, abi_version, device_report, lib, last_error
from .decoder import B200QwenDecoder, create_b200_qwen_decoder
from .quantization import (
    QuantizedLinear,
    fused_attention_step,
    fused_swiglu_mlp,
    fused_swiglu_mlp_batched,
    quantize_weight_int4_grouped,
    w4a32_grouped_linear,
)

__all__ = [
    "TorchBurnB200Error", "abi_version", "device_report", "lib", "last_error",
    "B200QwenDecoder", "create_b200_qwen_decoder", "QuantizedLinear", "fused_attention_step",
    "fused_swiglu_mlp", "fused_swiglu_mlp_batched", "quantize_weight_int4_grouped",
    "w4a32_grouped_linear",
]
