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
from .speculative import BatchedDecoder, SpeculativeDecoder
from .quantization import (
    QuantizedLinear,
    dequantize_int4_grouped_v2,
    fused_attention_step,
    fused_swiglu_mlp,
    fused_swiglu_mlp_batched,
    fused_transformer_layer_step,
    quantize_weight_int4_grouped,
    quantize_weight_int4_grouped_v2,
    w4a32_grouped_linear,
    w4a32_grouped_linear_v2,
)

__all__ = [
    "TorchBurnB200Error", "abi_version", "device_report", "lib", "last_error",
    "B200QwenDecoder", "create_b200_qwen_decoder", "SpeculativeDecoder", "BatchedDecoder", "QuantizedLinear", "fused_attention_step",
    "fused_swiglu_mlp", "fused_swiglu_mlp_batched", "fused_transformer_layer_step", "quantize_weight_int4_grouped",
    "w4a32_grouped_linear", "quantize_weight_int4_grouped_v2", "dequantize_int4_grouped_v2", "w4a32_grouped_linear_v2",
]
