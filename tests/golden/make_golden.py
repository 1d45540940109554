"""Generate golden fixtures by running the REFERENCE's own Python code.

Run once, where the torchburn source tree is available:

    python tests/golden/make_golden.py /path/to/torchburn

The reference's Python package cannot be imported normally without its compiled
Rust extension (``torchburn/__init__.py`` imports ``_torchburn``), but the two
modules that define this path's arithmetic are pure torch:

* ``python/torchburn/quantization.py``  -> ``quantize_weight_int4_grouped``
  (the production quantizer, lines 53-118);
* ``python/torchburn/llm/model.py``     -> ``UniversalTransformer`` with
  ``StaticKVCache`` (RMSNorm, RoPE, GQA attention, SwiGLU MLP, lm_head).

They are loaded from the reference tree with an empty stand-in for the native
module, so every number written here is produced by reference code, not by a
restatement.  The decoder fixtures run the reference model in fp32 with each
linear's weight replaced by dequant(quantize(weight)) - the definition of the
W4A32 linear (tests/test_parity.py:51-64) - one token at a time through the
static KV cache, which is what ``RustQwenDecoder.step_internal`` computes.

Outputs (committed): quantizer_golden.npz, layout_v2_golden.npz, decoder_qwen_tiny_g32.npz,
decoder_llama_tiny_g64.npz.
"""
from __future__ import annotations

import importlib
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def load_reference(ref_root: str):
    pkg_dir = os.path.join(ref_root, "python", "torchburn")
    pkg = types.ModuleType("torchburn")
    pkg.__path__ = [pkg_dir]
    sys.modules["torchburn"] = pkg
    native = types.ModuleType("torchburn._torchburn")  # empty stand-in; nothing here calls it
    sys.modules["torchburn._torchburn"] = native
    pkg._torchburn = native
    llm = types.ModuleType("torchburn.llm")
    llm.__path__ = [os.path.join(pkg_dir, "llm")]
    sys.modules["torchburn.llm"] = llm
    quant = importlib.import_module("torchburn.quantization")
    config = importlib.import_module("torchburn.llm.config")
    model = importlib.import_module("torchburn.llm.model")
    return quant, config, model


def dequant(packed: torch.Tensor, scales: torch.Tensor, group_size: int) -> torch.Tensor:
    # same definition as the reference's tests/test_parity.py:51-64
    n, pc = packed.shape
    lo = (packed & 0x0F).to(torch.int8)
    hi = ((packed >> 4) & 0x0F).to(torch.int8)
    q = torch.stack([lo, hi], dim=2).reshape(n, pc * 2) - 8
    return q.float() * scales.repeat_interleave(group_size, dim=1)


def quantizer_cases(quant):
    out = {}
    g = torch.Generator().manual_seed(1234)
    cases = {
        "normal_g32": (torch.randn(24, 256, generator=g) * 0.02, 32),
        "normal_g64": (torch.randn(24, 256, generator=g) * 0.02, 64),
        "wide_g32": (torch.randn(8, 128, generator=g) * 3.0, 32),
        "g128": (torch.randn(4, 256, generator=g), 128),
    }
    # exact ties: w/scale lands on x.5 -> torch.round is half-to-even
    t = torch.zeros(4, 64)
    t[:, 0] = 7.0  # scale = 1.0
    t[0, 1:9] = torch.tensor([0.5, 1.5, 2.5, 3.5, -0.5, -1.5, -2.5, -6.5])
    t[1, 1:5] = torch.tensor([6.5, -7.5, 4.5, -4.5])
    t[2, 0] = -7.0  # negative extreme -> scale from |w|
    t[2, 1] = 7.0
    t[3, :] = 0.0  # all-zero group -> scale clamps to 1e-8, codes 0 -> nibble 8
    t[3, 32:] = 1e-9  # below the clamp
    cases["ties_zero_g32"] = (t, 32)
    # lower clamp: value that would round below -8 cannot occur (scale=max/7) but +max -> 7, -max -> -7
    big = torch.tensor([[1e30, -1e30] + [0.0] * 30, [3.4e38, 1.0] + [1e-30] * 30])
    cases["huge_g32"] = (big, 32)
    for name, (w, gs) in cases.items():
        packed, scales = quant.quantize_weight_int4_grouped(w, group_size=gs)
        out[f"{name}__w"] = w.numpy()
        out[f"{name}__g"] = np.int32(gs)
        out[f"{name}__packed"] = packed.numpy()
        out[f"{name}__scales"] = scales.numpy()
    # chunked branch (N > chunk_size): must equal the single-shot branch
    w = torch.randn(40, 64, generator=g) * 0.02
    packed, scales = quant.quantize_weight_int4_grouped(w, group_size=32, chunk_size=16)
    out["chunked_g32__w"] = w.numpy()
    out["chunked_g32__g"] = np.int32(32)
    out["chunked_g32__packed"] = packed.numpy()
    out["chunked_g32__scales"] = scales.numpy()
    return out


def decoder_case(quant, config, model, *, seed, group_size, cfg_kwargs, tokens, max_seq_len, tied):
    torch.manual_seed(seed)
    cfg = config.ModelConfig(**cfg_kwargs)
    m = model.UniversalTransformer(cfg)  # fp32, init N(0, 0.02) (model.py:509-515)
    m.fuse_qkv()
    m.eval()
    out = {}
    g = torch.Generator().manual_seed(seed + 1)
    with torch.no_grad():
        # non-trivial norm weights and (if present) qkv bias so those paths are exercised
        for norm in [m.norm] + [l.input_layernorm for l in m.layers] + [l.post_attention_layernorm for l in m.layers]:
            norm.weight.copy_(1.0 + 0.1 * torch.randn(norm.weight.shape, generator=g))

        def q_replace(linear, key):
            packed, scales = quant.quantize_weight_int4_grouped(linear.weight.data, group_size=group_size)
            linear.weight.data.copy_(dequant(packed, scales, group_size))
            out[f"{key}_w"] = packed.numpy()
            out[f"{key}_s"] = scales.numpy()

        for i, layer in enumerate(m.layers):
            att = layer.self_attn
            if att.qkv_proj.bias is not None:
                att.qkv_proj.bias.copy_(0.05 * torch.randn(att.qkv_proj.bias.shape, generator=g))
                out[f"l{i}_qkv_b"] = att.qkv_proj.bias.detach().numpy().copy()
            q_replace(att.qkv_proj, f"l{i}_qkv")
            q_replace(att.o_proj, f"l{i}_o")
            q_replace(layer.mlp.gate_proj, f"l{i}_gate")
            q_replace(layer.mlp.up_proj, f"l{i}_up")
            q_replace(layer.mlp.down_proj, f"l{i}_down")
            out[f"l{i}_input_norm_w"] = layer.input_layernorm.weight.detach().numpy().copy()
            out[f"l{i}_post_norm_w"] = layer.post_attention_layernorm.weight.detach().numpy().copy()
        out["embed_tokens"] = m.embed_tokens.weight.detach().numpy().copy()
        if tied:
            # tied embeddings: lm_head is a separately quantized copy of the embedding
            # (python/torchburn/llm/loader.py:502-512)
            m.lm_head = torch.nn.Linear(cfg.hidden_size, cfg.vocab_size, bias=False)
            m.lm_head.weight.data.copy_(m.embed_tokens.weight.data)
        q_replace(m.lm_head, "lm_head")
        out["final_norm_w"] = m.norm.weight.detach().numpy().copy()

        caches = m.create_static_kv_caches(max_batch_size=1, max_seq_len=max_seq_len)
        logits = []
        for off, tok in enumerate(tokens):
            lg, _ = m(torch.tensor([[tok]]), caches, offset=off)
            logits.append(lg[0, 0].numpy().copy())
        out["logits"] = np.stack(logits)
        out["k_cache_l0"] = caches[0].k[0, :, : len(tokens)].numpy().copy()
        out["v_cache_l0"] = caches[0].v[0, :, : len(tokens)].numpy().copy()
    out["tokens"] = np.asarray(tokens, dtype=np.int64)
    out["cfg"] = np.asarray(
        [cfg.vocab_size, cfg.hidden_size, cfg.intermediate_size, cfg.num_hidden_layers,
         cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, group_size, max_seq_len],
        dtype=np.int64)
    out["cfg_f"] = np.asarray([cfg.rms_norm_eps, cfg.rope_theta], dtype=np.float64)
    return out


def v2_cases(quant):
    """The reference's own v2 quantizer and dequantizer (quantization.py:121-169)."""
    g = torch.Generator().manual_seed(77)
    w = torch.randn(6, 256, generator=g) * 0.05
    w[0, :64] *= 1e-4   # a group whose scale is a binary16 subnormal
    w[1, 64:128] *= 40  # a large scale
    packed, scales = quant.quantize_weight_int4_grouped(w, group_size=64)
    blocked = quant.quantize_weight_int4_grouped_v2(w, group_size=64)
    deq = quant.dequantize_int4_grouped_v2(blocked, 64)
    vals = torch.tensor([0.0, -0.0, 1.0, -1.0, 0.5, 2.0, 65504.0, -3.75, 1234.5, 1e-4, 6.0e-5, 6.1e-8, 1e6, -1e6,
                         0.1, 3.1415927, 2.0 ** -14, 2.0 ** -24, 2.0 ** -25, 65519.0, 65520.0, 1.00048828125])
    half_bits = vals.half().view(torch.int16).numpy().astype(np.uint16)
    return {"w": w.numpy(), "packed": packed.numpy(), "scales": scales.numpy(), "blocked": blocked.numpy(),
            "dequant": deq.numpy(), "f16_inputs": vals.numpy(), "f16_bits": half_bits,
            "f16_back": vals.half().float().numpy()}


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/torchburn")
    ref_root = sys.argv[1]
    quant, config, model = load_reference(ref_root)
    np.savez_compressed(os.path.join(HERE, "quantizer_golden.npz"), **quantizer_cases(quant))
    np.savez_compressed(os.path.join(HERE, "layout_v2_golden.npz"), **v2_cases(quant))
    qwen = decoder_case(
        quant, config, model, seed=11, group_size=32,
        cfg_kwargs=dict(vocab_size=320, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                        num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=64,
                        rms_norm_eps=1e-6, rope_theta=1000000.0, qkv_bias=True, tie_word_embeddings=True),
        tokens=[5, 17, 300, 0, 42, 255, 17, 9], max_seq_len=16, tied=True)
    np.savez_compressed(os.path.join(HERE, "decoder_qwen_tiny_g32.npz"), **qwen)
    llama = decoder_case(
        quant, config, model, seed=23, group_size=64,
        cfg_kwargs=dict(vocab_size=256, hidden_size=256, intermediate_size=448, num_hidden_layers=2,
                        num_attention_heads=8, num_key_value_heads=2, head_dim=32, max_position_embeddings=64,
                        rms_norm_eps=1e-5, rope_theta=500000.0, qkv_bias=False, tie_word_embeddings=False,
                        architectures=["LlamaForCausalLM"]),
        tokens=[1, 200, 33, 34, 35, 7, 7, 128, 64, 2], max_seq_len=12, tied=False)
    np.savez_compressed(os.path.join(HERE, "decoder_llama_tiny_g64.npz"), **llama)
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")


if __name__ == "__main__":
    main()
