"""Checkpoint -> INT4 cache -> decoder, the load side of the hot path.

Mirrors the parts of python/torchburn/llm/loader.py that stand in front of the decoder:

* ``quantize_checkpoint`` - ``_stream_quantize_safetensors`` (:376-537): walks a Llama / Qwen style
  checkpoint layer by layer, fuses q/k/v into one ``qkv_proj`` (rows concatenated in that order,
  biases too), quantizes every linear with ``quantize_weight_int4_grouped`` (on the GPU) and, for
  tied embeddings, quantizes a separate copy of the embedding as ``lm_head``.  The result uses the
  reference model's ``state_dict`` names, so the two caches are interchangeable.
* ``save_cache`` / ``load_cache`` - the safetensors disk cache ``torchburn_int4_g64.safetensors``
  (:150-173, :520-535) and its v2 twin ``torchburn_int4_g64_v2.safetensors`` whose ``qweight``
  tensors hold 34-byte blocks and which carries no ``scales`` (:542-560, :563-606); a v2 file is
  migrated to v1 tensors in memory when it is loaded.
* ``decoder_from_state_dict`` - ``create_rust_qwen_decoder`` (python/torchburn/quantization.py:
  560-660) for ``B200QwenDecoder``.
"""
from __future__ import annotations

import os
from typing import Callable, Dict, Mapping, Optional, Sequence

import numpy as np
import torch

from ._lib import check, lib
from .quantization import quantize_weight_int4_grouped

# The reference's literal file names: "g64" is part of the name whatever the group size of the
# file's contents (python/torchburn/llm/loader.py:92-95, 150-153), so that a cache written by
# either side is found by the other; the group size is read from the shape of the scales.
CACHE_V1 = "torchburn_int4_g64.safetensors"
CACHE_V2 = "torchburn_int4_g64_v2.safetensors"

# Names under which the pieces of a layer appear in checkpoints (loader.py:236-330).
_PREFIXES = ("model.", "transformer.", "")
_ALIASES = {
    "gate_proj": ("gate_proj", "w1"),
    "up_proj": ("up_proj", "w3"),
    "down_proj": ("down_proj", "w2"),
}


def _find(tensors: Mapping[str, torch.Tensor], candidates: Sequence[str]) -> Optional[torch.Tensor]:
    for c in candidates:
        if c in tensors:
            return tensors[c]
    return None


def _layer_names(idx: int, rest: str):
    return [f"{p}layers.{idx}.{rest}" for p in _PREFIXES] + [f"transformer.h.{idx}.{rest}"]


def _require(tensors, candidates, what: str) -> torch.Tensor:
    t = _find(tensors, candidates)
    if t is None:
        raise KeyError(f"Required tensor '{what}' is missing from the checkpoint; "
                       "the model architecture is not compatible with TorchBurn's decoder")  # loader.py:366-372
    return t


def quantize_checkpoint(tensors: Mapping[str, torch.Tensor], num_layers: int, group_size: int = 64,
                        tie_word_embeddings: bool = False, qkv_bias: bool = False,
                        quantize: Optional[Callable] = None) -> Dict[str, torch.Tensor]:
    """Float checkpoint tensors -> the quantized state dict (CPU tensors, reference key names)."""
    q = quantize or (lambda w: quantize_weight_int4_grouped(w, group_size=group_size))

    def qlin(w: torch.Tensor):
        pw, ps = q(w.float())
        return pw.cpu().contiguous(), ps.cpu().float().contiguous()

    sd: Dict[str, torch.Tensor] = {}
    emb = _require(tensors, [f"{p}embed_tokens.weight" for p in _PREFIXES] + ["transformer.wte.weight"], "embed_tokens")
    sd["embed_tokens.weight"] = emb.float().cpu().contiguous()
    sd["norm.weight"] = _require(tensors, [f"{p}norm.weight" for p in _PREFIXES] + ["transformer.ln_f.weight"],
                                 "norm").float().cpu().contiguous()
    for i in range(num_layers):
        pre = f"layers.{i}."
        sd[pre + "input_layernorm.weight"] = _require(
            tensors, _layer_names(i, "input_layernorm.weight"), pre + "input_layernorm.weight").float().cpu().contiguous()
        qkv = [_require(tensors, _layer_names(i, f"self_attn.{n}_proj.weight"), pre + f"self_attn.{n}_proj.weight")
               for n in ("q", "k", "v")]
        sd[pre + "self_attn.qkv_proj.qweight"], sd[pre + "self_attn.qkv_proj.scales"] = qlin(
            torch.cat([t.float() for t in qkv], dim=0))  # loader.py:408-423
        if qkv_bias:
            bs = [_find(tensors, _layer_names(i, f"self_attn.{n}_proj.bias")) for n in ("q", "k", "v")]
            if all(b is not None for b in bs):
                sd[pre + "self_attn.qkv_proj.bias"] = torch.cat([b.float() for b in bs], dim=0).cpu().contiguous()
        sd[pre + "self_attn.o_proj.qweight"], sd[pre + "self_attn.o_proj.scales"] = qlin(
            _require(tensors, _layer_names(i, "self_attn.o_proj.weight"), pre + "self_attn.o_proj.weight"))
        post = _find(tensors, _layer_names(i, "post_attention_layernorm.weight"))
        if post is not None:
            sd[pre + "post_attention_layernorm.weight"] = post.float().cpu().contiguous()
        for proj, names in _ALIASES.items():
            cands = [c for n in names for c in _layer_names(i, f"mlp.{n}.weight")]
            sd[pre + f"mlp.{proj}.qweight"], sd[pre + f"mlp.{proj}.scales"] = qlin(
                _require(tensors, cands, pre + f"mlp.{proj}.weight"))
    if tie_word_embeddings:
        # the lm_head of a tied model is a separately quantized copy of the embedding (loader.py:500-509)
        sd["lm_head.qweight"], sd["lm_head.scales"] = qlin(sd["embed_tokens.weight"])
    else:
        sd["lm_head.qweight"], sd["lm_head.scales"] = qlin(_require(tensors, ["lm_head.weight", "model.lm_head.weight"], "lm_head"))
    return sd


def migrate_state_dict_to_v2(sd: Mapping[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """v1 tensors -> the v2 cache form (migrate_cache_to_v2, loader.py:563-606): every (qweight, scales)
    pair of group size 64 becomes one tensor of 34-byte blocks; the scales tensors are dropped."""
    out: Dict[str, torch.Tensor] = {}
    for key, t in sd.items():
        if key.endswith(".qweight") and key.replace(".qweight", ".scales") in sd:
            sc = sd[key.replace(".qweight", ".scales")]
            n, k = t.shape[0], t.shape[1] * 2
            if sc.shape != (n, k // 64):
                raise ValueError(f"{key}: the v2 layout needs group size 64 (scales {tuple(sc.shape)})")
            p = np.ascontiguousarray(t.cpu().numpy())
            s = np.ascontiguousarray(sc.cpu().numpy(), dtype=np.float32)
            blocks = np.empty((n, (k // 64) * 34), np.uint8)
            check(lib().tb_pack_v1_to_v2(p.ctypes.data, s.ctypes.data, n, k, blocks.ctypes.data))
            out[key] = torch.from_numpy(blocks)
        elif key.endswith(".scales") and key.replace(".scales", ".qweight") in sd:
            continue
        else:
            out[key] = t.contiguous()
    return out


def migrate_v2_state_dict(sd: Mapping[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """_migrate_v2_state_dict (loader.py:542-560): blocks -> qweight (N, K/2) + scales (N, K/64) f32."""
    out: Dict[str, torch.Tensor] = {}
    for key, t in sd.items():
        if key.endswith(".qweight") and t.ndim == 2 and t.shape[1] % 34 == 0 and key.replace(".qweight", ".scales") not in sd:
            b = np.ascontiguousarray(t.cpu().numpy())
            n, ng = b.shape[0], b.shape[1] // 34
            packed = np.empty((n, ng * 32), np.uint8)
            scales = np.empty((n, ng), np.float32)
            check(lib().tb_unpack_v2_to_v1(b.ctypes.data, n, ng * 64, packed.ctypes.data, scales.ctypes.data))
            out[key] = torch.from_numpy(packed)
            out[key.replace(".qweight", ".scales")] = torch.from_numpy(scales)
        else:
            out[key] = t
    return out


def save_cache(sd: Mapping[str, torch.Tensor], path: str) -> str:
    import safetensors.torch

    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    safetensors.torch.save_file({k: v.contiguous() for k, v in sd.items()}, path)
    return path


def find_cache(model_dir: str, group_size: int = 64) -> Optional[str]:
    """The cache the reference would pick for this directory: v2 first, then v1 (loader.py:92-112)."""
    for name in ([CACHE_V2] if group_size == 64 else []) + [CACHE_V1]:
        for cand in (os.path.join(model_dir, name),
                     os.path.join(os.path.expanduser("~/.cache/torchburn"), f"{os.path.basename(os.path.normpath(model_dir))}_{name}")):
            if os.path.isfile(cand):
                return cand
    return None


def load_cache(path: str) -> Dict[str, torch.Tensor]:
    """Reads a v1 or v2 cache file; the result is always in v1 tensors."""
    import safetensors.torch

    sd = safetensors.torch.load_file(path, device="cpu")
    if os.path.basename(path) == CACHE_V2 or any(
            k.endswith(".qweight") and k.replace(".qweight", ".scales") not in sd for k in sd):
        sd = migrate_v2_state_dict(sd)
    return sd


def decoder_from_state_dict(sd: Mapping[str, torch.Tensor], num_layers: int, hidden_size: int, intermediate_size: int,
                            num_heads: int, num_kv_heads: int, head_dim: int, group_size: int = 64,
                            rms_norm_eps: float = 1e-6, max_seq_len: int = 4096, rope_theta: float = 1e6, **kw):
    """create_rust_qwen_decoder (quantization.py:560-660) on a quantized state dict."""
    from .decoder import B200QwenDecoder

    layers = []
    for i in range(num_layers):
        pre = f"layers.{i}."
        post = sd.get(pre + "post_attention_layernorm.weight")
        if post is None:
            post = torch.ones(hidden_size)
        caps = [sd[pre + "input_layernorm.weight"], sd[pre + "self_attn.qkv_proj.qweight"], sd[pre + "self_attn.qkv_proj.scales"],
                sd[pre + "self_attn.o_proj.qweight"], sd[pre + "self_attn.o_proj.scales"], post,
                sd[pre + "mlp.gate_proj.qweight"], sd[pre + "mlp.gate_proj.scales"], sd[pre + "mlp.up_proj.qweight"],
                sd[pre + "mlp.up_proj.scales"], sd[pre + "mlp.down_proj.qweight"], sd[pre + "mlp.down_proj.scales"]]
        if pre + "self_attn.qkv_proj.bias" in sd:
            caps.append(sd[pre + "self_attn.qkv_proj.bias"])
        layers.append(caps)
    return B200QwenDecoder(sd["embed_tokens.weight"], layers, sd["norm.weight"], sd["lm_head.qweight"], sd["lm_head.scales"],
                           num_layers, hidden_size, intermediate_size, num_heads, num_kv_heads, head_dim, group_size,
                           rms_norm_eps, max_seq_len, rope_theta, **kw)
