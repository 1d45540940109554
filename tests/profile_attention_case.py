"""Small fixed workload for ncu captures of the decode-attention kernel (see profiles/):
Llama-3-8B head shape, context 4100, 8 distinct KV caches (273 MB), 24 launches.

    python tests/profile_attention_case.py
"""
import os
import sys
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch
import torchburn_b200 as tb
dev = torch.device("cuda", 0)
L = tb.lib()
nh, nkv, hd, S, off, layers, B = 32, 8, 128, 4160, 4100, 8, 1
kc = [torch.randn(B, nkv, S, hd, device=dev)*0.5 for _ in range(layers)]
vc = [torch.randn(B, nkv, S, hd, device=dev) for _ in range(layers)]
qkv = torch.randn(B, (nh+2*nkv)*hd, device=dev)
cos = torch.randn(S, hd, device=dev); sin = torch.randn(S, hd, device=dev)
offs = torch.full((B,), off, dtype=torch.int32, device=dev)
out = torch.empty(B, nh*hd, device=dev)
scratch = torch.zeros(L.tb_attention_scratch_bytes(B, nh, nkv, hd, S), dtype=torch.uint8, device=dev)
st = torch.cuda.current_stream(dev).cuda_stream
for rep in range(3):
    for l in range(layers):
        assert L.tb_attention_decode(qkv.data_ptr(), kc[l].data_ptr(), vc[l].data_ptr(), cos.data_ptr(), sin.data_ptr(), offs.data_ptr(), out.data_ptr(), scratch.data_ptr(), B, nh, nkv, hd, S, st) == 0
torch.cuda.synchronize(); print("ok")
