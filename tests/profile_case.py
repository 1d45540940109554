"""Small fixed workload for ncu captures of the GEMV kernels (see profiles/): a few distinct
weight copies of one shape, launched back to back through the C ABI.

    python tests/profile_case.py {c1|qkv|down|gateup|lm_head} [M]      (M > 1: the batched product)
"""
import os
import sys
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch
import torchburn_b200 as tb
dev = torch.device("cuda", 0)
L = tb.lib()
name = sys.argv[1]
M = int(sys.argv[2]) if len(sys.argv) > 2 else 1
shapes = {"c1": (4096, 4096, False), "qkv": (6144, 4096, False), "down": (4096, 14336, False), "gateup": (14336, 4096, True), "lm_head": (128256, 4096, False)}
n, k, swi = shapes[name]
per = (n*k//2 + n*(k//32)*4) * (2 if swi else 1)
copies = max(2, int(400e6 // per))
ws = []
for i in range(copies*(2 if swi else 1)):
    ws.append((torch.randint(0, 256, (n, k//2), dtype=torch.uint8, device=dev), torch.rand(n, k//32, device=dev)*0.01))
x = torch.randn(M,k,device=dev); out = torch.empty(M,n,device=dev)
st = torch.cuda.current_stream(dev).cuda_stream
for rep in range(3):
    for i in range(copies):
        if swi:
            a,b = ws[2*i], ws[2*i+1]
            rc = L.tb_swiglu_gemv_w4a32(x.data_ptr(), a[0].data_ptr(), a[1].data_ptr(), None, b[0].data_ptr(), b[1].data_ptr(), None, out.data_ptr(), M, n, k, 32, st)
        else:
            a = ws[i]
            rc = L.tb_gemm_w4a32_grouped(x.data_ptr(), a[0].data_ptr(), a[1].data_ptr(), None, out.data_ptr(), M, n, k, 32, st)
        assert rc == 0, tb.last_error()
torch.cuda.synchronize()
print("ok", name, copies)
