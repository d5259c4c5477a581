"""Small case for profiler captures: two forward + backward steps of the parallel mLSTM at
B=4, NH=8, S=4096, D=256 in bf16 (q, k, v are 201 MB together, larger than L2).

    python profiles/run_small_case.py [B]
"""
import importlib
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch

pkg = importlib.import_module("xlstm-triton-cuda-implementation_b200")
B = int(sys.argv[1]) if len(sys.argv) > 1 else 4
NH, S, D = 8, 4096, 256
dev = torch.device("cuda", 0)
g = torch.Generator().manual_seed(0)
mk = lambda *s: torch.randn(*s, generator=g)
q, k, v = ((mk(B, NH, S, D) * D ** -0.5).bfloat16().to(dev) for _ in range(3))
f, i = (3.0 + mk(B, NH, S)).bfloat16().to(dev), mk(B, NH, S).bfloat16().to(dev)
dh = mk(B, NH, S, D).bfloat16().to(dev)
for _ in range(2):
    h, m, b = pkg.mlstm_matmul_forward(q, k, v, f, i, h_dtype=torch.bfloat16)
    grads = pkg.mlstm_matmul_backward(dh, q, k, v, f, i, h, m, b)
torch.cuda.synchronize()
print("ok", float(h.float().abs().max()), float(grads[0].float().abs().max()))
