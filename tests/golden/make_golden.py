"""Generate the golden vectors under tests/golden/ from the reference project itself.

Run where the reference checkout is present, with MLSTM_REF pointing at it, and where
oracle/_ref/libmlstm_ref.so has been built (``make -C oracle ref REF=$MLSTM_REF``):

    MLSTM_REF=<reference checkout> python tests/golden/make_golden.py

It imports the reference's own PyTorch functions (mlstm_matmul.py:104-118, 336-365;
mlstm_scan.py:343-372) on CPU and calls the reference's own host C++ forward (mlstmCpu,
cuda-src/cpu_utils.cuh:126-170) through oracle/_ref, on small seeded inputs, and stores inputs
and outputs as .npz files.  The tests read only those files.
"""
import ctypes
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF = os.environ.get("MLSTM_REF")
if not REF or not os.path.isfile(os.path.join(REF, "mlstm_matmul.py")):
    raise SystemExit("set MLSTM_REF to the reference checkout (the directory that holds mlstm_matmul.py)")
sys.path.insert(0, REF)

import mlstm_matmul as ref_mm  # noqa: E402  (the reference module)
import mlstm_scan as ref_scan  # noqa: E402


def gen_matmul(name, B, NH, S, D, f_mean, seed):
    g = torch.Generator().manual_seed(seed)
    q, k, v = (torch.randn(B, NH, S, D, generator=g) for _ in range(3))
    f = f_mean + torch.randn(B, NH, S, generator=g)
    i = torch.randn(B, NH, S, generator=g)
    dh = torch.randn(B, NH, S, D, generator=g)
    ref_mm.DEVICE = torch.device("cpu")
    h = ref_mm.mlstm_matmul_pytorch(q, k, v, f, i)
    dq, dk, dv, df, di = ref_mm.mlstm_matmul_backward_pytorch(dh, q, k, v, f, i)
    np.savez(os.path.join(HERE, name), q=q.numpy(), k=k.numpy(), v=v.numpy(), f=f.numpy(),
             i=i.numpy(), dh=dh.numpy(), h=h.numpy(), dq=dq.numpy(), dk=dk.numpy(),
             dv=dv.numpy(), df=df.numpy(), di=di.numpy())
    print(name, "h max", float(h.abs().max()))


def gen_scan(name, B, NH, S, D, f_mean, seed):
    g = torch.Generator().manual_seed(seed)
    q, k, v = (torch.randn(B, NH, S, D, generator=g) for _ in range(3))
    f = f_mean + torch.randn(B, NH, S, generator=g)
    i = torch.randn(B, NH, S, generator=g)
    o = torch.randn(B, NH, S, D, generator=g)
    h = ref_scan.mlstm_scan_pytorch(q, k, v, f, i, o)
    np.savez(os.path.join(HERE, name), q=q.numpy(), k=k.numpy(), v=v.numpy(), f=f.numpy(),
             i=i.numpy(), o=o.numpy(), h=h.numpy())
    print(name, "h max", float(h.abs().max()))


def gen_long_bf16(name, S, D, f_mean, seed):
    """One head of a long 16-bit case (the chunkwise path's shape): inputs are bf16 values (stored as their bit
    patterns), outputs come from the reference's PyTorch forward (mlstm_matmul.py:104-118) and backward
    (mlstm_matmul.py:336-365) in fp32 on exactly those values and are stored as float16."""
    g = torch.Generator().manual_seed(seed)
    mk = lambda *s: torch.randn(*s, generator=g)
    q, k, v = ((mk(1, 1, S, D) * D ** -0.5).bfloat16() for _ in range(3))
    f, i = (f_mean + mk(1, 1, S)).bfloat16(), mk(1, 1, S).bfloat16()
    dh = mk(1, 1, S, D).bfloat16()
    ref_mm.DEVICE = torch.device("cpu")
    x = [t.float() for t in (q, k, v, f, i)]
    h = ref_mm.mlstm_matmul_pytorch(*x)
    dq, dk, dv, df, di = ref_mm.mlstm_matmul_backward_pytorch(dh.float(), *x)
    bits = lambda t: t.view(torch.int16).numpy()
    np.savez(os.path.join(HERE, name), q=bits(q), k=bits(k), v=bits(v), f=bits(f), i=bits(i), dh=bits(dh),
             h=h.half().numpy(), dq=dq.half().numpy(), dk=dk.half().numpy(), dv=dv.half().numpy(),
             df=df.float().numpy(), di=di.float().numpy())
    print(name, "h max", float(h.abs().max()), "dq max", float(dq.abs().max()))


def gen_cpp(name, S, D, seed):
    lib = ctypes.CDLL(os.path.join(ROOT, "oracle", "_ref", "libmlstm_ref.so"))
    mk = lambda n: np.zeros(n, dtype=np.float16)
    Q, K, V, F, I, H = mk(S * D), mk(S * D), mk(S * D), mk(S), mk(S), mk(S * D)
    p = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    lib.ref_fill(ctypes.c_uint(seed), p(Q), p(K), p(V), p(F), p(I), ctypes.c_uint(S), ctypes.c_uint(D))
    lib.ref_mlstm_cpu(p(Q), p(K), p(V), p(F), p(I), p(H), ctypes.c_uint(S), ctypes.c_uint(D))
    np.savez(os.path.join(HERE, name), Q=Q.reshape(S, D), K=K.reshape(S, D), V=V.reshape(S, D),
             F=F, I=I, H=H.reshape(S, D))
    print(name, "sum H", float(H.astype(np.float64).sum()), H[0], H[-1])


def gen_cpp_backward(name, S, D, seed):
    """Inputs in the backward driver's recipe (uniform [-1, 1) halves, srand(seed); cuda-src/mlstm_backward.cu:
    580-586), gradients from the reference's PyTorch backward (mlstm_matmul.py:336-365) in fp32 on those values.
    The reference's C++ host backward covers dB, dQ and dK only and is not used."""
    lib = ctypes.CDLL(os.path.join(ROOT, "oracle", "_ref", "libmlstm_ref.so"))
    mk = lambda n: np.zeros(n, dtype=np.float16)
    Q, K, V, F, I, dH, scratch = mk(S * D), mk(S * D), mk(S * D), mk(S), mk(S), mk(S * D), mk(S * D)
    p = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    lib.ref_fill(ctypes.c_uint(seed), p(Q), p(K), p(V), p(F), p(I), ctypes.c_uint(S), ctypes.c_uint(D))
    lib.ref_fill(ctypes.c_uint(seed + 1), p(dH), p(scratch), p(scratch), p(mk(S)), p(mk(S)), ctypes.c_uint(S), ctypes.c_uint(D))
    t = lambda a, *shape: torch.from_numpy(a.astype(np.float32)).reshape(1, 1, *shape)
    ref_mm.DEVICE = torch.device("cpu")
    dq, dk, dv, df, di = ref_mm.mlstm_matmul_backward_pytorch(t(dH, S, D), t(Q, S, D), t(K, S, D), t(V, S, D), t(F, S), t(I, S))
    np.savez(os.path.join(HERE, name), Q=Q.reshape(S, D), K=K.reshape(S, D), V=V.reshape(S, D), F=F, I=I,
             dH=dH.reshape(S, D), dQ=dq[0, 0].numpy(), dK=dk[0, 0].numpy(), dV=dv[0, 0].numpy(), dF=df[0, 0].numpy(),
             dI=di[0, 0].numpy())
    print(name, "max |dQ|", float(dq.abs().max()), "max |dF|", float(df.abs().max()))


if __name__ == "__main__":
    gen_matmul("matmul_s128_d32_f0.npz", 1, 2, 128, 32, 0.0, 0)
    gen_matmul("matmul_s192_d64_f3.npz", 2, 1, 192, 64, 3.0, 1)
    # one mid-size case per path: all large-shape parity otherwise rests on the (pinned) port
    gen_matmul("matmul_s768_d32_f1.npz", 1, 1, 768, 32, 1.0, 4)
    gen_scan("scan_s512_d32_f1.npz", 1, 1, 512, 32, 1.0, 5)
    gen_long_bf16("long_bf16_s1024_d128_f3.npz", 1024, 128, 3.0, 6)
    gen_scan("scan_s96_d16_f0.npz", 1, 2, 96, 16, 0.0, 2)
    gen_scan("scan_s64_d32_f3.npz", 1, 1, 64, 32, 3.0, 3)
    # the reference demo's own recipe: srand(100), S = 640 (the README's value), D = 128
    gen_cpp("cpp_forward_seed100_s640_d128.npz", 640, 128, 100)
    gen_cpp("cpp_forward_seed100_s128_d128.npz", 128, 128, 100)
    # the backward driver's recipe: srand(1678), D = 128 (S = 192 keeps the fixture small and is not a tile multiple)
    gen_cpp_backward("cpp_backward_seed1678_s192_d128.npz", 192, 128, 1678)
