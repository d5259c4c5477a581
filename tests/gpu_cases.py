"""Shared helpers of the GPU parity tests: seeded inputs in the configurations' recipes, calls
through the C ABI, and comparison with the CPU oracle."""
import importlib
import math

import torch

from oracle import mlstm_oracle as orc

PKG = importlib.import_module("xlstm-triton-cuda-implementation_b200")
_lib = PKG._lib


def make_inputs(B, NH, S, D, dtype, f_mean=0.0, qkv_scale=1.0, seed=0, with_o=False):
    """CPU-generator randn in the order q, k, v, f, i, (o), dh, then rounded to ``dtype``."""
    g = torch.Generator().manual_seed(seed)
    q, k, v = ((torch.randn(B, NH, S, D, generator=g) * qkv_scale).to(dtype) for _ in range(3))
    f = (f_mean + torch.randn(B, NH, S, generator=g)).to(dtype)
    i = torch.randn(B, NH, S, generator=g).to(dtype)
    out = dict(q=q, k=k, v=v, f=f, i=i)
    if with_o:
        out["o"] = torch.randn(B, NH, S, D, generator=g).to(dtype)
    out["dh"] = torch.randn(B, NH, S, D, generator=g)
    return out


def run_forward(x, h_dtype=torch.float32, flags=0):
    dev = torch.device("cuda", 0)
    args = [x[n].to(dev) for n in ("q", "k", "v", "f", "i")]
    h, m, b = PKG.mlstm_matmul_forward(*args, h_dtype=h_dtype, flags=flags)
    torch.cuda.synchronize()
    return h, m, b


def run_backward(x, h, m, b, flags=0):
    dev = torch.device("cuda", 0)
    args = [x[n].to(dev) for n in ("q", "k", "v", "f", "i")]
    dh = x["dh"].to(dev).to(h.dtype)
    out = PKG.mlstm_matmul_backward(dh, *args, h, m, b, flags=flags)
    torch.cuda.synchronize()
    return out


def oracle_forward(x):
    return orc.matmul_forward(x["q"], x["k"], x["v"], x["f"], x["i"], return_state=True)


def oracle_backward(x, h_dtype):
    dh = x["dh"].to(h_dtype)
    return orc.matmul_backward(dh, x["q"], x["k"], x["v"], x["f"], x["i"])


def errors_forward(x, h, m, b):
    """max-abs-rel per output, plus for h the fraction of elements outside the reference's elementwise
    comparator (utils.py:4: atol = rtol = 1e-2) and the worst row-wise relative error of the first tile
    (early rows have small magnitudes that a norm-wise measure hides)."""
    h_ref, m_ref, b_ref, _ = oracle_forward(x)
    hf = h.float().cpu().double()
    rows = min(128, hf.shape[-2])
    row_err = (hf[..., :rows, :] - h_ref[..., :rows, :]).abs().amax(-1) / h_ref[..., :rows, :].abs().amax(-1).clamp_min(1e-30)
    return {"h": orc.max_abs_rel(h.float(), h_ref), "m": orc.max_abs_rel(m, m_ref), "b": orc.max_abs_rel(b, b_ref),
            "h_check_frac": orc.check(h.float(), h_ref)[1], "h_first_tile_row_rel": float(row_err.max())}


def errors_backward(x, grads, h_dtype):
    ref = oracle_backward(x, h_dtype)
    out = {n: orc.max_abs_rel(g.float(), r) for n, g, r in zip(("dq", "dk", "dv", "df", "di"), grads, ref)}
    out["check_frac"] = max(orc.check(g.float(), r)[1] for g, r in zip(grads[:3], ref[:3]))
    return out


# bounds for the 16-bit tensor-core path beside max-abs-rel <= 1e-2: share of elements outside the reference's
# elementwise comparator, and the worst relative row error in the first tile
CHECK_FRAC_16 = 2e-3
ROW_REL_16 = 3e-2
