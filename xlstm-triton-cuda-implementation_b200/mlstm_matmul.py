"""Parallel (matmul) mLSTM forward and backward on the B200 kernels.

Same names, arguments and results as the reference module of this name
(mlstm_matmul.py:121-129 ``mlstm_matmul``; :368-405 ``Triton_mLSTM``):

    h = Triton_mLSTM.apply(q, k, v, f, i, SB, NUM_WARPS)
    h.backward(dh)          # q.grad, k.grad, v.grad, f.grad, i.grad

q, k, v: [B, NH, S, D]; f, i: [B, NH, S]; CUDA, contiguous, float32 / float16 / bfloat16.
``h`` is float32 whatever the inputs are, as in the reference (mlstm_matmul.py:373); gradients have
the inputs' type (:389-393).  ``SB`` and ``num_warps`` are the reference's tiling hints: they are
checked (positive integers) and otherwise ignored, the kernels pick their own tiles.

float32 inputs keep fp32-level accuracy, like the reference's ``tl.dot(..., allow_tf32=False)``
(mlstm_matmul.py:19): at D = 64 and 128 they run on the tensor cores with every operand split into two
bf16 halves and three products per fp32 product (error about 1e-5); at other head dimensions with IEEE
fp32 dot products on the CUDA cores.  Setting the environment variable ``MLSTM_B200_TF32=1`` (or passing
``flags=_lib.F_ALLOW_TF32`` to the two plain functions) trades accuracy for speed: single tf32 products
(D in {64, 128, 256}; error about 5e-4).  ``fp32_math_mode(D)`` says which of these a call will use.

Head dimensions above 256 (multiples of 256 up to 4096), 16-bit inputs, or float32 inputs with tf32 allowed:
forward (float32 ``h``) and backward run on the tensor cores in two passes each (gated S x S matrices to scratch,
then plain contractions: W V forward; dT K, dT^T Q, W^T dH backward).
"""
import os
import torch

from . import _lib

__all__ = ["Triton_mLSTM", "mlstm_matmul", "mlstm_matmul_forward", "mlstm_matmul_backward", "fp32_math_mode",
           "output_gate_forward", "output_gate_backward"]


_DEFAULT_FLAGS = _lib.F_ALLOW_TF32 if os.environ.get("MLSTM_B200_TF32", "0") not in ("", "0") else 0


def fp32_math_mode(D, flags=None):
    """The arithmetic float32 inputs get at head dimension D with the given flags (default: the module's)."""
    flags = _DEFAULT_FLAGS if flags is None else flags
    if flags & _lib.F_FORCE_SIMT:
        return "IEEE fp32 FMA on the CUDA cores"
    if (flags & _lib.F_ALLOW_TF32) and D in (64, 128, 256):
        return "single tf32 products on the tensor cores, fp32 accumulate"
    if (flags & _lib.F_ALLOW_TF32) and 256 < D <= 4096 and D % 256 == 0:
        return "single tf32 products on the tensor cores (two passes per direction), fp32 accumulate"
    if not (flags & _lib.F_NO_SPLIT) and D in (64, 128):
        return "split bf16 products (hi*hi + hi*mid + mid*hi) on the tensor cores, fp32 accumulate"
    return "IEEE fp32 FMA on the CUDA cores"


def _check_hints(SB, num_warps):
    if int(SB) <= 0 or int(num_warps) <= 0:
        raise ValueError("SB and num_warps must be positive")


def _check_shapes(q, k, v, f, i):
    if q.dim() != 4 or k.shape != q.shape or v.shape != q.shape:
        raise ValueError("q, k, v must share the shape [B, NH, S, D]")
    if f.shape != q.shape[:3] or i.shape != q.shape[:3]:
        raise ValueError("f, i must have the shape [B, NH, S]")
    if not (k.dtype == v.dtype == f.dtype == i.dtype == q.dtype):
        raise TypeError("q, k, v, f, i must share one element type")


def mlstm_matmul_forward(q, k, v, f, i, h_dtype=torch.float32, flags=0):
    """Run the forward; returns (h, m, b) with m, b the float32 stabiliser and row sums."""
    _check_shapes(q, k, v, f, i)
    dev = _lib.require_cuda(q, k, v, f, i)
    B, NH, S, D = q.shape
    dt = _lib.dtype_code(q)
    h = torch.empty((B, NH, S, D), device=dev, dtype=h_dtype)
    m = torch.empty((B, NH, S), device=dev, dtype=torch.float32)
    b = torch.empty((B, NH, S), device=dev, dtype=torch.float32)
    L = _lib.lib()
    ws = _lib.workspace(L.mlstm_mm_fwd_workspace(B, NH, S, D, dt, flags), dev)
    with torch.cuda.device(dev):
        rc = L.mlstm_mm_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), f.data_ptr(), i.data_ptr(), h.data_ptr(),
                            m.data_ptr(), b.data_ptr(), ws.data_ptr(), ws.numel(), B, NH, S, D, dt,
                            _lib.dtype_code(h), flags, _lib.stream_ptr(dev))
    _lib.check(rc, "mlstm_mm_fwd")
    _lib.maybe_read_status(ws, dev, "mlstm_mm_fwd")
    return h, m, b


def mlstm_matmul_backward(dh, q, k, v, f, i, h, m, b, flags=0):
    """Run the backward; returns (dq, dk, dv, df, di) in the inputs' element type."""
    dev = _lib.require_cuda(dh, q, k, v, f, i, h, m, b)
    B, NH, S, D = q.shape
    if dh.shape != q.shape or dh.dtype != h.dtype:
        raise ValueError("dh must match h in shape and element type")
    dt, hdt = _lib.dtype_code(q), _lib.dtype_code(h)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    df, di = torch.empty_like(f), torch.empty_like(i)
    L = _lib.lib()
    ws = _lib.workspace(L.mlstm_mm_bwd_workspace(B, NH, S, D, dt, hdt, flags), dev)
    with torch.cuda.device(dev):
        rc = L.mlstm_mm_bwd(dh.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), f.data_ptr(), i.data_ptr(),
                            h.data_ptr(), m.data_ptr(), b.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                            df.data_ptr(), di.data_ptr(), ws.data_ptr(), ws.numel(), B, NH, S, D, dt, hdt, flags,
                            _lib.stream_ptr(dev))
    _lib.check(rc, "mlstm_mm_bwd")
    _lib.maybe_read_status(ws, dev, "mlstm_mm_bwd")
    return dq, dk, dv, df, di


def output_gate_forward(h_inner, o):
    """h = h_inner * silu(o) (mlstm_scan.py:273-278), one elementwise kernel."""
    dev = _lib.require_cuda(h_inner, o)
    h = torch.empty_like(h_inner)
    with torch.cuda.device(dev):
        rc = _lib.lib().mlstm_ogate_fwd(h_inner.data_ptr(), o.data_ptr(), h.data_ptr(), h_inner.numel(),
                                        _lib.dtype_code(h_inner), _lib.dtype_code(o), _lib.stream_ptr(dev))
    _lib.check(rc, "mlstm_ogate_fwd")
    return h


def output_gate_backward(dh, h_inner, o):
    """(dh_inner, do) of h = h_inner * silu(o): dh_inner = dh silu(o), do = dh h_inner silu'(o)."""
    dev = _lib.require_cuda(dh, h_inner, o)
    dh_inner = torch.empty_like(h_inner)
    do = torch.empty_like(o)
    with torch.cuda.device(dev):
        rc = _lib.lib().mlstm_ogate_bwd(dh.data_ptr(), h_inner.data_ptr(), o.data_ptr(), dh_inner.data_ptr(), do.data_ptr(),
                                        h_inner.numel(), _lib.dtype_code(h_inner), _lib.dtype_code(o), _lib.stream_ptr(dev))
    _lib.check(rc, "mlstm_ogate_bwd")
    return dh_inner, do


class Triton_mLSTM(torch.autograd.Function):
    """Drop-in for the reference's autograd function (mlstm_matmul.py:368-405); the name is kept.

    One argument more than the reference takes: ``o`` ([B, NH, S, D], optional, after the two tiling hints) is the
    output gate the reference leaves as a note ("Integrate o", mlstm_matmul.py:36): the result is then
    h * silu(o) as in its scan path (mlstm_scan.py:273-278), and ``o`` gets its gradient."""

    @staticmethod
    def forward(ctx, q, k, v, f, i, SB=16, num_warps=8, o=None):
        _check_hints(SB, num_warps)
        if o is not None and (o.shape != q.shape or o.dtype != q.dtype):
            raise ValueError("o must match q in shape and element type")
        h, m, b = mlstm_matmul_forward(q, k, v, f, i, flags=_DEFAULT_FLAGS)
        ctx.gated = o is not None
        ctx.sb = SB
        if o is None:
            ctx.save_for_backward(q, k, v, f, i, m, b, h)
            return h
        ctx.save_for_backward(q, k, v, f, i, m, b, h, o)
        return output_gate_forward(h, o)

    @staticmethod
    def backward(ctx, dh):
        assert dh.is_contiguous()  # mlstm_matmul.py:385
        if ctx.gated:
            q, k, v, f, i, m, b, h, o = ctx.saved_tensors
            dh, do = output_gate_backward(dh, h, o)
        else:
            q, k, v, f, i, m, b, h = ctx.saved_tensors
            do = None
        dq, dk, dv, df, di = mlstm_matmul_backward(dh, q, k, v, f, i, h, m, b, flags=_DEFAULT_FLAGS)
        return dq, dk, dv, df, di, None, None, do


def mlstm_matmul(q, k, v, f, i, SB=16, num_warps=8):
    """Forward without autograd (mlstm_matmul.py:121-129)."""
    _check_hints(SB, num_warps)
    return mlstm_matmul_forward(q, k, v, f, i, flags=_DEFAULT_FLAGS)[0]
