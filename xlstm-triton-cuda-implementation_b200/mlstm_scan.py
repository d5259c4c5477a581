"""Forward mLSTM scan with output gate on the B200 kernels.

Same name, arguments and result as the reference's ``mlstm_scan`` (mlstm_scan.py:281-327):

    h = mlstm_scan(q, k, v, f, i, o, reduce_block_size=4, value_block_size=4)

q, k, v, o: [B, NH, S, D]; f, i: [B, NH, S]; CUDA, contiguous; h is float32 (mlstm_scan.py:303).
The block-size arguments are the reference's tiling hints: they are validated the way the
reference's grid needs them (positive, dividing D, mlstm_scan.py:297, 309-310) and otherwise ignored.

The library picks one of three forms by shape (``mlstm_scan_fwd`` in include/mlstm_b200.h):
  * D above 256 (the reference demo, D = 1024): two tensor-core passes, the gated S x S matrix once
    and then W V; the quadratic form is the cheapest there because the D x D state is larger than S x S;
  * S much longer than D (16-bit inputs, D = 128 or 256): chunkwise, i.e. per-block (C, n) states with the
    stabiliser known up front, an inter-block carry and the output from the carried state, which is
    the mechanism of the reference's three scan kernels (mlstm_scan.py:74-137, 143-195, 200-278);
  * otherwise the parallel forward with silu(o) in its epilogue.
``initial`` / ``return_state`` expose the carried state (S [B*NH, D, D] key-major, z [B*NH, D], F, A
[B*NH] float64; see ``mlstm_chunkwise``) and need the chunkwise form's shapes.

Arithmetic: 16-bit inputs always run on the tensor cores.  float32 inputs: at D = 64 and 128 the split
tensor-core form (three bf16 products per fp32 product, error about 1e-5, as fast as tf32 there), whatever
``allow_tf32`` says; at D = 256 and at multiples of 256 up to 4096 single tf32 products with fp32
accumulation when ``allow_tf32`` is true (the default here; measured max-abs-rel error about 5e-4 to 2e-3,
inside the reference's own 1e-2 check), IEEE fp32 dot products on the CUDA cores (much slower) when it is
false or at any other D.

The reference's scan is forward only (README.md:97).  Here inputs that require gradients get them, behind
the output gate's own derivative: long 16-bit sequences at D = 128 or 256 through the chunkwise forward and the
chunkwise backward (states carried forward for dQ and back for dK, dV; linear in S), everything else
through the parallel kernels (``mlstm_matmul_backward``), whose cost is quadratic in S.
"""
import torch

from . import _lib
from .mlstm_matmul import mlstm_matmul_backward, mlstm_matmul_forward, output_gate_backward, output_gate_forward

__all__ = ["mlstm_scan", "output_gate_forward", "output_gate_backward"]


def _chunkwise_shape(q):
    """Whether the scan entry's chunkwise form (and with it the chunkwise backward) serves this input."""
    B, NH, S, D = q.shape
    return q.dtype in (torch.float16, torch.bfloat16) and D in (128, 256) and S > 2 * D and S > 512


class _ScanWithGrad(torch.autograd.Function):
    """mLSTM(q, k, v, f, i) * silu(o) with gradients for all six inputs.  Long 16-bit sequences at D = 128, 256 take
    the chunkwise forward and backward (linear in S); everything else the parallel kernels (quadratic)."""

    @staticmethod
    def forward(ctx, q, k, v, f, i, o, flags):
        ctx.chunked = _chunkwise_shape(q)
        if ctx.chunked:
            from .mlstm_chunkwise import ChunkSegment
            seg = ChunkSegment(q, k, v, f, i, 256, shared_workspace=True)
            seg.prepare(None)
            h_inner = seg.apply(None)
            m, b = seg.read_mb()
        else:
            h_inner, m, b = mlstm_matmul_forward(q, k, v, f, i, flags=flags)
        ctx.save_for_backward(q, k, v, f, i, o, m, b, h_inner)
        ctx.flags = flags
        return output_gate_forward(h_inner, o)

    @staticmethod
    def backward(ctx, dh):
        q, k, v, f, i, o, m, b, h_inner = ctx.saved_tensors
        dh_inner, do = output_gate_backward(dh.contiguous(), h_inner, o)
        if ctx.chunked:
            from .mlstm_chunkwise import mlstm_chunkwise_backward
            dq, dk, dv, df, di = mlstm_chunkwise_backward(dh_inner, q, k, v, f, i, h_inner, m, b, 256)
        else:
            dq, dk, dv, df, di = mlstm_matmul_backward(dh_inner, q, k, v, f, i, h_inner, m, b, flags=ctx.flags)
        return dq, dk, dv, df, di, do, None


def mlstm_scan(q, k, v, f, i, o, reduce_block_size=4, value_block_size=4, num_warps=8, allow_tf32=True, flags=0,
               initial=None, return_state=False):
    if q.dim() != 4 or k.shape != q.shape or v.shape != q.shape or o.shape != q.shape:
        raise ValueError("q, k, v, o must share the shape [B, NH, S, D]")
    if f.shape != q.shape[:3] or i.shape != q.shape[:3]:
        raise ValueError("f, i must have the shape [B, NH, S]")
    if not (k.dtype == v.dtype == o.dtype == f.dtype == i.dtype == q.dtype):
        raise TypeError("q, k, v, f, i, o must share one element type")
    B, NH, S, D = q.shape
    for name, val in (("reduce_block_size", reduce_block_size), ("value_block_size", value_block_size),
                      ("num_warps", num_warps)):
        if int(val) <= 0:
            raise ValueError(f"{name} must be positive")
    if D % int(reduce_block_size) or D % int(value_block_size):
        raise ValueError("reduce_block_size and value_block_size must divide D")
    dev = _lib.require_cuda(q, k, v, f, i, o)
    if allow_tf32 and D not in (64, 128):   # at D = 64, 128 the split form is as fast and at fp32 accuracy
        flags |= _lib.F_ALLOW_TF32
    if initial is not None or return_state:
        from .mlstm_chunkwise import mlstm_chunkwise
        return mlstm_chunkwise(q, k, v, f, i, chunk_size=256, initial=initial, return_state=return_state, o=o)
    if torch.is_grad_enabled() and any(t.requires_grad for t in (q, k, v, f, i, o)):
        return _ScanWithGrad.apply(q, k, v, f, i, o, flags)
    dt = _lib.dtype_code(q)
    h = torch.empty((B, NH, S, D), device=dev, dtype=torch.float32)
    L = _lib.lib()
    ws = _lib.workspace(L.mlstm_scan_fwd_workspace(B, NH, S, D, dt, flags), dev)
    with torch.cuda.device(dev):
        rc = L.mlstm_scan_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), f.data_ptr(), i.data_ptr(), o.data_ptr(),
                              h.data_ptr(), ws.data_ptr(), ws.numel(), B, NH, S, D, dt, flags, _lib.stream_ptr(dev))
    _lib.check(rc, "mlstm_scan_fwd")
    _lib.maybe_read_status(ws, dev, "mlstm_scan_fwd")
    return h
