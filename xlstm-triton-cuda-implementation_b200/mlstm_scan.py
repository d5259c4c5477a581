"""Forward mLSTM scan with output gate on the B200 kernels.

Same name, arguments and result as the reference's ``mlstm_scan`` (mlstm_scan.py:281-327):

    h = mlstm_scan(q, k, v, f, i, o, reduce_block_size=4, value_block_size=4)

q, k, v, o: [B, NH, S, D]; f, i: [B, NH, S]; CUDA, contiguous; h is float32 (mlstm_scan.py:303).
The block-size arguments are the reference's tiling hints: they are validated the way the
reference's grid needs them (positive, dividing D, mlstm_scan.py:297, 309-310) and otherwise ignored.
Forward only, like the reference (README.md:97).

Arithmetic: 16-bit inputs always run on the tensor cores.  float32 inputs run on them with tf32
operands and fp32 accumulation when ``allow_tf32`` is true (the default here: max-abs-rel error about
5e-4, inside the reference's own 1e-2 check) and D is 64, 128, 256 or a multiple of 256 up to 4096;
``allow_tf32=False`` gives IEEE fp32 dot products on the CUDA cores (error about 1e-6, much slower).
"""
import torch

from . import _lib

__all__ = ["mlstm_scan"]


def mlstm_scan(q, k, v, f, i, o, reduce_block_size=4, value_block_size=4, num_warps=8, allow_tf32=True, flags=0):
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
    if allow_tf32:
        flags |= _lib.F_ALLOW_TF32
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
