"""ctypes binding of libmlstm_b200.so (the C ABI declared in include/mlstm_b200.h).

torch is used for device memory and streams only: every call hands raw device pointers and the
current CUDA stream to the library.  There is no fallback: a missing library or a failed call raises.
"""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libmlstm_b200.so")

DT_F32, DT_F16, DT_BF16 = 0, 1, 2
F_FORCE_SIMT, F_FORCE_TC, F_ALLOW_TF32, F_NO_SPLIT = 1, 2, 4, 8
_DTYPES = {torch.float32: DT_F32, torch.float16: DT_F16, torch.bfloat16: DT_BF16}

_lib = None


class MlstmError(RuntimeError):
    def __init__(self, code, where):
        self.code = code
        msg = lib().mlstm_status_string(code).decode()
        if code == -6:
            detail = lib().mlstm_last_error_detail().decode()
            if detail:
                msg += " [" + detail + "]"
        super().__init__(f"{where}: {msg} (status {code})")


def lib():
    """Load the library once.  Raises if it has not been built: there is no other code path."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python {os.path.join(_HERE, 'build.py')}` "
            "(nvcc, sm_100a).  This library has no CPU or PyTorch fallback.")
    L = ctypes.CDLL(LIB_PATH)
    vp, i32, u32, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_uint, ctypes.c_size_t
    L.mlstm_status_string.restype = ctypes.c_char_p
    L.mlstm_status_string.argtypes = [i32]
    L.mlstm_last_error_detail.restype = ctypes.c_char_p
    L.mlstm_last_error_detail.argtypes = []
    L.mlstm_tc_supported.restype = i32
    L.mlstm_tc_supported.argtypes = [i32, i32, i32]
    L.mlstm_mm_fwd_workspace.restype = sz
    L.mlstm_mm_fwd_workspace.argtypes = [i32] * 6
    L.mlstm_mm_fwd.restype = i32
    L.mlstm_mm_fwd.argtypes = [vp] * 8 + [vp, sz] + [i32] * 7 + [vp]
    L.mlstm_mm_bwd_workspace.restype = sz
    L.mlstm_mm_bwd_workspace.argtypes = [i32] * 7
    L.mlstm_mm_bwd.restype = i32
    L.mlstm_mm_bwd.argtypes = [vp] * 14 + [vp, sz] + [i32] * 7 + [vp]
    L.mlstm_scan_fwd_workspace.restype = sz
    L.mlstm_scan_fwd_workspace.argtypes = [i32] * 6
    L.mlstm_scan_fwd.restype = i32
    L.mlstm_scan_fwd.argtypes = [vp] * 7 + [vp, sz] + [i32] * 6 + [vp]
    L.mlstm_forward_f16_workspace.restype = sz
    L.mlstm_forward_f16_workspace.argtypes = [u32, u32]
    L.mlstm_forward_f16.restype = i32
    L.mlstm_forward_f16.argtypes = [vp] * 6 + [u32, u32, vp, sz, vp]
    L.mlstm_backward_f16_workspace.restype = sz
    L.mlstm_backward_f16_workspace.argtypes = [u32, u32]
    L.mlstm_backward_f16.restype = i32
    L.mlstm_backward_f16.argtypes = [vp] * 11 + [u32, u32, vp, sz, vp]
    L.mlstm_forward_f16_static.restype = i32
    L.mlstm_forward_f16_static.argtypes = [vp] * 6 + [u32, u32, vp]
    L.mlstm_chunk_workspace.restype = sz
    L.mlstm_chunk_workspace.argtypes = [i32] * 6
    L.mlstm_chunk_gate_summary.restype = i32
    L.mlstm_chunk_gate_summary.argtypes = [vp, vp, vp, vp, sz] + [i32] * 6 + [vp]
    L.mlstm_chunk_prepare.restype = i32
    L.mlstm_chunk_prepare.argtypes = [vp] * 6 + [vp, sz] + [i32] * 6 + [vp]
    L.mlstm_chunk_local_state.restype = i32
    L.mlstm_chunk_local_state.argtypes = [vp, sz, vp, vp] + [i32] * 6 + [vp]
    L.mlstm_chunk_apply.restype = i32
    L.mlstm_chunk_apply.argtypes = [vp] * 7 + [i32, vp, vp, vp, sz] + [i32] * 6 + [vp]
    L.mlstm_chunk_sp_record_floats.restype = sz
    L.mlstm_chunk_sp_record_floats.argtypes = [i32]
    L.mlstm_chunk_sp_local.restype = i32
    L.mlstm_chunk_sp_local.argtypes = [vp] * 5 + [vp, sz] + [i32] * 6 + [vp]
    L.mlstm_chunk_sp_apply.restype = i32
    L.mlstm_chunk_sp_apply.argtypes = [vp] * 5 + [i32, i32, vp, i32, vp, vp, sz] + [i32] * 6 + [vp]
    L.mlstm_chunk_read_mb.restype = i32
    L.mlstm_chunk_read_mb.argtypes = [vp, sz, vp, vp] + [i32] * 6 + [vp]
    L.mlstm_chunk_bwd_workspace.restype = sz
    L.mlstm_chunk_bwd_workspace.argtypes = [i32] * 7
    L.mlstm_chunk_bwd.restype = i32
    L.mlstm_chunk_bwd.argtypes = [vp] * 14 + [vp, sz] + [i32] * 7 + [vp]
    L.mlstm_forward_f16_static_status.restype = i32
    L.mlstm_forward_f16_static_status.argtypes = [ctypes.POINTER(i32), vp]
    L.mlstm_ogate_fwd.restype = i32
    L.mlstm_ogate_fwd.argtypes = [vp, vp, vp, ctypes.c_longlong, i32, i32, vp]
    L.mlstm_ogate_bwd.restype = i32
    L.mlstm_ogate_bwd.argtypes = [vp] * 5 + [ctypes.c_longlong, i32, i32, vp]
    L.mlstm_selftest_wait_timeout.restype = i32
    L.mlstm_selftest_wait_timeout.argtypes = [vp, sz, ctypes.c_longlong, vp]
    L.mlstm_read_status.restype = i32
    L.mlstm_read_status.argtypes = [vp, ctypes.POINTER(i32), vp]
    _lib = L
    return L


EXPORTS = [
    "mlstm_status_string", "mlstm_last_error_detail", "mlstm_tc_supported", "mlstm_mm_fwd_workspace", "mlstm_mm_fwd",
    "mlstm_mm_bwd_workspace", "mlstm_mm_bwd", "mlstm_scan_fwd_workspace", "mlstm_scan_fwd",
    "mlstm_forward_f16_workspace", "mlstm_forward_f16", "mlstm_forward_f16_static", "mlstm_backward_f16_workspace",
    "mlstm_backward_f16", "mlstm_read_status",
    "mlstm_chunk_workspace", "mlstm_chunk_gate_summary", "mlstm_chunk_prepare", "mlstm_chunk_local_state",
    "mlstm_chunk_apply", "mlstm_chunk_sp_record_floats", "mlstm_chunk_sp_local", "mlstm_chunk_sp_apply",
    "mlstm_chunk_read_mb", "mlstm_chunk_bwd_workspace", "mlstm_chunk_bwd",
    "mlstm_forward_f16_static_status", "mlstm_selftest_wait_timeout", "mlstm_ogate_fwd", "mlstm_ogate_bwd",
]


def dtype_code(t: torch.Tensor) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise TypeError(f"unsupported element type {t.dtype}; use float32, float16 or bfloat16") from None


def require_cuda(*tensors):
    dev = tensors[0].device
    if dev.type != "cuda":
        raise RuntimeError("mLSTM B200 kernels need CUDA tensors; there is no CPU path")
    for t in tensors:
        if t.device != dev:
            raise RuntimeError("all tensors must live on the same CUDA device")
        if not t.is_contiguous():
            raise RuntimeError("tensors must be contiguous (the reference indexes them with fixed strides)")
    return dev


def stream_ptr(dev) -> int:
    return torch.cuda.current_stream(dev).cuda_stream


_WS_CACHE = {}


def workspace(nbytes: int, dev) -> torch.Tensor:
    """Scratch memory for one library call: a grow-only buffer per (device, stream).

    Calls that share a stream run in order, so they can share one buffer; calls on different
    streams get different buffers.  Keeping it avoids a large allocation per call (hundreds of MB
    at the largest configurations)."""
    if nbytes <= 0:
        raise MlstmError(-2, "workspace query")
    dev = torch.device(dev)
    key = (dev.index if dev.index is not None else torch.cuda.current_device(), stream_ptr(dev))
    buf = _WS_CACHE.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        _WS_CACHE[key] = buf
    return buf


def check(code: int, where: str):
    if code != 0:
        raise MlstmError(code, where)


_CHECK_STATUS = os.environ.get("MLSTM_B200_CHECK", "0") not in ("", "0")


def maybe_read_status(ws: torch.Tensor, dev, where: str):
    """With MLSTM_B200_CHECK=1 every call synchronises and reads the kernels' status word."""
    if _CHECK_STATUS:
        read_status(ws, dev, where)


def read_status(ws: torch.Tensor, dev, where: str):
    st = ctypes.c_int(0)
    check(lib().mlstm_read_status(ws.data_ptr(), ctypes.byref(st), stream_ptr(dev)), where)
