"""B200-native mLSTM kernels behind the reference project's operator API.

    from <this package>.mlstm_matmul import Triton_mLSTM, mlstm_matmul
    from <this package>.mlstm_scan import mlstm_scan

The compute lives in libmlstm_b200.so (CUDA for sm_100a, C ABI in include/mlstm_b200.h), loaded on
first use.  There is no CPU, PyTorch or Triton fallback: without the built library calls raise.
"""
from . import _lib
from .mlstm_matmul import Triton_mLSTM, fp32_math_mode, mlstm_matmul, mlstm_matmul_backward, mlstm_matmul_forward
from .mlstm_scan import mlstm_scan, output_gate_backward, output_gate_forward
from .mlstm_chunkwise import mlstm_chunkwise, mlstm_chunkwise_backward, mlstm_chunkwise_sequence_parallel
from .partition import shard_slices, slice_range, unshard_slices

__all__ = ["Triton_mLSTM", "mlstm_matmul", "mlstm_matmul_forward", "mlstm_matmul_backward", "fp32_math_mode", "mlstm_scan",
           "output_gate_forward", "output_gate_backward", "mlstm_chunkwise", "mlstm_chunkwise_backward",
           "mlstm_chunkwise_sequence_parallel",
           "slice_range", "shard_slices", "unshard_slices", "_lib"]
