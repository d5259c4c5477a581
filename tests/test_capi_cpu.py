"""CPU tests of the boundary: the library loads without a GPU, exports every declared symbol, and
rejects bad arguments before touching a device."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol(pkg):
    L = pkg._lib.lib()
    header = open(os.path.join(ROOT, "include", "mlstm_b200.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)  # declarations only, not the comments
    declared = set(re.findall(r"\b(mlstm_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    assert declared == set(pkg._lib.EXPORTS)
    for name in declared:
        assert hasattr(L, name), name


def test_workspace_sizes_and_support_matrix(pkg):
    L = pkg._lib.lib()
    assert L.mlstm_mm_fwd_workspace(1, 1, 128, 64, 2, 0) >= 256 + 2 * 128 * 4
    assert L.mlstm_mm_fwd_workspace(0, 1, 128, 64, 2, 0) == 0
    assert L.mlstm_mm_bwd_workspace(1, 1, 100, 64, 2, 0, 0) > L.mlstm_mm_bwd_workspace(1, 1, 100, 64, 2, 2, 0)
    assert L.mlstm_mm_fwd_workspace(1, 1, 128, 64, 0, 4) > L.mlstm_mm_fwd_workspace(1, 1, 128, 64, 0, 0)   # tf32 copies
    assert L.mlstm_tc_supported(4096, 256, 2) == 1
    assert L.mlstm_tc_supported(4096, 256, 0) == 2   # fp32: only with MLSTM_F_ALLOW_TF32
    assert L.mlstm_tc_supported(4096, 96, 2) == 0


def test_bad_arguments_rejected_without_a_device(pkg):
    L = pkg._lib.lib()
    one = ctypes.c_void_p(16)  # non-null, aligned; never dereferenced because checks fail first
    assert L.mlstm_mm_fwd(None, one, one, one, one, one, one, one, one, 1 << 20, 1, 1, 8, 8, 0, 0, 0, None) == -1
    assert L.mlstm_mm_fwd(one, one, one, one, one, one, one, one, one, 1 << 20, 1, 1, 8, 12, 0, 0, 0, None) == -2
    assert L.mlstm_mm_fwd(ctypes.c_void_p(8), one, one, one, one, one, one, one, one, 1 << 20, 1, 1, 8, 8, 0, 0, 0, None) == -3
    assert L.mlstm_mm_fwd(one, one, one, one, one, one, one, one, one, 16, 1, 1, 8, 8, 0, 0, 0, None) == -5
    assert L.mlstm_mm_fwd(one, one, one, one, one, one, one, one, one, 1 << 20, 1, 1, 8, 8, 7, 0, 0, None) == -1
    assert b"aligned" in L.mlstm_status_string(-3)


def test_python_wrappers_refuse_cpu_tensors(pkg):
    q = torch.zeros(1, 1, 8, 8)
    f = torch.zeros(1, 1, 8)
    with pytest.raises(RuntimeError, match="no CPU path"):
        pkg.mlstm_matmul(q, q, q, f, f)
    with pytest.raises(RuntimeError, match="no CPU path"):
        pkg.mlstm_scan(q, q, q, f, f, q)
    with pytest.raises(ValueError):
        pkg.mlstm_scan(q, q, q, f, f, q, reduce_block_size=3)
