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
    # fp32 inputs on the tensor cores work on converted operand copies (split bf16 by default, tf32 on request)
    assert L.mlstm_mm_fwd_workspace(1, 1, 128, 64, 0, 4) > L.mlstm_mm_fwd_workspace(1, 1, 128, 64, 0, 1)
    assert L.mlstm_mm_fwd_workspace(1, 1, 128, 64, 0, 0) > L.mlstm_mm_fwd_workspace(1, 1, 128, 64, 0, 8)
    assert L.mlstm_mm_fwd_workspace(1, 1, 128, 256, 0, 0) == L.mlstm_mm_fwd_workspace(1, 1, 128, 256, 0, 1)   # no split form at D = 256
    # the scan entry: two-pass scratch above D = 256, chunkwise scratch for long 16-bit sequences at D = 128
    assert L.mlstm_scan_fwd_workspace(1, 4, 2048, 1024, 0, 4) > 4 * 2048 * 2048 * 4
    assert L.mlstm_scan_fwd_workspace(1, 2, 4096, 128, 2, 0) == L.mlstm_chunk_workspace(1, 2, 4096, 128, 2, 256)
    assert L.mlstm_chunk_sp_record_floats(128) == 128 * 128 + 128 + 4
    # the chunkwise form (forward and backward) takes D = 128 and 256, 16-bit inputs
    assert L.mlstm_chunk_workspace(1, 2, 4096, 256, 2, 256) > L.mlstm_chunk_workspace(1, 2, 4096, 128, 2, 256) > 0
    assert L.mlstm_chunk_bwd_workspace(1, 2, 4096, 256, 2, 0, 256) > 0
    assert L.mlstm_chunk_workspace(1, 2, 4096, 64, 2, 256) == 0 and L.mlstm_chunk_workspace(1, 2, 4096, 128, 0, 256) == 0
    assert L.mlstm_scan_fwd_workspace(1, 2, 4096, 256, 2, 0) == L.mlstm_chunk_workspace(1, 2, 4096, 256, 2, 256)
    # the parallel path above D = 256 (multiples of 256): two passes per direction with the gated S x S matrices in scratch;
    # float32 inputs only where tf32 is allowed; forced CUDA-core calls need none of it
    S, Spad = 300, 384
    assert L.mlstm_mm_fwd_workspace(1, 2, S, 512, 2, 0) >= 2 * Spad * Spad * 2
    assert L.mlstm_mm_fwd_workspace(1, 2, S, 512, 2, 1) < Spad * Spad * 2
    assert L.mlstm_mm_fwd_workspace(1, 2, S, 512, 0, 0) < Spad * Spad * 4 <= L.mlstm_mm_fwd_workspace(1, 2, S, 512, 0, 4) // 2
    assert L.mlstm_mm_bwd_workspace(1, 2, S, 512, 2, 0, 0) >= 4 * Spad * Spad * 2
    assert L.mlstm_mm_bwd_workspace(1, 2, S, 384, 2, 2, 0) < Spad * Spad * 2   # not a multiple of 256: CUDA cores
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


def test_static_scratch_figure_matches_the_workspace_query(pkg):
    """The built-in scratch of mlstm_forward_f16_static is exactly the forward scratch at its length limit."""
    L = pkg._lib.lib()
    header = open(os.path.join(ROOT, "include", "mlstm_b200.h")).read()
    max_s = int(re.search(r"#define MLSTM_STATIC_MAX_S (\d+)u", header).group(1))
    nbytes = int(re.search(r"#define MLSTM_STATIC_SCRATCH_BYTES (\d+)u", header).group(1))
    assert L.mlstm_forward_f16_workspace(max_s, 128) == nbytes
    assert L.mlstm_forward_f16_workspace(max_s + 1, 128) > nbytes


def test_slice_partition_is_contiguous_and_complete(pkg):
    for n, world in ((128, 1), (128, 8), (10, 4), (3, 8)):
        edges = [pkg.slice_range(n, r, world) for r in range(world)]
        assert edges[0][0] == 0 and edges[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(edges, edges[1:]))
        sizes = [hi - lo for lo, hi in edges]
        assert max(sizes) - min(sizes) <= 1
    t = torch.arange(2 * 3 * 5).reshape(2, 3, 5)
    parts = [pkg.shard_slices(t, r, 4) for r in range(4)]
    assert torch.equal(pkg.unshard_slices(parts, 2, 3), t)


def _partition_worker(rank, world, port, out):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import importlib
        pkg = importlib.import_module("xlstm-triton-cuda-implementation_b200")
        g = torch.Generator().manual_seed(0)
        full = torch.randn(3, 4, 6, 2, generator=g)            # every rank holds the same global problem
        mine = pkg.shard_slices(full, rank, world).contiguous() * 2.0   # stand-in for the per-slice computation
        sizes = [torch.zeros(1, dtype=torch.long) for _ in range(world)]
        dist.all_gather(sizes, torch.tensor([mine.shape[1]]))
        parts = [torch.empty((1, int(n), 6, 2)) for n in sizes]
        dist.all_gather(parts, mine)
        out[rank] = bool(torch.equal(pkg.unshard_slices(parts, 3, 4), full * 2.0))
    finally:
        dist.destroy_process_group()


def test_slice_partition_over_gloo():
    """Two ranks shard one global problem by (batch, head) slices, work on their shards and the shards tile the
    problem exactly (the collective here only carries the check; the data path has none)."""
    import socket
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    out = mp.Manager().dict()
    mp.spawn(_partition_worker, args=(2, port, out), nprocs=2, join=True)
    assert dict(out) == {0: True, 1: True}
