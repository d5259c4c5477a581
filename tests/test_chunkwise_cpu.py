"""CPU tests of the chunkwise / sequence-parallel host logic: the carry folds and the one-all-gather
protocol, driven over gloo with a dense fp64 model of the per-segment stages."""
import importlib
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import mlstm_oracle as orc
from tests import kernel_model as km

PKG = "xlstm-triton-cuda-implementation_b200"


def _inputs(B, NH, S, D, f_mean, seed):
    g = torch.Generator().manual_seed(seed)
    q, k, v = (torch.randn(B, NH, S, D, generator=g) for _ in range(3))
    f = f_mean + torch.randn(B, NH, S, generator=g)
    i = torch.randn(B, NH, S, generator=g)
    return q, k, v, f, i


def test_segment_model_alone_matches_oracle():
    x = _inputs(1, 2, 96, 16, 1.0, 0)
    seg = km.ChunkSegmentModel(*x)
    seg.prepare(None)
    assert orc.max_abs_rel(seg.apply(h_dtype=torch.float64), orc.matmul_forward(*x)) < 1e-10


@pytest.mark.parametrize("cuts", [(40,), (17, 60), (32, 33, 80)])
def test_folds_reproduce_the_full_sequence(cuts):
    """Serial emulation of G ranks: split, summaries, folds, apply; compare with the unsplit oracle."""
    mc = importlib.import_module(PKG + ".mlstm_chunkwise")
    x = _inputs(1, 2, 96, 16, 2.0, 1)
    S = x[0].shape[2]
    edges = (0,) + tuple(cuts) + (S,)
    segs = [km.ChunkSegmentModel(*[t[:, :, a:b] for t in x]) for a, b in zip(edges[:-1], edges[1:])]
    carry = mc.fold_gate_summaries(torch.stack([s.gate_summary() for s in segs]))
    assert torch.isinf(carry[0, :, 1]).all() and (carry[0, :, 0] == 0).all()
    summaries = [s.prepare(carry[g] if g else None) for g, s in enumerate(segs)]
    states = [s.local_state() for s in segs]
    S_all, z_all = torch.stack([a for a, _ in states]), torch.stack([b for _, b in states])
    A_end = torch.stack([s[:, 1] for s in summaries])
    assert (A_end[1:] >= A_end[:-1]).all()
    h = torch.cat([s.apply(mc.fold_states(S_all, z_all, A_end, g), h_dtype=torch.float64) for g, s in enumerate(segs)], 2)
    assert orc.max_abs_rel(h, orc.matmul_forward(*x)) < 1e-5   # the carried state passes through float32


@pytest.mark.parametrize("cuts", [(40,), (17, 60), (32, 33, 80)])
def test_record_fold_reproduces_the_full_sequence(cuts):
    """Serial emulation of the one-exchange protocol: every segment's record with no carry, fold_records,
    apply; compare with the unsplit oracle."""
    x = _inputs(1, 2, 96, 16, 2.0, 4)
    S = x[0].shape[2]
    edges = (0,) + tuple(cuts) + (S,)
    segs = [km.ChunkSegmentModel(*[t[:, :, a:b] for t in x]) for a, b in zip(edges[:-1], edges[1:])]
    gathered = torch.stack([s.sp_local() for s in segs])
    h = torch.cat([s.sp_apply(gathered, g, h_dtype=torch.float64) for g, s in enumerate(segs)], 2)
    assert orc.max_abs_rel(h, orc.matmul_forward(*x)) < 1e-5   # the carried state passes through float32


def test_fold_state_agrees_with_the_recurrent_oracle_state():
    """The carried (S, z, F, A) is the oracle's (C, n, m) up to the stabiliser convention:
    C* = exp(m) C = exp(F + A) S^T / sqrt(D)."""
    x = _inputs(1, 1, 48, 8, 0.5, 2)
    q, k, v, f, i = x
    _, (C, n, m) = orc.scan_forward(q, k, v, f, i, torch.zeros_like(q), return_state=True)
    seg = km.ChunkSegmentModel(*x)
    F_end, A_end = seg.prepare(None)[0]
    S_loc, z_loc = seg.local_state()
    true_C = torch.exp(m)[0, 0] * C[0, 0]
    mine = torch.exp(F_end + A_end) * S_loc[0].double().T / 8 ** 0.5
    assert orc.max_abs_rel(mine, true_C) < 1e-5


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, x, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        mc = importlib.import_module(PKG + ".mlstm_chunkwise")
        S = x[0].shape[2]
        a, b = rank * S // world, (rank + 1) * S // world
        seg = km.ChunkSegmentModel(*[t[:, :, a:b] for t in x])
        h = mc.sequence_parallel_forward(seg, h_dtype=torch.float64)
        ref = orc.matmul_forward(*x)[:, :, a:b]
        out[rank] = orc.max_abs_rel(h, ref)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sequence_parallel_protocol_over_gloo(world):
    x = _inputs(1, 2, 90, 8, 2.0, 3)
    out = mp.Manager().dict()
    mp.spawn(_worker, args=(world, _free_port(), x, out), nprocs=world, join=True)
    assert len(out) == world and all(e < 1e-5 for e in out.values()), dict(out)
