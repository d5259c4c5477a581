"""Partition of one mLSTM problem over the GPUs of a box.

Every (batch, head) slice of the parallel forward and backward is independent in both directions (the
reference offsets every pointer per (batch, head): mlstm_matmul.py:46-50, 145-149, 213-217), so a problem
[B, NH, S, D] is split by giving each rank a contiguous range of the B*NH flattened slices.  No rank needs
anything from another one: there is no collective on the data path.
"""
import torch

__all__ = ["slice_range", "shard_slices", "unshard_slices"]


def slice_range(n_slices: int, rank: int, world: int):
    """[lo, hi) of rank's slices: contiguous, sizes differ by at most one, lower ranks get the extra ones."""
    if not 0 <= rank < world:
        raise ValueError("rank outside the group")
    base, extra = divmod(int(n_slices), int(world))
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_slices(t: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """t [B, NH, ...] -> this rank's slices as [1, n_local, ...] (a view when t is contiguous)."""
    B, NH = t.shape[:2]
    lo, hi = slice_range(B * NH, rank, world)
    return t.reshape((1, B * NH) + tuple(t.shape[2:]))[:, lo:hi]


def unshard_slices(parts, B: int, NH: int) -> torch.Tensor:
    """Inverse of shard_slices over the list of all ranks' results (rank order)."""
    cat = torch.cat(list(parts), dim=1)
    return cat.reshape((B, NH) + tuple(cat.shape[2:]))
