"""Sharding of independent work units (GEMM problems, attention heads) over ranks.

The hot path has no exchange step: each GPU runs the single-GPU kernels on its own contiguous block of
units (unit u belongs to rank floor(u * world / units)), and the only collective is the all-gather that
gives every rank the full output.  The partition arithmetic and the gather are kept free of CUDA so that
they can be exercised with the gloo backend on CPU; on GPUs the same gather runs over NCCL.
"""
import torch
import torch.distributed as dist


def unit_range(units, world, rank):
    """Contiguous block [begin, end) of `units` owned by `rank`: unit u goes to rank floor(u * world / units)."""
    if units < 0 or world <= 0 or not (0 <= rank < world):
        raise ValueError("bad partition arguments")
    begin = -(-rank * units // world)        # ceil(rank * units / world)
    end = -(-(rank + 1) * units // world)
    return begin, end


def owner_of(unit, units, world):
    return unit * world // units


def all_gather_units(local, units, group=None):
    """Gathers per-rank blocks of unit outputs (first dimension = units of this rank) into the full
    [units, ...] tensor on every rank.  Blocks may differ in size by one unit; they are padded to the
    largest block for the collective and trimmed afterwards."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    b, e = unit_range(units, world, rank)
    if local.shape[0] != e - b:
        raise ValueError(f"rank {rank} holds {local.shape[0]} units, expected {e - b}")
    biggest = max(unit_range(units, world, r)[1] - unit_range(units, world, r)[0] for r in range(world))
    if all(unit_range(units, world, r)[1] - unit_range(units, world, r)[0] == biggest for r in range(world)):
        out = torch.empty((units,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(out, local.contiguous(), group=group)
        return out
    padded = torch.zeros((biggest,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    padded[: e - b] = local
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded, group=group)
    chunks = []
    for r in range(world):
        rb, re_ = unit_range(units, world, r)
        chunks.append(parts[r][: re_ - rb])
    return torch.cat(chunks, dim=0)
