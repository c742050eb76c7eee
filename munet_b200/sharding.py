"""Host-side logic of the multi-GPU inference path: how a global batch is split over
ranks and how a whole-job time is formed. The decoder shards by independent sequences
(the reference's Engine::run_batch is a loop over independent inputs,
src/inference.hpp:618-627), so there is no data-path collective; only the timing and
the optional result gather touch torch.distributed."""
from __future__ import annotations


def shard_bounds(n_items: int, rank: int, world: int) -> tuple[int, int]:
    """Half-open range of the items rank owns: contiguous, sizes differ by at most one,
    ragged tails go to the first ranks."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank/world {rank}/{world}")
    base, extra = divmod(n_items, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def max_over_ranks(value: float, device="cpu") -> float:
    """MAX all-reduce of a per-rank measurement (device time in ms); identity without a group."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def gather_shards(local, n_items: int, device="cpu"):
    """All-gather per-rank result rows (a [n_local, ...] tensor) back into global order."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return local
    world = dist.get_world_size()
    sizes = [shard_bounds(n_items, r, world) for r in range(world)]
    width = max(hi - lo for lo, hi in sizes)
    pad = torch.zeros((width,) + tuple(local.shape[1:]), dtype=local.dtype, device=device)
    pad[: local.shape[0]] = local
    parts = [torch.empty_like(pad) for _ in range(world)]
    dist.all_gather(parts, pad)
    return torch.cat([p[: hi - lo] for p, (lo, hi) in zip(parts, sizes)], dim=0)
