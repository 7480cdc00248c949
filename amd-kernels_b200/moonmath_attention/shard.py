"""Multi-GPU use of `forward`: independent (batch x head) slices, one process per GPU.

The reference has no multi-GPU path at all (no collective, no process group
anywhere in its sources).  Attention needs none on the hot path: every
(batch, head) slice is a closed problem (the reference's grid makes the same
point, csrc/attention_kernel.hip:505-529: one work-group = one query block of
one slice).  So ranks take contiguous ranges of slices and run the single-GPU
kernel on them; a collective appears only if the caller wants the whole output
on every rank (`gather_slices`, an all-gather over NCCL or gloo).
"""

from __future__ import annotations

import torch


def slice_range(rank: int, world: int, n_slices: int) -> range:
    """Contiguous, balanced range of (batch*heads) slice indices owned by `rank`."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank/world: {rank}/{world}")
    if n_slices < 0:
        raise ValueError("n_slices must be non-negative")
    base, extra = divmod(n_slices, world)
    begin = rank * base + min(rank, extra)
    return range(begin, begin + base + (1 if rank < extra else 0))


def max_over_ranks(value: float, group=None) -> float:
    """Largest `value` over the ranks of the (initialised) process group; used for step times."""
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return float(value)
    backend = dist.get_backend(group)
    dev = torch.device("cuda", torch.cuda.current_device()) if backend == "nccl" else torch.device("cpu")
    t = torch.tensor([float(value)], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


def gather_slices(local: torch.Tensor, n_slices: int, group=None) -> torch.Tensor:
    """All-gathers per-rank outputs shaped [1, n_local, S, D] into [1, n_slices, S, D] on every rank.

    Outside the hot path: only for callers that want the full result everywhere.
    Ranks may own different slice counts; shorter ones are padded for the exchange.
    """
    import torch.distributed as dist

    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    counts = [len(slice_range(r, world, n_slices)) for r in range(world)]
    if local.size(1) != counts[rank]:
        raise ValueError(f"rank {rank} holds {local.size(1)} slices, expected {counts[rank]}")
    pad = max(counts)
    buf = local
    if local.size(1) < pad:
        buf = torch.zeros(1, pad, *local.shape[2:], dtype=local.dtype, device=local.device)
        buf[:, : local.size(1)] = local
    # bf16 is exchanged as raw bytes so that every backend (gloo has no 16-bit types) moves exact bit patterns
    raw = buf.contiguous().view(torch.uint8)
    parts = [torch.empty_like(raw) for _ in range(world)]
    dist.all_gather(parts, raw, group=group)
    return torch.cat([p.view(local.dtype)[:, :c] for p, c in zip(parts, counts)], dim=1)
