"""Lane-level data parallelism across the GPUs of one node: replicated weights, each rank owns a
contiguous block of lanes, no collective on the decode step.  The only exchange is the gather of
the sampled token ids (4 bytes per lane) that the caller wants on one host, which the reference's
single-request driver never needed (engine/decode_run.cpp runs one request on device 0,
engine/loader.cpp:481)."""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_lanes(total_lanes: int, world: int, rank: int) -> tuple[int, int]:
    """(first lane, lane count) of `rank`: blocks differ by at most one lane, lower ranks first."""
    if not (0 <= rank < world) or total_lanes < 0:
        raise ValueError("bad rank / world / lanes")
    base, extra = divmod(total_lanes, world)
    count = base + (1 if rank < extra else 0)
    first = rank * base + min(rank, extra)
    return first, count


def gather_tokens(local_tokens: torch.Tensor, total_lanes: int, dst: int = 0):
    """Gather every rank's int32 token ids (any device) into lane order on rank `dst`.
    Works on the gloo (host) and nccl (device) backends; returns None on the other ranks."""
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return local_tokens.clone()
    world, rank = dist.get_world_size(), dist.get_rank()
    counts = [shard_lanes(total_lanes, world, r)[1] for r in range(world)]
    if local_tokens.numel() != counts[rank]:
        raise ValueError(f"rank {rank} holds {local_tokens.numel()} lanes, expected {counts[rank]}")
    width = max(counts)
    buf = torch.full((width,), -1, dtype=torch.int32, device=local_tokens.device)
    buf[:counts[rank]] = local_tokens.to(torch.int32)
    out = [torch.empty_like(buf) for _ in range(world)] if rank == dst else None
    dist.gather(buf, out, dst=dst)
    if rank != dst:
        return None
    return torch.cat([o[:c] for o, c in zip(out, counts)])
