"""Partitioning of the compressed-attention work across the GPUs of one box.

The unit of work is a lane: one (sequence, KV head) pair.  A lane's packed codes, norms and
fp16 sink/recent tokens are read by exactly one CTA group, and the attention outputs of the
query heads that share that KV head depend on nothing else, so lanes can be dealt to ranks
with no data-path collective.  Two plans:

* by sequence (``plan_lanes(..., split_heads=False)``): whole sequences per rank; nothing is
  exchanged.  This is what ``bench.py --gpus N`` times.
* by sequence and KV head (``split_heads=True``): used when there are fewer sequences than
  ranks; each rank then holds the caches of its KV heads only and the per-head outputs are
  gathered once per step (``gather_heads``), the only collective on the path.

``job_time_ms`` is the barrier-free max over ranks that multi-GPU timings must use.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class LanePlan:
    """Half-open ranges of sequences and KV heads owned by one rank."""
    seq_begin: int
    seq_end: int
    head_begin: int
    head_end: int

    @property
    def n_lanes(self) -> int:
        return (self.seq_end - self.seq_begin) * (self.head_end - self.head_begin)


def _even_range(n: int, parts: int, index: int) -> tuple[int, int]:
    """Range `index` of `n` items dealt to `parts` owners, sizes differing by at most one."""
    base, extra = divmod(n, parts)
    begin = index * base + min(index, extra)
    return begin, begin + base + (1 if index < extra else 0)


def plan_lanes(n_sequences: int, n_kv_heads: int, world: int, rank: int, split_heads: bool | None = None) -> LanePlan:
    """Lanes of rank `rank` out of `world`.

    With ``split_heads`` None the plan splits by sequence whenever every rank can get at least one
    sequence, otherwise by (sequence, head group): ranks are arranged as `n_sequences` rows of
    ``world // n_sequences`` head groups, which must divide evenly."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    if n_sequences < 1 or n_kv_heads < 1:
        raise ValueError("need at least one sequence and one KV head")
    if split_heads is None:
        split_heads = n_sequences < world
    if not split_heads:
        b, e = _even_range(n_sequences, world, rank)
        return LanePlan(b, e, 0, n_kv_heads)
    if world % n_sequences:
        raise ValueError(f"{world} ranks cannot be arranged as {n_sequences} sequences x head groups")
    groups = world // n_sequences
    if n_kv_heads % groups:
        raise ValueError(f"{n_kv_heads} KV heads do not split into {groups} equal groups")
    seq, grp = divmod(rank, groups)
    per = n_kv_heads // groups
    return LanePlan(seq, seq + 1, grp * per, (grp + 1) * per)


def gather_heads(local_out: torch.Tensor, group: dist.ProcessGroup | None = None) -> torch.Tensor:
    """Concatenate per-rank attention outputs (B, H_q_local, 1, D) along the head axis.

    Only needed under a head-split plan; ranks of one sequence row must form `group` in head order."""
    world = dist.get_world_size(group)
    if world == 1:
        return local_out
    parts = [torch.empty_like(local_out) for _ in range(world)]
    dist.all_gather(parts, local_out.contiguous(), group=group)
    return torch.cat(parts, dim=1)


def job_time_ms(local_ms: float, device: torch.device | None = None, group: dist.ProcessGroup | None = None) -> float:
    """Max over ranks of a device-measured duration."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return float(local_ms)
    t = torch.tensor([local_ms], dtype=torch.float64, device=device if device is not None else "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())
