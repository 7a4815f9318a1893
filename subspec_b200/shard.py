"""Data-parallel sharding of independent sequences over the GPUs of one box.

The reference runs one request at a time (every generator asserts batch size 1,
e.g. generators/classic_sd.py:169) and has no distributed code at all.  Requests
are independent, so the batched kernels scale by giving each rank (one process
per GPU) a contiguous block of sequences: there is no exchange step and no
collective on the hot path.  The only communication is the reduction of a
handful of statistics after the timed region.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List

import torch


@dataclass
class Shard:
    rank: int
    world: int
    first: int       # first global sequence id of this rank
    count: int       # sequences owned by this rank
    wave: int        # sequences per kernel launch
    total: int       # sequences in the whole job after rounding to whole waves

    @property
    def n_waves(self) -> int:
        return self.count // self.wave

    def wave_ids(self, w: int) -> List[int]:
        if not 0 <= w < self.n_waves:
            raise IndexError(w)
        start = self.first + w * self.wave
        return list(range(start, start + self.wave))


def shard_sequences(total: int, world: int, rank: int, wave: int) -> Shard:
    """Contiguous blocks of `total // world` sequences per rank, rounded down to whole waves."""
    if world < 1 or not 0 <= rank < world or total < world or wave < 1:
        raise ValueError(f"bad sharding request: total={total} world={world} rank={rank} wave={wave}")
    per_rank = total // world
    wave = min(wave, per_rank)
    per_rank = (per_rank // wave) * wave
    return Shard(rank=rank, world=world, first=rank * per_rank, count=per_rank, wave=wave, total=per_rank * world)


def device_for_rank(local_rank: int, local_world: int, visible: int) -> int:
    """Which of the box's `visible` GPUs the rank with this local rank takes.

    With as many ranks as GPUs it is the rank's own ordinal.  With fewer, the ranks are spread over the box
    (stride visible // local_world) instead of packed onto GPUs 0 .. n-1: neighbouring GPUs share PCIe
    switches and host links, and a job whose steps start with a host-to-device copy of its inputs is bound by
    exactly those when its ranks sit side by side."""
    if local_world < 1 or visible < 1 or not 0 <= local_rank < local_world:
        raise ValueError(f"bad placement request: local_rank={local_rank} local_world={local_world} visible={visible}")
    if local_world >= visible:
        return local_rank % visible
    return local_rank * (visible // local_world)


def reduce_stats(times_ms: Dict[str, float], counts: Dict[str, float], device="cpu") -> Dict[str, float]:
    """MAX over ranks of the timings, SUM over ranks of the counters (identity when not distributed)."""
    import torch.distributed as dist

    out = dict(times_ms)
    out.update(counts)
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return out
    tk, ck = sorted(times_ms), sorted(counts)
    t = torch.tensor([times_ms[k] for k in tk], dtype=torch.float64, device=device)
    c = torch.tensor([counts[k] for k in ck], dtype=torch.float64, device=device)
    if tk:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if ck:
        dist.all_reduce(c, op=dist.ReduceOp.SUM)
    out.update(dict(zip(tk, t.tolist())))
    out.update(dict(zip(ck, c.tolist())))
    return out
