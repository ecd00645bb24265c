"""Data-parallel plumbing for the decode path: one process per GPU, one weight replica per GPU,
sessions sharded across ranks, no collective on the data path.

The reference scales the same way: its sessions are independent (one KV cache, one RNG stream
each, `native/qwen3-tts-native/src/session_bench.rs` runs them side by side against one model),
so a rank never needs another rank's activations.  The only cross-rank traffic is the timing
protocol of the benchmark: a barrier on each side of the timed region and a MAX over ranks of the
elapsed time, from which the whole-job throughput follows.

Everything here works on any `torch.distributed` backend (nccl on GPUs, gloo in the CPU tests).
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np


@dataclass(frozen=True)
class RankInfo:
    rank: int
    local_rank: int
    world: int

    @staticmethod
    def from_env(env=None) -> "RankInfo":
        """RANK / LOCAL_RANK / WORLD_SIZE as torchrun exports them; a plain launch is rank 0 of 1."""
        env = os.environ if env is None else env
        rank = int(env.get("RANK", "0"))
        world = int(env.get("WORLD_SIZE", "1"))
        local = int(env.get("LOCAL_RANK", str(rank)))
        if world < 1 or not 0 <= rank < world:
            raise ValueError(f"inconsistent rank environment: RANK={rank} WORLD_SIZE={world}")
        return RankInfo(rank, local, world)


def shard_session_seeds(rank: int, sessions_per_gpu: int, base: int = 1) -> List[int]:
    """Seeds of the sessions a rank owns.  Ranks get disjoint, reproducible streams: session j of
    rank r is seeded base + 1000 r + j (a batch is at most 64 sessions, so blocks never touch)."""
    if not 0 < sessions_per_gpu <= 1000:
        raise ValueError("sessions_per_gpu must be in 1..1000")
    return [base + 1000 * rank + j for j in range(sessions_per_gpu)]


def shard_kv_lengths(rank: int, sessions_per_gpu: int, low: int = 64, high: int = 2048, seed: int = 3) -> np.ndarray:
    """Ragged KV lengths of a rank's sessions, U[low, high], seeded per rank (weak scaling: every
    rank holds the same amount of work in expectation, none of it shared)."""
    return np.random.default_rng(seed + rank).integers(low, high + 1, size=sessions_per_gpu)


def assign_sessions(total_sessions: int, world: int) -> List[range]:
    """Contiguous split of a global session list over ranks (used when a host shards an existing
    population of sessions rather than creating them per rank): sizes differ by at most one."""
    if world < 1 or total_sessions < 0:
        raise ValueError("world must be >= 1 and total_sessions >= 0")
    base, extra = divmod(total_sessions, world)
    out, start = [], 0
    for r in range(world):
        n = base + (1 if r < extra else 0)
        out.append(range(start, start + n))
        start += n
    return out


def whole_job_throughput(local_elapsed_s: float, local_units: int, world: int, device: Optional[str] = None):
    """(units of all ranks) / (max over ranks of the elapsed time), and that max.

    `local_elapsed_s` is this rank's device-timed region; the MAX makes the slowest rank set the
    pace, which is what a user of the whole box observes."""
    if world == 1:
        return local_units / local_elapsed_s, local_elapsed_s, local_units
    import torch
    import torch.distributed as dist
    t = torch.tensor([local_elapsed_s], dtype=torch.float64, device=device or "cpu")
    u = torch.tensor([float(local_units)], dtype=torch.float64, device=device or "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dist.all_reduce(u, op=dist.ReduceOp.SUM)
    return float(u.item()) / float(t.item()), float(t.item()), int(round(float(u.item())))


def gather_rank_lines(line: dict, world: int) -> Sequence[dict]:
    """Every rank's small report on rank 0 (clock samples, launch counts); other ranks get []."""
    if world == 1:
        return [line]
    import torch.distributed as dist
    out = [None] * world if dist.get_rank() == 0 else None
    dist.gather_object(line, out, dst=0)
    return out if out is not None else []
