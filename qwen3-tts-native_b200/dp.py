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


def shard_kv_lengths(rank: int, sessions_per_gpu: int, low: int = 64, high: int = 2048, seed: int = 3,
                     per_rank: bool = True) -> np.ndarray:
    """Ragged KV lengths of a rank's sessions, U[low, high].  Seeded per rank by default (every rank
    holds the same amount of work in expectation, none of it shared); `per_rank=False` replicates
    one draw on every GPU, which is how the 64-session configuration is specified (the slowest
    rank then does not depend on the luck of its draw)."""
    return np.random.default_rng(seed + (rank if per_rank else 0)).integers(low, high + 1, size=sessions_per_gpu)


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


# ---- weight image: quantize on one rank, hand the decode-form tensors to the others -----------
#
# The reference quantizes the decode matrices on every GPU as the checkpoint is uploaded
# (talker.cu:564-668).  With one replica per GPU the bf16 checkpoint (3.8 GB) needs to reach only
# one rank: the others receive the int8 rows, the row scales and the bf16 leftovers (2.6 GB in all)
# straight into their own model's storage and adopt them.  This is a load-time edge, not a
# data-path collective.

class _DeviceSpan:
    """A raw device pointer dressed up for torch.as_tensor (CUDA array interface, bytes)."""

    def __init__(self, pointer: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (int(nbytes),), "typestr": "|u1",
                                         "data": (int(pointer), False), "version": 2}


def device_bytes(pointer, nbytes: int, device_index: int):
    """uint8 view of `nbytes` of device memory at `pointer` (no copy)."""
    import torch
    return torch.as_tensor(_DeviceSpan(pointer, nbytes), device=torch.device("cuda", device_index))


def image_spans(image) -> List[tuple]:
    """(pointer, bytes) of everything that makes up one tensor's decode form."""
    spans = [(image.data, int(image.data_bytes))]
    if image.quantized:
        spans.append((image.scales, int(image.scales_bytes)))
    return spans


def _settle(tensor) -> None:
    """The copies ran on torch's stream; the model reads the storage on its own streams."""
    if tensor is not None and getattr(tensor, "is_cuda", False):
        import torch
        torch.cuda.synchronize(tensor.device)


def broadcast_weight_image(model, names: Sequence[str], rank: int, src: int = 0, group=None,
                           view=device_bytes) -> int:
    """Rank `src` has uploaded (and thereby quantized) `names`; every other rank's model receives
    the decode-form bytes into its own storage and adopts them.  Returns the bytes broadcast.

    `view(pointer, nbytes, device_index)` turns a span into a tensor the backend can broadcast;
    the default wraps device memory for NCCL."""
    import torch.distributed as dist
    total = 0
    last = None
    for name in names:
        image = model.tensor_image(name)
        if rank == src and not image.loaded:
            raise RuntimeError(f"rank {src} has not uploaded {name}")
        for pointer, nbytes in image_spans(image):
            last = view(pointer, nbytes, image.device_index)
            dist.broadcast(last, src, group=group)
            total += nbytes
        if rank != src:
            model.adopt_tensor(name)
    _settle(last)
    return total


def copy_weight_image(source, destination, names: Sequence[str], view=device_bytes) -> int:
    """The same hand-over inside one process (two replicas, one or two GPUs): device-to-device
    copies of the decode-form tensors, then adoption.  Returns the bytes copied."""
    total = 0
    last = None
    for name in names:
        src_image = source.tensor_image(name)
        dst_image = destination.tensor_image(name)
        if not src_image.loaded:
            raise RuntimeError(f"the source model has not uploaded {name}")
        src_spans, dst_spans = image_spans(src_image), image_spans(dst_image)
        if [n for _, n in src_spans] != [n for _, n in dst_spans]:
            raise RuntimeError(f"{name}: the two models disagree on the tensor's size")
        for (sp, n), (dp_, _) in zip(src_spans, dst_spans):
            last = view(dp_, n, dst_image.device_index)
            last.copy_(view(sp, n, src_image.device_index))
            total += n
        destination.adopt_tensor(name)
    _settle(last)
    return total
