"""The data-parallel launcher logic on CPU: two gloo ranks on 127.0.0.1 run the sharding and the
timing protocol that bench.py uses on GPUs, and each rank decodes its own shard with the CPU
oracle's sampler so that the 'no shared state between ranks' claim is exercised end to end."""
import importlib
import os
import socket
import sys

import numpy as np
import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def worker(rank: int, world: int, port: int, results):
    import torch.distributed as dist
    sys.path.insert(0, REPO)
    dp = importlib.import_module("qwen3-tts-native_b200.dp")
    from oracle import oracle
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        info = dp.RankInfo.from_env({"RANK": str(rank), "WORLD_SIZE": str(world), "LOCAL_RANK": str(rank)})
        seeds = dp.shard_session_seeds(info.rank, 4)
        lengths = dp.shard_kv_lengths(info.rank, 4)
        # each rank samples one token per session from the same logits with its own seeds
        rng = np.random.default_rng(0)
        logits = oracle.to_bf16(rng.standard_normal(3072).astype(np.float32))
        tokens = []
        for seed in seeds:
            token, _ = oracle.sample(logits, seed, suppress=True, do_sample=1, top_k=50, top_p=0.9,
                                     temperature=0.9, penalty=1.0)
            tokens.append(int(token))
        dist.barrier()
        elapsed = 0.010 * (rank + 1)          # rank 1 is the slow one
        value, slowest, units = dp.whole_job_throughput(elapsed, 4 * 10, world)
        dist.barrier()
        lines = dp.gather_rank_lines({"rank": rank, "seeds": seeds, "tokens": tokens,
                                      "lengths": [int(x) for x in lengths]}, world)
        results[rank] = dict(value=value, slowest=slowest, units=units, lines=list(lines))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_two_ranks_shard_and_aggregate():
    import torch.multiprocessing as mp
    world = 2
    port = free_port()
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(worker, args=(world, port, results), nprocs=world, join=True)
        r0, r1 = results[0], results[1]
    # whole-job value = units of all ranks / slowest rank's time, identical on every rank
    assert r0["units"] == r1["units"] == 80
    assert r0["slowest"] == pytest.approx(0.020) and r1["slowest"] == pytest.approx(0.020)
    assert r0["value"] == pytest.approx(80 / 0.020) and r1["value"] == pytest.approx(r0["value"])
    # rank 0 holds every rank's report; the shards do not overlap and differ in content
    assert len(r0["lines"]) == 2 and r1["lines"] == []
    a, b = r0["lines"]
    assert set(a["seeds"]).isdisjoint(b["seeds"])
    assert a["lengths"] != b["lengths"]
    assert a["tokens"] != b["tokens"]          # different seeds, different samples
    assert all(0 <= t < 3072 for t in a["tokens"] + b["tokens"])


def test_sharding_helpers():
    sys.path.insert(0, REPO)
    dp = importlib.import_module("qwen3-tts-native_b200.dp")
    assert [list(r) for r in dp.assign_sessions(10, 4)] == [[0, 1, 2], [3, 4, 5], [6, 7], [8, 9]]
    assert [len(r) for r in dp.assign_sessions(3, 8)] == [1, 1, 1, 0, 0, 0, 0, 0]
    assert sum(len(r) for r in dp.assign_sessions(512, 8)) == 512
    with pytest.raises(ValueError):
        dp.assign_sessions(4, 0)
    seeds = [dp.shard_session_seeds(r, 64) for r in range(8)]
    flat = [s for block in seeds for s in block]
    assert len(set(flat)) == len(flat) == 512
    assert np.array_equal(dp.shard_kv_lengths(3, 64), dp.shard_kv_lengths(3, 64))
    assert not np.array_equal(dp.shard_kv_lengths(3, 64), dp.shard_kv_lengths(4, 64))
    assert np.array_equal(dp.shard_kv_lengths(3, 64, per_rank=False), dp.shard_kv_lengths(0, 64))   # replicated draw
    lens = dp.shard_kv_lengths(0, 64)
    assert lens.min() >= 64 and lens.max() <= 2048
    assert dp.RankInfo.from_env({}) == dp.RankInfo(0, 0, 1)
    assert dp.RankInfo.from_env({"RANK": "5", "WORLD_SIZE": "8", "LOCAL_RANK": "5"}).local_rank == 5
    with pytest.raises(ValueError):
        dp.RankInfo.from_env({"RANK": "2", "WORLD_SIZE": "2"})
    value, slowest, units = dp.whole_job_throughput(0.5, 100, 1)
    assert (value, slowest, units) == (200.0, 0.5, 100)


class _HostImage:
    """Stand-in for Q3tTensorImage whose 'pointers' are numpy arrays (no GPU in this test)."""

    def __init__(self, data, scales, loaded):
        self.data, self.data_bytes = data, data.nbytes
        self.scales, self.scales_bytes = scales, 0 if scales is None else scales.nbytes
        self.quantized, self.loaded, self.device_index = scales is not None, loaded, 0


class _HostModel:
    """The two calls broadcast_weight_image needs, over host memory."""

    def __init__(self, shapes, fill):
        self.tensors, self.adopted = {}, []
        for i, (name, (rows, cols, quantized)) in enumerate(shapes.items()):
            rng = np.random.default_rng(100 + i)
            if quantized:
                data = rng.integers(-127, 128, (rows, cols), dtype=np.int8) if fill else np.zeros((rows, cols), np.int8)
                scales = rng.random(rows, dtype=np.float32) if fill else np.zeros(rows, np.float32)
            else:
                data = rng.integers(0, 65536, (rows, cols), dtype=np.uint16) if fill else np.zeros((rows, cols), np.uint16)
                scales = None
            self.tensors[name] = [data, scales, fill]

    def tensor_image(self, name):
        data, scales, loaded = self.tensors[name]
        return _HostImage(data, scales, loaded)

    def adopt_tensor(self, name):
        if self.tensors[name][2]:
            raise RuntimeError("duplicate tensor upload: " + name)
        self.tensors[name][2] = True
        self.adopted.append(name)


IMAGE_SHAPES = {"layer.q_proj.weight": (48, 64, True), "layer.norm.weight": (1, 64, False),
                "layer.down_proj.weight": (64, 96, True)}


def image_worker(rank: int, world: int, port: int, results):
    import torch
    import torch.distributed as dist
    sys.path.insert(0, REPO)
    dp = importlib.import_module("qwen3-tts-native_b200.dp")
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        model = _HostModel(IMAGE_SHAPES, fill=(rank == 0))
        host_view = lambda array, nbytes, device: torch.from_numpy(array.reshape(-1).view(np.uint8))
        total = dp.broadcast_weight_image(model, list(IMAGE_SHAPES), rank, src=0, view=host_view)
        digest = {n: (int(t[0].astype(np.int64).sum()), None if t[1] is None else float(t[1].sum()), t[2])
                  for n, t in model.tensors.items()}
        second = None
        if rank == 1:
            try:
                model.adopt_tensor("layer.norm.weight")
            except RuntimeError as e:
                second = str(e)
        results[rank] = dict(total=total, digest=digest, adopted=list(model.adopted), second=second)
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_weight_image_reaches_the_other_rank():
    import torch.multiprocessing as mp
    world = 2
    port = free_port()
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(image_worker, args=(world, port, results), nprocs=world, join=True)
        r0, r1 = results[0], results[1]
    expected = 48 * 64 + 48 * 4 + 64 * 2 + 64 * 96 + 64 * 4
    assert r0["total"] == r1["total"] == expected
    assert r0["digest"] == r1["digest"]                    # same bytes, everything marked loaded
    assert all(v[2] for v in r1["digest"].values())
    assert r0["adopted"] == [] and r1["adopted"] == list(IMAGE_SHAPES)
    assert "duplicate" in r1["second"]


def test_source_rank_must_have_uploaded():
    sys.path.insert(0, REPO)
    dp = importlib.import_module("qwen3-tts-native_b200.dp")
    empty = _HostModel(IMAGE_SHAPES, fill=False)
    with pytest.raises(RuntimeError, match="has not uploaded"):
        dp.broadcast_weight_image(empty, list(IMAGE_SHAPES), rank=0, src=0, view=None)
    with pytest.raises(RuntimeError, match="has not uploaded"):
        dp.copy_weight_image(empty, _HostModel(IMAGE_SHAPES, fill=False), list(IMAGE_SHAPES), view=None)
