"""Two GPUs, one checkpoint: rank 0 uploads (and quantizes) the bf16 tensors, rank 1 receives the
decode form over NCCL into its own model's storage, and both replicas decode the same frames.
Skipped on boxes with one GPU.  No data-path collective is involved: this is the load-time edge."""
import importlib
import os
import socket
import sys

import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def worker(rank: int, world: int, port: int, results):
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import torch
    import torch.distributed as dist
    sys.path.insert(0, REPO)
    q3t = importlib.import_module("qwen3-tts-native_b200")
    dp = importlib.import_module("qwen3-tts-native_b200.dp")
    synth = importlib.import_module("qwen3-tts-native_b200.synth")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    model = q3t.NativeTalkerModel.create(rank)
    try:
        names = list(synth.tensor_shapes(128).keys())
        if rank == 0:
            for name, bits in synth.checkpoint_cuda(0, seed=0):
                model.upload_tensor(name, bits)
        sent = dp.broadcast_weight_image(model, names, rank, src=0)
        memory = model.finalize()
        model.set_option("mask_eos", 1)
        t = q3t.SamplingConfig(True, 50, 0.9, 0.9, 1.05)
        p = q3t.SamplingConfig(True, 50, 1.0, 0.9, 1.0)
        session = model.start_prompt([1501, 77, 151935, -1, 9000, 42, 31337, 8], [-1, 2148, 3, 2049, -1, 100, 7, 2000], 64, 777, t, p)
        frames = [tuple(session.next_frame(9).codes) for _ in range(3)]
        session.close()
        # placement independence: the sessions every rank owns under the data-parallel sharding
        # (dp.shard_session_seeds), decoded here as lockstep batches whatever this rank is
        by_owner = {}
        for owner in range(world):
            group = [model.start_prompt([1501, 77, 9000, 42], [-1, 2148, -1, 100], 64, seed, t, p)
                     for seed in dp.shard_session_seeds(owner, 3)]
            codes = [[] for _ in group]
            for _ in range(3):
                pending = model.batch_begin_device_frames(group, [9] * len(group))
                for i, pf in enumerate(pending):
                    frame = pf.finish_without_consumer()
                    codes[i].append(int(frame.next_semantic_token))
            by_owner[owner] = codes
            for x in group:
                x.close()
        results[rank] = dict(sent=sent, tensors=int(memory.tensor_count), frames=frames, by_owner=by_owner,
                             errors=int(q3t.native.library().q3t_kernel_error_count()))
        dist.barrier()
    finally:
        model.close()
        dist.destroy_process_group()


@pytest.mark.timeout(600)
def test_broadcast_image_then_decode_on_two_gpus():
    import torch
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world = 2
    port = free_port()
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(worker, args=(world, port, results), nprocs=world, join=True)
        r0, r1 = results[0], results[1]
    assert r0["tensors"] == r1["tensors"] == 404
    assert r0["sent"] == r1["sent"] > 2_000_000_000
    assert r0["frames"] == r1["frames"]
    # a session's tokens depend on its seed and prompt, not on the GPU or rank that decodes it
    assert r0["by_owner"] == r1["by_owner"]
    assert r0["by_owner"][0] != r0["by_owner"][1]          # different seeds do give different sessions
    assert r0["errors"] == r1["errors"] == 0
