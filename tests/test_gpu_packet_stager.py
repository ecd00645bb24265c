"""The hand-over after the path: frames begun on the device are staged into the codec's packet
without a host copy, with the events and the refusals of the reference host's stager
(native/qwen3-tts-runtime/src/cuda_packet_stager.rs:230-340)."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

PROMPT_TEXT = [1501, 77, 151935, -1, 9000, 42, 31337, 8]
PROMPT_CODEC = [-1, 2148, 3, 2049, -1, 100, 7, 2000]


def read_device_u16(torch, pointer: int, count: int) -> np.ndarray:
    cudart = C.CDLL("libcudart.so")
    host = np.zeros(count, dtype=np.uint16)
    torch.cuda.synchronize()
    rc = cudart.cudaMemcpy(host.ctypes.data_as(C.c_void_p), C.c_void_p(pointer), C.c_size_t(count * 2), C.c_int(2))
    assert rc == 0
    return host


def make_session(q3t, gpu_model):
    gpu_model.set_option("mask_eos", 1)
    t = q3t.SamplingConfig(True, 50, 0.9, 0.9, 1.05)
    p = q3t.SamplingConfig(True, 50, 1.0, 0.9, 1.0)
    return gpu_model.start_prompt(PROMPT_TEXT, PROMPT_CODEC, 64, 31, t, p)


@pytest.fixture()
def session(q3t, gpu_model):
    s = make_session(q3t, gpu_model)
    yield s
    s.close()


@pytest.fixture()
def twin(q3t, gpu_model):
    """The same session stepped through the host-copy call: what each frame's codes are."""
    s = make_session(q3t, gpu_model)
    yield s
    s.close()


def test_packet_of_four_frames_matches_the_host_copies(q3t, session, twin):
    import torch
    stager = q3t.native.PacketStager(0)
    try:
        assert stager.device_bytes == 128 and stager.staged_frames == 0
        with pytest.raises(q3t.native.PacketStagerError, match="empty"):
            stager.packet_view()
        frames = []
        for i in range(4):
            pending = session.begin_device_frame(9)
            copied = stager.stage(pending)
            assert copied != 0 and stager.staged_frames == i + 1
            # the copy event is the consumer-done event of the frame's lease
            pending.finish(copied)              # codes stay on the device in this call
            frames.append(twin.next_frame(9))
        view = stager.packet_view()
        assert view.frame_count == 4 and view.ready_event == copied
        packet = read_device_u16(torch, view.device_codes, 64).reshape(4, 16)
        for row, frame in zip(packet, frames):
            assert tuple(int(c) for c in row) == tuple(frame.codes)

        pending = session.begin_device_frame(9)
        with pytest.raises(q3t.native.PacketStagerError, match="full"):
            stager.stage(pending)
        pending.finish_without_consumer()
        fifth = twin.next_frame(9)

        with pytest.raises(q3t.native.PacketStagerError, match="consume event is required"):
            stager.release_after_consumer(0)
        done = torch.cuda.Event()
        done.record()
        stager.release_after_consumer(done.cuda_event)
        assert stager.staged_frames == 0
        with pytest.raises(q3t.native.PacketStagerError, match="no staged packet"):
            stager.release_after_consumer(done.cuda_event)

        # the next packet starts at slot 0 again
        pending = session.begin_device_frame(9)
        copied = stager.stage(pending)
        pending.finish(copied)
        sixth = twin.next_frame(9)
        view = stager.packet_view()
        assert view.frame_count == 1
        first = read_device_u16(torch, view.device_codes, 16)
        assert tuple(int(c) for c in first) == tuple(sixth.codes) != tuple(fifth.codes)
    finally:
        stager.close()


def test_refusals(q3t, session):
    stager = q3t.native.PacketStager(0)
    try:
        pending = session.begin_device_frame(9)
        with pytest.raises(q3t.native.PacketStagerError, match="does not match stager device"):
            stager.stage_frame(pending.device_codes, pending.ready_event, source_device=3)
        with pytest.raises(q3t.native.PacketStagerError, match="are required"):
            stager.stage_frame(0, pending.ready_event)
        with pytest.raises(q3t.native.PacketStagerError, match="are required"):
            stager.stage_frame(pending.device_codes, 0)
        with pytest.raises(q3t.native.PacketStagerError, match="returned 15 codes; expected 16"):
            stager.stage_frame(pending.device_codes, pending.ready_event, code_count=15)
        assert stager.staged_frames == 0
        pending.finish_without_consumer()
    finally:
        stager.close()
