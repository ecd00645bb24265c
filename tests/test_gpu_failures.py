"""Failure paths of the engine, driven from the host (nothing here makes a GPU fault, trap or hang).

The reference poisons a session whose frame could not be enqueued (talker.cu:1245-1252) and, in a
lockstep batch, every session of that batch (talker.cu:1946-1956); a poisoned session refuses all
further work with STATUS_STATE while sessions outside the failed call keep decoding the same codes
as before.  The library's test hooks make the engine see a failed launch, a failed allocation, or a
bounded device-side wait that ran out, without any CUDA call failing."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TEXT = [1501, 77, 151935, -1, 9000, 42, 31337, 8]
CODEC = [-1, 2148, 3, 2049, -1, 100, 7, 2000]


def start(q3t, model, seed, max_seq=64):
    t = q3t.SamplingConfig(True, 50, 0.9, 0.9, 1.05)
    p = q3t.SamplingConfig(True, 50, 1.0, 0.9, 1.0)
    return model.start_prompt(TEXT, CODEC, max_seq, seed, t, p)


@pytest.fixture(scope="module")
def model(gpu_model):
    gpu_model.set_option("mask_eos", 1)
    return gpu_model


@pytest.fixture()
def no_graphs(model):
    """Launch kernels one by one, so that the n-th launch of a frame exists on every frame."""
    model.set_option("use_graphs", 0)
    yield model
    model.set_option("use_graphs", 1)


def frames_of(session, count):
    return [(tuple(f.codes), f.next_semantic_token) for f in (session.next_frame(100 + i) for i in range(count))]


def test_failed_launch_poisons_the_session_only(q3t, no_graphs):
    model, lib = no_graphs, q3t.library()
    reference = start(q3t, model, 31)
    expected = frames_of(reference, 3)
    reference.close()

    victim, sibling = start(q3t, model, 30), start(q3t, model, 31)
    got = frames_of(sibling, 1)
    lib.q3t_test_fail_launch_after(37)             # somewhere inside the predictor of the next frame
    with pytest.raises(q3t.NativeTalkerStatusError) as e:
        victim.next_frame(100)
    lib.q3t_test_fail_launch_after(0)
    assert e.value.status == q3t.native.STATUS_CUDA
    for _ in range(2):                             # poisoned: every later call is refused, nothing runs
        with pytest.raises(q3t.NativeTalkerStatusError) as e:
            victim.next_frame(100)
        assert e.value.status == q3t.native.STATUS_STATE and "poisoned" in e.value.message
    with pytest.raises(q3t.NativeTalkerStatusError):
        victim.prefill(TEXT, CODEC)
    got += [(tuple(f.codes), f.next_semantic_token) for f in (sibling.next_frame(101 + i) for i in range(2))]
    assert got == expected                         # the sibling never noticed
    victim.close()
    sibling.close()
    assert lib.q3t_kernel_error_count() == 0


def test_failed_launch_poisons_the_whole_batch(q3t, no_graphs):
    model, lib = no_graphs, q3t.library()
    reference = start(q3t, model, 41)
    expected = frames_of(reference, 2)
    reference.close()

    batch = [start(q3t, model, 50 + i) for i in range(3)]
    outsider = start(q3t, model, 41)
    lib.q3t_test_fail_launch_after(200)
    with pytest.raises(q3t.NativeTalkerStatusError) as e:
        model.batch_begin_device_frames(batch, [100] * 3)
    lib.q3t_test_fail_launch_after(0)
    assert e.value.status == q3t.native.STATUS_CUDA
    for s in batch:
        with pytest.raises(q3t.NativeTalkerStatusError) as e:
            s.next_frame(100)
        assert e.value.status == q3t.native.STATUS_STATE and "poisoned" in e.value.message
    with pytest.raises(q3t.NativeTalkerStatusError):       # a poisoned member makes the next batch fail early,
        model.batch_begin_device_frames([batch[0], outsider], [100, 100])   # before anything is enqueued
    assert frames_of(outsider, 2) == expected
    for s in batch + [outsider]:
        s.close()


def test_failed_allocation_is_reported_and_leaves_the_model_usable(q3t, model):
    lib = q3t.library()
    lib.q3t_test_fail_allocation_after(2)
    with pytest.raises(q3t.NativeTalkerStatusError) as e:
        model.create_session(64, 1)
    lib.q3t_test_fail_allocation_after(0)
    assert e.value.status == q3t.native.STATUS_ALLOCATION
    s = start(q3t, model, 7)                       # pages of the failed attempt went back to the pool
    assert len(frames_of(s, 1)) == 1
    s.close()


def test_a_device_wait_that_ran_out_is_seen_at_the_next_host_sync(q3t, model):
    """The kernels bump a host-visible word when one of their bounded waits gives up; the engine
    compares it at finish / prefill / frame-loop time and refuses to hand out the results."""
    lib = q3t.library()
    single = start(q3t, model, 60)
    pair = [start(q3t, model, 61), start(q3t, model, 62)]
    bystander = start(q3t, model, 63)
    pending_single = single.begin_device_frame(100)
    pending_pair = model.batch_begin_device_frames(pair, [100, 100])
    assert lib.q3t_test_report_device_wait_failure(0) == 0
    with pytest.raises(q3t.NativeTalkerStatusError) as e:
        pending_single.finish_without_consumer()
    assert e.value.status == q3t.native.STATUS_CUDA and "wait" in e.value.message
    for p in pending_pair:                          # every session whose frame was in flight
        with pytest.raises(q3t.NativeTalkerStatusError) as e:
            p.finish_without_consumer()
        assert e.value.status == q3t.native.STATUS_CUDA
    for s in [single] + pair:
        with pytest.raises(q3t.NativeTalkerStatusError) as e:
            s.next_frame(100)
        assert e.value.status == q3t.native.STATUS_STATE
    assert len(frames_of(bystander, 1)) == 1       # begun after the event: not affected
    for s in [single, bystander] + pair:
        s.close()


def test_session_rebuilt_at_the_same_address_gets_its_own_pages(q3t, model):
    """A session is destroyed after its prompt and the next one, with another capacity, usually lands
    at the same heap address with another page list: its prompt must go through its own pages.  The
    second session's frames equal those of the same session created in a quiet model."""
    prompt = ([int(t) for t in np.random.default_rng(4).integers(0, 151936, size=40)], [-1] * 40)

    def run(max_seq, seed):
        t = q3t.SamplingConfig(True, 50, 0.9, 0.9, 1.05)
        p = q3t.SamplingConfig(True, 50, 1.0, 0.9, 1.0)
        s = model.start_prompt(prompt[0], prompt[1], max_seq, seed, t, p)
        out = frames_of(s, 2)
        s.close()
        return out

    quiet = run(96, 5)
    for capacity in (64, 256, 48):                 # churn: different page counts, freed in between
        t = q3t.SamplingConfig(True, 50, 0.9, 0.9, 1.05)
        s = model.start_prompt(prompt[0], prompt[1], capacity, 9, t, t)
        s.close()
    assert run(96, 5) == quiet
    a = run(128, 5)                                # capacity does not change what a session decodes
    assert a == quiet
