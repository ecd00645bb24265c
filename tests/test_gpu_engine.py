"""GPU tests of the drop-in boundary itself: the native talker ABI v3 driven the way the
reference's host crate drives it (prefill, next_frame, begin/finish leases, lockstep batch),
checked against the CPU oracle's restatement of the frame algorithm and against the
self-consistency protocol of the reference's session benchmark (same seed => same codes
whatever the batching; different seeds differ; a dropped session does not disturb siblings;
lease misuse is a STATE error that leaves the GPU alone)."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

PROMPT_TEXT = [1501, 77, 151935, -1, 9000, 42, 31337, 8]
PROMPT_CODEC = [-1, 2148, 3, 2049, -1, 100, 7, 2000]


def cfgs(q3t, sampled=True):
    if sampled:
        return (q3t.SamplingConfig(True, 50, 0.9, 0.9, 1.05), q3t.SamplingConfig(True, 50, 1.0, 0.9, 1.0))
    return q3t.SamplingConfig.greedy(), q3t.SamplingConfig.greedy()


def start(q3t, model, seed, sampled=True, max_seq=64, prompt=(PROMPT_TEXT, PROMPT_CODEC)):
    t, p = cfgs(q3t, sampled)
    return model.start_prompt(prompt[0], prompt[1], max_seq, seed, t, p)


def as_kwargs(c):
    return dict(do_sample=int(c.do_sample), top_k=c.top_k, top_p=c.top_p, temperature=c.temperature,
                penalty=c.repetition_penalty)


@pytest.fixture(scope="module")
def model(gpu_model):
    gpu_model.set_option("mask_eos", 1)      # random logits would end sessions at random
    return gpu_model


def test_model_memory_and_state(q3t, model):
    assert model.memory.tensor_count == 404
    assert model.memory.shared_weight_bytes == 3_833_352_704     # the reference's README figure
    s = model.create_session(64, 1)
    st = s.runtime_state()
    assert (st.abi_version, st.phase, st.talker_position) == (3, 1, 0)     # READY
    assert s.memory.max_sequence_length == 64
    assert s.memory.talker_kv_bytes == 4 * 28 * 2 * 16 * 1024 * 2          # 4 pages
    assert s.memory.predictor_kv_bytes == 5 * 2 * 16 * 1024 * 2
    s.close()


class KernelBackend:
    """The oracle's primitive interface served by the kernels under test, one operator-level
    launch per call.  Running the oracle's frame composition over it gives, bit for bit, what the
    engine must produce: every operator is pinned against the oracle and the reference kernels
    on its own (test_gpu_gemv / _rowops / _attention / _sampler), and the engine's fused and paged
    launches are pinned against these stand-alone launches there too."""

    def __init__(self, ops, pad_rows=1):
        # pad_rows > 1 repeats the activation row so that the launch takes the path (SIMT or
        # tensor cores, tile width, K-slices) that a lockstep batch of that many sessions takes;
        # a row's result does not depend on what the other rows hold
        self.ops = ops
        self.pad_rows = pad_rows

    def rms_norm_rows(self, x, w):
        return self.ops.rms_norm_rows(x, w)

    def _padded(self, a):
        a = np.ascontiguousarray(a).reshape(1, -1)
        return np.repeat(a, self.pad_rows, axis=0)

    def int8_gemm_rows(self, w, s, x, y_in=None, mode=0):
        if self.pad_rows == 1:
            return self.ops.int8_gemm_rows(w, s, x, y_in=y_in, mode=mode, cache_weights=True)
        out = self.ops.int8_gemm_rows(w, s, self._padded(x), y_in=None if y_in is None else self._padded(y_in),
                                      mode=mode, cache_weights=True)
        return out[:1].copy()

    def int8_gate_up_silu_rows(self, w, s, x):
        return self.int8_gemm_rows(w, s, x, mode=2)

    def head_rms_norm(self, v, w, hd):
        v = np.ascontiguousarray(v)
        return self.ops.head_rms_norm_rows(v, w, 1, v.size // hd, hd)

    def rope_rows_at(self, v, rows, heads, hd, positions):
        return self.ops.rope_rows_at(v, rows, heads, hd, positions)

    def attention(self, q, k, v, positions, qh, kvh, hd, fast=True):
        return self.ops.attention_contiguous(q, k, v, positions, qh, kvh, hd)

    def bias_activation_rows(self, v, bias, silu):
        return self.ops.bias_activation_rows(v, bias, silu)

    def add(self, a, b):
        return self.ops.add_in_place(a, b)

    def sample(self, logits, rng, **kw):
        return self.ops.sample(logits, rng, **kw)


@pytest.fixture(scope="module")
def oracle_model(orc, checkpoint):
    return orc.OracleModel(checkpoint)


def test_cpu_oracle_tracks_the_kernels(orc, ops, oracle_model):
    """The same frame composition on the CPU oracle and on the kernels stays close through a
    whole prompt and a predictor pass.  (Exact equality is not expected: libm and CUDA differ by an
    ulp in rsqrtf/expf/cosf/sinf, and a flipped bf16 rounding spreads through 28 layers.)"""
    cfg = as_kwargs(cfgs_greedy())
    cpu = orc.OracleSession(oracle_model, 64, 9)
    gpu = orc.OracleSession(oracle_model, 64, 9, backend=KernelBackend(ops))
    cpu.prefill(PROMPT_TEXT[:4], PROMPT_CODEC[:4], cfg)
    gpu.prefill(PROMPT_TEXT[:4], PROMPT_CODEC[:4], cfg)
    a, b = orc.from_bf16(cpu.last_hidden), orc.from_bf16(gpu.last_hidden)
    cos = float(np.dot(a, b) / (np.linalg.norm(a) * np.linalg.norm(b)))
    assert cos > 0.999, cos
    la, lb = orc.from_bf16(cpu.trace["talker_logits"]), orc.from_bf16(gpu.trace["talker_logits"])
    assert np.abs(la - lb).max() < 0.15 * la.std() + 1e-3, (np.abs(la - lb).max(), la.std())


def cfgs_greedy():
    class G:
        do_sample, top_k, top_p, temperature, repetition_penalty = False, 0, 1.0, 1.0, 1.0
    return G


@pytest.mark.parametrize("sampled", [False, True])
def test_frames_match_the_oracle(q3t, orc, ops, model, oracle_model, sampled):
    """Prefill + two frames through the C ABI equal, bit for bit, the oracle's frame algorithm
    evaluated with this library's operators: first semantic token, all 16 codes of each frame,
    the next semantic tokens, the final-normed hidden state and the RNG state."""
    tcfg, pcfg = cfgs(q3t, sampled)
    seed = 4242
    s = start(q3t, model, seed, sampled)
    o = orc.OracleSession(oracle_model, 64, seed, backend=KernelBackend(ops))
    o.mask_eos = True
    first = o.prefill(PROMPT_TEXT, PROMPT_CODEC, as_kwargs(tcfg))
    hidden, _, rng = s.read_state()
    assert np.array_equal(hidden, o.last_hidden), int(orc.bf16_ulp_distance(hidden, o.last_hidden).max())
    assert s.current_semantic_token == first
    assert rng == o.rng
    for frame in range(2):
        want_codes, want_next = o.frame(555 + frame, as_kwargs(tcfg), as_kwargs(pcfg))
        got = s.next_frame(555 + frame)
        assert list(got.codes) == want_codes, (frame, got.codes, want_codes)
        assert got.next_semantic_token == want_next
        assert got.talker_position == len(PROMPT_TEXT) + frame
    assert s.read_state()[2] == o.rng
    st = s.runtime_state()
    assert (st.frames_generated, st.device_sample_count, st.host_sync_count) == (2, 1 + 2 * 16, 1 + 2)
    assert st.semantic_history_count == 3 and st.talker_position == len(PROMPT_TEXT) + 2
    s.close()


def run_solo(q3t, model, seed, frames, sampled=True):
    s = start(q3t, model, seed, sampled)
    out = []
    for f in range(frames):
        fr = s.next_frame(100 + f)
        out.append((fr.codes, fr.next_semantic_token))
    s.close()
    return out


def lockstep(q3t, model, seeds, frames):
    n = len(seeds)
    sessions = [start(q3t, model, seed) for seed in seeds]
    got = {i: [] for i in range(n)}
    for f in range(frames):
        pending = model.batch_begin_device_frames(sessions, [100 + f] * n)
        assert len({p.lease_id for p in pending}) <= n
        for i, (s, p) in enumerate(zip(sessions, pending)):
            assert p.device_codes and p.ready_event and p.view.code_count == 16
            fr = p.finish_without_consumer()
            _, tokens, _ = s.read_state()
            got[i].append((tuple(int(t) for t in tokens), fr.next_semantic_token))
    return sessions, {seed: got[i] for i, seed in enumerate(seeds)} if len(set(seeds)) == n else got


@pytest.mark.parametrize("n", [2, 3, 8, 9, 20])
def test_lockstep_batch_equals_solo(q3t, model, n):
    """session_bench.rs protocol: identical code sequences with and without batching."""
    frames = 3
    seeds = [1000 + i for i in range(n)]
    # Bit-identity with the solo run needs the reference's summation order, which the SIMT
    # kernels keep and the tensor-core kernels (the default for every row count) do not promise.
    model.set_option("tc_min_rows", 65)
    model.set_option("gemv_mode", 0)
    try:
        solo = {seed: run_solo(q3t, model, seed, frames) for seed in seeds[:3]}
        sessions, got = lockstep(q3t, model, seeds, frames)
    finally:
        model.set_option("tc_min_rows", 9)
        model.set_option("gemv_mode", 1)
    for seed in seeds[:3]:
        assert got[seed] == solo[seed], seed
    # duplicate seed => identical, different seeds => different (session_bench.rs:228-232)
    assert got[seeds[0]] != got[seeds[1]]
    for s in sessions:
        s.close()


@pytest.mark.parametrize("n", [12, 64])
def test_lockstep_on_the_tensor_cores(q3t, orc, model, n):
    """Nine rows and up run the tcgen05 GEMM: K-slices are summed in a fixed order, so a run
    repeats bit for bit and rows with the same seed agree with each other."""
    seeds = [2000 + (i % (n - 2)) for i in range(n)]        # the last two repeat seeds 2000, 2001
    frames = 3
    s1, a = lockstep(q3t, model, seeds, frames)
    hidden = [s.read_state()[0] for s in s1]
    for s in s1:
        s.close()
    s2, b = lockstep(q3t, model, seeds, frames)
    for s in s2:
        s.close()
    assert a == b
    assert a[0] == a[n - 2] and a[1] == a[n - 1] and a[0] != a[1]
    assert np.array_equal(hidden[0], hidden[n - 2])
    assert q3t.library().q3t_kernel_error_count() == 0


@pytest.mark.parametrize("n", [12, 40])
def test_tensor_core_frames_match_the_oracle(q3t, orc, ops, model, oracle_model, n):
    """A lockstep batch on the tensor-core path equals, bit for bit, the oracle's frame algorithm
    evaluated with this library's operators launched at the same row count."""
    tcfg, pcfg = cfgs(q3t, True)
    seed = 777
    sessions = [start(q3t, model, seed + 13 * i) for i in range(n)]
    o = orc.OracleSession(oracle_model, 64, seed, backend=KernelBackend(ops))
    o.mask_eos = True
    o.prefill(PROMPT_TEXT, PROMPT_CODEC, as_kwargs(tcfg))        # prompts run one session at a time
    o.b = KernelBackend(ops, pad_rows=n)
    for frame in range(2):
        want_codes, want_next = o.frame(300 + frame, as_kwargs(tcfg), as_kwargs(pcfg))
        pending = model.batch_begin_device_frames(sessions, [300 + frame] * n)
        got = [p.finish_without_consumer() for p in pending][0]
        _, tokens, _ = sessions[0].read_state()
        assert [int(t) for t in tokens] == want_codes, (frame, list(tokens), want_codes)
        assert got.next_semantic_token == want_next
    assert sessions[0].read_state()[2] == o.rng
    assert q3t.library().q3t_kernel_error_count() == 0
    for s_ in sessions:
        s_.close()


def test_duplicate_seed_and_dropped_sibling(q3t, model):
    a, b, c = start(q3t, model, 7), start(q3t, model, 7), start(q3t, model, 8)
    seq = {0: [], 1: []}
    for f in range(2):
        pend = model.batch_begin_device_frames([a, b, c], [5, 5, 5])
        for i, p in enumerate(pend):
            fr = p.finish_without_consumer()
            if i < 2:
                seq[i].append(fr.next_semantic_token)
    assert seq[0] == seq[1]
    c.close()                                   # drop one participant mid-stream
    want = run_solo(q3t, model, 7, 4)
    for f in range(2, 4):
        pend = model.batch_begin_device_frames([a, b], [100 + f, 100 + f])
        for p in pend:
            p.finish_without_consumer()
    # a and b continued with trailing ids 5,5 then 102,103; re-run solo with the same ids
    s = start(q3t, model, 7)
    nxt = [s.next_frame(5).next_semantic_token, s.next_frame(5).next_semantic_token,
           s.next_frame(102).next_semantic_token, s.next_frame(103).next_semantic_token]
    assert a.current_semantic_token == b.current_semantic_token == nxt[-1]
    assert want  # solo run with other trailing ids simply has to complete
    for x in (a, b, s):
        x.close()


def test_run_frames_equals_stepping(q3t, model):
    a, b = start(q3t, model, 31), start(q3t, model, 31)
    for f in range(3):
        a.next_frame(9)
    total_ms, per_frame = model.run_frames([b], 3, trailing_text_id=9, want_frame_ms=True)
    assert total_ms > 0 and per_frame.shape == (3,) and (per_frame > 0).all()
    ha, ta, ra = a.read_state()
    hb, tb, rb = b.read_state()
    assert np.array_equal(ta, tb) and ra == rb and np.array_equal(ha, hb)
    assert a.runtime_state().talker_position == b.runtime_state().talker_position
    # and both continue identically through the normal API
    assert a.next_frame(1).codes == b.next_frame(1).codes
    a.close()
    b.close()


def test_chunked_prompt_equals_position_by_position(q3t, orc, model):
    """A prompt run as rows of one decoder pass (64 positions per pass) leaves the session where the
    position-by-position path leaves it: bit for bit while every GEMM stays on the SIMT kernels,
    and within bf16 noise when the 9+ row passes go to the tensor cores."""
    rng = np.random.default_rng(5)
    n = 75                                  # two passes: 64 + 11 rows
    text = [int(t) for t in rng.integers(0, 1000, size=n)]
    codec = [int(c) if i % 3 else -1 for i, c in enumerate(rng.integers(0, 2048, size=n))]
    text = [t if i % 5 else -1 for i, t in enumerate(text)]
    text[0], codec[0] = 17, 5               # every position needs text or codec
    for i in range(n):
        if text[i] < 0 and codec[i] < 0:
            codec[i] = 7

    def run(chunk, tc_min_rows):
        model.set_option("prefill_chunk", chunk)
        model.set_option("tc_min_rows", tc_min_rows)
        model.set_option("gemv_mode", 0 if tc_min_rows > 64 else 1)     # 65: SIMT kernels everywhere
        try:
            s = start(q3t, model, 31, max_seq=128, prompt=(text, codec))
            first = s.current_semantic_token
            hidden, _, rng_state = s.read_state()
            frames = [s.next_frame(3).codes for _ in range(2)]
            s.close()
            return first, hidden, rng_state, frames
        finally:
            model.set_option("prefill_chunk", 64)
            model.set_option("tc_min_rows", 9)
            model.set_option("gemv_mode", 1)

    one = run(1, 65)
    rows = run(64, 65)
    assert rows[0] == one[0] and rows[2] == one[2]
    assert np.array_equal(rows[1], one[1])
    assert rows[3] == one[3]                # the KV cache they left behind is the same too
    tc = run(64, 9)
    again = run(64, 9)
    assert tc[0] == again[0] and np.array_equal(tc[1], again[1]) and tc[3] == again[3]
    a, b = orc.from_bf16(tc[1]).ravel(), orc.from_bf16(one[1]).ravel()
    assert float(a @ b / np.sqrt((a @ a) * (b @ b))) > 0.995
    assert q3t.library().q3t_kernel_error_count() == 0


def test_host_pump_equals_stepping(q3t, model):
    """The compiled host loop over the exported ABI produces what the same calls made one by one do."""
    for n in (1, 3):
        a = [start(q3t, model, 900 + i) for i in range(n)]
        b = [start(q3t, model, 900 + i) for i in range(n)]
        for f in range(3):
            if n == 1:
                a[0].next_frame(9)
            else:
                for p in model.batch_begin_device_frames(a, [9] * n):
                    p.finish_without_consumer()
        wall_ms = model.host_pump_frames(b, 3, trailing_text_id=9)
        assert wall_ms > 0
        for x, y in zip(a, b):
            hx, tx, rx = x.read_state()
            hy, ty, ry = y.read_state()
            assert np.array_equal(tx, ty) and rx == ry and np.array_equal(hx, hy)
            assert x.current_semantic_token == y.current_semantic_token
        for s_ in a + b:
            s_.close()


def test_frame_pump_batches_concurrent_owners(q3t, model):
    """Twelve owner threads ask for frames through the C++ rendezvous: the first frame of each
    bypasses it, later frames share lockstep batches, and every session ends where it ends when
    stepped alone (SIMT kernels for every row count, so batching cannot change a bit)."""
    import threading
    n, frames = 12, 4
    model.set_option("tc_min_rows", 65)
    model.set_option("gemv_mode", 0)
    pump = q3t.native.BatchFramePump(model, max_batch=64, window_us=20000)
    try:
        solo = [run_solo(q3t, model, 400 + i, frames) for i in range(n)]
        sessions = [start(q3t, model, 400 + i) for i in range(n)]
        got = [[] for _ in range(n)]
        errors = []

        def owner(i):
            try:
                pump.register()
                for f in range(frames):
                    pending = pump.begin(sessions[i], 100 + f)
                    fr = pending.finish_without_consumer()
                    _, tokens, _ = sessions[i].read_state()
                    got[i].append((tuple(int(t) for t in tokens), fr.next_semantic_token))
            except Exception as exc:      # surfaced below, on the main thread
                errors.append(exc)
            finally:
                pump.unregister()

        threads = [threading.Thread(target=owner, args=(i,)) for i in range(n)]
        for t in threads:
            t.start()
        for t in threads:
            t.join(timeout=120)
        assert not errors, errors
        for i in range(n):
            assert [(tuple(c), nxt) for c, nxt in solo[i]] == got[i], i
        batches, pumped = pump.statistics()
        assert pumped == n * (frames - 1)              # first frames went around the pump
        assert batches < pumped                        # and later ones were really shared
        for s_ in sessions:
            s_.close()
    finally:
        pump.close()
        model.set_option("tc_min_rows", 9)
        model.set_option("gemv_mode", 1)
    assert q3t.native.pick_device([3, 1, 1, 2]) == 1 and q3t.native.pick_device([0]) == 0
    assert q3t.native.pick_device([]) == -1


def test_device_frame_lease_protocol(q3t, model):
    s = start(q3t, model, 55)
    err = C.create_string_buffer(256)
    lib = q3t.library()
    p = s.begin_device_frame(3)
    assert p.lease_id >= 1 and p.view.device_index == 0
    # a second begin, a prefill or a reset while the lease is out: STATE, nothing enqueued
    with pytest.raises(q3t.NativeTalkerStatusError) as e:
        s.begin_device_frame(3)
    assert e.value.status == q3t.native.STATUS_STATE
    with pytest.raises(q3t.NativeTalkerStatusError):
        s.reset(1)
    # stale lease id
    nxt = C.c_uint16()
    info = q3t.native.FrameInfoC()
    rc = lib.qwen3_tts_session_next_frame_finish_v2(s._handle, p.lease_id + 17, None, C.byref(nxt),
                                                   C.byref(info), err, 256)
    assert rc == q3t.native.STATUS_STATE and b"lease" in err.value
    fr = p.finish_without_consumer()
    assert fr.predictor_gpu_milliseconds > 0 and fr.talker_gpu_milliseconds > 0
    # finish without begin
    rc = lib.qwen3_tts_session_next_frame_finish_v2(s._handle, p.lease_id, None, C.byref(nxt),
                                                   C.byref(info), err, 256)
    assert rc == q3t.native.STATUS_STATE
    # view with a wrong struct_size / reserved field: INVALID_ARGUMENT
    view = q3t.native.DeviceFrameViewV2C()
    view.struct_size = 8
    rc = lib.qwen3_tts_session_next_frame_begin_v2(s._handle, 0, s.talker_sampling.to_c(),
                                                  s.predictor_sampling.to_c(), C.byref(view), err, 256)
    assert rc == q3t.native.STATUS_INVALID_ARGUMENT
    s.close()


def test_argument_and_state_errors(q3t, model):
    lib = q3t.library()
    err = C.create_string_buffer(256)
    s = model.create_session(16, 3)
    # frame before prefill
    with pytest.raises(q3t.NativeTalkerStatusError) as e:
        s.next_frame(0)
    assert e.value.status == q3t.native.STATUS_STATE and "prefill" in e.value.message
    # prompt longer than the KV capacity, empty prompt, position without input
    for text, codec in (([1] * 17, [1] * 17), ([], []), ([-1], [-1])):
        with pytest.raises(q3t.NativeTalkerStatusError):
            s.prefill(text, codec)
    s.prefill([5, 6], [-1, 7])
    # invalid sampling configurations (talker.cu:3588-3591)
    for bad in (q3t.SamplingConfig(True, -1, 1.0, 1.0, 1.0), q3t.SamplingConfig(True, 5, 0.0, 1.0, 1.0),
                q3t.SamplingConfig(True, 5, 1.5, 1.0, 1.0), q3t.SamplingConfig(True, 5, 1.0, 0.0, 1.0),
                q3t.SamplingConfig(True, 5, 1.0, 1.0, 0.0)):
        s.talker_sampling = bad
        with pytest.raises(q3t.NativeTalkerStatusError):
            s.next_frame(0)
    s.talker_sampling = q3t.SamplingConfig.official_talker_defaults()
    # wrong semantic token, text id out of range, undersized code buffer
    codes = (C.c_uint16 * 16)()
    nxt = C.c_uint16()
    info = q3t.native.FrameInfoC()
    wrong = (s.current_semantic_token + 1) % 2048
    rc = lib.qwen3_tts_session_next_frame(s._handle, wrong, 0, s.talker_sampling.to_c(),
                                          s.predictor_sampling.to_c(), codes, 16, C.byref(nxt),
                                          C.byref(info), err, 256)
    assert rc == q3t.native.STATUS_STATE and b"does not match" in err.value
    with pytest.raises(q3t.NativeTalkerStatusError):
        s.next_frame(151936)
    rc = lib.qwen3_tts_session_next_frame(s._handle, s.current_semantic_token, 0,
                                          s.talker_sampling.to_c(), s.predictor_sampling.to_c(), codes,
                                          15, C.byref(nxt), C.byref(info), err, 256)
    assert rc == q3t.native.STATUS_INVALID_ARGUMENT
    # the session is still usable and fills its KV capacity exactly
    frames = 0
    while True:
        try:
            s.next_frame(1)
            frames += 1
        except q3t.NativeTalkerStatusError as full:
            assert "full" in full.message
            break
    assert frames == 16 - 2
    # out-of-range session capacity, batch of zero and of 65
    with pytest.raises(q3t.NativeTalkerStatusError):
        model.create_session(15, 0)
    with pytest.raises(q3t.NativeTalkerStatusError):
        model.create_session(8193, 0)
    views = (q3t.native.DeviceFrameViewV2C * 1)()
    rc = lib.qwen3_tts_model_batch_next_frame_begin_v2(model._handle, None, 0, None, None, None, views,
                                                      err, 256)
    assert rc == q3t.native.STATUS_INVALID_ARGUMENT
    s.close()


def test_upload_validation(q3t, synth):
    m = q3t.NativeTalkerModel.create(0)
    good = synth.make_tensor("talker.model.norm.weight", (2048,), 0)
    with pytest.raises(q3t.NativeTalkerStatusError) as e:
        m.upload_tensor("talker.model.norm.weight", good[:100].copy())
    assert e.value.status == q3t.native.STATUS_MODEL and "shape" in e.value.message
    with pytest.raises(q3t.NativeTalkerStatusError):
        m.upload_tensor("not.a.tensor", good)
    m.upload_tensor("talker.model.norm.weight", good)
    with pytest.raises(q3t.NativeTalkerStatusError) as e:
        m.upload_tensor("talker.model.norm.weight", good)
    assert "duplicate" in e.value.message
    with pytest.raises(q3t.NativeTalkerStatusError) as e:
        m.finalize()
    assert "missing" in e.value.message or "404" in e.value.message
    with pytest.raises(q3t.NativeTalkerStatusError):
        m.create_session(64, 0)                 # not finalized
    m.close()


def test_seed_zero_and_reset(q3t, model):
    a = start(q3t, model, 0)
    b = start(q3t, model, 0x9E3779B97F4A7C15)   # what seed 0 is replaced by (talker.cu:1022)
    assert a.next_frame(2).codes == b.next_frame(2).codes
    first = a.current_semantic_token
    a.reset(0)
    assert a.runtime_state().phase == 1 and a.runtime_state().talker_position == 0
    a.prefill(PROMPT_TEXT, PROMPT_CODEC)
    b.reset(0)
    b.prefill(PROMPT_TEXT, PROMPT_CODEC)
    assert a.current_semantic_token == b.current_semantic_token
    assert a.next_frame(2).codes == b.next_frame(2).codes
    assert first >= 0
    a.close()
    b.close()


def test_weight_image_hand_over(q3t, model, checkpoint):
    """A second replica built from the first one's decode-form tensors (int8 rows, row scales, bf16
    leftovers copied device to device and adopted) counts the same 404 tensors and decodes the same
    frames; a tensor can be adopted only once, unknown names are refused, and a replica with a
    tensor missing does not finalize."""
    import importlib
    dp = importlib.import_module("qwen3-tts-native_b200.dp")
    names = list(checkpoint.keys())
    image = model.tensor_image("talker.model.layers.3.self_attn.k_proj.weight")
    assert image.quantized == 1 and image.loaded == 1
    assert image.data_bytes == 1024 * 2048 and image.scales_bytes == 1024 * 4
    norm = model.tensor_image("talker.model.norm.weight")
    assert norm.quantized == 0 and norm.data_bytes == 2048 * 2 and not norm.scales

    replica = q3t.NativeTalkerModel.create(0)
    try:
        copied = dp.copy_weight_image(model, replica, names[:-1])
        with pytest.raises(q3t.NativeTalkerStatusError, match="duplicate"):
            replica.adopt_tensor(names[0])
        with pytest.raises(q3t.NativeTalkerStatusError, match="not part of"):
            replica.tensor_image("talker.no_such.weight")
        with pytest.raises(q3t.NativeTalkerStatusError):
            replica.finalize()                                   # one tensor still missing
        copied += dp.copy_weight_image(model, replica, names[-1:])
        memory = replica.finalize()
        assert memory.tensor_count == 404
        assert memory.shared_weight_bytes == model.memory.shared_weight_bytes
        assert 2_000_000_000 < copied < memory.shared_weight_bytes   # the image is smaller than the checkpoint
        replica.set_option("mask_eos", 1)
        a, b = start(q3t, model, 4242), start(q3t, replica, 4242)
        for _ in range(3):
            fa, fb = a.next_frame(9), b.next_frame(9)
            assert np.array_equal(fa.codes, fb.codes)
        ha, ta, ra = a.read_state()
        hb, tb, rb = b.read_state()
        assert np.array_equal(ha, hb) and np.array_equal(ta, tb) and ra == rb
        a.close()
        b.close()
    finally:
        replica.close()
