"""CPU-only checks of the drop-in boundary: the shared library loads without a GPU, exports
every symbol the headers in include/ declare, and the host-side structs have the layouts the
reference's Rust host pins (native_talker.rs:1733-1743: 20/12/16/16/32/40/40 bytes)."""
import ctypes as C
import os
import re

import pytest

from conftest import ROOT


def _declared_symbols():
    names = []
    for header in ("qwen3_tts_native.h", "q3t_ops.h"):
        text = open(os.path.join(ROOT, "include", header)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names += re.findall(r"QWEN3_TTS_API\s+[\w\s\*]+?\b(q(?:wen3_tts|3t)_\w+)\s*\(", text)
    return names


def test_headers_declare_the_reference_surface():
    names = _declared_symbols()
    assert len(names) == len(set(names))
    for required in ("qwen3_tts_talker_abi_version", "qwen3_tts_model_create",
                     "qwen3_tts_model_upload_tensor", "qwen3_tts_model_finalize",
                     "qwen3_tts_session_create", "qwen3_tts_session_prefill",
                     "qwen3_tts_session_next_frame", "qwen3_tts_session_next_frame_begin_v2",
                     "qwen3_tts_session_next_frame_finish_v2",
                     "qwen3_tts_model_batch_next_frame_begin_v2", "qwen3_tts_session_state_info"):
        assert required in names


def test_library_exports_every_declared_symbol(q3t):
    lib = q3t.library()
    declared = _declared_symbols()
    assert set(declared) == set(q3t.native.EXPORTED_SYMBOLS)
    for name in declared:
        assert getattr(lib, name) is not None, name


def test_abi_version_and_limits(q3t):
    assert q3t.library().qwen3_tts_talker_abi_version() == 3
    header = open(os.path.join(ROOT, "include", "qwen3_tts_native.h")).read()
    assert "#define QWEN3_TTS_MAX_BATCH_SESSIONS 64" in header
    assert q3t.native.MAX_BATCH_SESSIONS == 64


def test_struct_layouts(q3t):
    n = q3t.native
    assert C.sizeof(n.SamplingConfigC) == 20
    assert C.sizeof(n.PrefillResultC) == 12
    assert C.sizeof(n.FrameInfoC) == 16
    assert C.sizeof(n.ModelMemoryC) == 16
    assert C.sizeof(n.SessionMemoryC) == 32
    assert C.sizeof(n.StateInfoC) == 40
    assert C.sizeof(n.DeviceFrameViewV2C) == 40 and C.alignment(n.DeviceFrameViewV2C) == 8
    assert C.sizeof(n.ArgmaxBenchmarkC) == 24
    assert C.sizeof(n.WeightUploadMetricsC) == 64
    assert n.DeviceFrameViewV2C.lease_id.offset == 24
    assert n.DeviceFrameViewV2C.device_index.offset == 32


def test_sampling_defaults(q3t):
    t = q3t.SamplingConfig.official_talker_defaults()
    p = q3t.SamplingConfig.official_predictor_defaults()
    g = q3t.SamplingConfig.greedy()
    assert (t.do_sample, t.top_k, t.top_p, t.temperature, t.repetition_penalty) == (True, 50, 1.0, 0.9, 1.05)
    assert p.repetition_penalty == 1.0 and p.top_k == 50
    assert not g.do_sample and g.top_k == 0


def test_null_arguments_are_rejected_without_touching_cuda(q3t):
    lib = q3t.library()
    err = C.create_string_buffer(128)
    # null output pointers: INVALID_ARGUMENT before any CUDA call (talker.cu:3825, 3877)
    assert lib.qwen3_tts_model_create(0, None, err, 128) == q3t.native.STATUS_INVALID_ARGUMENT
    assert err.value
    assert lib.qwen3_tts_session_create(None, 64, 0, None, None, err, 128) == q3t.native.STATUS_INVALID_ARGUMENT
    assert lib.qwen3_tts_session_state_info(None, None, err, 128) == q3t.native.STATUS_INVALID_ARGUMENT
    # a null handle is a STATE error with a message, not a crash
    info = q3t.native.StateInfoC()
    assert lib.qwen3_tts_session_state_info(None, C.byref(info), err, 128) == q3t.native.STATUS_STATE
    assert b"null" in err.value
    # capacity 0 / null error buffer are tolerated
    assert lib.qwen3_tts_session_state_info(None, C.byref(info), None, 0) == q3t.native.STATUS_STATE
    one = C.create_string_buffer(1)
    assert lib.qwen3_tts_session_state_info(None, C.byref(info), one, 1) == q3t.native.STATUS_STATE
    assert one.raw == b"\x00"


def test_synthetic_checkpoint_inventory(synth):
    shapes = synth.tensor_shapes()
    assert len(shapes) == 404                       # talker.cu:488
    assert shapes["talker.model.text_embedding.weight"] == (151936, 2048)
    assert shapes["talker.code_predictor.model.layers.0.self_attn.q_proj.weight"] == (2048, 1024)
    assert shapes["talker.code_predictor.lm_head.14.weight"] == (2048, 1024)
    small = synth.tensor_shapes(predictor_head_dim=64)
    assert small["talker.code_predictor.model.layers.0.self_attn.k_proj.weight"] == (512, 1024)
    a = synth.make_tensor("talker.model.norm.weight", (2048,), 0)
    b = synth.make_tensor("talker.model.norm.weight", (2048,), 0)
    assert (a == b).all() and a.dtype.name == "uint16"


def test_missing_library_fails_loudly(q3t, monkeypatch):
    monkeypatch.setenv("QWEN3_TTS_TALKER_LIBRARY", "/nonexistent/libqwen3_tts_cuda.so")
    monkeypatch.setattr(q3t.native, "_lib", None)
    with pytest.raises(ImportError):
        q3t.native.library()


# ---- shared-memory plan of the 1..8-row projection kernel (host arithmetic, no GPU) ----------

# (in_features, out_features, gate/up, norm prologue): every projection shape of the model
PROJECTION_SHAPES = [
    (2048, 4096, 0, 1), (2048, 2048, 0, 0), (2048, 6144, 1, 1), (6144, 2048, 0, 0),      # talker layer
    (1024, 4096, 0, 1), (2048, 1024, 0, 0), (1024, 3072, 1, 1), (3072, 1024, 0, 0),      # predictor layer
    (2048, 3072, 0, 1), (1024, 2048, 0, 1), (2048, 1024, 0, 0), (2048, 2048, 0, 0),      # heads, input and text projections
    (2048, 6144, 0, 0),                                                                  # the benchmark's configs[0]
]


@pytest.mark.parametrize("k,n,gate_up,norm", PROJECTION_SHAPES)
def test_projection_plan_keeps_every_stage_inside_the_allocation(q3t, k, n, gate_up, norm):
    """The kernel's tile loop reads all sixteen rows of a weight stage whatever was copied into it, so
    a launch is safe only if every stage, read at full height, lies inside its dynamic shared memory;
    a tile group must not be larger than the ring (its tiles are all resident before it starts); and
    the launch must fit what one SM has.  (A plan that let a short last stage stick out of the
    allocation once ended in an illegal shared-memory access on a one-row launch.)"""
    lib = q3t.library()
    lib.q3t_test_gemv_plan.argtypes = [C.c_int32] * 5 + [C.POINTER(C.c_int64)]
    taken = 0
    for rows in range(1, 9):
        f = (C.c_int64 * 8)()
        if not lib.q3t_test_gemv_plan(k, n, rows, gate_up, norm, f):
            continue
        taken += 1
        grid, stages, group, tiles, per_launch, stage_bytes, ring_bytes, shared_bytes = (int(v) for v in f)
        assert 1 <= grid <= 148 and tiles >= 1
        assert 1 <= group <= stages <= max(tiles, 1)
        assert stage_bytes == 2 * (8 * k + 64)
        assert stages * stage_bytes <= shared_bytes, (rows, stages, stage_bytes, shared_bytes)
        assert ring_bytes % 16 == 0 and ring_bytes <= shared_bytes <= 200 * 1024
        assert 1 <= per_launch <= 8
        if rows <= 2 and shared_bytes <= 113 * 1024:
            assert 2 * shared_bytes <= 227 * 1024          # room for the next launch's CTA beside this one
    # every shape of the model is taken at one row (larger row counts may run as several launches)
    f = (C.c_int64 * 8)()
    assert lib.q3t_test_gemv_plan(k, n, 1, gate_up, norm, f) == 1
    assert taken >= 1


def test_projection_plan_refuses_what_the_kernel_does_not_take(q3t):
    lib = q3t.library()
    lib.q3t_test_gemv_plan.argtypes = [C.c_int32] * 5 + [C.POINTER(C.c_int64)]
    f = (C.c_int64 * 8)()
    assert lib.q3t_test_gemv_plan(1536, 300, 1, 0, 0, f) == 0        # K = 512 * 3 is not built
    assert lib.q3t_test_gemv_plan(3072, 1024, 1, 0, 1, f) == 0       # norm prologue only for K = 1024, 2048
    assert lib.q3t_test_gemv_plan(2048, 4096, 9, 0, 0, f) == 0       # more than eight rows per launch
    assert lib.q3t_test_gemv_plan(2000, 4096, 1, 0, 0, f) == 0
