"""Host-side binding of libqwen3_tts_cuda.so.

Python counterpart of the reference's Rust host wrapper
(native/qwen3-tts-native/src/native_talker.rs): the same objects and method names
(NativeTalkerModel.load / start_prompt, NativeTalkerSession.next_frame /
begin_device_frame / finish, SamplingConfig.official_*_defaults, NativeTalkerStatusError)
over the same C symbols, resolved by name from the shared library exactly as the Rust
crate does with libloading (native_talker.rs:776-821).  There is no CPU fallback: if the
library is missing, import fails with the build command to run.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass
from typing import Iterable, Optional, Sequence, Tuple

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIBRARY_NAME = "libqwen3_tts_cuda.so"
LIBRARY_PATH = os.path.join(_HERE, LIBRARY_NAME)

ABI_VERSION = 3
MAX_BATCH_SESSIONS = 64
CODEBOOKS = 16
EOS = 2150
TALKER_VOCAB = 3072
TEXT_VOCAB = 151936

STATUS_OK, STATUS_INVALID_ARGUMENT, STATUS_CUDA, STATUS_STATE, STATUS_ALLOCATION, STATUS_MODEL = (
    0, -1, -2, -3, -4, -5)


class SamplingConfigC(C.Structure):   # qwen3_tts_native.h Qwen3TtsSamplingConfig (20 bytes)
    _fields_ = [("do_sample", C.c_int32), ("top_k", C.c_int32), ("top_p", C.c_float),
                ("temperature", C.c_float), ("repetition_penalty", C.c_float)]


class PrefillResultC(C.Structure):    # 12 bytes
    _fields_ = [("first_semantic_token", C.c_uint16), ("reserved", C.c_uint16),
                ("prompt_tokens", C.c_uint32), ("talker_gpu_milliseconds", C.c_float)]


class FrameInfoC(C.Structure):        # 16 bytes
    _fields_ = [("talker_position", C.c_uint32), ("ended_by_eos", C.c_uint32),
                ("predictor_gpu_milliseconds", C.c_float), ("talker_gpu_milliseconds", C.c_float)]


class DeviceFrameViewV2C(C.Structure):   # 40 bytes, align 8
    _fields_ = [("struct_size", C.c_uint32), ("code_count", C.c_uint32),
                ("device_codes", C.c_void_p), ("ready_event", C.c_void_p),
                ("lease_id", C.c_uint64), ("device_index", C.c_int32), ("reserved", C.c_uint32)]


class StateInfoC(C.Structure):        # 40 bytes
    _fields_ = [("abi_version", C.c_uint32), ("phase", C.c_uint32),
                ("talker_position", C.c_uint32), ("semantic_history_count", C.c_uint32),
                ("frames_generated", C.c_uint64), ("device_sample_count", C.c_uint64),
                ("host_sync_count", C.c_uint64)]


class TensorImageC(C.Structure):      # q3t_ops.h Q3tTensorImage
    _fields_ = [("struct_size", C.c_uint32), ("device_index", C.c_int32), ("data", C.c_void_p),
                ("data_bytes", C.c_uint64), ("scales", C.c_void_p), ("scales_bytes", C.c_uint64),
                ("quantized", C.c_int32), ("loaded", C.c_int32)]


class ModelMemoryC(C.Structure):      # 16 bytes
    _fields_ = [("shared_weight_bytes", C.c_uint64), ("tensor_count", C.c_uint32),
                ("device_index", C.c_int32)]


class SessionMemoryC(C.Structure):    # 32 bytes
    _fields_ = [("talker_kv_bytes", C.c_uint64), ("predictor_kv_bytes", C.c_uint64),
                ("workspace_bytes", C.c_uint64), ("max_sequence_length", C.c_uint32),
                ("reserved", C.c_uint32)]


class PrimitiveParityC(C.Structure):
    _fields_ = [("rms_norm_max_absolute_error", C.c_float), ("rope_max_absolute_error", C.c_float),
                ("attention_max_absolute_error", C.c_float), ("silu_gate_max_absolute_error", C.c_float)]


class GemvBenchmarkC(C.Structure):
    _fields_ = [("input_features", C.c_int32), ("output_features", C.c_int32),
                ("iterations", C.c_int32), ("reserved", C.c_int32), ("weight_bytes", C.c_uint64),
                ("cold_launch_microseconds", C.c_float), ("mean_launch_microseconds", C.c_float),
                ("tera_operations_per_second", C.c_float)]


class DeviceInfoC(C.Structure):
    _fields_ = [("device_index", C.c_int32), ("compute_major", C.c_int32),
                ("compute_minor", C.c_int32), ("total_global_memory_bytes", C.c_uint64),
                ("runtime_free_memory_bytes", C.c_uint64), ("runtime_total_memory_bytes", C.c_uint64),
                ("device_name", C.c_char * 256)]


# every symbol the headers in include/ declare
EXPORTED_SYMBOLS = (
    "qwen3_tts_talker_abi_version", "qwen3_tts_probe_device",
    "qwen3_tts_benchmark_bf16_argmax", "qwen3_tts_benchmark_bf16_gemv",
    "qwen3_tts_device_buffer_create", "qwen3_tts_device_buffer_upload", "qwen3_tts_device_buffer_finish",
    "qwen3_tts_device_buffer_read", "qwen3_tts_device_buffer_data", "qwen3_tts_device_buffer_destroy",
    "qwen3_tts_validate_transformer_primitives", "qwen3_tts_model_create",
    "qwen3_tts_model_destroy", "qwen3_tts_model_upload_tensor", "qwen3_tts_model_finalize",
    "qwen3_tts_session_create", "qwen3_tts_session_destroy", "qwen3_tts_session_reset",
    "qwen3_tts_session_prefill", "qwen3_tts_session_next_frame",
    "qwen3_tts_session_next_frame_begin_v2", "qwen3_tts_session_next_frame_finish_v2",
    "qwen3_tts_model_batch_next_frame_begin_v2", "qwen3_tts_session_state_info",
    "q3t_launch_int8_gemm_rows", "q3t_launch_int8_gemm_rows_add",
    "q3t_launch_int8_gate_up_silu_rows", "q3t_launch_int8_gemm_ex",
    "q3t_launch_quantize_weight_rows", "q3t_benchmark_int8_gemv", "q3t_launch_rms_norm_rows",
    "q3t_set_gemv_mode", "q3t_test_gemv_plan", "q3t_set_attention_mode", "q3t_benchmark_decode_attention", "q3t_attention_range_error_count", "q3t_test_fail_launch_after", "q3t_test_fail_allocation_after",
    "q3t_test_report_device_wait_failure", "q3t_host_pump_frames",
    "q3t_pump_create", "q3t_pump_destroy", "q3t_pump_register", "q3t_pump_unregister",
    "q3t_pump_begin_frame", "q3t_pump_statistics", "q3t_pick_device",
    "q3t_launch_head_rms_norm_rows", "q3t_launch_rope_rows_at", "q3t_launch_kv_scatter_rows",
    "q3t_launch_bias_activation_rows", "q3t_launch_add_in_place", "q3t_launch_silu_gate",
    "q3t_launch_gather_embedding_rows", "q3t_launch_add_embedding_rows",
    "q3t_attention_scratch_bytes", "q3t_launch_batch_causal_gqa_attention_fast",
    "q3t_launch_decode_attention_ex", "q3t_launch_sample_logits", "q3t_launch_sample_logits_at",
    "q3t_model_set_option", "q3t_model_run_frames", "q3t_session_read_state", "q3t_session_read_kv",
    "q3t_session_synthetic_prefill", "q3t_model_kernel_launches", "q3t_session_current_token",
    "q3t_launch_batch_causal_gqa_attention_fast_noalloc", "q3t_attention_static_scratch_capacity",
    "q3t_kernel_error_count", "q3t_model_tensor_image", "q3t_model_adopt_tensor",
    "q3t_packet_stager_create", "q3t_packet_stager_destroy", "q3t_packet_stager_device_bytes",
    "q3t_packet_stager_staged_frames", "q3t_packet_stager_stage_frame", "q3t_packet_stager_packet_view",
    "q3t_packet_stager_release_after_consumer",
)

_lib: Optional[C.CDLL] = None


def library() -> C.CDLL:
    """dlopen the CUDA library; fails loudly when it has not been built."""
    global _lib
    if _lib is None:
        path = os.environ.get("QWEN3_TTS_TALKER_LIBRARY", LIBRARY_PATH)
        if not os.path.exists(path):
            raise ImportError(
                f"{path} is missing: build it with `python qwen3-tts-native_b200/build.py` "
                "(there is no CPU fallback for the decode path)")
        lib = C.CDLL(path)
        lib.qwen3_tts_talker_abi_version.restype = C.c_uint32
        # (a library that exports only the reference's own ABI may be loaded through
        # QWEN3_TTS_TALKER_LIBRARY for side-by-side runs: the q3t_* additions are then absent)
        for name, restype in (("q3t_attention_scratch_bytes", C.c_size_t),
                              ("q3t_attention_static_scratch_capacity", C.c_size_t),
                              ("q3t_kernel_error_count", C.c_uint32),
                              ("q3t_test_fail_launch_after", None),
                              ("q3t_test_fail_allocation_after", None)):
            if hasattr(lib, name):
                getattr(lib, name).restype = restype
        lib.qwen3_tts_model_destroy.restype = None
        lib.qwen3_tts_session_destroy.restype = None
        lib.qwen3_tts_model_destroy.argtypes = [C.c_void_p]
        lib.qwen3_tts_session_destroy.argtypes = [C.c_void_p]
        lib.qwen3_tts_session_next_frame.argtypes = [
            C.c_void_p, C.c_uint16, C.c_int32, SamplingConfigC, SamplingConfigC,
            C.POINTER(C.c_uint16), C.c_size_t, C.POINTER(C.c_uint16), C.POINTER(FrameInfoC),
            C.c_char_p, C.c_size_t]
        lib.qwen3_tts_session_next_frame_begin_v2.argtypes = [
            C.c_void_p, C.c_int32, SamplingConfigC, SamplingConfigC, C.POINTER(DeviceFrameViewV2C),
            C.c_char_p, C.c_size_t]
        lib.qwen3_tts_session_next_frame_finish_v2.argtypes = [
            C.c_void_p, C.c_uint64, C.c_void_p, C.POINTER(C.c_uint16), C.POINTER(FrameInfoC),
            C.c_char_p, C.c_size_t]
        lib.qwen3_tts_session_prefill.argtypes = [
            C.c_void_p, C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.c_int32, SamplingConfigC,
            C.POINTER(PrefillResultC), C.c_char_p, C.c_size_t]
        lib.qwen3_tts_model_batch_next_frame_begin_v2.argtypes = [
            C.c_void_p, C.POINTER(C.c_void_p), C.c_int32, C.POINTER(C.c_int32),
            C.POINTER(SamplingConfigC), C.POINTER(SamplingConfigC), C.POINTER(DeviceFrameViewV2C),
            C.c_char_p, C.c_size_t]
        lib.qwen3_tts_model_upload_tensor.argtypes = [
            C.c_void_p, C.c_char_p, C.c_void_p, C.c_uint64, C.c_int32, C.POINTER(C.c_uint64),
            C.c_char_p, C.c_size_t]
        lib.qwen3_tts_session_create.argtypes = [
            C.c_void_p, C.c_int32, C.c_uint64, C.POINTER(C.c_void_p), C.POINTER(SessionMemoryC),
            C.c_char_p, C.c_size_t]
        lib.qwen3_tts_session_reset.argtypes = [C.c_void_p, C.c_uint64, C.c_char_p, C.c_size_t]
        lib.qwen3_tts_session_state_info.argtypes = [C.c_void_p, C.POINTER(StateInfoC), C.c_char_p,
                                                     C.c_size_t]
        lib.qwen3_tts_model_create.argtypes = [C.c_int32, C.POINTER(C.c_void_p), C.c_char_p, C.c_size_t]
        lib.qwen3_tts_model_finalize.argtypes = [C.c_void_p, C.POINTER(ModelMemoryC), C.c_char_p,
                                                 C.c_size_t]
        for name, argtypes in (
                ("q3t_model_run_frames", [
                    C.c_void_p, C.POINTER(C.c_void_p), C.c_int32, C.c_int32, C.c_int32, SamplingConfigC,
                    SamplingConfigC, C.POINTER(C.c_float), C.POINTER(C.c_float), C.c_char_p, C.c_size_t]),
                ("q3t_model_set_option", [C.c_void_p, C.c_char_p, C.c_int32, C.c_char_p, C.c_size_t]),
                ("q3t_session_read_state", [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_char_p,
                                            C.c_size_t]),
                ("q3t_session_read_kv", [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p,
                                         C.c_char_p, C.c_size_t]),
                ("q3t_session_synthetic_prefill", [C.c_void_p, C.c_int32, C.c_uint64, C.c_char_p, C.c_size_t]),
                ("q3t_model_kernel_launches", [C.c_void_p, C.POINTER(C.c_uint64), C.c_char_p, C.c_size_t])):
            if hasattr(lib, name):
                getattr(lib, name).argtypes = argtypes
        _lib = lib
    return _lib


class NativeTalkerStatusError(RuntimeError):
    """A call across the C ABI returned a negative status (native_talker.rs:32-57)."""

    def __init__(self, status: int, message: str):
        super().__init__(f"native talker status {status}: {message}")
        self.status = status
        self.message = message


_ERR_CAP = 512


def _check(status: int, err) -> None:
    if status != STATUS_OK:
        raise NativeTalkerStatusError(status, err.value.decode("utf-8", "replace"))


@dataclass(frozen=True)
class SamplingConfig:
    """native_talker.rs:404-445"""
    do_sample: bool = True
    top_k: int = 50
    top_p: float = 1.0
    temperature: float = 0.9
    repetition_penalty: float = 1.0

    @staticmethod
    def official_talker_defaults() -> "SamplingConfig":
        return SamplingConfig(True, 50, 1.0, 0.9, 1.05)

    @staticmethod
    def official_predictor_defaults() -> "SamplingConfig":
        return SamplingConfig(True, 50, 1.0, 0.9, 1.0)

    @staticmethod
    def greedy() -> "SamplingConfig":
        return SamplingConfig(False, 0, 1.0, 1.0, 1.0)

    def to_c(self) -> SamplingConfigC:
        return SamplingConfigC(int(self.do_sample), int(self.top_k), float(self.top_p),
                               float(self.temperature), float(self.repetition_penalty))


@dataclass(frozen=True)
class StreamingCodecFrame:
    codes: Tuple[int, ...]
    next_semantic_token: int
    ended_by_eos: bool
    talker_position: int
    predictor_gpu_milliseconds: float
    talker_gpu_milliseconds: float


@dataclass(frozen=True)
class SessionRuntimeState:
    abi_version: int
    phase: int
    talker_position: int
    semantic_history_count: int
    frames_generated: int
    device_sample_count: int
    host_sync_count: int


class PendingTalkerFrame:
    """A begun frame whose codes live on the device until finish (native_talker.rs:548-626)."""

    def __init__(self, session: "NativeTalkerSession", view: DeviceFrameViewV2C):
        self._session = session
        self.view = view

    @property
    def lease_id(self) -> int:
        return int(self.view.lease_id)

    @property
    def device_codes(self) -> int:
        return int(self.view.device_codes or 0)

    @property
    def ready_event(self) -> int:
        return int(self.view.ready_event or 0)

    def finish(self, consumer_done_event: int = 0) -> StreamingCodecFrame:
        return self._session._finish(self.lease_id, consumer_done_event)

    def finish_without_consumer(self) -> StreamingCodecFrame:
        return self.finish(0)


class NativeTalkerModel:
    """Shared weights on one GPU (native_talker.rs:705-1215)."""

    def __init__(self, handle: int, memory: ModelMemoryC, device_index: int):
        self._handle = C.c_void_p(handle)
        self.memory = memory
        self.device_index = device_index

    @staticmethod
    def create(device_index: int = 0) -> "NativeTalkerModel":
        lib = library()
        err = C.create_string_buffer(_ERR_CAP)
        handle = C.c_void_p()
        _check(lib.qwen3_tts_model_create(device_index, C.byref(handle), err, _ERR_CAP), err)
        return NativeTalkerModel(handle.value, ModelMemoryC(), device_index)

    @staticmethod
    def load(device_index: int, tensors: Iterable[Tuple[str, np.ndarray]]) -> "NativeTalkerModel":
        """Uploads every (name, bf16 bit-pattern array) pair and finalizes."""
        model = NativeTalkerModel.create(device_index)
        try:
            for name, array in tensors:
                model.upload_tensor(name, array)
            model.finalize()
        except Exception:
            model.close()
            raise
        return model

    def upload_tensor(self, name: str, array: np.ndarray) -> None:
        a = np.ascontiguousarray(array)
        if a.dtype != np.uint16:
            raise TypeError("tensors are passed as bf16 bit patterns (uint16)")
        shape = (C.c_uint64 * a.ndim)(*a.shape)
        err = C.create_string_buffer(_ERR_CAP)
        _check(library().qwen3_tts_model_upload_tensor(
            self._handle, name.encode(), a.ctypes.data_as(C.c_void_p), a.nbytes, a.ndim, shape,
            err, _ERR_CAP), err)

    def tensor_image(self, name: str) -> TensorImageC:
        """Device storage of a checkpoint tensor in decode form (int8 rows + fp32 row scales, or bf16)."""
        image = TensorImageC()
        image.struct_size = C.sizeof(TensorImageC)
        err = C.create_string_buffer(_ERR_CAP)
        _check(library().q3t_model_tensor_image(self._handle, name.encode(), C.byref(image), err, _ERR_CAP), err)
        return image

    def adopt_tensor(self, name: str) -> None:
        """Declares the tensor's device storage filled by the caller (broadcast, peer copy, file)."""
        err = C.create_string_buffer(_ERR_CAP)
        _check(library().q3t_model_adopt_tensor(self._handle, name.encode(), err, _ERR_CAP), err)

    def finalize(self) -> ModelMemoryC:
        err = C.create_string_buffer(_ERR_CAP)
        _check(library().qwen3_tts_model_finalize(self._handle, C.byref(self.memory), err, _ERR_CAP), err)
        return self.memory

    def set_option(self, key: str, value: int) -> None:
        err = C.create_string_buffer(_ERR_CAP)
        _check(library().q3t_model_set_option(self._handle, key.encode(), int(value), err, _ERR_CAP), err)

    def kernel_launches(self) -> int:
        out = C.c_uint64(0)
        err = C.create_string_buffer(_ERR_CAP)
        _check(library().q3t_model_kernel_launches(self._handle, C.byref(out), err, _ERR_CAP), err)
        return int(out.value)

    def talker_abi_version(self) -> int:
        return int(library().qwen3_tts_talker_abi_version())

    def supports_device_frames(self) -> bool:
        return True

    def supports_batch_frames(self) -> bool:
        return True

    def create_session(self, max_sequence_length: int, seed: int) -> "NativeTalkerSession":
        err = C.create_string_buffer(_ERR_CAP)
        handle = C.c_void_p()
        memory = SessionMemoryC()
        _check(library().qwen3_tts_session_create(self._handle, max_sequence_length, seed,
                                                  C.byref(handle), C.byref(memory), err, _ERR_CAP), err)
        return NativeTalkerSession(self, handle.value, memory)

    def start_prompt(self, text_ids: Sequence[int], codec_ids: Sequence[int],
                     max_sequence_length: int, seed: int,
                     talker_sampling: SamplingConfig = SamplingConfig.official_talker_defaults(),
                     predictor_sampling: SamplingConfig = SamplingConfig.official_predictor_defaults(),
                     ) -> "NativeTalkerSession":
        """create + prefill (native_talker.rs:911-980)"""
        session = self.create_session(max_sequence_length, seed)
        try:
            session.talker_sampling = talker_sampling
            session.predictor_sampling = predictor_sampling
            session.prefill(text_ids, codec_ids)
        except Exception:
            session.close()
            raise
        return session

    def batch_begin_device_frames(self, sessions: Sequence["NativeTalkerSession"],
                                  trailing_text_ids: Sequence[int]) -> list:
        """One lockstep frame for all sessions (native_talker.rs:314-380)."""
        n = len(sessions)
        handles = (C.c_void_p * n)(*[s._handle for s in sessions])
        trailing = (C.c_int32 * n)(*[int(t) for t in trailing_text_ids])
        talker = (SamplingConfigC * n)(*[s.talker_sampling.to_c() for s in sessions])
        predictor = (SamplingConfigC * n)(*[s.predictor_sampling.to_c() for s in sessions])
        views = (DeviceFrameViewV2C * n)()
        for v in views:
            v.struct_size = C.sizeof(DeviceFrameViewV2C)
            v.reserved = 0
        err = C.create_string_buffer(_ERR_CAP)
        _check(library().qwen3_tts_model_batch_next_frame_begin_v2(
            self._handle, handles, n, trailing, talker, predictor, views, err, _ERR_CAP), err)
        out = []
        for s, v in zip(sessions, views):
            copy = DeviceFrameViewV2C.from_buffer_copy(v)
            out.append(PendingTalkerFrame(s, copy))
        return out

    def host_pump_frames(self, sessions: Sequence["NativeTalkerSession"], frames: int,
                         trailing_text_id: int = 0) -> float:
        """The reference host's per-frame ABI call sequence as a compiled loop; returns wall ms."""
        n = len(sessions)
        handles = (C.c_void_p * n)(*[s._handle for s in sessions])
        last = (C.c_uint16 * n)()
        wall = C.c_double(0.0)
        err = C.create_string_buffer(_ERR_CAP)
        lib = library()
        lib.q3t_host_pump_frames.argtypes = [C.c_void_p, C.POINTER(C.c_void_p), C.c_int32, C.c_int32, C.c_int32,
                                             SamplingConfigC, SamplingConfigC, C.POINTER(C.c_uint16),
                                             C.POINTER(C.c_double), C.c_char_p, C.c_size_t]
        lib.q3t_host_pump_frames.restype = C.c_int32
        _check(lib.q3t_host_pump_frames(self._handle, handles, n, frames, trailing_text_id,
                                        sessions[0].talker_sampling.to_c(), sessions[0].predictor_sampling.to_c(),
                                        last, C.byref(wall), err, _ERR_CAP), err)
        for s, tok in zip(sessions, last):
            s.current_semantic_token = int(tok)
            s.frames_emitted += frames
            s.ended = s.current_semantic_token == EOS
        return float(wall.value)

    def run_frames(self, sessions: Sequence["NativeTalkerSession"], frames: int,
                   trailing_text_id: int = 0, want_frame_ms: bool = False):
        """Frame loop with no host round trip per frame; returns (total_ms, frame_ms|None)."""
        n = len(sessions)
        handles = (C.c_void_p * n)(*[s._handle for s in sessions])
        per_frame = (C.c_float * frames)() if want_frame_ms else None
        total = C.c_float(0.0)
        err = C.create_string_buffer(_ERR_CAP)
        _check(library().q3t_model_run_frames(
            self._handle, handles, n, frames, trailing_text_id,
            sessions[0].talker_sampling.to_c(), sessions[0].predictor_sampling.to_c(),
            per_frame, C.byref(total), err, _ERR_CAP), err)
        for s in sessions:
            tok = C.c_uint16(0)
            _check(library().q3t_session_current_token(s._handle, C.byref(tok), err, _ERR_CAP), err)
            s.current_semantic_token = int(tok.value)
            s.frames_emitted += frames
            s.ended = s.current_semantic_token == EOS
        return float(total.value), (np.array(per_frame[:], dtype=np.float32) if want_frame_ms else None)

    def close(self) -> None:
        if self._handle:
            library().qwen3_tts_model_destroy(self._handle)
            self._handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class NativeTalkerSession:
    """One utterance: KV cache, RNG, history (native_talker.rs:720-762, 1217-1648)."""

    def __init__(self, model: NativeTalkerModel, handle: int, memory: SessionMemoryC):
        self._model = model
        self._handle = C.c_void_p(handle)
        self.memory = memory
        self.talker_sampling = SamplingConfig.official_talker_defaults()
        self.predictor_sampling = SamplingConfig.official_predictor_defaults()
        self.current_semantic_token = 0
        self.frames_emitted = 0
        self.ended = False

    def memory_usage(self) -> SessionMemoryC:
        return self.memory

    def reset(self, seed: int) -> None:
        err = C.create_string_buffer(_ERR_CAP)
        _check(library().qwen3_tts_session_reset(self._handle, seed, err, _ERR_CAP), err)
        self.current_semantic_token = 0
        self.frames_emitted = 0
        self.ended = False

    def prefill(self, text_ids: Sequence[int], codec_ids: Sequence[int]) -> PrefillResultC:
        n = len(text_ids)
        if len(codec_ids) != n:
            raise ValueError("text and codec id arrays differ in length")
        t = (C.c_int32 * max(n, 1))(*[int(x) for x in text_ids])
        c = (C.c_int32 * max(n, 1))(*[int(x) for x in codec_ids])
        out = PrefillResultC()
        err = C.create_string_buffer(_ERR_CAP)
        _check(library().qwen3_tts_session_prefill(self._handle, t, c, n, self.talker_sampling.to_c(),
                                                   C.byref(out), err, _ERR_CAP), err)
        self.current_semantic_token = int(out.first_semantic_token)
        self.ended = self.current_semantic_token == EOS
        self.prefill_result = out
        return out

    def synthetic_prefill(self, position: int, seed: int) -> None:
        """Benchmark harness: PREFILLED at `position` with seeded random KV (no prompt run)."""
        err = C.create_string_buffer(_ERR_CAP)
        _check(library().q3t_session_synthetic_prefill(self._handle, position, seed, err, _ERR_CAP), err)
        self.current_semantic_token = seed % 2048
        self.ended = False

    def next_frame(self, trailing_text_id: int = 0) -> Optional[StreamingCodecFrame]:
        """Host-visible frame (native_talker.rs:1279-1334)."""
        if self.ended:
            return None
        codes = (C.c_uint16 * CODEBOOKS)()
        nxt = C.c_uint16(0)
        info = FrameInfoC()
        err = C.create_string_buffer(_ERR_CAP)
        _check(library().qwen3_tts_session_next_frame(
            self._handle, self.current_semantic_token, trailing_text_id, self.talker_sampling.to_c(),
            self.predictor_sampling.to_c(), codes, CODEBOOKS, C.byref(nxt), C.byref(info), err,
            _ERR_CAP), err)
        return self._advance(tuple(int(c) for c in codes), nxt.value, info)

    def begin_device_frame(self, trailing_text_id: int = 0) -> Optional[PendingTalkerFrame]:
        """Device-resident frame (native_talker.rs:1340-1420)."""
        if self.ended:
            return None
        view = DeviceFrameViewV2C()
        view.struct_size = C.sizeof(DeviceFrameViewV2C)
        view.reserved = 0
        err = C.create_string_buffer(_ERR_CAP)
        _check(library().qwen3_tts_session_next_frame_begin_v2(
            self._handle, trailing_text_id, self.talker_sampling.to_c(),
            self.predictor_sampling.to_c(), C.byref(view), err, _ERR_CAP), err)
        return PendingTalkerFrame(self, view)

    def _finish(self, lease_id: int, consumer_done_event: int) -> StreamingCodecFrame:
        nxt = C.c_uint16(0)
        info = FrameInfoC()
        err = C.create_string_buffer(_ERR_CAP)
        _check(library().qwen3_tts_session_next_frame_finish_v2(
            self._handle, lease_id, C.c_void_p(consumer_done_event or None), C.byref(nxt),
            C.byref(info), err, _ERR_CAP), err)
        return self._advance((), nxt.value, info)

    def _advance(self, codes, nxt: int, info: FrameInfoC) -> StreamingCodecFrame:
        self.current_semantic_token = int(nxt)
        self.frames_emitted += 1
        self.ended = bool(info.ended_by_eos)
        return StreamingCodecFrame(codes, int(nxt), bool(info.ended_by_eos), int(info.talker_position),
                                   float(info.predictor_gpu_milliseconds),
                                   float(info.talker_gpu_milliseconds))

    def runtime_state(self) -> SessionRuntimeState:
        out = StateInfoC()
        err = C.create_string_buffer(_ERR_CAP)
        _check(library().qwen3_tts_session_state_info(self._handle, C.byref(out), err, _ERR_CAP), err)
        return SessionRuntimeState(out.abi_version, out.phase, out.talker_position,
                                   out.semantic_history_count, out.frames_generated,
                                   out.device_sample_count, out.host_sync_count)

    def read_state(self):
        """(last_hidden bf16[2048], frame_tokens int32[16], rng_state) -- test hook."""
        hidden = np.zeros(2048, dtype=np.uint16)
        tokens = np.zeros(CODEBOOKS, dtype=np.int32)
        rng = np.zeros(1, dtype=np.uint64)
        err = C.create_string_buffer(_ERR_CAP)
        _check(library().q3t_session_read_state(self._handle, hidden.ctypes.data_as(C.c_void_p),
                                                tokens.ctypes.data_as(C.c_void_p),
                                                rng.ctypes.data_as(C.c_void_p), err, _ERR_CAP), err)
        return hidden, tokens, int(rng[0])

    def read_kv(self, layer: int, first: int, count: int):
        """(keys, values) of talker positions [first, first + count) of one layer, bf16 bits
        [count][1024] each, as the cache holds them -- test hook."""
        keys = np.zeros((count, 1024), dtype=np.uint16)
        values = np.zeros((count, 1024), dtype=np.uint16)
        err = C.create_string_buffer(_ERR_CAP)
        _check(library().q3t_session_read_kv(self._handle, layer, first, count,
                                             keys.ctypes.data_as(C.c_void_p),
                                             values.ctypes.data_as(C.c_void_p), err, _ERR_CAP), err)
        return keys, values

    def close(self) -> None:
        if self._handle:
            library().qwen3_tts_session_destroy(self._handle)
            self._handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def validate_transformer_primitives(device_index: int = 0) -> PrimitiveParityC:
    out = PrimitiveParityC()
    err = C.create_string_buffer(_ERR_CAP)
    _check(library().qwen3_tts_validate_transformer_primitives(device_index, C.byref(out), err,
                                                               _ERR_CAP), err)
    return out


def probe_device(device_index: int = 0) -> DeviceInfoC:
    out = DeviceInfoC()
    err = C.create_string_buffer(_ERR_CAP)
    _check(library().qwen3_tts_probe_device(device_index, C.byref(out), err, _ERR_CAP), err)
    return out


def set_gemv_mode(mode: int) -> int:
    """Kernel for projections of 1..8 rows: 0 SIMT (bit-identical to the reference's summation order),
    1 int8 tensor-core kernel where the shape allows (default).  Returns the previous mode."""
    return int(library().q3t_set_gemv_mode(int(mode)))


def set_attention_mode(mode: int) -> int:
    """Decode attention kernel: 1 split-KV on tensor cores (default), 0 sums in the reference's order
    (parity mode, bit-identical to the reference's kernel, slow).  Returns the previous mode."""
    return int(library().q3t_set_attention_mode(int(mode)))


def benchmark_decode_attention(device_index: int, rows: int = 64, min_length: int = 64, max_length: int = 2048,
                               seed: int = 3, iterations: int = 20):
    """(mean microseconds per launch, K+V bytes one launch reads) of the decode attention on a seeded
    ragged batch of contiguous caches -- the operator-level case profiles are taken on."""
    us = C.c_float(0.0)
    nbytes = C.c_uint64(0)
    err = C.create_string_buffer(_ERR_CAP)
    lib = library()
    lib.q3t_benchmark_decode_attention.argtypes = [C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_uint64, C.c_int32,
                                                   C.POINTER(C.c_float), C.POINTER(C.c_uint64), C.c_char_p, C.c_size_t]
    _check(lib.q3t_benchmark_decode_attention(device_index, rows, min_length, max_length, seed, iterations,
                                              C.byref(us), C.byref(nbytes), err, _ERR_CAP), err)
    return float(us.value), int(nbytes.value)


def benchmark_int8_gemv(device_index: int, in_features: int, out_features: int, rows: int = 1,
                        buffers: int = 16, iterations: int = 2000) -> GemvBenchmarkC:
    out = GemvBenchmarkC()
    err = C.create_string_buffer(_ERR_CAP)
    _check(library().q3t_benchmark_int8_gemv(device_index, in_features, out_features, rows, buffers,
                                             iterations, C.byref(out), err, _ERR_CAP), err)
    return out


# ---- entry points only the reference's command-line tools use (cli_compat.cu) -----------------

class ArgmaxBenchmarkC(C.Structure):        # qwen3_tts_native.h Qwen3TtsArgmaxBenchmark
    _fields_ = [("vocabulary_size", C.c_int32), ("iterations", C.c_int32), ("selected_token", C.c_int32),
                ("expected_token", C.c_int32), ("cold_launch_microseconds", C.c_float),
                ("mean_launch_microseconds", C.c_float)]


class WeightUploadMetricsC(C.Structure):    # qwen3_tts_native.h Qwen3TtsWeightUploadMetrics
    _fields_ = [("device_index", C.c_int32), ("reserved", C.c_int32), ("allocation_bytes", C.c_uint64),
                ("pinned_staging_bytes", C.c_uint64), ("uploaded_bytes", C.c_uint64),
                ("upload_calls", C.c_uint64), ("free_before_bytes", C.c_uint64),
                ("free_after_allocation_bytes", C.c_uint64), ("allocation_microseconds", C.c_float),
                ("upload_microseconds", C.c_float)]


def benchmark_bf16_argmax(device_index: int, vocabulary_size: int, iterations: int = 100):
    out = ArgmaxBenchmarkC()
    err = C.create_string_buffer(_ERR_CAP)
    rc = library().qwen3_tts_benchmark_bf16_argmax(C.c_int32(device_index), C.c_int32(vocabulary_size),
                                                   C.c_int32(iterations), C.byref(out), err, C.c_size_t(_ERR_CAP))
    return rc, out, err.value.decode()


def benchmark_bf16_gemv(device_index: int, in_features: int, out_features: int, iterations: int = 100):
    out = GemvBenchmarkC()
    err = C.create_string_buffer(_ERR_CAP)
    rc = library().qwen3_tts_benchmark_bf16_gemv(C.c_int32(device_index), C.c_int32(in_features),
                                                 C.c_int32(out_features), C.c_int32(iterations), C.byref(out),
                                                 err, C.c_size_t(_ERR_CAP))
    return rc, out, err.value.decode()


class DeviceWeightBuffer:
    """The upload arena of the reference's weight loader (src/device_weights.rs)."""

    def __init__(self, device_index: int, capacity_bytes: int, staging_bytes: int):
        lib = library()
        lib.qwen3_tts_device_buffer_data.restype = C.c_void_p
        lib.qwen3_tts_device_buffer_data.argtypes = [C.c_void_p]
        lib.qwen3_tts_device_buffer_destroy.restype = None
        lib.qwen3_tts_device_buffer_destroy.argtypes = [C.c_void_p]
        self._lib = lib
        self._handle = C.c_void_p()
        self.metrics = WeightUploadMetricsC()
        self.error = C.create_string_buffer(_ERR_CAP)
        self.status = lib.qwen3_tts_device_buffer_create(
            C.c_int32(device_index), C.c_uint64(capacity_bytes), C.c_uint64(staging_bytes), C.byref(self._handle),
            C.byref(self.metrics), self.error, C.c_size_t(_ERR_CAP))

    def upload(self, offset: int, data: bytes) -> int:
        return self._lib.qwen3_tts_device_buffer_upload(self._handle, C.c_uint64(offset), data,
                                                        C.c_uint64(len(data)), self.error, C.c_size_t(_ERR_CAP))

    def finish(self) -> int:
        return self._lib.qwen3_tts_device_buffer_finish(self._handle, C.byref(self.metrics), self.error,
                                                        C.c_size_t(_ERR_CAP))

    def read(self, offset: int, count: int):
        out = C.create_string_buffer(count)
        rc = self._lib.qwen3_tts_device_buffer_read(self._handle, C.c_uint64(offset), out, C.c_uint64(count),
                                                    self.error, C.c_size_t(_ERR_CAP))
        return rc, out.raw

    def data(self) -> int:
        return self._lib.qwen3_tts_device_buffer_data(self._handle) or 0

    def close(self) -> None:
        if self._handle:
            self._lib.qwen3_tts_device_buffer_destroy(self._handle)
            self._handle = C.c_void_p()


class BatchFramePump:
    """The lockstep rendezvous of the reference's host (native_talker.rs:267-401), C++ side in
    csrc/host_pump.cu.  Owner threads call begin(); each then finishes its own frame."""

    def __init__(self, model: "NativeTalkerModel", max_batch: int = MAX_BATCH_SESSIONS, window_us: int = 2000):
        lib = library()
        lib.q3t_pump_begin_frame.argtypes = [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, SamplingConfigC,
                                             SamplingConfigC, C.POINTER(DeviceFrameViewV2C), C.c_char_p, C.c_size_t]
        lib.q3t_pump_begin_frame.restype = C.c_int32
        lib.q3t_pump_destroy.argtypes = [C.c_void_p]
        lib.q3t_pump_destroy.restype = None
        lib.q3t_pump_register.argtypes = [C.c_void_p]
        lib.q3t_pump_register.restype = None
        lib.q3t_pump_unregister.argtypes = [C.c_void_p]
        lib.q3t_pump_unregister.restype = None
        self._lib = lib
        self._handle = C.c_void_p()
        err = C.create_string_buffer(_ERR_CAP)
        _check(lib.q3t_pump_create(model._handle, C.c_int32(max_batch), C.c_int32(window_us), C.byref(self._handle),
                                   err, C.c_size_t(_ERR_CAP)), err)

    def register(self) -> None:
        self._lib.q3t_pump_register(self._handle)

    def unregister(self) -> None:
        self._lib.q3t_pump_unregister(self._handle)

    def begin(self, session: "NativeTalkerSession", trailing_text_id: int) -> "PendingTalkerFrame":
        view = DeviceFrameViewV2C()
        view.struct_size = C.sizeof(DeviceFrameViewV2C)
        view.reserved = 0
        err = C.create_string_buffer(_ERR_CAP)
        _check(self._lib.q3t_pump_begin_frame(self._handle, session._handle, session.frames_emitted,
                                              trailing_text_id, session.talker_sampling.to_c(),
                                              session.predictor_sampling.to_c(), C.byref(view), err, _ERR_CAP), err)
        return PendingTalkerFrame(session, view)

    def statistics(self):
        batches, frames = C.c_uint64(0), C.c_uint64(0)
        self._lib.q3t_pump_statistics(self._handle, C.byref(batches), C.byref(frames))
        return int(batches.value), int(frames.value)

    def close(self) -> None:
        if self._handle:
            self._lib.q3t_pump_destroy(self._handle)
            self._handle = C.c_void_p()


def pick_device(active_sessions_per_device: Sequence[int]) -> int:
    n = len(active_sessions_per_device)
    arr = (C.c_int32 * max(n, 1))(*[int(v) for v in active_sessions_per_device])
    return int(library().q3t_pick_device(arr, C.c_int32(n)))


class StagedPacketViewC(C.Structure):      # q3t_ops.h Q3tStagedPacketView
    _fields_ = [("device_codes", C.c_void_p), ("frame_count", C.c_uint64), ("ready_event", C.c_void_p)]


class PacketStagerError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(message)
        self.status = status


class PacketStager:
    """Device-to-device hand-over of begun frames to the codec (cuda_packet_stager.rs:167-340 of
    the reference host): stage up to four frames, let the codec read the packet, release."""
    CODEBOOKS = 16
    MAX_PACKET_FRAMES = 4

    def __init__(self, device_index: int = 0):
        lib = library()
        lib.q3t_packet_stager_create.restype = C.c_void_p
        lib.q3t_packet_stager_device_bytes.restype = C.c_uint64
        err = C.create_string_buffer(_ERR_CAP)
        self._handle = lib.q3t_packet_stager_create(C.c_int32(device_index), err, _ERR_CAP)
        if not self._handle:
            raise PacketStagerError(2, err.value.decode(errors="replace"))
        self.device_index = device_index

    def _raise(self, status: int, err) -> None:
        if status != 0:
            raise PacketStagerError(status, err.value.decode(errors="replace"))

    @property
    def device_bytes(self) -> int:
        return int(library().q3t_packet_stager_device_bytes(C.c_void_p(self._handle)))

    @property
    def staged_frames(self) -> int:
        return int(library().q3t_packet_stager_staged_frames(C.c_void_p(self._handle)))

    def stage_frame(self, device_codes: int, ready_event: int, source_device: Optional[int] = None,
                    code_count: int = 16) -> int:
        """Returns the event that fires once the frame's codes are in the packet."""
        copied = C.c_void_p()
        err = C.create_string_buffer(_ERR_CAP)
        self._raise(library().q3t_packet_stager_stage_frame(
            C.c_void_p(self._handle), C.c_void_p(device_codes), C.c_size_t(code_count),
            C.c_void_p(ready_event), C.c_int32(self.device_index if source_device is None else source_device),
            C.byref(copied), err, _ERR_CAP), err)
        return int(copied.value or 0)

    def stage(self, pending: "PendingTalkerFrame") -> int:
        return self.stage_frame(pending.device_codes, pending.ready_event)

    def packet_view(self) -> StagedPacketViewC:
        view = StagedPacketViewC()
        err = C.create_string_buffer(_ERR_CAP)
        self._raise(library().q3t_packet_stager_packet_view(C.c_void_p(self._handle), C.byref(view), err,
                                                            _ERR_CAP), err)
        return view

    def release_after_consumer(self, consumer_done_event: int) -> None:
        err = C.create_string_buffer(_ERR_CAP)
        self._raise(library().q3t_packet_stager_release_after_consumer(
            C.c_void_p(self._handle), C.c_void_p(consumer_done_event), err, _ERR_CAP), err)

    def close(self) -> None:
        if self._handle:
            library().q3t_packet_stager_destroy(C.c_void_p(self._handle))
            self._handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
