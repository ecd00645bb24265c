"""B200-native decode hot path of Qwen3-TTS: libqwen3_tts_cuda.so and its host binding.

The directory name is not a Python identifier; load the package with

    import importlib
    q3t = importlib.import_module("qwen3-tts-native_b200")

Submodules: `native` (the C ABI binding, mirrors the reference's native_talker.rs),
`ops` (operator-level drivers), `synth` (seeded synthetic checkpoint), `build` (nvcc recipe).
"""
from . import native  # noqa: F401
from .native import (  # noqa: F401
    NativeTalkerModel,
    NativeTalkerSession,
    NativeTalkerStatusError,
    SamplingConfig,
    library,
)

__all__ = ["native", "NativeTalkerModel", "NativeTalkerSession", "NativeTalkerStatusError",
           "SamplingConfig", "library"]
