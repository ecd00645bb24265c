"""Shared fixtures.  GPU tests are marked `gpu`; everything else runs on CPU only."""
import importlib
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

PACKAGE = "qwen3-tts-native_b200"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200 box)")


@pytest.fixture(scope="session")
def orc():
    """The CPU oracle (oracle/oracle.py over oracle/q3t_oracle.c)."""
    from oracle import oracle
    oracle.build()
    return oracle


@pytest.fixture(scope="session")
def q3t():
    """The product package (binding of libqwen3_tts_cuda.so)."""
    return importlib.import_module(PACKAGE)


@pytest.fixture(scope="session")
def ops(q3t):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return importlib.import_module(PACKAGE + ".ops")


@pytest.fixture(scope="session")
def synth():
    return importlib.import_module(PACKAGE + ".synth")


@pytest.fixture(scope="session")
def ref(orc):
    """The reference project's kernels compiled for sm_100a, when oracle/_ref was built."""
    if not orc.ref_available():
        pytest.skip("oracle/_ref/libq3t_ref.so not built (needs a reference checkout)")
    orc.ref()
    return orc


def rand_bf16(rng, shape, scale=1.0):
    from oracle import oracle
    return oracle.to_bf16((rng.standard_normal(shape) * scale).astype(np.float32))


@pytest.fixture(scope="session")
def checkpoint(synth):
    """All 404 synthetic tensors as {name: bf16 bits}; about 3.8 GB of host memory."""
    return dict(synth.checkpoint(seed=0))


@pytest.fixture(scope="session")
def gpu_model(q3t, checkpoint):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    model = q3t.NativeTalkerModel.load(0, checkpoint.items())
    yield model
    model.close()
