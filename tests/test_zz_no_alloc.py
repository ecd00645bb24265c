"""The attention entry point for hosts that cannot allocate device memory.

q3t_launch_batch_causal_gqa_attention_fast_noalloc serves callers such as a real-time audio
thread, a process whose GPU memory budget is fixed and policed after start-up, or a plugin that
is only lent streams and buffers: it takes inputs and outputs and keeps its split-KV scratch in
an array built into the library, so nothing is allocated by the call or asked of the caller.

Checked here through the C ABI: two calls in a row give exactly the output of the regular entry
point (which works from a caller-provided scratch buffer) -- the second call runs over whatever the
first left in the shared array -- and a shape whose scratch would not fit is refused with a
message instead of being run.  Collected last on purpose (file name), and self-contained so that
it passes alone in a fresh process as well as after the other tests.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _case(orc, seed, rows, qh, kvh, hd, cap, positions):
    rng = np.random.default_rng(seed)
    q = orc.to_bf16(rng.standard_normal((rows, qh * hd)).astype(np.float32))
    k = orc.to_bf16(rng.standard_normal((rows, cap, kvh * hd)).astype(np.float32))
    v = orc.to_bf16(rng.standard_normal((rows, cap, kvh * hd)).astype(np.float32))
    return q, k, v, np.asarray(positions, dtype=np.int32)


def test_two_calls_in_a_row_match_the_regular_entry_point(orc, ops):
    qh, kvh, hd = 16, 8, 128
    # first call: long rows, many splits, fills the built-in array with partials and tickets
    q, k, v, pos = _case(orc, 1, 4, qh, kvh, hd, 700, [699, 64, 300, 0])
    want = ops.attention_contiguous(q, k, v, pos, qh, kvh, hd)
    status, message, got = ops.attention_contiguous_noalloc(q, k, v, pos, qh, kvh, hd)
    assert status == 0 and message == ""
    assert np.array_equal(got, want)       # same kernel, same arithmetic: bit-identical
    # second call, other shape and lengths, over the leftovers of the first
    q, k, v, pos = _case(orc, 2, 3, qh, kvh, hd, 450, [449, 129, 17])
    want = ops.attention_contiguous(q, k, v, pos, qh, kvh, hd)
    status, message, got = ops.attention_contiguous_noalloc(q, k, v, pos, qh, kvh, hd)
    assert status == 0 and message == ""
    assert np.array_equal(got, want)
    # and against the CPU oracle, with the tolerance the attention tests use
    ref = orc.from_bf16(orc.attention(q, k, v, pos, qh, kvh, hd, fast=True)).reshape(-1, hd)
    out = orc.from_bf16(got).reshape(-1, hd)
    rms = np.sqrt((ref ** 2).mean(axis=1, keepdims=True))
    assert (np.abs(out - ref) <= 2.0 ** -7 * np.maximum(np.abs(ref), 0.25 * rms)).all()


def test_oversized_shape_is_refused(q3t, orc, ops):
    lib = q3t.library()
    capacity = int(lib.q3t_attention_static_scratch_capacity())
    assert capacity == 4 << 20
    qh, kvh, hd = 16, 8, 128
    need = int(lib.q3t_attention_scratch_bytes(64, qh, kvh, hd, 8192))
    assert need > capacity
    # 64 rows of up to 1024 positions need 64*16*16*130*4 bytes of partials: too much
    q, k, v, pos = _case(orc, 3, 64, qh, kvh, hd, 1024, [5] * 64)
    status, message, _ = ops.attention_contiguous_noalloc(q, k, v, pos, qh, kvh, hd)
    assert status == q3t.native.STATUS_INVALID_ARGUMENT
    assert "scratch" in message and str(capacity) in message


FRESH_PROCESS_SCRIPT = r"""
import importlib, sys
import numpy as np
sys.path.insert(0, sys.argv[1])
from oracle import oracle as orc
orc.build()
ops = importlib.import_module("qwen3-tts-native_b200.ops")
rng = np.random.default_rng(5)
rows, qh, kvh, hd, cap = 3, 16, 8, 128, 520
q = orc.to_bf16(rng.standard_normal((rows, qh * hd)).astype(np.float32))
k = orc.to_bf16(rng.standard_normal((rows, cap, kvh * hd)).astype(np.float32))
v = orc.to_bf16(rng.standard_normal((rows, cap, kvh * hd)).astype(np.float32))
pos = np.asarray([519, 77, 0], dtype=np.int32)
# the very first call this process makes into the library: nothing has resolved the built-in
# array's address or configured a kernel before it
status, message, got = ops.attention_contiguous_noalloc(q, k, v, pos, qh, kvh, hd)
assert status == 0 and message == "", (status, message)
want = ops.attention_contiguous(q, k, v, pos, qh, kvh, hd)
assert np.array_equal(got, want)
print("fresh-process first call ok")
"""


def test_first_call_in_a_fresh_process(ops):
    """The entry point as the first thing a new process asks of the library (address of the built-in
    array not yet resolved, kernels not yet configured), which running after other tests cannot show."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    proc = subprocess.run([sys.executable, "-c", FRESH_PROCESS_SCRIPT, root], capture_output=True, text=True,
                          timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert "fresh-process first call ok" in proc.stdout
