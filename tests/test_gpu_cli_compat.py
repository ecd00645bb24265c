"""The entry points only the reference's command-line tools call: the weight-upload arena
(weights.cu:98-340 semantics: sequential uploads, chunked through pinned staging, reads limited to
what was uploaded) and the two bf16 microbenchmarks with their built-in correctness checks."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_device_buffer_round_trip_and_rules(q3t):
    n = q3t.native
    rng = np.random.default_rng(0)
    payload = rng.integers(0, 256, size=1_000_003, dtype=np.uint8).tobytes()
    buf = n.DeviceWeightBuffer(0, len(payload), 64 * 1024 + 7)     # odd staging size: ragged chunks
    assert buf.status == 0 and buf.data() != 0
    assert buf.metrics.allocation_bytes == len(payload) and buf.metrics.pinned_staging_bytes == 64 * 1024 + 7
    assert buf.finish() == -2                                       # nothing uploaded yet
    assert buf.upload(5, payload[:10]) == -3                        # must start at the current end
    assert buf.upload(0, payload[:300_000]) == 0
    assert buf.upload(0, payload[:10]) == -3                        # not sequential
    assert buf.upload(300_000, payload[300_000:] + b"x") == -4      # past the capacity
    rc, got = buf.read(100, 1000)
    assert rc == 0 and got == payload[100:1100]
    assert buf.read(299_999, 2)[0] == -2                            # beyond what has been uploaded
    assert buf.upload(300_000, payload[300_000:]) == 0
    assert buf.finish() == 0
    assert buf.metrics.uploaded_bytes == len(payload) and buf.metrics.upload_calls >= 2
    rc, got = buf.read(0, len(payload))
    assert rc == 0 and got == payload
    buf.close()
    bad = n.DeviceWeightBuffer(0, 0, 1024)
    assert bad.status == -2
    bad = n.DeviceWeightBuffer(0, 1024, 0)
    assert bad.status == -3


def test_bf16_microbenchmarks(q3t):
    n = q3t.native
    for vocab in (2048, 3072, 100):
        rc, out, err = n.benchmark_bf16_argmax(0, vocab, 20)
        assert rc == 0, err
        assert out.selected_token == out.expected_token == min(1729, vocab - 1)
        assert out.mean_launch_microseconds > 0
    assert n.benchmark_bf16_argmax(0, 0, 5)[0] == -2
    assert n.benchmark_bf16_argmax(0, 100, 0)[0] == -3
    rc, out, err = n.benchmark_bf16_gemv(0, 2048, 6144, 20)
    assert rc == 0, err
    assert out.weight_bytes == 2048 * 6144 * 2 and out.mean_launch_microseconds > 0
    assert out.tera_operations_per_second > 0
    rc, out, err = n.benchmark_bf16_gemv(0, 100, 33, 3)            # K not a multiple of 8
    assert rc == 0, err
    assert n.benchmark_bf16_gemv(0, 0, 10, 1)[0] == -2
