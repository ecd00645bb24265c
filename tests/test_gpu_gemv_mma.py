"""GPU parity of the default kernel for projections of 1..8 rows (gemv_int8_mma.cu: weights
bulk-copied ahead of the launch dependency, int8 mma.sync arithmetic on byte limbs of the activations)
through the operator-level C ABI.

The products are the reference's (int8 weight x bf16 activation) and they are summed exactly, as
integers, per eighth of K; what differs from the reference's kernel is the order and rounding of the
few fp32 steps that remain, so the checks are the north-star tolerance stated two ways and a
rounding-step bound on the bf16 output:

  * fp32 value before the final round within 1e-3 of fp64 truth, element-wise relative error on
    every element whose magnitude is at least 0.1 x the row's RMS (smaller ones are cancellations,
    where a relative error has no meaning) and, for every element, relative to |truth| + RMS;
    both figures are expected around 1e-7;
  * bf16 output == bf16(that fp32 value), and within one bf16 rounding step of the oracle's output
    with few mismatching elements;
  * a row's result does not depend on the rows beside it (batch of R == R solo calls, bit for bit),
    and repeated calls agree bit for bit.
"""
import json
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def report(**fields):
    """Appends one JSON line of measured errors to the file named by Q3T_PARITY_REPORT, if set."""
    path = os.environ.get("Q3T_PARITY_REPORT")
    if path:
        with open(path, "a") as f:
            f.write(json.dumps(fields) + "\n")

SHAPES = [  # (out_features, in_features)
    (6144, 2048),   # config 0 / gate, up
    (4096, 2048),   # stacked q|k|v
    (2048, 6144),   # talker down: four chunks of K
    (1024, 2048),   # small_to_mtp
    (3072, 2048),   # codec head
    (4096, 1024),   # predictor q|k|v
    (2048, 1024),   # predictor lm_head
    (1024, 3072),   # predictor down: two chunks of K
    (131, 1024), (77, 3072), (5, 6144), (1, 2048), (40, 4096), (300, 1536),
]


@pytest.fixture(autouse=True)
def mma_kernels(q3t):
    before = q3t.native.set_gemv_mode(1)
    yield
    q3t.native.set_gemv_mode(before)


def case(orc, seed, n, k, rows, scale=None):
    rng = np.random.default_rng(seed)
    w = rng.integers(-127, 128, size=(n, k), dtype=np.int8)
    s = (rng.uniform(0.5, 1.5, size=n) * (scale or 1.0 / (73.6 * np.sqrt(k)))).astype(np.float32)
    x = orc.to_bf16(rng.standard_normal((rows, k)).astype(np.float32))
    return w, s, x


def relative_errors(value, truth):
    rms = np.sqrt((truth ** 2).mean(axis=-1, keepdims=True))
    guarded = np.abs(value - truth) / (np.abs(truth) + rms)
    big = np.abs(truth) >= 0.1 * rms
    plain = np.abs(value - truth)[big] / np.abs(truth)[big]
    return float(plain.max()) if plain.size else 0.0, float(guarded.max())


def check_bf16(orc, got, want, summand=None):
    g, w = orc.from_bf16(got), orc.from_bf16(want)
    rms = np.sqrt((w ** 2).mean(axis=-1, keepdims=True))
    mag = np.maximum(np.abs(w), 0.25 * rms)
    if summand is not None:
        mag = np.maximum(mag, np.abs(orc.from_bf16(summand)).reshape(mag.shape))
    bad = np.abs(g - w) > 2.0 ** -7 * mag
    assert not bad.any(), (int(bad.sum()), float(np.abs(g - w).max()))
    assert (g != w).mean() < 0.02, float((g != w).mean())


@pytest.mark.parametrize("n,k", SHAPES)
@pytest.mark.parametrize("rows", [1, 2, 5, 8])
def test_plain_within_tolerance(orc, ops, n, k, rows):
    if rows > 2 and n * k > 8_000_000:
        rows = 3
    w, s, x = case(orc, rows, n, k, rows)
    out = ops.int8_gemm(w, s, x, want_f32=True)
    truth = orc.int8_gemm_rows_f64(w, s, x)
    plain, guarded = relative_errors(out["f32"], truth)
    report(test="gemv_mma_plain", n=n, k=k, rows=rows, plain_relative=plain, guarded_relative=guarded)
    assert plain <= 1.0e-3 and guarded <= 1.0e-3, (plain, guarded)     # north-star tolerance
    assert plain <= 1.0e-4 and guarded <= 1.0e-5, (plain, guarded)     # what fp32 accumulation should give
    assert np.array_equal(out["y"], orc.to_bf16(out["f32"]))
    check_bf16(orc, out["y"], orc.int8_gemm_rows(w, s, x))


@pytest.mark.parametrize("n,k,rows", [(2048, 2048, 1), (2048, 6144, 4), (1024, 3072, 8), (131, 1024, 3)])
def test_residual_epilogue(orc, ops, n, k, rows):
    w, s, x = case(orc, 2, n, k, rows)
    base = orc.to_bf16(np.random.default_rng(3).standard_normal((rows, n)).astype(np.float32))
    got = ops.int8_gemm_rows(w, s, x, y_in=base, mode=1)
    check_bf16(orc, got, orc.int8_gemm_rows(w, s, x, y_in=base, mode=1), summand=base)


@pytest.mark.parametrize("n,k,rows", [(6144, 2048, 1), (3072, 1024, 8), (6144, 2048, 6), (45, 1024, 2), (9, 2048, 1)])
def test_gate_up_silu(orc, ops, n, k, rows):
    rng = np.random.default_rng(4)
    w = rng.integers(-127, 128, size=(2 * n, k), dtype=np.int8)
    s = (rng.uniform(0.5, 1.5, size=2 * n) / (73.6 * np.sqrt(k))).astype(np.float32)
    x = orc.to_bf16(rng.standard_normal((rows, k)).astype(np.float32))
    out = ops.int8_gemm(w, s, x, epilogue=ops.EPI_GATE_UP_SILU, want_f32=True)
    gate = orc.int8_gemm_rows_f64(w[:n], s[:n], x)
    up = orc.int8_gemm_rows_f64(w[n:], s[n:], x)
    truth = gate / (1.0 + np.exp(-gate)) * up
    plain, guarded = relative_errors(out["f32"], truth)
    assert plain <= 1.0e-3 and guarded <= 1.0e-3, (plain, guarded)
    assert np.array_equal(out["y"], orc.to_bf16(out["f32"]))
    check_bf16(orc, out["y"], orc.int8_gate_up_silu_rows(w, s, x))


@pytest.mark.parametrize("k,n,rows", [(2048, 4096, 1), (1024, 2048, 3), (2048, 3072, 8), (2048, 12288, 2)])
def test_norm_prologue(orc, ops, k, n, rows):
    """The RMSNorm folded into the launch produces the stand-alone norm's rows bit for bit, and the
    projection of those rows."""
    rng = np.random.default_rng(6)
    gateup = n == 12288
    w, s, x = case(orc, 6, n, k, rows)
    x = orc.to_bf16((rng.standard_normal((rows, k)) * 3.0).astype(np.float32))
    nw = orc.to_bf16((1.0 + 0.02 * rng.standard_normal(k)).astype(np.float32))
    epi = ops.EPI_GATE_UP_SILU if gateup else ops.EPI_PLAIN
    fused = ops.int8_gemm(w, s, x, norm_w=nw, want_norm=True, epilogue=epi)
    normed = ops.rms_norm_rows(x, nw)
    assert np.array_equal(fused["norm"], normed)
    assert np.array_equal(fused["y"], ops.int8_gemm(w, s, normed, epilogue=epi)["y"])
    if not gateup:
        check_bf16(orc, fused["y"], orc.int8_gemm_rows(w, s, normed))


@pytest.mark.parametrize("rows", [1, 4, 8])
def test_bias_epilogues(orc, ops, rows):
    k, n = 2048, 1024
    rng = np.random.default_rng(7)
    w, s, x = case(orc, 7, n, k, rows)
    bias = orc.to_bf16((0.1 * rng.standard_normal(n)).astype(np.float32))
    resid = orc.to_bf16(rng.standard_normal((rows, n)).astype(np.float32))
    plain = ops.int8_gemm_rows(w, s, x)           # this kernel's own plain output
    got = ops.int8_gemm(w, s, x, epilogue=ops.EPI_BIAS, bias=bias)["y"]
    assert np.array_equal(got, orc.bias_activation_rows(plain, bias, False))
    got = ops.int8_gemm(w, s, x, epilogue=ops.EPI_BIAS_SILU, bias=bias)["y"]
    d = orc.bf16_ulp_distance(got, orc.bias_activation_rows(plain, bias, True))
    assert d.max() <= 1 and (d > 0).mean() < 0.01
    got = ops.int8_gemm(w, s, x, epilogue=ops.EPI_BIAS_ADD, bias=bias, resid=resid)["resid"]
    want = orc.add(resid, orc.bias_activation_rows(plain, bias, False))
    assert np.array_equal(got, want.reshape(rows, n))


@pytest.mark.parametrize("n,k", [(4096, 2048), (1024, 3072), (2048, 6144), (6144, 1024)])
def test_rows_do_not_depend_on_their_neighbours(orc, ops, n, k):
    """Each activation row is its own pair of tensor-core columns with its own power of two, and every
    product and partial sum is an exact integer, so a row computed beside other rows equals the row
    computed alone, bit for bit, whatever the row count (1..2 rows and 3..8 rows run different
    instantiations, K = 6144 takes several launches of fewer rows).  Repeated calls agree too."""
    w, s, x = case(orc, 8, n, k, 8)
    x[3] = orc.to_bf16(np.random.default_rng(9).standard_normal(k).astype(np.float32) * 1.0e4)   # another scale
    x[5] = orc.to_bf16(np.random.default_rng(10).standard_normal(k).astype(np.float32) * 1.0e-6)
    batch = ops.int8_gemm_rows(w, s, x)
    again = ops.int8_gemm_rows(w, s, x)
    assert np.array_equal(batch, again)
    for rows in ([0], [3], [5], [7], [2, 3], [2, 3, 4], [1, 2, 3, 4, 5], [0, 1, 2, 3, 4, 5, 6]):
        alone = ops.int8_gemm_rows(w, s, x[rows[0]:rows[-1] + 1])
        assert np.array_equal(alone, batch[rows[0]:rows[-1] + 1]), rows


def test_activation_range(orc, ops):
    """bf16 activations far outside fp16's range (per-part power-of-two scaling), zeros, and a row
    whose parts differ by many orders of magnitude."""
    n, k = 512, 2048
    rng = np.random.default_rng(11)
    w, s, _ = case(orc, 11, n, k, 1, scale=1.0)
    rows = []
    for magnitude in (1.0e30, 1.0e-30, 70000.0, 1.0):
        rows.append(rng.standard_normal(k) * magnitude)
    mixed = rng.standard_normal(k)
    mixed[: k // 2] *= 1.0e12
    mixed[k // 2:] *= 1.0e-12
    rows.append(mixed)
    sparse = np.zeros(k)
    sparse[[3, 700, 2047]] = [1.5, -2.25, 1.0e-20]
    rows.append(sparse)
    rows.append(np.zeros(k))
    x = orc.to_bf16(np.asarray(rows, dtype=np.float32))
    out = ops.int8_gemm(w, s, x, want_f32=True)
    truth = orc.int8_gemm_rows_f64(w, s, x)
    assert np.isfinite(out["f32"]).all()
    for r in range(len(rows) - 1):
        plain, guarded = relative_errors(out["f32"][r:r + 1], truth[r:r + 1])
        assert plain <= 1.0e-4 and guarded <= 1.0e-5, (r, plain, guarded)
    assert not out["f32"][-1].any()


def test_no_device_wait_ran_out(q3t, ops):
    assert q3t.library().q3t_kernel_error_count() == 0
