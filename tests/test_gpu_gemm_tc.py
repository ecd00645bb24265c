"""GPU parity of the tensor-core (tcgen05) skinny GEMM used for 9..64 activation rows.

The contraction runs on the tensor cores in K-slices, so the fp32 summation order differs from
the SIMT kernels and from the reference: the checks are the north-star tolerance (fp32 value
before the final round within 1e-3 of fp64 truth, relative to |value| + the row's RMS) and bf16
outputs within one rounding step of bf16(oracle).  Rows are independent in the reference kernel,
so the oracle for more than 8 rows is the reference arithmetic applied row by row."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

MODEL_SHAPES = [  # (out_features, in_features)
    (4096, 2048), (2048, 2048), (2048, 6144), (3072, 2048), (1024, 2048),
    (4096, 1024), (1024, 3072), (2048, 1024),
    (200, 64), (129, 128), (64, 192),      # ragged channel counts, short K
]


def case(orc, seed, n, k, rows):
    rng = np.random.default_rng(seed)
    w = rng.integers(-127, 128, size=(n, k), dtype=np.int8)
    s = (rng.uniform(0.5, 1.5, size=n) / (73.6 * np.sqrt(k))).astype(np.float32)
    x = orc.to_bf16(rng.standard_normal((rows, k)).astype(np.float32))
    return w, s, x


def check_bf16(orc, got, want, summand=None):
    """One bf16 rounding step of the value, or of the largest summand that was itself rounded
    to bf16 on the way (a residual add can cancel down to a small value)."""
    g, w = orc.from_bf16(got), orc.from_bf16(want)
    rms = np.sqrt((w ** 2).mean(axis=-1, keepdims=True))
    mag = np.maximum(np.abs(w), 0.25 * rms)
    if summand is not None:
        mag = np.maximum(mag, np.abs(orc.from_bf16(summand)).reshape(mag.shape))
    step = 2.0 ** -7 * mag
    bad = np.abs(g - w) > step
    assert not bad.any(), (int(bad.sum()), float(np.abs(g - w).max()))
    assert (g != w).mean() < 0.02, float((g != w).mean())


@pytest.mark.parametrize("n,k", MODEL_SHAPES)
@pytest.mark.parametrize("rows", [9, 16, 17, 33, 64])
def test_plain(orc, ops, n, k, rows):
    w, s, x = case(orc, rows, n, k, rows)
    out = ops.int8_gemm(w, s, x, want_f32=True)
    truth = orc.int8_gemm_rows_f64(w, s, x)
    rel = np.abs(out["f32"] - truth) / (np.abs(truth) + np.sqrt((truth ** 2).mean()))
    assert rel.max() <= 1.0e-3, rel.max()
    assert np.array_equal(out["y"], orc.to_bf16(out["f32"]))
    check_bf16(orc, out["y"], orc.int8_gemm_rows(w, s, x))


@pytest.mark.parametrize("n,k,rows", [(2048, 2048, 64), (2048, 6144, 20), (130, 256, 12)])
def test_residual(orc, ops, n, k, rows):
    w, s, x = case(orc, 1, n, k, rows)
    base = orc.to_bf16(np.random.default_rng(2).standard_normal((rows, n)).astype(np.float32))
    got = ops.int8_gemm_rows(w, s, x, y_in=base, mode=1)
    check_bf16(orc, got, orc.int8_gemm_rows(w, s, x, y_in=base, mode=1), summand=base)


@pytest.mark.parametrize("n,k,rows", [(6144, 2048, 64), (3072, 1024, 16), (100, 128, 9), (64, 64, 33)])
def test_gate_up_silu(orc, ops, n, k, rows):
    rng = np.random.default_rng(3)
    w = rng.integers(-127, 128, size=(2 * n, k), dtype=np.int8)
    s = (rng.uniform(0.5, 1.5, size=2 * n) / (73.6 * np.sqrt(k))).astype(np.float32)
    x = orc.to_bf16(rng.standard_normal((rows, k)).astype(np.float32))
    got = ops.int8_gemm_rows(w, s, x, mode=2)
    check_bf16(orc, got, orc.int8_gate_up_silu_rows(w, s, x))


@pytest.mark.parametrize("rows", [12, 64])
def test_bias_epilogues_and_norm(orc, ops, rows):
    k, n = 2048, 1024
    rng = np.random.default_rng(4)
    w, s, x = case(orc, 4, n, k, rows)
    bias = orc.to_bf16((0.1 * rng.standard_normal(n)).astype(np.float32))
    resid = orc.to_bf16(rng.standard_normal((rows, n)).astype(np.float32))
    plain = orc.int8_gemm_rows(w, s, x)
    check_bf16(orc, ops.int8_gemm(w, s, x, epilogue=ops.EPI_BIAS, bias=bias)["y"],
               orc.bias_activation_rows(plain, bias, False))
    check_bf16(orc, ops.int8_gemm(w, s, x, epilogue=ops.EPI_BIAS_SILU, bias=bias)["y"],
               orc.bias_activation_rows(plain, bias, True))
    got = ops.int8_gemm(w, s, x, epilogue=ops.EPI_BIAS_ADD, bias=bias, resid=resid)["resid"]
    check_bf16(orc, got, orc.add(resid, orc.bias_activation_rows(plain, bias, False)).reshape(rows, n),
               summand=resid)
    # RMSNorm in front: same normalised rows as the stand-alone operator
    nw = orc.to_bf16((1.0 + 0.02 * rng.standard_normal(k)).astype(np.float32))
    fused = ops.int8_gemm(w, s, x, norm_w=nw, want_norm=True)
    normed = ops.rms_norm_rows(x, nw)
    assert np.array_equal(fused["norm"], normed)
    assert np.array_equal(fused["y"], ops.int8_gemm_rows(w, s, normed))


def test_deterministic_and_healthy(q3t, orc, ops):
    w, s, x = case(orc, 5, 2048, 2048, 64)
    a = ops.int8_gemm_rows(w, s, x)
    b = ops.int8_gemm_rows(w, s, x)
    assert np.array_equal(a, b)                       # K-slices are summed in slice order
    # a row's result does not depend on how many rows ride along, as long as the tile width is the same
    c = ops.int8_gemm_rows(w, s, x[:40])
    assert np.array_equal(a[:40], c)
    assert q3t.library().q3t_kernel_error_count() == 0
