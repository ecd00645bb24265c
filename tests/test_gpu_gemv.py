"""GPU parity of the int8 weight-only GEMV / skinny GEMM (plain, residual, gate/up/SiLU and norm-fused forms) through the
operator-level C ABI, against the CPU oracle, against fp64 truth, and against the reference's
own kernels compiled for sm_100a when oracle/_ref is present.

Tolerances: the SIMT kernel keeps the reference's summation order, so bf16 outputs must be
bit-identical to the oracle for the plain and residual epilogues; epilogues that go through
expf may differ from the CPU by one bf16 ulp on a few elements (libm vs CUDA expf) but must be
bit-identical to the reference kernels run on the same GPU.  The fp32 value before the final
round must be within 1e-3 relative of fp64 truth (the north-star tolerance)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def simt_kernels(q3t):
    """These tests pin the kernel that keeps the reference's summation order (gemv mode 0); the
    default kernel for 1..8 rows has its own file, test_gpu_gemv_mma.py."""
    before = q3t.native.set_gemv_mode(0)
    yield
    q3t.native.set_gemv_mode(before)


SHAPES = [  # (out_features, in_features)
    (8, 16), (5, 32), (33, 64), (130, 272),
    (6144, 2048),   # config 0 / gate, up
    (2048, 6144),   # down
    (1024, 2048),   # k, v, small_to_mtp
    (3072, 2048),   # codec head
    (2048, 1024),   # predictor lm_head / q
    (1024, 3072),   # predictor down
    (131, 1024), (77, 3072), (5, 6144),   # odd channel counts
]


def case(orc, seed, n, k, rows, scale=1.0 / 127.0):
    rng = np.random.default_rng(seed)
    w = rng.integers(-127, 128, size=(n, k), dtype=np.int8)
    s = (rng.uniform(0.5, 1.5, size=n) * scale).astype(np.float32)
    x = orc.to_bf16(rng.standard_normal((rows, k)).astype(np.float32))
    return w, s, x


def ulp_report(orc, got, want):
    d = orc.bf16_ulp_distance(got, want)
    return int(d.max()), float((d > 0).mean())


@pytest.mark.parametrize("n,k", SHAPES)
@pytest.mark.parametrize("rows", [1, 3, 8])
def test_plain_bit_exact_vs_oracle(orc, ops, n, k, rows):
    if rows > 1 and n * k > 4_000_000:
        rows = 2
    w, s, x = case(orc, 0, n, k, rows)
    got = ops.int8_gemm_rows(w, s, x)
    want = orc.int8_gemm_rows(w, s, x)
    assert np.array_equal(got, want), ulp_report(orc, got, want)


@pytest.mark.parametrize("rows", [1, 2, 7, 9, 16, 17, 64])
def test_rows_up_to_64(orc, ops, rows):
    w, s, x = case(orc, 1, 272, 528, rows)
    got = ops.int8_gemm_rows(w, s, x)
    want = orc.int8_gemm_rows(w, s, x)     # rows are independent in the reference kernel
    assert np.array_equal(got, want), ulp_report(orc, got, want)


@pytest.mark.parametrize("n,k,rows", [(64, 128, 1), (2048, 2048, 1), (2048, 6144, 4), (272, 528, 20)])
def test_residual_epilogue_bit_exact(orc, ops, n, k, rows):
    w, s, x = case(orc, 2, n, k, rows)
    base = orc.to_bf16(np.random.default_rng(3).standard_normal((rows, n)).astype(np.float32))
    got = ops.int8_gemm_rows(w, s, x, y_in=base, mode=1)
    want = orc.int8_gemm_rows(w, s, x, y_in=base, mode=1)
    assert np.array_equal(got, want), ulp_report(orc, got, want)


@pytest.mark.parametrize("n,k,rows", [(24, 96, 2), (6144, 2048, 1), (3072, 1024, 8), (40, 80, 11)])
def test_gate_up_silu(orc, ops, n, k, rows):
    rng = np.random.default_rng(4)
    w = rng.integers(-127, 128, size=(2 * n, k), dtype=np.int8)
    s = (rng.uniform(0.5, 1.5, size=2 * n) / (73.6 * np.sqrt(k))).astype(np.float32)
    x = orc.to_bf16(rng.standard_normal((rows, k)).astype(np.float32))
    got = ops.int8_gemm_rows(w, s, x, mode=2)
    want = orc.int8_gate_up_silu_rows(w, s, x)
    worst, frac = ulp_report(orc, got, want)
    assert worst <= 1 and frac < 0.01, (worst, frac)


@pytest.mark.parametrize("n,k,rows", [(6144, 2048, 1), (2048, 6144, 1), (130, 272, 5)])
def test_fp32_accumulator_within_1e3_of_fp64(orc, ops, n, k, rows):
    w, s, x = case(orc, 5, n, k, rows)
    out = ops.int8_gemm(w, s, x, want_f32=True)
    truth = orc.int8_gemm_rows_f64(w, s, x)
    rel = np.abs(out["f32"] - truth) / (np.abs(truth) + np.sqrt((truth ** 2).mean()))
    assert rel.max() <= 1.0e-3, rel.max()      # north-star tolerance; expected ~1e-6
    assert np.array_equal(out["y"], orc.to_bf16(out["f32"]))


@pytest.mark.parametrize("k,n,rows", [(2048, 4096, 1), (1024, 2048, 3), (2048, 3072, 8), (64, 40, 10)])
def test_norm_prologue(orc, ops, k, n, rows):
    """RMSNorm folded into the GEMV must equal the stand-alone norm followed by the GEMV."""
    rng = np.random.default_rng(6)
    w, s, x = case(orc, 6, n, k, rows, scale=1.0 / (73.6 * np.sqrt(k)))
    x = orc.to_bf16((rng.standard_normal((rows, k)) * 3.0).astype(np.float32))
    nw = orc.to_bf16((1.0 + 0.02 * rng.standard_normal(k)).astype(np.float32))
    fused = ops.int8_gemm(w, s, x, norm_w=nw, want_norm=True)
    normed = ops.rms_norm_rows(x, nw)
    assert np.array_equal(fused["norm"], normed)
    assert np.array_equal(fused["y"], ops.int8_gemm_rows(w, s, normed))
    # and against the CPU oracle (rsqrtf may differ from the correctly rounded value by an ulp)
    want = orc.int8_gemm_rows(w, s, orc.rms_norm_rows(x, nw))
    worst, frac = ulp_report(orc, fused["y"], want)
    assert worst <= 2 and frac < 0.05, (worst, frac)


@pytest.mark.parametrize("rows", [1, 4, 8])
def test_bias_epilogues(orc, ops, rows):
    k, n = 2048, 1024
    rng = np.random.default_rng(7)
    w, s, x = case(orc, 7, n, k, rows, scale=1.0 / (73.6 * np.sqrt(k)))
    bias = orc.to_bf16((0.1 * rng.standard_normal(n)).astype(np.float32))
    resid = orc.to_bf16(rng.standard_normal((rows, n)).astype(np.float32))
    plain = orc.int8_gemm_rows(w, s, x)
    got = ops.int8_gemm(w, s, x, epilogue=ops.EPI_BIAS, bias=bias)["y"]
    assert np.array_equal(got, orc.bias_activation_rows(plain, bias, False))
    got = ops.int8_gemm(w, s, x, epilogue=ops.EPI_BIAS_SILU, bias=bias)["y"]
    worst, frac = ulp_report(orc, got, orc.bias_activation_rows(plain, bias, True))
    assert worst <= 1 and frac < 0.01, (worst, frac)
    got = ops.int8_gemm(w, s, x, epilogue=ops.EPI_BIAS_ADD, bias=bias, resid=resid)["resid"]
    want = orc.add(resid, orc.bias_activation_rows(plain, bias, False))
    assert np.array_equal(got, want.reshape(rows, n))


def test_invalid_arguments_are_rejected(orc, ops):
    w, s, x = case(orc, 8, 8, 16, 1)
    with pytest.raises(RuntimeError):
        ops.int8_gemm_rows(w[:, :8].copy(), s, x[:, :8].copy())    # K % 16 != 0 (int8_gemv.cu:329)
    with pytest.raises(RuntimeError):
        ops.int8_gemm_rows(w, s, np.zeros((65, 16), dtype=np.uint16))   # more rows than the batch limit


def test_quantizer_matches_oracle(orc, ops):
    rng = np.random.default_rng(9)
    wt = orc.to_bf16((rng.standard_normal((96, 256)) * 0.03).astype(np.float32))
    wt[5] = 0
    q, s = ops.quantize_rows(wt)
    oq, os_ = orc.quantize_rows(wt)
    assert np.array_equal(q, oq) and np.array_equal(s, os_)


# ---- against the reference's own kernels on the same GPU ------------------------------------

@pytest.mark.parametrize("n,k,rows", [(6144, 2048, 1), (2048, 6144, 8), (130, 272, 3)])
def test_bit_exact_vs_reference_kernels(orc, ops, ref, n, k, rows):
    w, s, x = case(orc, 10, n, k, rows, scale=1.0 / (73.6 * np.sqrt(k)))
    base = orc.to_bf16(np.random.default_rng(11).standard_normal((rows, n)).astype(np.float32))
    assert np.array_equal(ops.int8_gemm_rows(w, s, x), ref.ref_int8_gemm(w, s, x))
    assert np.array_equal(ops.int8_gemm_rows(w, s, x, y_in=base, mode=1),
                          ref.ref_int8_gemm(w, s, x, y_in=base, mode=1))
    if n % 2 == 0:
        # the same matrix read as a stacked [gate; up] pair of n/2 channels each
        assert np.array_equal(ops.int8_gemm_rows(w, s, x, mode=2), ref.ref_int8_gemm(w, s, x, mode=2))
    # the oracle itself is pinned by the same comparison
    assert np.array_equal(orc.int8_gemm_rows(w, s, x), ref.ref_int8_gemm(w, s, x))


def test_quantizer_vs_reference_kernel(orc, ops, ref):
    rng = np.random.default_rng(12)
    wt = orc.to_bf16((rng.standard_normal((64, 512)) * 0.05).astype(np.float32))
    q, s = ops.quantize_rows(wt)
    rq, rs = ref.ref_quantize_rows(wt)
    assert np.array_equal(q, rq) and np.array_equal(s, rs)


def test_no_device_wait_ran_out(q3t, ops):
    """Every wait on a bulk copy or a tensor-core barrier is bounded; a healthy run never exhausts one."""
    assert q3t.library().q3t_kernel_error_count() == 0
