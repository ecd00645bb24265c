"""The persistent chain of batch-1 GEMVs against the single-launch SIMT kernel: same descriptors,
same bits.  (The SIMT kernel is itself pinned against the oracle and the reference's kernels in
test_gpu_gemv.py.)"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def weights(rng, n, k):
    w = rng.integers(-127, 128, size=(n, k), dtype=np.int8)
    s = (rng.uniform(0.5, 1.5, size=n) / (73.6 * np.sqrt(k))).astype(np.float32)
    return w, s


def test_decoder_layer_tail_matches_single_launches(orc, ops):
    """attention output (+residual) -> RMSNorm + gate/up/SiLU -> down (+residual) -> RMSNorm + q/k/v:
    the chain a talker layer issues at batch 1, with the talker's shapes."""
    rng = np.random.default_rng(21)
    H, Q, I, QKV = 2048, 2048, 6144, 4096
    wo, so = weights(rng, H, Q)
    wg, sg = weights(rng, 2 * I, H)
    wd, sd = weights(rng, H, I)
    wq, sq = weights(rng, QKV, H)
    attn = orc.to_bf16(rng.standard_normal(Q).astype(np.float32))
    hidden = orc.to_bf16(rng.standard_normal(H).astype(np.float32))
    n1 = orc.to_bf16((1.0 + 0.02 * rng.standard_normal(H)).astype(np.float32))
    n2 = orc.to_bf16((1.0 + 0.02 * rng.standard_normal(H)).astype(np.float32))
    # one launch per projection
    h1 = ops.int8_gemm(wo, so, attn, epilogue=ops.EPI_ADD, y_in=hidden)["y"]
    g = ops.int8_gemm(wg, sg, h1, epilogue=ops.EPI_GATE_UP_SILU, norm_w=n1)["y"]
    h2 = ops.int8_gemm(wd, sd, g, epilogue=ops.EPI_ADD, y_in=h1)["y"]
    qkv = ops.int8_gemm(wq, sq, h2, norm_w=n2)["y"]
    # the same four as one chain
    out = ops.int8_gemv_chain([
        dict(w=wo, scales=so, x=attn, y="hidden", epilogue=ops.EPI_ADD, init={"hidden": hidden}),
        dict(w=wg, scales=sg, x="hidden", y="gate", epilogue=ops.EPI_GATE_UP_SILU, norm_w=n1),
        dict(w=wd, scales=sd, x="gate", y="hidden", epilogue=ops.EPI_ADD),
        dict(w=wq, scales=sq, x="hidden", y="qkv", norm_w=n2),
    ])
    assert np.array_equal(out["gate"], g)
    assert np.array_equal(out["hidden"], h2)
    assert np.array_equal(out["qkv"], qkv)


def test_bias_epilogues_and_predictor_shapes(orc, ops):
    rng = np.random.default_rng(22)
    w1, s1 = weights(rng, 1024, 2048)       # small_to_mtp: bias
    w2, s2 = weights(rng, 4096, 1024)       # predictor q/k/v
    w3, s3 = weights(rng, 1024, 3072)       # predictor down
    w4, s4 = weights(rng, 2048, 1024)       # head / fc: bias + SiLU, then bias + residual
    x = orc.to_bf16(rng.standard_normal(2048).astype(np.float32))
    x3 = orc.to_bf16(rng.standard_normal(3072).astype(np.float32))
    b1 = orc.to_bf16((0.1 * rng.standard_normal(1024)).astype(np.float32))
    b4 = orc.to_bf16((0.1 * rng.standard_normal(2048)).astype(np.float32))
    nw = orc.to_bf16((1.0 + 0.02 * rng.standard_normal(1024)).astype(np.float32))
    res = orc.to_bf16(rng.standard_normal(2048).astype(np.float32))
    a = ops.int8_gemm(w1, s1, x, epilogue=ops.EPI_BIAS, bias=b1)["y"]
    b = ops.int8_gemm(w2, s2, a, norm_w=nw)["y"]
    c = ops.int8_gemm(w3, s3, x3, epilogue=ops.EPI_ADD, y_in=a)["y"]
    d = ops.int8_gemm(w4, s4, c, epilogue=ops.EPI_BIAS_SILU, bias=b4)["y"]
    e = ops.int8_gemm(w4, s4, c, epilogue=ops.EPI_BIAS_ADD, bias=b4, resid=res)["resid"]
    out = ops.int8_gemv_chain([
        dict(w=w1, scales=s1, x=x, y="a", epilogue=ops.EPI_BIAS, bias=b1),
        dict(w=w2, scales=s2, x="a", y="b", norm_w=nw),
        dict(w=w3, scales=s3, x=x3, y="a", epilogue=ops.EPI_ADD),
        dict(w=w4, scales=s4, x="a", y="d", epilogue=ops.EPI_BIAS_SILU, bias=b4),
        dict(w=w4, scales=s4, x="a", resid="e", epilogue=ops.EPI_BIAS_ADD, bias=b4, init={"e": res}),
    ])
    assert np.array_equal(out["b"], b)
    assert np.array_equal(out["a"], c)
    assert np.array_equal(out["d"], d)
    assert np.array_equal(out["e"], e)


def test_repeated_launches_and_odd_channel_counts(q3t, orc, ops):
    rng = np.random.default_rng(23)
    w, s = weights(rng, 77, 1024)
    x = orc.to_bf16(rng.standard_normal(1024).astype(np.float32))
    want = ops.int8_gemm(w, s, x)["y"]
    for _ in range(3):      # the barrier counters return to zero after every launch
        out = ops.int8_gemv_chain([dict(w=w, scales=s, x=x, y="y"), dict(w=w, scales=s, x=x, y="z")])
        assert np.array_equal(out["y"], want) and np.array_equal(out["z"], want)
    assert q3t.library().q3t_kernel_error_count() == 0


def test_unsupported_shapes_are_refused(orc, ops):
    rng = np.random.default_rng(24)
    w, s = weights(rng, 64, 528)
    x = orc.to_bf16(rng.standard_normal(528).astype(np.float32))
    with pytest.raises(RuntimeError):
        ops.int8_gemv_chain([dict(w=w, scales=s, x=x, y="y")])     # K not a multiple of 1024
