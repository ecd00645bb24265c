"""GPU parity of the row operators (norms, RoPE, KV append, elementwise glue): RMSNorm, per-head
RMSNorm, RoPE, KV append, bias/activation, SiLU gate, residual add, embedding gather/add,
plus the reference's four closed-form known-answer cases run through this library.

The operators keep the reference's fp32 order and use the same CUDA math functions, so they
must be bit-identical to the reference kernels on the same GPU; against the CPU oracle a
transcendental (rsqrtf, powf, cosf, sinf, expf) may differ by an ulp and flip a bf16 rounding
on a few elements."""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def bf(orc, a):
    return orc.to_bf16(np.asarray(a, dtype=np.float32))


def vp(a):
    import ctypes
    return ctypes.c_void_p(a.ctypes.data)


def ulps(orc, got, want):
    d = orc.bf16_ulp_distance(got, want)
    return int(d.max()), float((d > 0).mean())


def test_known_answer_cases(q3t):
    """qwen3_tts_validate_transformer_primitives: tolerance 0.016 as in the reference."""
    r = q3t.native.validate_transformer_primitives(0)
    assert r.rms_norm_max_absolute_error <= 0.016
    assert r.rope_max_absolute_error <= 0.016
    assert r.attention_max_absolute_error <= 0.016
    assert r.silu_gate_max_absolute_error <= 0.016


def test_golden_fixtures_through_the_abi(orc, ops):
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "primitive_parity.npz"))
    y = ops.rms_norm_rows(g["rms_x"][None, :], g["rms_w"])
    assert np.abs(orc.from_bf16(y)[0] - g["rms_expected"]).max() <= 0.016
    v = ops.rope_rows_at(g["rope_v"], 1, 2, 128, [37])
    assert np.abs(orc.from_bf16(v) - g["rope_expected"]).max() <= 0.016
    a = ops.attention_contiguous(g["att_q"], g["att_k"].reshape(1, 7, 64), g["att_v"].reshape(1, 7, 64),
                                 [6], 4, 2, 32)
    assert np.abs(orc.from_bf16(a)[0] - g["att_expected"]).max() <= 0.016
    s = ops.silu_gate(g["silu_gate"], g["silu_up"])
    assert np.abs(orc.from_bf16(s) - g["silu_expected"]).max() <= 0.016


@pytest.mark.parametrize("rows,width", [(1, 128), (1, 2048), (5, 1024), (64, 2048), (3, 100)])
def test_rms_norm_rows(orc, ops, rows, width):
    rng = np.random.default_rng(0)
    x = bf(orc, rng.standard_normal((rows, width)) * 2.5)
    w = bf(orc, 1.0 + 0.05 * rng.standard_normal(width))
    got = ops.rms_norm_rows(x, w)
    worst, frac = ulps(orc, got, orc.rms_norm_rows(x, w))
    assert worst <= 1 and frac < 0.01, (worst, frac)


@pytest.mark.parametrize("rows,heads,hd", [(1, 16, 128), (3, 8, 128), (2, 16, 64), (1, 4, 32), (64, 8, 128)])
def test_head_rms_norm_rows(orc, ops, rows, heads, hd):
    rng = np.random.default_rng(1)
    v = bf(orc, rng.standard_normal(rows * heads * hd) * 1.7)
    w = bf(orc, 1.0 + 0.05 * rng.standard_normal(hd))
    got = ops.head_rms_norm_rows(v, w, rows, heads, hd)
    worst, frac = ulps(orc, got, orc.head_rms_norm(v, w, hd))
    assert worst <= 1 and frac < 0.01, (worst, frac)


@pytest.mark.parametrize("rows,heads,hd", [(1, 16, 128), (4, 8, 128), (2, 16, 64)])
def test_rope_rows_at(orc, ops, rows, heads, hd):
    rng = np.random.default_rng(2)
    v = bf(orc, rng.standard_normal(rows * heads * hd))
    positions = rng.integers(0, 8192, size=rows).astype(np.int32)
    positions[0] = 0
    got = ops.rope_rows_at(v, rows, heads, hd, positions)
    worst, frac = ulps(orc, got, orc.rope_rows_at(v, rows, heads, hd, positions))
    assert worst <= 2 and frac < 0.03, (worst, frac)
    zero = ops.rope_rows_at(v, rows, heads, hd, np.zeros(rows, dtype=np.int32))
    assert np.array_equal(zero, v)            # angle 0: cos 1, sin 0


def test_kv_scatter_rows(orc, ops):
    rng = np.random.default_rng(3)
    rows, cap, width = 5, 12, 1024
    caches = bf(orc, rng.standard_normal((rows, cap, width)))
    new = bf(orc, rng.standard_normal((rows, width)))
    positions = np.array([0, 11, 3, 7, 5], dtype=np.int32)
    got = ops.kv_scatter_rows(new, caches, positions)
    want = caches.copy()
    for r in range(rows):
        want[r, positions[r]] = new[r]
    assert np.array_equal(got, want)


@pytest.mark.parametrize("silu", [False, True])
def test_bias_activation_rows(orc, ops, silu):
    rng = np.random.default_rng(4)
    v = bf(orc, rng.standard_normal((6, 1024)) * 2)
    b = bf(orc, rng.standard_normal(1024) * 0.2)
    got = ops.bias_activation_rows(v, b, silu)
    worst, frac = ulps(orc, got, orc.bias_activation_rows(v, b, silu))
    assert worst <= (1 if silu else 0) and frac < 0.01, (worst, frac)


def test_add_and_silu_gate(orc, ops):
    rng = np.random.default_rng(5)
    a = bf(orc, rng.standard_normal(4097))
    b = bf(orc, rng.standard_normal(4097))
    assert np.array_equal(ops.add_in_place(a, b), orc.add(a, b))
    worst, frac = ulps(orc, ops.silu_gate(a, b), orc.silu_gate(a, b))
    assert worst <= 1 and frac < 0.01, (worst, frac)


def test_embedding_gather_and_add(orc, ops):
    rng = np.random.default_rng(6)
    table = bf(orc, rng.standard_normal((300, 256)))
    tokens = np.array([[5, 299, 0], [17, -1, 4], [300, 2, 2]], dtype=np.int32)
    got = ops.gather_embedding_rows(table, tokens, 0)
    assert np.array_equal(got[0], table[5]) and np.array_equal(got[1], table[17])
    assert not got[2].any()                   # out-of-range token: row left untouched
    acc = ops.gather_embedding_rows(table, tokens, 1, out=got)
    assert np.array_equal(acc[0], orc.add(table[5], table[299]))
    assert np.array_equal(acc[1], table[17])  # -1 skipped
    assert np.array_equal(acc[2], orc.add(np.zeros(256, dtype=np.uint16), table[2]))


# ---- against the reference's own kernels on the same GPU ------------------------------------

def test_row_operators_bit_exact_vs_reference_kernels(orc, ops, ref):
    rng = np.random.default_rng(7)
    x = bf(orc, rng.standard_normal((8, 2048)) * 2.0)
    w = bf(orc, 1.0 + 0.05 * rng.standard_normal(2048))
    assert np.array_equal(ops.rms_norm_rows(x, w), ref.ref_rms_norm_rows(x, w))
    for heads, hd in ((16, 128), (8, 128), (16, 64)):
        v = bf(orc, rng.standard_normal(8 * heads * hd))
        hw = bf(orc, 1.0 + 0.05 * rng.standard_normal(hd))
        assert np.array_equal(ops.head_rms_norm_rows(v, hw, 8, heads, hd),
                              ref.ref_head_rms_norm_rows(v, hw, 8, heads, hd))
        pos = rng.integers(0, 8192, size=8).astype(np.int32)
        assert np.array_equal(ops.rope_rows_at(v, 8, heads, hd, pos),
                              ref.ref_rope_rows_at(v, 8, heads, hd, pos))
    b = bf(orc, rng.standard_normal(2048) * 0.3)
    for silu in (0, 1):
        got = ops.bias_activation_rows(x, b, silu)
        want = x.copy()
        assert ref.ref().ref_bias_activation_rows(vp(want), vp(b), 8, 2048, silu) == 0
        assert np.array_equal(got, want)
    g, u = x[0].copy(), x[1].copy()
    want = g.copy()
    assert ref.ref().ref_silu_gate(vp(want), vp(u), 2048) == 0
    assert np.array_equal(ops.silu_gate(g, u), want)
