"""CPU checks of the oracle itself: the reference's closed-form known-answer cases
(tests/golden/primitive_parity.npz, regenerated from primitive_parity.cu's formulas),
agreement between its fp32 restatement and fp64 truth, and the sampler's branch structure."""
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "primitive_parity.npz")
TOL = 0.016   # the reference's own tolerance for these four cases (primitive_parity.cu)


@pytest.fixture(scope="module")
def golden():
    return np.load(GOLDEN)


def test_golden_rms_norm(orc, golden):
    y = orc.rms_norm_rows(golden["rms_x"][None, :], golden["rms_w"])
    assert np.abs(orc.from_bf16(y)[0] - golden["rms_expected"]).max() <= TOL


def test_golden_rope(orc, golden):
    v = orc.rope_rows_at(golden["rope_v"], 1, 2, 128, [37])
    assert np.abs(orc.from_bf16(v) - golden["rope_expected"]).max() <= TOL


@pytest.mark.parametrize("fast", [True, False])
def test_golden_attention(orc, golden, fast):
    k = golden["att_k"].reshape(1, 7, 64)
    v = golden["att_v"].reshape(1, 7, 64)
    out = orc.attention(golden["att_q"], k, v, [6], 4, 2, 32, fast=fast)
    assert np.abs(orc.from_bf16(out)[0] - golden["att_expected"]).max() <= TOL


def test_golden_silu_gate(orc, golden):
    g = orc.silu_gate(golden["silu_gate"], golden["silu_up"])
    assert np.abs(orc.from_bf16(g) - golden["silu_expected"]).max() <= TOL


def _gemv_case(orc, seed, n, k, rows=1):
    rng = np.random.default_rng(seed)
    w = rng.integers(-127, 128, size=(n, k), dtype=np.int8)
    s = (rng.uniform(0.5, 1.5, size=n) / 127.0).astype(np.float32)
    x = orc.to_bf16(rng.standard_normal((rows, k)).astype(np.float32))
    return w, s, x


@pytest.mark.parametrize("n,k,rows", [(8, 16, 1), (33, 64, 3), (256, 2048, 1), (64, 6144, 8)])
def test_gemv_fp32_against_fp64(orc, n, k, rows):
    w, s, x = _gemv_case(orc, 0, n, k, rows)
    y, acc = orc.int8_gemm_rows(w, s, x, want_acc=True)
    truth = orc.int8_gemm_rows_f64(w, s, x)
    # fp32 accumulate versus exact: relative to the row's scale of values
    err = np.abs(acc - truth) / (np.abs(truth) + np.sqrt((truth ** 2).mean()))
    assert err.max() < 1.0e-5
    assert np.array_equal(y, orc.to_bf16(acc))


def test_gemv_matches_plain_numpy(orc):
    w, s, x = _gemv_case(orc, 1, 40, 128)
    truth = (w.astype(np.float64) @ orc.from_bf16(x)[0].astype(np.float64)) * s
    assert np.allclose(orc.int8_gemm_rows_f64(w, s, x)[0], truth, rtol=1e-12)


def test_gemv_add_is_one_fma(orc):
    w, s, x = _gemv_case(orc, 2, 32, 64)
    base = orc.to_bf16(np.linspace(-3, 3, 32, dtype=np.float32))
    _, acc = orc.int8_gemm_rows(w, s, x, want_acc=True)
    y, val = orc.int8_gemm_rows(w, s, x, y_in=base, mode=1, want_acc=True)
    raw = acc[0] / s   # not exact, so recompute the fused form in float64 and round once
    truth = orc.int8_gemm_rows_f64(w, s, x)[0] + orc.from_bf16(base).astype(np.float64)
    assert np.abs(val[0] - truth).max() < 1e-4
    assert raw.shape == (32,)
    assert np.array_equal(y, orc.to_bf16(val))


def test_gate_up_silu(orc):
    rng = np.random.default_rng(3)
    n, k = 24, 96
    w = rng.integers(-127, 128, size=(2 * n, k), dtype=np.int8)
    s = (rng.uniform(0.5, 1.5, size=2 * n) / (127.0 * 8)).astype(np.float32)
    x = orc.to_bf16(rng.standard_normal((2, k)).astype(np.float32))
    y, val = orc.int8_gate_up_silu_rows(w, s, x, want_acc=True)
    both = orc.int8_gemm_rows_f64(w, s, x)
    g, u = both[:, :n], both[:, n:]
    truth = g / (1.0 + np.exp(-g)) * u
    assert np.abs(val - truth).max() < 1e-4 * (1 + np.abs(truth).max())
    assert np.array_equal(y, orc.to_bf16(val))


def test_quantizer(orc):
    rng = np.random.default_rng(4)
    w = orc.to_bf16((rng.standard_normal((16, 64)) * 0.05).astype(np.float32))
    w[3] = 0   # an all-zero row keeps scale 1 (int8_gemv.cu:41)
    q, s = orc.quantize_rows(w)
    wf = orc.from_bf16(w)
    assert s[3] == 1.0 and not q[3].any()
    mask = np.arange(16) != 3
    assert np.allclose(s[mask], np.abs(wf[mask]).max(axis=1) / 127.0, rtol=1e-6)
    assert np.abs(q).max() == 127
    assert np.abs(q[mask].astype(np.float32) * s[mask, None] - wf[mask]).max() <= s[mask].max() * 0.5001


def test_attention_fast_close_to_exact(orc):
    rng = np.random.default_rng(5)
    rows, qh, kvh, hd, cap = 2, 4, 2, 64, 40
    q = orc.to_bf16(rng.standard_normal((rows, qh * hd)).astype(np.float32))
    k = orc.to_bf16(rng.standard_normal((rows, cap, kvh * hd)).astype(np.float32))
    v = orc.to_bf16(rng.standard_normal((rows, cap, kvh * hd)).astype(np.float32))
    pos = [39, 12]
    fast = orc.from_bf16(orc.attention(q, k, v, pos, qh, kvh, hd, fast=True))
    exact = orc.from_bf16(orc.attention(q, k, v, pos, qh, kvh, hd, fast=False))
    assert np.abs(fast - exact).max() < 0.05   # bf16 rounding of scores/probabilities only


def _xorshift(state):
    mask = (1 << 64) - 1
    v = state or 0x9E3779B97F4A7C15
    v ^= v >> 12
    v ^= (v << 25) & mask
    v ^= v >> 27
    return v, ((v * 0x2545F4914F6CDD1D) & mask)


def test_xorshift_stream(orc):
    import ctypes as C
    state = C.c_uint64(orc.seed_state(0))
    py_state = orc.seed_state(0)
    for _ in range(5):
        u = orc.lib().orc_uniform(C.byref(state))
        py_state, out = _xorshift(py_state)
        assert state.value == py_state
        assert u == np.float32((out >> 11) * (1.0 / 9007199254740992.0))
        assert 0.0 <= u < 1.0 or u == 1.0


def test_sampler_greedy_and_ties(orc):
    logits = orc.to_bf16(np.array([0.5, 2.0, -1.0, 2.0, 1.0] + [0.0] * 11, dtype=np.float32))
    tok, st = orc.sample(logits, 123, do_sample=0, top_k=0)
    assert tok == 1 and st == 123            # ties go to the lower index, no RNG draw
    tok, st = orc.sample(logits, 123, do_sample=1, top_k=1)
    assert tok == 1 and st != 123            # a sampled call advances the state exactly once
    _, st2 = orc.sample(logits, 123, do_sample=1, top_k=0, top_p=1.0)
    assert st2 == st


def test_sampler_suppress_and_penalty(orc):
    rng = np.random.default_rng(6)
    logits = orc.to_bf16(rng.standard_normal(3072).astype(np.float32))
    big = orc.to_bf16(np.float32(50.0))
    logits[2500] = big          # reserved token: masked for talker rows
    logits[2150] = orc.to_bf16(np.float32(40.0))   # EOS stays selectable
    tok, _ = orc.sample(logits, 1, suppress=True, do_sample=0)
    assert tok == 2150
    tok, _ = orc.sample(logits, 1, suppress=False, do_sample=0)
    assert tok == 2500
    # repetition penalty only bites on tokens in the history and only for talker rows
    logits[7] = orc.to_bf16(np.float32(45.0))
    tok, _ = orc.sample(logits, 1, suppress=True, do_sample=0, history=[7], penalty=2.0)
    assert tok == 2150
    tok, _ = orc.sample(logits, 1, suppress=True, do_sample=0, history=[8], penalty=2.0)
    assert tok == 7


def test_sampler_top_p_keeps_head(orc):
    logits = orc.to_bf16(np.array([10.0, 9.0, 1.0, 0.0] + [-5.0] * 60, dtype=np.float32))
    seen = set()
    state = 99
    for _ in range(200):
        tok, state = orc.sample(logits, state, top_k=50, top_p=0.5, temperature=1.0)
        seen.add(tok)
    assert seen == {0}           # p(0) = 0.73 >= 0.5: only the first candidate is retained
    seen = set()
    for _ in range(300):
        tok, state = orc.sample(logits, state, top_k=2, top_p=1.0, temperature=1.0)
        seen.add(tok)
    assert seen == {0, 1}


def test_sampler_distribution(orc):
    logits = orc.to_bf16(np.log(np.array([0.5, 0.3, 0.2] + [1e-9] * 13, dtype=np.float32)))
    counts = np.zeros(16)
    state = 2024
    n = 4000
    for _ in range(n):
        tok, state = orc.sample(logits, state, top_k=0, top_p=1.0, temperature=1.0)
        counts[tok] += 1
    assert np.abs(counts[:3] / n - np.array([0.5, 0.3, 0.2])).max() < 0.03
