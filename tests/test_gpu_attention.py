"""GPU parity of the split-KV decode attention (stand-alone and with head-norm, RoPE and KV append fused).

Semantic reference: the reference's fast kernel (fp32 scores).  The split-KV kernel sums in a
different order, so the comparison is the north-star tolerance: the fp32 value before the final
round within 1e-3 (relative to |value| + the head's RMS), and the bf16 output within one ulp of
bf16(oracle) with fewer than 1 % of elements differing at all."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def bf(orc, a):
    return orc.to_bf16(np.asarray(a, dtype=np.float32))


def make(orc, seed, rows, qh, kvh, hd, cap, positions):
    rng = np.random.default_rng(seed)
    q = bf(orc, rng.standard_normal((rows, qh * hd)))
    k = bf(orc, rng.standard_normal((rows, cap, kvh * hd)))
    v = bf(orc, rng.standard_normal((rows, cap, kvh * hd)))
    return q, k, v, np.asarray(positions, dtype=np.int32)


def check_bf16(orc, got_bf16, want_bf16, hd):
    """bf16 outputs: fewer than 1 % of elements differ at all, and where they do the difference
    is one rounding step (2^-7 relative) of the element -- or, for elements that are small
    against their head (cancellation), of a quarter of the head's RMS."""
    got = orc.from_bf16(got_bf16).reshape(-1, hd)
    want = orc.from_bf16(want_bf16).reshape(-1, hd)
    rms = np.sqrt((want ** 2).mean(axis=1, keepdims=True))
    step = 2.0 ** -7 * np.maximum(np.abs(want), 0.25 * rms)
    bad = np.abs(got - want) > step
    assert not bad.any(), (int(bad.sum()), float(np.abs(got - want).max()))
    assert (got != want).mean() < 0.01, float((got != want).mean())


def check(orc, got_bf16, got_f32, want_bf16, want_f32, hd):
    heads = want_f32.reshape(-1, hd)
    rms = np.sqrt((heads ** 2).mean(axis=1, keepdims=True))
    rel = np.abs(got_f32.reshape(-1, hd) - heads) / (np.abs(heads) + rms)
    assert rel.max() <= 1.0e-3, rel.max()
    check_bf16(orc, got_bf16, want_bf16, hd)


@pytest.mark.parametrize("length", [1, 2, 15, 16, 17, 63, 64, 65, 128, 513, 2048])
def test_talker_shape_lengths(orc, ops, length):
    rows, qh, kvh, hd = 2, 16, 8, 128
    cap = max(length, 16)
    q, k, v, pos = make(orc, length, rows, qh, kvh, hd, cap, [length - 1, max(0, length // 2 - 1)])
    out = ops.attention_ex(q, pos, qh, kvh, hd, k=k, v=v, want_f32=True)
    want, want32 = orc.attention(q, k, v, pos, qh, kvh, hd, fast=True, want_f32=True)
    check(orc, out["out"], out["f32"], want, want32, hd)


@pytest.mark.parametrize("qh,kvh,hd", [(16, 8, 64), (4, 2, 32), (8, 8, 128), (8, 2, 64)])
def test_other_head_shapes(orc, ops, qh, kvh, hd):
    rows, cap = 3, 200
    q, k, v, pos = make(orc, 7, rows, qh, kvh, hd, cap, [199, 0, 70])
    out = ops.attention_ex(q, pos, qh, kvh, hd, k=k, v=v, want_f32=True)
    want, want32 = orc.attention(q, k, v, pos, qh, kvh, hd, fast=True, want_f32=True)
    check(orc, out["out"], out["f32"], want, want32, hd)


def test_ragged_batch_of_64(orc, ops):
    rows, qh, kvh, hd, cap = 64, 16, 8, 128, 320
    positions = np.random.default_rng(3).integers(0, cap, size=rows)
    q, k, v, pos = make(orc, 8, rows, qh, kvh, hd, cap, positions)
    out = ops.attention_ex(q, pos, qh, kvh, hd, k=k, v=v, want_f32=True)
    want, want32 = orc.attention(q, k, v, pos, qh, kvh, hd, fast=True, want_f32=True)
    check(orc, out["out"], out["f32"], want, want32, hd)
    # a row's result does not depend on its neighbours: run row 5 alone
    alone = ops.attention_ex(q[5:6], pos[5:6], qh, kvh, hd, k=k[5:6], v=v[5:6])
    assert np.array_equal(alone["out"][0], out["out"][5])


def test_reference_shaped_entry_point(orc, ops):
    rows, qh, kvh, hd, cap = 3, 16, 8, 128, 300
    q, k, v, pos = make(orc, 9, rows, qh, kvh, hd, cap, [299, 5, 64])
    got = ops.attention_contiguous(q, k, v, pos, qh, kvh, hd)
    full = ops.attention_ex(q, pos, qh, kvh, hd, k=k, v=v)
    assert np.array_equal(got, full["out"])


def paged_copy(k, v, kvw, rng, per_slab, hd=128):
    """Scatters contiguous caches [rows][cap][kvw] into shuffled 16-token pages of two slabs.  A page is
    head-major: [kv head][16 tokens][head_dim], so that a head's 16 tokens are one contiguous block."""
    rows, cap, _ = k.shape
    heads = kvw // hd
    pages_per_row = (cap + 15) // 16
    total = rows * pages_per_row
    slabs = [np.zeros((2, per_slab, heads, 16, hd), dtype=np.uint16) for _ in range((total + per_slab - 1) // per_slab + 1)]
    ids = rng.permutation(len(slabs) * per_slab)[:total]
    table = ids.reshape(rows, pages_per_row).astype(np.int32)
    for r in range(rows):
        for p in range(pages_per_row):
            pid = int(table[r, p])
            s, i = divmod(pid, per_slab)
            n = min(16, cap - p * 16)
            slabs[s][0, i, :, :n] = k[r, p * 16:p * 16 + n].reshape(n, heads, hd).transpose(1, 0, 2)
            slabs[s][1, i, :, :n] = v[r, p * 16:p * 16 + n].reshape(n, heads, hd).transpose(1, 0, 2)
    return slabs, table


def test_paged_equals_contiguous(orc, ops):
    rows, qh, kvh, hd, cap = 5, 16, 8, 128, 176
    q, k, v, pos = make(orc, 10, rows, qh, kvh, hd, cap, [175, 0, 15, 16, 100])
    contiguous = ops.attention_ex(q, pos, qh, kvh, hd, k=k, v=v)
    slabs, table = paged_copy(k, v, kvh * hd, np.random.default_rng(4), per_slab=32)
    paged = ops.attention_ex(q, pos, qh, kvh, hd, pages=slabs, page_table=table, slab_shift=5)
    assert np.array_equal(paged["out"], contiguous["out"])


@pytest.mark.parametrize("hd,qh,kvh", [(128, 16, 8), (64, 16, 8)])
def test_fused_norm_rope_append(orc, ops, hd, qh, kvh):
    """Fused launch == head-norm, RoPE, append, attention run one after the other."""
    rows, cap = 4, 150
    rng = np.random.default_rng(11)
    qw, kvw = qh * hd, kvh * hd
    positions = np.array([149, 0, 64, 17], dtype=np.int32)
    q, k, v, pos = make(orc, 12, rows, qh, kvh, hd, cap, positions)
    stride = qw + 2 * kvw
    qkv = bf(orc, rng.standard_normal((rows, stride)) * 1.5)
    qn = bf(orc, 1.0 + 0.05 * rng.standard_normal(hd))
    kn = bf(orc, 1.0 + 0.05 * rng.standard_normal(hd))
    fused = ops.attention_ex(qkv, pos, qh, kvh, hd, k=k, v=v, q_norm_w=qn, k_norm_w=kn, fused=True,
                             q_stride=stride, new_stride=stride)
    # step by step with the stand-alone operators
    q2 = np.ascontiguousarray(qkv[:, :qw])
    k2 = np.ascontiguousarray(qkv[:, qw:qw + kvw])
    v2 = np.ascontiguousarray(qkv[:, qw + kvw:])
    q2 = ops.rope_rows_at(ops.head_rms_norm_rows(q2, qn, rows, qh, hd), rows, qh, hd, pos).reshape(rows, qw)
    k2 = ops.rope_rows_at(ops.head_rms_norm_rows(k2, kn, rows, kvh, hd), rows, kvh, hd, pos).reshape(rows, kvw)
    kc = ops.kv_scatter_rows(k2, k, pos)
    vc = ops.kv_scatter_rows(v2, v, pos)
    plain = ops.attention_ex(q2, pos, qh, kvh, hd, k=kc, v=vc)
    assert np.array_equal(fused["k"], kc) and np.array_equal(fused["v"], vc)
    assert np.array_equal(fused["out"], plain["out"])


def test_fused_paged_append(orc, ops):
    rows, qh, kvh, hd, cap = 3, 16, 8, 128, 80
    rng = np.random.default_rng(13)
    qw, kvw = qh * hd, kvh * hd
    q, k, v, pos = make(orc, 14, rows, qh, kvh, hd, cap, [79, 31, 32])
    stride = qw + 2 * kvw
    qkv = bf(orc, rng.standard_normal((rows, stride)))
    qn = bf(orc, np.ones(hd))
    kn = bf(orc, np.ones(hd))
    a = ops.attention_ex(qkv, pos, qh, kvh, hd, k=k, v=v, q_norm_w=qn, k_norm_w=kn, fused=True,
                         q_stride=stride, new_stride=stride)
    slabs, table = paged_copy(k, v, kvw, np.random.default_rng(5), per_slab=16)
    b = ops.attention_ex(qkv, pos, qh, kvh, hd, pages=slabs, page_table=table, slab_shift=4,
                         q_norm_w=qn, k_norm_w=kn, fused=True, q_stride=stride, new_stride=stride)
    assert np.array_equal(a["out"], b["out"])
    for r in range(rows):   # the appended row landed in the right page
        pid = int(table[r, pos[r] // 16])
        s, i = divmod(pid, 16)
        assert np.array_equal(b["pages"][s][0, i, :, pos[r] % 16].reshape(-1), a["k"][r, pos[r]])
        assert np.array_equal(b["pages"][s][1, i, :, pos[r] % 16].reshape(-1), a["v"][r, pos[r]])


def test_repeated_launches_reuse_scratch(orc, ops):
    """The ticket counters reset themselves: two launches in a row give the same answer."""
    rows, qh, kvh, hd, cap = 2, 16, 8, 128, 400
    q, k, v, pos = make(orc, 15, rows, qh, kvh, hd, cap, [399, 130])
    first = ops.attention_ex(q, pos, qh, kvh, hd, k=k, v=v)["out"]
    second = ops.attention_ex(q, pos, qh, kvh, hd, k=k, v=v)["out"]
    assert np.array_equal(first, second)


# ---- against the reference's own kernels on the same GPU ------------------------------------

@pytest.mark.parametrize("length", [7, 64, 513])
def test_vs_reference_fast_kernel(orc, ops, ref, length):
    rows, qh, kvh, hd = 2, 16, 8, 128
    q, k, v, pos = make(orc, 16, rows, qh, kvh, hd, length, [length - 1, length // 3])
    out = ops.attention_ex(q, pos, qh, kvh, hd, k=k, v=v, want_f32=True)
    fast = ref.ref_attention(q, k, v, pos, qh, kvh, hd, fast=True)
    check_bf16(orc, out["out"], fast, hd)
    # the oracle restates that kernel: pin it here too (expf and rsqrtf differ by an ulp
    # between libm and CUDA, which shows on elements that nearly cancel)
    check_bf16(orc, orc.attention(q, k, v, pos, qh, kvh, hd, fast=True), fast, hd)
    # distance to the reference's bf16-rounding "exact" kernel, reported for context
    exact = ref.ref_attention(q, k, v, pos, qh, kvh, hd, fast=False)
    d = orc.bf16_ulp_distance(out["out"], exact)
    print(f"L={length}: max ulp distance to the exact kernel {int(d.max())}, "
          f"{100 * float((d > 0).mean()):.1f}% of elements differ")


# ---- parity mode: sums in the reference's order ----------------------------------------------

@pytest.fixture
def reference_order(q3t):
    before = q3t.native.set_attention_mode(0)
    yield
    q3t.native.set_attention_mode(before)


@pytest.mark.parametrize("length", [1, 2, 7, 64, 257, 513, 1100])
def test_reference_order_is_bit_identical(orc, ops, ref, reference_order, length):
    """Attention mode 0 against the reference's fast kernel run on the same GPU: equal bits."""
    rows, qh, kvh, hd = 3, 16, 8, 128
    q, k, v, pos = make(orc, 21, rows, qh, kvh, hd, length, [length - 1, length // 3, 0])
    got = ops.attention_ex(q, pos, qh, kvh, hd, k=k, v=v)["out"]
    want = ref.ref_attention(q, k, v, pos, qh, kvh, hd, fast=True)
    assert np.array_equal(got.reshape(-1), want.reshape(-1))
    slabs, table = paged_copy(k, v, kvh * hd, np.random.default_rng(6), per_slab=32)
    paged = ops.attention_ex(q, pos, qh, kvh, hd, pages=slabs, page_table=table, slab_shift=5)["out"]
    assert np.array_equal(paged.reshape(-1), want.reshape(-1))


def test_reference_order_fused(orc, ops, ref, reference_order):
    """Fused call in mode 0 == the stand-alone operators one after the other, then the reference's
    fast kernel over the caches they produced."""
    rows, qh, kvh, hd, cap = 4, 16, 8, 128, 150
    rng = np.random.default_rng(22)
    qw, kvw = qh * hd, kvh * hd
    q, k, v, pos = make(orc, 23, rows, qh, kvh, hd, cap, [149, 0, 64, 17])
    stride = qw + 2 * kvw
    qkv = bf(orc, rng.standard_normal((rows, stride)) * 1.5)
    qn = bf(orc, 1.0 + 0.05 * rng.standard_normal(hd))
    kn = bf(orc, 1.0 + 0.05 * rng.standard_normal(hd))
    fused = ops.attention_ex(qkv, pos, qh, kvh, hd, k=k, v=v, q_norm_w=qn, k_norm_w=kn, fused=True,
                             q_stride=stride, new_stride=stride)
    q2 = np.ascontiguousarray(qkv[:, :qw])
    k2 = np.ascontiguousarray(qkv[:, qw:qw + kvw])
    v2 = np.ascontiguousarray(qkv[:, qw + kvw:])
    q2 = ops.rope_rows_at(ops.head_rms_norm_rows(q2, qn, rows, qh, hd), rows, qh, hd, pos).reshape(rows, qw)
    k2 = ops.rope_rows_at(ops.head_rms_norm_rows(k2, kn, rows, kvh, hd), rows, kvh, hd, pos).reshape(rows, kvw)
    kc = ops.kv_scatter_rows(k2, k, pos)
    vc = ops.kv_scatter_rows(v2, v, pos)
    assert np.array_equal(fused["k"], kc) and np.array_equal(fused["v"], vc)
    want = ref.ref_attention(q2, kc, vc, pos, qh, kvh, hd, fast=True)
    assert np.array_equal(fused["out"].reshape(-1), want.reshape(-1))


def test_position_outside_the_launch_is_clamped_and_counted(q3t, orc, ops):
    """A position at or past max_sequence_length (the caller's device memory said so) must not run the
    kernel over scratch and tickets it was not sized for: the row is computed over the clamped length,
    the library's range-error counter rises, and the next launch is unaffected."""
    rows, qh, kvh, hd, cap = 2, 16, 8, 128, 128
    q, k, v, pos = make(orc, 31, rows, qh, kvh, hd, cap, [127, 40])
    lib = q3t.library()
    before = int(lib.q3t_attention_range_error_count())
    good = ops.attention_ex(q, pos, qh, kvh, hd, k=k, v=v)["out"]
    assert int(lib.q3t_attention_range_error_count()) == before
    bad_pos = np.array([5000, 40], dtype=np.int32)       # row 0 claims a length the launch was not sized for
    out = ops.attention_ex(q, bad_pos, qh, kvh, hd, k=k, v=v)["out"]
    assert int(lib.q3t_attention_range_error_count()) > before
    assert np.array_equal(out.reshape(rows, -1)[0], good.reshape(rows, -1)[0])      # clamped to position 127
    assert np.array_equal(out.reshape(rows, -1)[1], good.reshape(rows, -1)[1])
    again = ops.attention_ex(q, pos, qh, kvh, hd, k=k, v=v)["out"]
    assert np.array_equal(again, good)


def test_operator_benchmark_case_runs(q3t):
    """The paged, ragged case `bench.py --leg attn` profiles: runs, reports the bytes it read."""
    us, kv_bytes = q3t.native.benchmark_decode_attention(0, rows=4, min_length=10, max_length=300, seed=5, iterations=2)
    assert us > 0.0
    assert kv_bytes % (1024 * 2 * 2) == 0 and 4 * 10 <= kv_bytes // 4096 <= 4 * 300      # tokens x 1024 x bf16 x (K, V)
