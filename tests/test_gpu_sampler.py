"""GPU parity of the sampler (temperature / top-k / top-p / repetition penalty / EOS suppression): token IDs and the post-call RNG state must be
bit-exact given identical logits, history and seed -- against the CPU oracle and, when
oracle/_ref is present, against the reference's own sample_logits_kernel on the same GPU."""
import itertools

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def logits_case(orc, rng, vocab, kind):
    if kind == "normal":
        x = rng.standard_normal(vocab) * 3.0
    elif kind == "ties":                       # few distinct values: many exact ties
        x = rng.integers(-3, 4, size=vocab).astype(np.float64) * 0.5
    elif kind == "all_equal":
        x = np.full(vocab, 1.25)
    elif kind == "zeros":                      # +0 and -0 must tie
        x = np.where(rng.random(vocab) < 0.5, 0.0, -0.0)
    elif kind == "peaked":
        x = rng.standard_normal(vocab)
        x[rng.integers(0, vocab)] = 30.0
    else:                                      # -inf tail
        x = rng.standard_normal(vocab) * 2.0
        x[rng.random(vocab) < 0.7] = -np.inf
        x[0] = 0.5
    return orc.to_bf16(x.astype(np.float32))


KINDS = ["normal", "ties", "all_equal", "zeros", "peaked", "inf_tail"]


def sweep(orc, seed, count):
    rng = np.random.default_rng(seed)
    for i in range(count):
        vocab = int(rng.choice([2048, 3072, 3072, 17, 513]))
        kind = KINDS[i % len(KINDS)]
        suppress = bool(vocab == 3072 and rng.random() < 0.6)
        history = rng.integers(0, min(vocab, 2048), size=int(rng.choice([0, 1, 40, 900]))).astype(np.int32)
        cfg = dict(
            do_sample=int(rng.random() < 0.9),
            top_k=int(rng.choice([0, 1, 2, 50, 50, 50, 512, 513, 1024, 1025, vocab, vocab + 5])),
            top_p=float(rng.choice([0.5, 0.9, 0.9, 1.0, 1.0, 0.999])),
            temperature=float(rng.choice([0.5, 0.9, 0.9, 1.5])),
            penalty=float(rng.choice([1.0, 1.05, 1.05, 2.0, 0.8])),
        )
        state = int(rng.integers(0, 2 ** 63)) if i % 7 else 0     # state 0 is re-seeded in place
        yield logits_case(orc, rng, vocab, kind), state, suppress, history, cfg


def test_bit_exact_vs_oracle(orc, ops):
    mismatches = []
    for i, (logits, state, suppress, history, cfg) in enumerate(sweep(orc, 0, 360)):
        want = orc.sample(logits, state, suppress=suppress, history=history, **cfg)
        got = ops.sample(logits, state, suppress=suppress, history=history, **cfg)
        if got != want:
            mismatches.append((i, logits.size, suppress, history.size, cfg, got, want))
    assert not mismatches, mismatches[:5]


def test_config_defaults_paths(orc, ops):
    """The three configurations the product uses, many seeds each."""
    rng = np.random.default_rng(1)
    configs = [
        (3072, True, dict(do_sample=1, top_k=50, top_p=0.9, temperature=0.9, penalty=1.0)),    # the talker configuration of the benchmark spec
        (3072, True, dict(do_sample=1, top_k=50, top_p=1.0, temperature=0.9, penalty=1.05)),   # official talker
        (2048, False, dict(do_sample=1, top_k=50, top_p=1.0, temperature=0.9, penalty=1.0)),   # official predictor
    ]
    for vocab, suppress, cfg in configs:
        state = 0x1234567
        history = []
        for _ in range(60):
            logits = orc.to_bf16((rng.standard_normal(vocab) * 2.5).astype(np.float32))
            want_tok, want_state = orc.sample(logits, state, suppress=suppress, history=history, **cfg)
            got_tok, got_state = ops.sample(logits, state, suppress=suppress, history=history, **cfg)
            assert (got_tok, got_state) == (want_tok, want_state)
            state = got_state
            if suppress:
                history.append(got_tok)


def test_greedy_does_not_draw(orc, ops):
    logits = orc.to_bf16(np.random.default_rng(2).standard_normal(2048).astype(np.float32))
    tok, state = ops.sample(logits, 777, do_sample=0, top_k=0)
    assert state == 777 and tok == int(np.argmax(orc.from_bf16(logits)))


def test_history_count_read_from_device(orc, ops):
    rng = np.random.default_rng(3)
    logits = orc.to_bf16((rng.standard_normal(3072) * 3).astype(np.float32))
    history = rng.integers(0, 2048, size=300).astype(np.int32)
    cfg = dict(do_sample=1, top_k=50, top_p=0.9, temperature=0.9, penalty=1.3)
    a = ops.sample(logits, 5, suppress=True, history=history, **cfg)
    b = ops.sample(logits, 5, suppress=True, history=history, count_on_device=True, **cfg)
    assert a == b == orc.sample(logits, 5, suppress=True, history=history, **cfg)


def test_invalid_vocabulary_rejected(orc, ops):
    with pytest.raises(RuntimeError):
        ops.sample(np.zeros(3073, dtype=np.uint16), 1)     # sampling_kernels.cu:476


# ---- against the reference's own kernel on the same GPU --------------------------------------

def test_bit_exact_vs_reference_kernel(orc, ops, ref):
    mismatches = []
    for i, (logits, state, suppress, history, cfg) in enumerate(sweep(orc, 4, 240)):
        if logits.size > 3072:
            continue
        want = ref.ref_sample(logits, state, suppress=suppress, history=history, **cfg)
        got = ops.sample(logits, state, suppress=suppress, history=history, **cfg)
        oracle = orc.sample(logits, state, suppress=suppress, history=history, **cfg)
        if got != want or oracle != want:
            mismatches.append((i, logits.size, suppress, history.size, cfg, got, want, oracle))
    assert not mismatches, mismatches[:5]
