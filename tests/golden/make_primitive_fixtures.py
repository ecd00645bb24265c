"""Regenerates tests/golden/primitive_parity.npz.

The reference project's only known-answer test for this path is
native/qwen3-tts-native/native/src/primitive_parity.cu:115-324: four closed-form
inputs (RMSNorm W=128; RoPE 2 heads x 128 at position 37, theta 1e6; GQA attention
4 query / 2 KV heads, head_dim 32, 7 positions; SiLU-gate W=257) with host fp32
expectations and an absolute tolerance of 0.016.  This script restates those formulas
(glibc float math through ctypes, as the reference's host code uses) and stores inputs
as bf16 bit patterns plus the expected bf16-rounded values.  Nothing is copied from the
reference; run it again whenever the formulas here change:

    python tests/golden/make_primitive_fixtures.py
"""
import ctypes
import ctypes.util
import os

import numpy as np

_m = ctypes.CDLL(ctypes.util.find_library("m"))
for _name in ("sinf", "cosf", "expf", "sqrtf"):
    getattr(_m, _name).restype = ctypes.c_float
    getattr(_m, _name).argtypes = [ctypes.c_float]
_m.powf.restype = ctypes.c_float
_m.powf.argtypes = [ctypes.c_float, ctypes.c_float]

f32 = np.float32


def sinf(x): return f32(_m.sinf(float(f32(x))))
def cosf(x): return f32(_m.cosf(float(f32(x))))
def expf(x): return f32(_m.expf(float(f32(x))))
def sqrtf(x): return f32(_m.sqrtf(float(f32(x))))
def powf(x, y): return f32(_m.powf(float(f32(x)), float(f32(y))))


def to_bf16(a):
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    r = (u + np.uint32(0x7FFF) + ((u >> 16) & 1)) >> 16
    return r.astype(np.uint16)


def from_bf16(b):
    return (b.astype(np.uint32) << 16).view(np.float32)


def rbf(a):
    return from_bf16(to_bf16(a))


def rms_norm():
    width = 128
    x = np.array([sinf(f32(i) * f32(0.071)) * f32(1.7) for i in range(width)], dtype=f32)
    w = np.array([f32(0.75) + cosf(f32(i) * f32(0.037)) * f32(0.2) for i in range(width)], dtype=f32)
    xb, wb = to_bf16(x), to_bf16(w)
    x, w = from_bf16(xb), from_bf16(wb)
    ss = f32(0.0)
    for v in x:
        ss = f32(ss + f32(v * v))
    inv = f32(1.0) / sqrtf(f32(ss / f32(width)) + f32(1.0e-6))
    expected = rbf(np.array([f32(f32(x[i] * inv) * w[i]) for i in range(width)], dtype=f32))
    return dict(rms_x=xb, rms_w=wb, rms_expected=expected)


def rope():
    heads, dim, half, position, theta = 2, 128, 64, 37, f32(1.0e6)
    v = np.array([sinf(f32(i) * f32(0.019)) for i in range(heads * dim)], dtype=f32)
    vb = to_bf16(v)
    v = from_bf16(vb)
    expected = np.zeros_like(v)
    for h in range(heads):
        for i in range(half):
            exponent = f32(2 * i) / f32(dim)
            angle = f32(position) * powf(theta, -exponent)
            first, second = v[h * dim + i], v[h * dim + i + half]
            c, s = cosf(angle), sinf(angle)
            expected[h * dim + i] = f32(f32(first * c) - f32(second * s))
            expected[h * dim + i + half] = f32(f32(second * c) + f32(first * s))
    return dict(rope_v=vb, rope_expected=rbf(expected))


def attention():
    qh, kvh, dim, seq = 4, 2, 32, 7
    q = np.array([sinf(f32(i) * f32(0.031)) * f32(0.4) for i in range(qh * dim)], dtype=f32)
    k = np.array([cosf(f32(i) * f32(0.023)) * f32(0.3) for i in range(seq * kvh * dim)], dtype=f32)
    v = np.array([sinf(f32(i) * f32(0.017)) * f32(0.5) for i in range(seq * kvh * dim)], dtype=f32)
    qb, kb, vb = to_bf16(q), to_bf16(k), to_bf16(v)
    q, k, v = from_bf16(qb), from_bf16(kb), from_bf16(vb)
    expected = np.zeros(qh * dim, dtype=f32)
    for h in range(qh):
        g = h // (qh // kvh)
        scores = np.zeros(seq, dtype=f32)
        maximum = f32(-np.inf)
        for p in range(seq):
            dot = f32(0.0)
            for i in range(dim):
                dot = f32(dot + f32(q[h * dim + i] * k[(p * kvh + g) * dim + i]))
            scores[p] = dot / sqrtf(f32(dim))
            maximum = max(maximum, scores[p])
        den = f32(0.0)
        for p in range(seq):
            scores[p] = expf(scores[p] - maximum)
            den = f32(den + scores[p])
        for i in range(dim):
            acc = f32(0.0)
            for p in range(seq):
                acc = f32(acc + f32(f32(scores[p] / den) * v[(p * kvh + g) * dim + i]))
            expected[h * dim + i] = acc
    return dict(att_q=qb, att_k=kb, att_v=vb, att_expected=rbf(expected))


def silu_gate():
    width = 257
    g = np.array([sinf(f32(i) * f32(0.043)) * f32(2.0) for i in range(width)], dtype=f32)
    u = np.array([cosf(f32(i) * f32(0.029)) for i in range(width)], dtype=f32)
    gb, ub = to_bf16(g), to_bf16(u)
    g, u = from_bf16(gb), from_bf16(ub)
    expected = np.array([f32(f32(g[i] / f32(f32(1.0) + expf(-g[i]))) * u[i]) for i in range(width)],
                        dtype=f32)
    return dict(silu_gate=gb, silu_up=ub, silu_expected=rbf(expected))


if __name__ == "__main__":
    data = {}
    for part in (rms_norm, rope, attention, silu_gate):
        data.update(part())
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "primitive_parity.npz")
    np.savez_compressed(out, **data)
    print("wrote", out, {k: v.shape for k, v in data.items()})
