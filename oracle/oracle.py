"""TEST INFRASTRUCTURE ONLY: numpy front end of the CPU restatement (q3t_oracle.c).

The checker used by tests/, by the smoke check and by the benchmark's CPU-baseline
legs.  The product package never imports this module.  bf16 tensors are numpy
uint16 arrays holding the bit patterns.

Composition helpers at the bottom (decoder_layer, predictor_position, frame) restate
the reference's fused INT8 batch path, luka-loehr/qwen3-tts-native
native/qwen3-tts-native/native/src/talker.cu:1495-1881 and :2038-2334.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libq3t_oracle.so")
_REF_PATH = os.path.join(_HERE, "_ref", "libq3t_ref.so")

EOS = 2150
RMS_EPS = 1.0e-6
ROPE_THETA = 1.0e6


def build(force: bool = False) -> str:
    """Compile the C restatement (seconds).  Returns the library path."""
    src = os.path.join(_HERE, "q3t_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "libq3t_oracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = C.CDLL(build())
        _lib.orc_uniform.restype = C.c_float
        _lib.orc_sample.restype = C.c_int
        _lib.orc_threads.restype = C.c_int
    return _lib


def _p(a: np.ndarray | None):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"], "oracle arguments must be C-contiguous"
    return a.ctypes.data_as(C.c_void_p)


def threads() -> int:
    return int(lib().orc_threads())


def set_threads(n: int) -> None:
    lib().orc_set_threads(C.c_int(n))


# ------------------------------------------------------------------ bf16 helpers

def to_bf16(x) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().orc_f2bf(_p(x), _p(out), C.c_long(x.size))
    return out


def from_bf16(b) -> np.ndarray:
    b = np.ascontiguousarray(b, dtype=np.uint16)
    return (b.astype(np.uint32) << 16).view(np.float32).reshape(b.shape)


def bf16_ulp_distance(a, b) -> np.ndarray:
    """Distance in bf16 units of least precision between two bf16 bit arrays."""
    def key(u):
        u = np.asarray(u, dtype=np.uint16).astype(np.int32)
        return np.where(u & 0x8000, -(u & 0x7FFF), u & 0x7FFF)
    return np.abs(key(a) - key(b))


# ------------------------------------------------------------------ primitives

def int8_gemm_rows(w, scales, x, y_in=None, mode=0, want_acc=False):
    """mode 0: y=bf16(scale*(W x)); mode 1: y=bf16(y_in + scale*(W x))."""
    n, k = w.shape
    x = np.ascontiguousarray(x, dtype=np.uint16).reshape(-1, k)
    rows = x.shape[0]
    y = np.zeros((rows, n), dtype=np.uint16) if y_in is None else np.array(y_in, dtype=np.uint16).reshape(rows, n).copy()
    acc = np.empty((rows, n), dtype=np.float32) if want_acc else None
    lib().orc_int8_gemm_rows(_p(np.ascontiguousarray(w, dtype=np.int8)),
                             _p(np.ascontiguousarray(scales, dtype=np.float32)),
                             _p(x), _p(y), _p(acc), C.c_int(k), C.c_int(n), C.c_int(rows),
                             C.c_int(mode))
    return (y, acc) if want_acc else y


def int8_gate_up_silu_rows(w, scales, x, want_acc=False):
    n2, k = w.shape
    n = n2 // 2
    x = np.ascontiguousarray(x, dtype=np.uint16).reshape(-1, k)
    rows = x.shape[0]
    y = np.zeros((rows, n), dtype=np.uint16)
    acc = np.empty((rows, n), dtype=np.float32) if want_acc else None
    lib().orc_int8_gate_up_silu_rows(_p(np.ascontiguousarray(w, dtype=np.int8)),
                                     _p(np.ascontiguousarray(scales, dtype=np.float32)),
                                     _p(x), _p(y), _p(acc), C.c_int(k), C.c_int(n), C.c_int(rows))
    return (y, acc) if want_acc else y


def int8_gemm_rows_f64(w, scales, x):
    n, k = w.shape
    x = np.ascontiguousarray(x, dtype=np.uint16).reshape(-1, k)
    out = np.empty((x.shape[0], n), dtype=np.float64)
    lib().orc_int8_gemm_rows_f64(_p(np.ascontiguousarray(w, dtype=np.int8)),
                                 _p(np.ascontiguousarray(scales, dtype=np.float32)),
                                 _p(x), _p(out), C.c_int(k), C.c_int(n), C.c_int(x.shape[0]))
    return out


def quantize_rows(weight_bf16):
    n, k = weight_bf16.shape
    q = np.empty((n, k), dtype=np.int8)
    s = np.empty((n,), dtype=np.float32)
    lib().orc_quantize_rows(_p(np.ascontiguousarray(weight_bf16, dtype=np.uint16)), _p(q), _p(s),
                            C.c_int(k), C.c_int(n))
    return q, s


def rms_norm_rows(x, w, eps=RMS_EPS):
    x = np.ascontiguousarray(x, dtype=np.uint16)
    width = x.shape[-1]
    rows = x.size // width
    y = np.empty_like(x)
    lib().orc_rms_norm_rows(_p(x), _p(np.ascontiguousarray(w, dtype=np.uint16)), _p(y),
                            C.c_int(rows), C.c_int(width), C.c_float(eps))
    return y


def head_rms_norm(v, w, head_dim, eps=RMS_EPS):
    v = np.array(v, dtype=np.uint16, copy=True)
    lib().orc_head_rms_norm(_p(v), _p(np.ascontiguousarray(w, dtype=np.uint16)),
                            C.c_int(v.size // head_dim), C.c_int(head_dim), C.c_float(eps))
    return v


def rope_rows_at(v, rows, heads, head_dim, positions, theta=ROPE_THETA):
    v = np.array(v, dtype=np.uint16, copy=True)
    pos = np.ascontiguousarray(positions, dtype=np.int32)
    lib().orc_rope_rows_at(_p(v), C.c_int(rows), C.c_int(heads), C.c_int(head_dim), _p(pos),
                           C.c_float(theta))
    return v


def attention(q, k, v, positions, q_heads, kv_heads, head_dim, fast=True, want_f32=False):
    """k, v: [rows][capacity][kv_heads*head_dim] bf16; positions[r] = last valid index."""
    q = np.ascontiguousarray(q, dtype=np.uint16)
    k = np.ascontiguousarray(k, dtype=np.uint16)
    v = np.ascontiguousarray(v, dtype=np.uint16)
    rows = k.shape[0]
    stride = k.size // rows
    pos = np.ascontiguousarray(positions, dtype=np.int32)
    out = np.empty((rows, q_heads * head_dim), dtype=np.uint16)
    if fast:
        f32 = np.empty((rows, q_heads * head_dim), dtype=np.float32) if want_f32 else None
        lib().orc_attention_fast(_p(q), _p(k), _p(v), _p(pos), _p(out), _p(f32), C.c_int(rows),
                                 C.c_int(q_heads), C.c_int(kv_heads), C.c_int(head_dim),
                                 C.c_long(stride))
        return (out, f32) if want_f32 else out
    lib().orc_attention_exact(_p(q), _p(k), _p(v), _p(pos), _p(out), C.c_int(rows),
                              C.c_int(q_heads), C.c_int(kv_heads), C.c_int(head_dim),
                              C.c_long(stride))
    return out


def bias_activation_rows(v, bias, silu):
    v = np.array(v, dtype=np.uint16, copy=True)
    width = bias.size
    lib().orc_bias_activation_rows(_p(v), _p(np.ascontiguousarray(bias, dtype=np.uint16)),
                                   C.c_int(v.size // width), C.c_int(width), C.c_int(int(silu)))
    return v


def silu_gate(gate, up):
    g = np.array(gate, dtype=np.uint16, copy=True)
    lib().orc_silu_gate(_p(g), _p(np.ascontiguousarray(up, dtype=np.uint16)), C.c_int(g.size))
    return g


def add(a, b):
    d = np.array(a, dtype=np.uint16, copy=True)
    lib().orc_add_in_place(_p(d), _p(np.ascontiguousarray(b, dtype=np.uint16)), C.c_long(d.size))
    return d


def seed_state(seed: int) -> int:
    """reset(): seed 0 is replaced by the golden-ratio constant (talker.cu:1022)."""
    return seed if seed != 0 else 0x9E3779B97F4A7C15


def sample(logits, rng_state: int, *, suppress=False, history=None, do_sample=1, top_k=50,
           top_p=1.0, temperature=0.9, penalty=1.0, eos=EOS):
    """Returns (token, new_rng_state)."""
    logits = np.ascontiguousarray(logits, dtype=np.uint16)
    hist = np.ascontiguousarray(history if history is not None else [], dtype=np.int32)
    st = C.c_uint64(rng_state)
    tok = lib().orc_sample(_p(logits), C.c_int(logits.size), C.c_int(int(suppress)), C.c_int(eos),
                           _p(hist) if hist.size else None, C.c_int(hist.size),
                           C.c_int(do_sample), C.c_int(top_k), C.c_float(top_p),
                           C.c_float(temperature), C.c_float(penalty), C.byref(st))
    return int(tok), int(st.value)


def embedding(table, token, out=None):
    width = table.shape[1]
    add_mode = out is not None
    o = np.zeros((width,), dtype=np.uint16) if out is None else np.array(out, dtype=np.uint16, copy=True)
    lib().orc_embedding(_p(np.ascontiguousarray(table, dtype=np.uint16)), C.c_int(table.shape[0]),
                        C.c_int(width), C.c_int(int(token)), _p(o), C.c_int(int(add_mode)))
    return o


# ------------------------------------------------------------------ reference kernels (GPU box)

_ref = None


def ref_available() -> bool:
    return os.path.exists(_REF_PATH)


def ref() -> C.CDLL:
    """The reference project's own kernels compiled for sm_100a (oracle/_ref)."""
    global _ref
    if _ref is None:
        _ref = C.CDLL(_REF_PATH)
        _ref.ref_time_int8_gemm.restype = C.c_float
    return _ref


def ref_int8_gemm(w, scales, x, y_in=None, mode=0):
    wr, k = w.shape
    n = wr // 2 if mode == 2 else wr
    x = np.ascontiguousarray(x, dtype=np.uint16).reshape(-1, k)
    rows = x.shape[0]
    y = np.zeros((rows, n), dtype=np.uint16) if y_in is None else np.array(y_in, dtype=np.uint16).reshape(rows, n).copy()
    rc = ref().ref_int8_gemm(_p(np.ascontiguousarray(w, dtype=np.int8)),
                             _p(np.ascontiguousarray(scales, dtype=np.float32)), _p(x), _p(y),
                             C.c_int(k), C.c_int(n), C.c_int(rows), C.c_int(mode))
    assert rc == 0, f"reference launch failed: cudaError {rc}"
    return y


def ref_quantize_rows(weight_bf16):
    n, k = weight_bf16.shape
    q = np.empty((n, k), dtype=np.int8)
    s = np.empty((n,), dtype=np.float32)
    rc = ref().ref_quantize_rows(_p(np.ascontiguousarray(weight_bf16, dtype=np.uint16)), _p(q),
                                 _p(s), C.c_int(k), C.c_int(n))
    assert rc == 0
    return q, s


def ref_rms_norm_rows(x, w, eps=RMS_EPS):
    x = np.ascontiguousarray(x, dtype=np.uint16)
    width = x.shape[-1]
    y = np.empty_like(x)
    rc = ref().ref_rms_norm_rows(_p(x), _p(np.ascontiguousarray(w, dtype=np.uint16)), _p(y),
                                 C.c_int(x.size // width), C.c_int(width), C.c_float(eps))
    assert rc == 0
    return y


def ref_head_rms_norm_rows(v, w, rows, heads, head_dim, eps=RMS_EPS):
    v = np.array(v, dtype=np.uint16, copy=True)
    rc = ref().ref_head_rms_norm_rows(_p(v), _p(np.ascontiguousarray(w, dtype=np.uint16)),
                                      C.c_int(rows), C.c_int(heads), C.c_int(head_dim),
                                      C.c_float(eps))
    assert rc == 0
    return v


def ref_rope_rows_at(v, rows, heads, head_dim, positions, theta=ROPE_THETA):
    v = np.array(v, dtype=np.uint16, copy=True)
    pos = np.ascontiguousarray(positions, dtype=np.int32)
    rc = ref().ref_rope_rows_at(_p(v), C.c_int(rows), C.c_int(heads), C.c_int(head_dim), _p(pos),
                                C.c_float(theta))
    assert rc == 0
    return v


def ref_attention(q, k, v, positions, q_heads, kv_heads, head_dim, fast=True):
    q = np.ascontiguousarray(q, dtype=np.uint16)
    k = np.ascontiguousarray(k, dtype=np.uint16)
    v = np.ascontiguousarray(v, dtype=np.uint16)
    rows, capacity = k.shape[0], k.shape[1]
    pos = np.ascontiguousarray(positions, dtype=np.int32)
    out = np.empty((rows, q_heads * head_dim), dtype=np.uint16)
    rc = ref().ref_attention(_p(q), _p(k), _p(v), _p(pos), _p(out), C.c_int(rows),
                             C.c_int(q_heads), C.c_int(kv_heads), C.c_int(head_dim),
                             C.c_int(capacity), C.c_int(int(fast)))
    assert rc == 0
    return out


def ref_sample(logits, rng_state: int, *, suppress=False, history=None, do_sample=1, top_k=50,
               top_p=1.0, temperature=0.9, penalty=1.0, eos=EOS):
    logits = np.ascontiguousarray(logits, dtype=np.uint16)
    hist = np.ascontiguousarray(history if history is not None else [], dtype=np.int32)
    st = C.c_uint64(rng_state)
    tok = C.c_int(-1)
    rc = ref().ref_sample(_p(logits), C.c_int(logits.size), C.c_int(int(suppress)), C.c_int(eos),
                          _p(hist) if hist.size else None, C.c_int(hist.size), C.c_int(do_sample),
                          C.c_int(top_k), C.c_float(top_p), C.c_float(temperature),
                          C.c_float(penalty), C.byref(st), C.byref(tok))
    assert rc == 0
    return int(tok.value), int(st.value)


def ref_time_int8_gemm(k, n, rows=1, mode=0, buffers=16, iterations=2000) -> float:
    """Mean microseconds per launch of the reference GEMV on this GPU."""
    return float(ref().ref_time_int8_gemm(C.c_int(k), C.c_int(n), C.c_int(rows), C.c_int(mode),
                                          C.c_int(buffers), C.c_int(iterations)))


# ------------------------------------------------------------------ frame composition

TALKER_DIMS = dict(hidden=2048, inter=6144, q_heads=16, kv_heads=8, head_dim=128, layers=28)


def predictor_dims(head_dim=128):
    return dict(hidden=1024, inter=3072, q_heads=16, kv_heads=8, head_dim=head_dim, layers=5)


class OracleModel:
    """int8 image of a checkpoint built the way the reference's finalize does
    (talker.cu:569-667): every decode matrix quantized per row, q/k/v stacked, gate/up stacked."""

    def __init__(self, tensors, predictor_head_dim=128):
        t = dict(tensors)
        self.t = t
        self.pd = predictor_dims(predictor_head_dim)
        self.q = {}

        def quant(name):
            self.q[name] = quantize_rows(t[name])

        def layers(prefix, count):
            out = []
            for l in range(count):
                p = f"{prefix}.{l}"
                qs = [quantize_rows(t[p + f".self_attn.{n}_proj.weight"]) for n in ("q", "k", "v")]
                gu = [quantize_rows(t[p + f".mlp.{n}_proj.weight"]) for n in ("gate", "up")]
                out.append(dict(
                    input_norm=t[p + ".input_layernorm.weight"],
                    qkv=(np.concatenate([a for a, _ in qs]), np.concatenate([s for _, s in qs])),
                    o=quantize_rows(t[p + ".self_attn.o_proj.weight"]),
                    q_norm=t[p + ".self_attn.q_norm.weight"], k_norm=t[p + ".self_attn.k_norm.weight"],
                    post_norm=t[p + ".post_attention_layernorm.weight"],
                    gate_up=(np.concatenate([a for a, _ in gu]), np.concatenate([s for _, s in gu])),
                    down=quantize_rows(t[p + ".mlp.down_proj.weight"])))
            return out

        self.talker_layers = layers("talker.model.layers", 28)
        self.predictor_layers = layers("talker.code_predictor.model.layers", 5)
        for name in ("talker.text_projection.linear_fc1.weight", "talker.text_projection.linear_fc2.weight",
                     "talker.codec_head.weight", "talker.code_predictor.small_to_mtp_projection.weight"):
            quant(name)
        self.heads = [quantize_rows(t[f"talker.code_predictor.lm_head.{g}.weight"]) for g in range(15)]
        self.pred_emb = [t[f"talker.code_predictor.model.codec_embedding.{g}.weight"] for g in range(15)]


import sys as _sys

_THIS = _sys.modules[__name__]


def decoder_layer(h, lw, dims, kcache, vcache, pos, b=None):
    """One layer of the fused int8 batch path (talker.cu:2054-2333) for a single row.
    kcache/vcache: [capacity][kv_width] and are appended in place.  `b` is the module or object
    that supplies the primitives (this module by default; the GPU tests pass an adapter over
    the operator-level C ABI to run the same composition on the kernels under test)."""
    b = b or _THIS
    qh, kvh, hd = dims["q_heads"], dims["kv_heads"], dims["head_dim"]
    qw, kvw = qh * hd, kvh * hd
    n = b.rms_norm_rows(h[None, :], lw["input_norm"])
    qkv = b.int8_gemm_rows(lw["qkv"][0], lw["qkv"][1], n)[0]
    q, k, v = qkv[:qw], qkv[qw:qw + kvw], qkv[qw + kvw:]
    q = b.rope_rows_at(b.head_rms_norm(q, lw["q_norm"], hd), 1, qh, hd, [pos])
    k = b.rope_rows_at(b.head_rms_norm(k, lw["k_norm"], hd), 1, kvh, hd, [pos])
    kcache[pos] = k.reshape(-1)
    vcache[pos] = v
    a = b.attention(q, kcache[None, :pos + 1], vcache[None, :pos + 1], [pos], qh, kvh, hd, fast=True)
    h = b.int8_gemm_rows(lw["o"][0], lw["o"][1], a, y_in=h[None, :], mode=1)
    n = b.rms_norm_rows(h, lw["post_norm"])
    g = b.int8_gate_up_silu_rows(lw["gate_up"][0], lw["gate_up"][1], n)
    h = b.int8_gemm_rows(lw["down"][0], lw["down"][1], g, y_in=h, mode=1)
    return h[0]


class OracleSession:
    """Single-session restatement of prefill + frame generation with the fused int8 semantics
    (frame algorithm: talker.cu:1495-1881; prompt embedding: talker.cu:2676-2748)."""

    def __init__(self, model: OracleModel, max_seq: int, seed: int, backend=None):
        self.m = model
        self.b = backend or _THIS   # supplier of the primitives (see decoder_layer)
        self.max_seq = max_seq
        kvw = 1024
        self.k = np.zeros((28, max_seq, kvw), dtype=np.uint16)
        self.v = np.zeros((28, max_seq, kvw), dtype=np.uint16)
        pkvw = model.pd["kv_heads"] * model.pd["head_dim"]
        self.pk = np.zeros((5, 16, pkvw), dtype=np.uint16)
        self.pv = np.zeros((5, 16, pkvw), dtype=np.uint16)
        self.rng = seed_state(seed)
        self.history = []
        self.position = 0
        self.current = 0
        self.last_hidden = np.zeros(2048, dtype=np.uint16)
        self.trace = {}

    def _project_text(self, token):
        t = self.m.t
        x = t["talker.model.text_embedding.weight"][token]
        w1, s1 = self.m.q["talker.text_projection.linear_fc1.weight"]
        w2, s2 = self.m.q["talker.text_projection.linear_fc2.weight"]
        p = self.b.bias_activation_rows(self.b.int8_gemm_rows(w1, s1, x), t["talker.text_projection.linear_fc1.bias"], True)
        return self.b.bias_activation_rows(self.b.int8_gemm_rows(w2, s2, p), t["talker.text_projection.linear_fc2.bias"], False)[0]

    def _talker_layers(self, h, pos):
        for l, lw in enumerate(self.m.talker_layers):
            h = decoder_layer(h, lw, TALKER_DIMS, self.k[l], self.v[l], pos, self.b)
        return h

    def _talker_head(self, h, cfg):
        t = self.m.t
        n = self.b.rms_norm_rows(h[None, :], t["talker.model.norm.weight"])[0]
        self.last_hidden = n.copy()
        w, s = self.m.q["talker.codec_head.weight"]
        logits = self.b.int8_gemm_rows(w, s, n)[0]
        self.trace["talker_logits"] = logits
        if getattr(self, "mask_eos", False):
            # harness option for random weights: EOS is masked like a reserved token
            logits = logits.copy()
            logits[EOS] = 0xFF80   # -inf
        tok, self.rng = self.b.sample(logits, self.rng, suppress=True, history=self.history, **cfg)
        self.history.append(tok)
        return tok

    def prefill(self, text_ids, codec_ids, cfg):
        t = self.m.t
        self.position = 0
        self.history = []
        h = None
        for i, (ti, ci) in enumerate(zip(text_ids, codec_ids)):
            h = self._project_text(ti) if ti >= 0 else np.zeros(2048, dtype=np.uint16)
            if ci >= 0:
                h = self.b.add(h, t["talker.model.codec_embedding.weight"][ci])
            h = self._talker_layers(h, i)
        self.position = len(text_ids)
        self.current = self._talker_head(h, cfg)
        return self.current

    def _predictor_position(self, x, pos, head):
        t = self.m.t
        w, s = self.m.q["talker.code_predictor.small_to_mtp_projection.weight"]
        h = self.b.bias_activation_rows(self.b.int8_gemm_rows(w, s, x), t["talker.code_predictor.small_to_mtp_projection.bias"], False)[0]
        for l, lw in enumerate(self.m.predictor_layers):
            h = decoder_layer(h, lw, self.m.pd, self.pk[l], self.pv[l], pos, self.b)
        if head < 0:
            return None
        n = self.b.rms_norm_rows(h[None, :], t["talker.code_predictor.model.norm.weight"])
        return self.b.int8_gemm_rows(self.m.heads[head][0], self.m.heads[head][1], n)[0]

    def frame(self, trailing_text, talker_cfg, predictor_cfg):
        """Returns (codes[16], next_semantic_token)."""
        t = self.m.t
        tok = [self.current]
        self._predictor_position(self.last_hidden, 0, -1)
        x = t["talker.model.codec_embedding.weight"][tok[0]]
        self.trace["predictor_logits"] = []
        for p in range(1, 16):
            logits = self._predictor_position(x, p, p - 1)
            self.trace["predictor_logits"].append(logits)
            nt, self.rng = self.b.sample(logits, self.rng, suppress=False, **predictor_cfg)
            tok.append(nt)
            if p < 15:
                x = self.m.pred_emb[p - 1][nt]
        h = t["talker.model.codec_embedding.weight"][tok[0]].copy()
        for r in range(15):
            h = self.b.add(h, self.m.pred_emb[r][tok[r + 1]])
        h = self.b.add(h, self._project_text(trailing_text))
        self.trace["talker_input"] = h
        h = self._talker_layers(h, self.position)
        self.trace["talker_hidden"] = h
        self.position += 1
        self.current = self._talker_head(h, talker_cfg)
        return tok, self.current
