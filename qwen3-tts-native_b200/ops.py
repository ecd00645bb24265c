"""numpy-in / numpy-out drivers of the operator-level C ABI (include/q3t_ops.h).

torch is used only to hold device memory: every function stages its numpy arguments in
CUDA tensors, passes the raw device pointers through the C ABI and brings the result back.
bf16 tensors are uint16 bit patterns.  Used by the GPU parity tests and the benchmark.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import numpy as np
import torch

from . import native

EPI_PLAIN, EPI_ADD, EPI_BIAS, EPI_BIAS_SILU, EPI_BIAS_ADD, EPI_GATE_UP_SILU = range(6)


class GemmDescC(C.Structure):     # include/q3t_ops.h Q3tGemmDesc
    _fields_ = [("struct_size", C.c_uint32), ("epilogue", C.c_int32), ("weight", C.c_void_p),
                ("scales", C.c_void_p), ("input", C.c_void_p), ("output", C.c_void_p),
                ("output_f32", C.c_void_p), ("norm_weight", C.c_void_p),
                ("norm_output", C.c_void_p), ("bias", C.c_void_p), ("residual", C.c_void_p),
                ("in_features", C.c_int32), ("out_features", C.c_int32), ("rows", C.c_int32),
                ("epsilon", C.c_float)]


class AttentionDescC(C.Structure):   # include/q3t_ops.h Q3tAttentionDesc
    _fields_ = [("struct_size", C.c_uint32), ("fused", C.c_int32), ("query", C.c_void_p),
                ("key_new", C.c_void_p), ("value_new", C.c_void_p),
                ("query_norm_weight", C.c_void_p), ("key_norm_weight", C.c_void_p),
                ("positions", C.c_void_p), ("output", C.c_void_p), ("output_f32", C.c_void_p),
                ("key_bases", C.c_void_p), ("value_bases", C.c_void_p), ("page_table", C.c_void_p),
                ("slabs", C.c_void_p), ("page_elements", C.c_int64), ("key_offset", C.c_int64),
                ("value_offset", C.c_int64), ("page_table_stride", C.c_int32),
                ("slab_shift", C.c_int32), ("query_stride", C.c_int32), ("new_stride", C.c_int32),
                ("rows", C.c_int32), ("query_heads", C.c_int32), ("key_value_heads", C.c_int32),
                ("head_dimension", C.c_int32), ("max_sequence_length", C.c_int32),
                ("epsilon", C.c_float), ("theta", C.c_float), ("scratch", C.c_void_p),
                ("scratch_bytes", C.c_size_t)]


def _dev(a: Optional[np.ndarray], device="cuda") -> Optional[torch.Tensor]:
    if a is None:
        return None
    a = np.ascontiguousarray(a)
    if a.dtype == np.uint16:
        return torch.from_numpy(a.view(np.int16)).to(device)
    if a.dtype == np.uint64:
        return torch.from_numpy(a.view(np.int64)).to(device)
    return torch.from_numpy(a).to(device)


def _ptr(t: Optional[torch.Tensor]):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def _u16(t: torch.Tensor) -> np.ndarray:
    return t.cpu().numpy().view(np.uint16)


def _ok(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} returned cudaError {rc}")
    torch.cuda.synchronize()


def int8_gemm(w, scales, x, *, epilogue=EPI_PLAIN, y_in=None, norm_w=None, bias=None, resid=None,
              want_f32=False, want_norm=False, eps=1.0e-6):
    """Returns dict(y=..., f32=..., norm=..., resid=...) for one fused GEMV/GEMM launch."""
    lib = native.library()
    wr, k = w.shape
    n = wr // 2 if epilogue == EPI_GATE_UP_SILU else wr
    x = np.ascontiguousarray(x, dtype=np.uint16).reshape(-1, k)
    rows = x.shape[0]
    dw, ds, dx = _dev(np.asarray(w, dtype=np.int8)), _dev(np.asarray(scales, dtype=np.float32)), _dev(x)
    y0 = np.zeros((rows, n), dtype=np.uint16) if y_in is None else np.asarray(y_in, dtype=np.uint16).reshape(rows, n)
    dy = _dev(y0)
    d32 = torch.zeros((rows, n), dtype=torch.float32, device="cuda") if want_f32 else None
    dn = _dev(np.asarray(norm_w, dtype=np.uint16)) if norm_w is not None else None
    dno = torch.zeros((rows, k), dtype=torch.int16, device="cuda") if want_norm else None
    db = _dev(np.asarray(bias, dtype=np.uint16)) if bias is not None else None
    dr = _dev(np.asarray(resid, dtype=np.uint16).reshape(rows, n)) if resid is not None else None
    d = GemmDescC()
    d.struct_size = C.sizeof(GemmDescC)
    d.epilogue = epilogue
    d.weight, d.scales, d.input, d.output = dw.data_ptr(), ds.data_ptr(), dx.data_ptr(), dy.data_ptr()
    d.output_f32 = d32.data_ptr() if d32 is not None else None
    d.norm_weight = dn.data_ptr() if dn is not None else None
    d.norm_output = dno.data_ptr() if dno is not None else None
    d.bias = db.data_ptr() if db is not None else None
    d.residual = dr.data_ptr() if dr is not None else None
    d.in_features, d.out_features, d.rows, d.epsilon = k, n, rows, eps
    _ok(lib.q3t_launch_int8_gemm_ex(C.byref(d), None), "q3t_launch_int8_gemm_ex")
    return dict(y=_u16(dy), f32=d32.cpu().numpy() if d32 is not None else None,
                norm=_u16(dno) if dno is not None else None,
                resid=_u16(dr) if dr is not None else None)


_weight_cache = {}


def _dev_cached(a: np.ndarray) -> torch.Tensor:
    """Device copy of a host array that is kept for the life of the process (weights that a
    test drives through many launches); keyed by the host buffer's address and shape."""
    key = (a.ctypes.data, a.shape, a.dtype.str)
    hit = _weight_cache.get(key)
    if hit is None:
        hit = (_dev(a), a)       # keep the host array alive so the address is not reused
        _weight_cache[key] = hit
    return hit[0]


def int8_gemm_rows(w, scales, x, y_in=None, mode=0, cache_weights=False):
    """The three reference-shaped entry points: mode 0 plain, 1 add, 2 gate/up/SiLU."""
    lib = native.library()
    wr, k = w.shape
    n = wr // 2 if mode == 2 else wr
    x = np.ascontiguousarray(x, dtype=np.uint16).reshape(-1, k)
    rows = x.shape[0]
    if cache_weights and w.dtype == np.int8 and w.flags["C_CONTIGUOUS"]:
        dw, ds = _dev_cached(w), _dev_cached(np.ascontiguousarray(scales, dtype=np.float32))
    else:
        dw, ds = _dev(np.asarray(w, dtype=np.int8)), _dev(np.asarray(scales, dtype=np.float32))
    dx = _dev(x)
    y0 = np.zeros((rows, n), dtype=np.uint16) if y_in is None else np.asarray(y_in, dtype=np.uint16).reshape(rows, n)
    dy = _dev(y0)
    fn = (lib.q3t_launch_int8_gemm_rows, lib.q3t_launch_int8_gemm_rows_add,
          lib.q3t_launch_int8_gate_up_silu_rows)[mode]
    _ok(fn(_ptr(dw), _ptr(ds), _ptr(dx), _ptr(dy), k, n, rows, None), "q3t_launch_int8_gemm_rows*")
    return _u16(dy)


def quantize_rows(weight_bf16):
    n, k = weight_bf16.shape
    dw = _dev(np.asarray(weight_bf16, dtype=np.uint16))
    dq = torch.zeros((n, k), dtype=torch.int8, device="cuda")
    ds = torch.zeros((n,), dtype=torch.float32, device="cuda")
    _ok(native.library().q3t_launch_quantize_weight_rows(_ptr(dw), _ptr(dq), _ptr(ds), k, n, None),
        "q3t_launch_quantize_weight_rows")
    return dq.cpu().numpy(), ds.cpu().numpy()


def rms_norm_rows(x, w, eps=1.0e-6):
    x = np.ascontiguousarray(x, dtype=np.uint16)
    width = x.shape[-1]
    dx, dw = _dev(x), _dev(np.asarray(w, dtype=np.uint16))
    dy = torch.zeros_like(dx)
    _ok(native.library().q3t_launch_rms_norm_rows(_ptr(dx), _ptr(dw), _ptr(dy), x.size // width,
                                                  width, C.c_float(eps), None), "rms_norm_rows")
    return _u16(dy).reshape(x.shape)


def head_rms_norm_rows(v, w, rows, heads, head_dim, eps=1.0e-6):
    dv, dw = _dev(np.asarray(v, dtype=np.uint16)), _dev(np.asarray(w, dtype=np.uint16))
    _ok(native.library().q3t_launch_head_rms_norm_rows(_ptr(dv), _ptr(dw), rows, heads, head_dim,
                                                       C.c_float(eps), None), "head_rms_norm_rows")
    return _u16(dv)


def rope_rows_at(v, rows, heads, head_dim, positions, theta=1.0e6):
    dv = _dev(np.asarray(v, dtype=np.uint16))
    dp = _dev(np.asarray(positions, dtype=np.int32))
    _ok(native.library().q3t_launch_rope_rows_at(_ptr(dv), rows, heads, head_dim, _ptr(dp),
                                                 C.c_float(theta), None), "rope_rows_at")
    return _u16(dv)


def bias_activation_rows(v, bias, silu):
    v = np.ascontiguousarray(v, dtype=np.uint16)
    width = np.asarray(bias).size
    dv, db = _dev(v), _dev(np.asarray(bias, dtype=np.uint16))
    _ok(native.library().q3t_launch_bias_activation_rows(_ptr(dv), _ptr(db), v.size // width, width,
                                                         int(silu), None), "bias_activation_rows")
    return _u16(dv).reshape(v.shape)


def add_in_place(a, b):
    da, db = _dev(np.asarray(a, dtype=np.uint16)), _dev(np.asarray(b, dtype=np.uint16))
    _ok(native.library().q3t_launch_add_in_place(_ptr(da), _ptr(db), da.numel(), None), "add_in_place")
    return _u16(da)


def silu_gate(gate, up):
    dg, du = _dev(np.asarray(gate, dtype=np.uint16)), _dev(np.asarray(up, dtype=np.uint16))
    _ok(native.library().q3t_launch_silu_gate(_ptr(dg), _ptr(du), dg.numel(), None), "silu_gate")
    return _u16(dg)


def kv_scatter_rows(rows_data, caches, positions):
    """caches: [rows][capacity][width]; returns the updated caches."""
    rows_data = np.ascontiguousarray(rows_data, dtype=np.uint16)
    caches = np.ascontiguousarray(caches, dtype=np.uint16)
    rows, width = rows_data.shape
    dc, dr = _dev(caches), _dev(rows_data)
    stride = dc[0].numel() * 2
    bases = torch.tensor([dc.data_ptr() + r * stride for r in range(rows)], dtype=torch.int64,
                         device="cuda")
    dp = _dev(np.asarray(positions, dtype=np.int32))
    _ok(native.library().q3t_launch_kv_scatter_rows(_ptr(dr), _ptr(bases), _ptr(dp), rows, width,
                                                    None), "kv_scatter_rows")
    return _u16(dc)


def gather_embedding_rows(table, tokens, token_offset, out=None):
    """tokens: [rows][m] int32 (one token array per row); out given -> add, else gather."""
    table = np.ascontiguousarray(table, dtype=np.uint16)
    tokens = np.ascontiguousarray(tokens, dtype=np.int32)
    rows = tokens.shape[0]
    width = table.shape[1]
    dt, dk = _dev(table), _dev(tokens)
    ptrs = torch.tensor([dk.data_ptr() + r * tokens.shape[1] * 4 for r in range(rows)],
                        dtype=torch.int64, device="cuda")
    do = _dev(np.zeros((rows, width), dtype=np.uint16) if out is None else np.asarray(out, dtype=np.uint16))
    fn = native.library().q3t_launch_gather_embedding_rows if out is None \
        else native.library().q3t_launch_add_embedding_rows
    _ok(fn(_ptr(dt), table.shape[0], width, _ptr(ptrs), token_offset, _ptr(do), rows, None),
        "gather/add_embedding_rows")
    return _u16(do)


def attention_contiguous(q, k, v, positions, q_heads, kv_heads, head_dim):
    """The reference-shaped entry point; k, v: [rows][capacity][kv_heads*head_dim]."""
    lib = native.library()
    k = np.ascontiguousarray(k, dtype=np.uint16)
    v = np.ascontiguousarray(v, dtype=np.uint16)
    rows, capacity = k.shape[0], k.shape[1]
    dq, dk, dv = _dev(np.asarray(q, dtype=np.uint16)), _dev(k), _dev(v)
    stride = dk[0].numel() * 2
    kb = torch.tensor([dk.data_ptr() + r * stride for r in range(rows)], dtype=torch.int64, device="cuda")
    vb = torch.tensor([dv.data_ptr() + r * stride for r in range(rows)], dtype=torch.int64, device="cuda")
    dp = _dev(np.asarray(positions, dtype=np.int32))
    do = torch.zeros((rows, q_heads * head_dim), dtype=torch.int16, device="cuda")
    nbytes = int(lib.q3t_attention_scratch_bytes(rows, q_heads, kv_heads, head_dim, capacity))
    scratch = torch.empty((max(nbytes, 16),), dtype=torch.uint8, device="cuda")
    _ok(lib.q3t_launch_batch_causal_gqa_attention_fast(
        _ptr(dq), _ptr(kb), _ptr(vb), _ptr(dp), _ptr(do), rows, q_heads, kv_heads, head_dim,
        capacity, _ptr(scratch), C.c_size_t(nbytes), None), "batch_causal_gqa_attention_fast")
    return _u16(do)


def attention_contiguous_noalloc(q, k, v, positions, q_heads, kv_heads, head_dim):
    """The entry point for hosts that may not allocate: same arguments as
    attention_contiguous minus the scratch buffer, which the library keeps in a built-in array.
    Returns (status, message, output)."""
    lib = native.library()
    k = np.ascontiguousarray(k, dtype=np.uint16)
    v = np.ascontiguousarray(v, dtype=np.uint16)
    rows, capacity = k.shape[0], k.shape[1]
    dq, dk, dv = _dev(np.asarray(q, dtype=np.uint16)), _dev(k), _dev(v)
    stride = dk[0].numel() * 2
    kb = torch.tensor([dk.data_ptr() + r * stride for r in range(rows)], dtype=torch.int64, device="cuda")
    vb = torch.tensor([dv.data_ptr() + r * stride for r in range(rows)], dtype=torch.int64, device="cuda")
    dp = _dev(np.asarray(positions, dtype=np.int32))
    do = torch.zeros((rows, q_heads * head_dim), dtype=torch.int16, device="cuda")
    err = C.create_string_buffer(256)
    torch.cuda.synchronize()
    status = lib.q3t_launch_batch_causal_gqa_attention_fast_noalloc(
        _ptr(dq), _ptr(kb), _ptr(vb), _ptr(dp), _ptr(do), rows, q_heads, kv_heads, head_dim, capacity,
        None, err, C.c_size_t(256))
    torch.cuda.synchronize()
    return int(status), err.value.decode(), _u16(do)


def attention_ex(q, positions, q_heads, kv_heads, head_dim, *, k=None, v=None, pages=None,
                 page_table=None, slab_shift=0, k_new=None, v_new=None, q_norm_w=None,
                 k_norm_w=None, fused=False, q_stride=0, new_stride=0, max_seq=None,
                 want_f32=False, theta=1.0e6, eps=1.0e-6):
    """Full-form attention.  Contiguous: k, v [rows][capacity][kvw].  Paged: `pages` is a list
    of slabs, each [2][pages_per_slab][kv_heads][16][head_dim] (K plane then V plane; a page is
    head-major: the 16 tokens of one KV head are contiguous), page_table
    [rows][stride].  Returns dict(out, f32, k, v | pages) with caches after the append."""
    lib = native.library()
    rows = np.asarray(positions).size
    kvw = kv_heads * head_dim
    d = AttentionDescC()
    d.struct_size = C.sizeof(AttentionDescC)
    d.fused = int(fused)
    keep = []
    dq = _dev(np.asarray(q, dtype=np.uint16)); keep.append(dq)
    d.query = dq.data_ptr()
    if fused:
        dqn, dkw = _dev(np.asarray(q_norm_w, dtype=np.uint16)), _dev(np.asarray(k_norm_w, dtype=np.uint16))
        keep += [dqn, dkw]
        d.query_norm_weight, d.key_norm_weight = dqn.data_ptr(), dkw.data_ptr()
        if k_new is None:
            # q is the packed [rows][q | k | v] projection output; k and v start inside it
            d.key_new = dq.data_ptr() + 2 * q_heads * head_dim
            d.value_new = dq.data_ptr() + 2 * (q_heads * head_dim + kvw)
        else:
            dkn, dvn = _dev(np.asarray(k_new, dtype=np.uint16)), _dev(np.asarray(v_new, dtype=np.uint16))
            keep += [dkn, dvn]
            d.key_new, d.value_new = dkn.data_ptr(), dvn.data_ptr()
    dp = _dev(np.asarray(positions, dtype=np.int32)); keep.append(dp)
    d.positions = dp.data_ptr()
    do = torch.zeros((rows, q_heads * head_dim), dtype=torch.int16, device="cuda")
    d.output = do.data_ptr()
    d32 = torch.zeros((rows, q_heads * head_dim), dtype=torch.float32, device="cuda") if want_f32 else None
    d.output_f32 = d32.data_ptr() if d32 is not None else None
    dk = dv = None
    dslabs = []
    if pages is None:
        dk, dv = _dev(np.asarray(k, dtype=np.uint16)), _dev(np.asarray(v, dtype=np.uint16))
        capacity = dk.shape[1]
        stride = dk[0].numel() * 2
        kb = torch.tensor([dk.data_ptr() + r * stride for r in range(rows)], dtype=torch.int64, device="cuda")
        vb = torch.tensor([dv.data_ptr() + r * stride for r in range(rows)], dtype=torch.int64, device="cuda")
        keep += [kb, vb]
        d.key_bases, d.value_bases = kb.data_ptr(), vb.data_ptr()
        max_seq = max_seq or capacity
    else:
        dslabs = [_dev(np.asarray(s, dtype=np.uint16)) for s in pages]
        per = dslabs[0].shape[1]
        slab_ptrs = torch.tensor([s.data_ptr() for s in dslabs], dtype=torch.int64, device="cuda")
        dpt = _dev(np.asarray(page_table, dtype=np.int32))
        keep += [slab_ptrs, dpt]
        d.page_table, d.slabs = dpt.data_ptr(), slab_ptrs.data_ptr()
        d.page_table_stride = np.asarray(page_table).shape[1]
        d.slab_shift = slab_shift
        d.page_elements = 16 * kvw
        d.key_offset, d.value_offset = 0, per * 16 * kvw
        max_seq = max_seq or d.page_table_stride * 16
    d.query_stride, d.new_stride = q_stride, new_stride
    d.rows, d.query_heads, d.key_value_heads, d.head_dimension = rows, q_heads, kv_heads, head_dim
    d.max_sequence_length = max_seq
    d.epsilon, d.theta = eps, theta
    nbytes = int(lib.q3t_attention_scratch_bytes(rows, q_heads, kv_heads, head_dim, max_seq))
    scratch = torch.empty((max(nbytes, 16),), dtype=torch.uint8, device="cuda")
    d.scratch, d.scratch_bytes = scratch.data_ptr(), nbytes
    _ok(lib.q3t_launch_decode_attention_ex(C.byref(d), None), "q3t_launch_decode_attention_ex")
    return dict(out=_u16(do), f32=d32.cpu().numpy() if d32 is not None else None,
                k=_u16(dk) if dk is not None else None, v=_u16(dv) if dv is not None else None,
                pages=[_u16(s) for s in dslabs])


def sample(logits, rng_state: int, *, suppress=False, history: Optional[Sequence[int]] = None,
           do_sample=1, top_k=50, top_p=1.0, temperature=0.9, penalty=1.0, eos=native.EOS,
           count_on_device=False):
    """One sampler launch; returns (token, new_rng_state)."""
    lib = native.library()
    dl = _dev(np.asarray(logits, dtype=np.uint16))
    hist = np.asarray(history if history is not None else [], dtype=np.int32)
    dh = _dev(hist) if hist.size else None
    dr = _dev(np.array([rng_state], dtype=np.uint64))
    dt = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    if count_on_device:
        dc = _dev(np.array([hist.size], dtype=np.int32))
        rc = lib.q3t_launch_sample_logits_at(_ptr(dl), dl.numel(), int(suppress), eos, _ptr(dh),
                                             _ptr(dc), do_sample, top_k, C.c_float(top_p),
                                             C.c_float(temperature), C.c_float(penalty), _ptr(dr),
                                             _ptr(dt), None)
    else:
        rc = lib.q3t_launch_sample_logits(_ptr(dl), dl.numel(), int(suppress), eos, _ptr(dh),
                                          int(hist.size), do_sample, top_k, C.c_float(top_p),
                                          C.c_float(temperature), C.c_float(penalty), _ptr(dr),
                                          _ptr(dt), None)
    _ok(rc, "q3t_launch_sample_logits")
    return int(dt.item()), int(dr.cpu().numpy().view(np.uint64)[0])
