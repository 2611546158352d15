"""ctypes/NumPy front end of the CPU oracle (oracle/ingot_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
CPU-baseline leg of the benchmark.  The product package never imports it.

Each wrapper names the reference code its C function restates; see the C
file for file:line citations.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libingot_oracle.so")
_REF_PATH = os.path.join(_HERE, "_ref", "libref_decode.so")


def build(force: bool = False) -> str:
    """Compile the oracle (and, when the reference tree is mounted, the
    reference's own scalar decoders) with the Makefile beside this file."""
    src = os.path.join(_HERE, "ingot_oracle.c")
    stale = (not os.path.exists(_LIB_PATH)) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src)
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "libingot_oracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return _LIB_PATH


_u8p = C.POINTER(C.c_uint8)
_f32p = C.POINTER(C.c_float)
_f64p = C.POINTER(C.c_double)
_u32p = C.POINTER(C.c_uint32)


def _load():
    build()
    lib = C.CDLL(_LIB_PATH)
    lib.oracle_half_to_float.restype = C.c_float
    lib.oracle_half_to_float.argtypes = [C.c_uint16]
    lib.oracle_float_to_half.restype = C.c_uint16
    lib.oracle_float_to_half.argtypes = [C.c_float]
    lib.oracle_float_to_bf16.restype = C.c_uint16
    lib.oracle_float_to_bf16.argtypes = [C.c_float]
    lib.oracle_geometry.restype = C.c_int
    lib.oracle_geometry.argtypes = [C.c_uint32, _u32p, _u32p]
    lib.oracle_weight_at.restype = C.c_float
    lib.oracle_weight_at.argtypes = [_u8p, C.c_uint32, C.c_uint32]
    lib.oracle_dequant_rows.restype = C.c_int
    lib.oracle_dequant_rows.argtypes = [_u8p, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint32, _f32p]
    mv = [_u8p, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint32, C.c_uint64, _f32p, C.c_uint64]
    lib.oracle_matvec_f64.restype = C.c_int
    lib.oracle_matvec_f64.argtypes = mv + [_f64p]
    lib.oracle_gemm_f16_f64.restype = C.c_int
    lib.oracle_gemm_f16_f64.argtypes = mv + [_f64p]
    lib.oracle_matvec_f32_mt.restype = C.c_int
    lib.oracle_matvec_f32_mt.argtypes = mv + [_f32p, C.c_uint32]
    lib.oracle_glu.restype = C.c_float
    lib.oracle_glu.argtypes = [C.c_float, C.c_float, C.c_int]
    lib.oracle_route.restype = C.c_int
    lib.oracle_route.argtypes = [_f32p, C.c_uint32, C.c_uint32, _u32p, _f32p]
    lib.oracle_moe_sum.restype = None
    lib.oracle_moe_sum.argtypes = [_f32p, _f32p, C.c_uint64, C.c_uint32, C.c_uint64, _f32p]
    lib.oracle_combine.restype = None
    lib.oracle_combine.argtypes = [_f32p, _f32p, _f32p, C.c_float, C.c_uint64, C.c_uint32, _f32p]
    lib.oracle_expert_layout.restype = C.c_int
    lib.oracle_expert_layout.argtypes = [_u32p, C.c_uint32, C.c_uint32, C.c_uint32, _u32p, _u32p,
                                         _u32p, _u32p]
    lib.oracle_combine_packed.restype = None
    lib.oracle_combine_packed.argtypes = [_f32p, _f32p, _f32p, _f32p, _u32p, C.c_uint64,
                                          C.c_uint32, C.c_uint64, _f32p]
    lib.oracle_add_rms.restype = None
    lib.oracle_add_rms.argtypes = [_f32p, _f32p, _f32p, C.c_uint64, C.c_float, C.c_int, _f32p,
                                   _f32p]
    lib.oracle_embedding.restype = C.c_int
    lib.oracle_embedding.argtypes = [_u8p, _u32p, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint32, C.c_uint64, _f32p]
    lib.oracle_qk_rope_cache.restype = None
    lib.oracle_qk_rope_cache.argtypes = [_f32p] * 9 + [C.c_uint32] * 5 + [C.c_float, C.c_int, C.c_int, C.c_int, C.c_float, C.c_int,
                                                                            C.c_float, C.c_uint32]
    lib.oracle_attention_decode.restype = None
    lib.oracle_attention_decode.argtypes = [_f32p] * 4 + [C.c_uint32] * 6
    lib.oracle_greedy.restype = None
    lib.oracle_greedy.argtypes = [_f32p, _u32p, C.c_uint64, C.c_uint64, _u32p]
    return lib


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = _load()
    return _lib


def _p(a: np.ndarray, t):
    return a.ctypes.data_as(t)


def _bytes(data) -> np.ndarray:
    a = np.ascontiguousarray(np.frombuffer(data, dtype=np.uint8) if not isinstance(data, np.ndarray)
                             else data.view(np.uint8).reshape(-1))
    return a


def _f32(x) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(x, dtype=np.float32))


def geometry(kind: int) -> tuple[int, int]:
    """(block elements, block bytes) for a GGML type id."""
    b, s = C.c_uint32(), C.c_uint32()
    if lib().oracle_geometry(kind, C.byref(b), C.byref(s)):
        raise ValueError(f"GGML type {kind} is unsupported")
    return b.value, s.value


def stride_of(kind: int, cols: int) -> int:
    block, size = geometry(kind)
    if cols % block:
        raise ValueError("cols is not a whole number of blocks")
    return cols // block * size


def dequant(data, cols: int, rows: int, kind: int) -> np.ndarray:
    """All rows (stacked experts included) as float32 [rows, cols] (read_rows)."""
    raw = _bytes(data)
    stride = stride_of(kind, cols)
    if raw.size != stride * rows:
        raise ValueError("invalid quantized matrix layout")
    out = np.empty((rows, cols), dtype=np.float32)
    if lib().oracle_dequant_rows(_p(raw, _u8p), cols, rows, stride, kind, _p(out, _f32p)):
        raise ValueError("invalid quantized matrix layout")
    return out


def matvec_f64(data, cols: int, rows: int, kind: int, x, expert: int = 0) -> np.ndarray:
    """float64 [count, rows]: f64 dot of the exactly dequantised weights."""
    raw, xv = _bytes(data), _f32(x).reshape(-1, cols)
    y = np.empty((xv.shape[0], rows), dtype=np.float64)
    rc = lib().oracle_matvec_f64(_p(raw, _u8p), cols, rows, stride_of(kind, cols), kind, expert,
                                 _p(xv, _f32p), xv.shape[0], _p(y, _f64p))
    if rc:
        raise ValueError("oracle_matvec_f64 failed")
    return y


def gemm_f16_f64(data, cols: int, rows: int, kind: int, x, expert: int = 0) -> np.ndarray:
    """float64 [count, rows] with weights and activations rounded to f16 first."""
    raw, xv = _bytes(data), _f32(x).reshape(-1, cols)
    y = np.empty((xv.shape[0], rows), dtype=np.float64)
    rc = lib().oracle_gemm_f16_f64(_p(raw, _u8p), cols, rows, stride_of(kind, cols), kind, expert,
                                   _p(xv, _f32p), xv.shape[0], _p(y, _f64p))
    if rc:
        raise ValueError("oracle_gemm_f16_f64 failed")
    return y


def matvec_f32(data, cols: int, rows: int, kind: int, x, expert: int = 0,
               threads: int = 1) -> np.ndarray:
    """float32 [count, rows]: scalar dequantise + fp32 dot, rows over threads."""
    raw, xv = _bytes(data), _f32(x).reshape(-1, cols)
    y = np.empty((xv.shape[0], rows), dtype=np.float32)
    rc = lib().oracle_matvec_f32_mt(_p(raw, _u8p), cols, rows, stride_of(kind, cols), kind, expert,
                                    _p(xv, _f32p), xv.shape[0], _p(y, _f32p), threads)
    if rc:
        raise ValueError("oracle_matvec_f32_mt failed")
    return y


def glu(gate, up, gelu: bool = False) -> np.ndarray:
    g, u = _f32(gate).reshape(-1), _f32(up).reshape(-1)
    f = lib().oracle_glu
    return np.array([f(float(a), float(b), int(gelu)) for a, b in zip(g, u)],
                    dtype=np.float32).reshape(np.shape(gate))


def route(logits, top: int) -> tuple[np.ndarray, np.ndarray]:
    """(ids uint32 [top], weights float32 [top]) for one token."""
    l = _f32(logits).reshape(-1)
    ids = np.empty(max(top, 1), dtype=np.uint32)
    w = np.empty(max(top, 1), dtype=np.float32)
    if lib().oracle_route(_p(l, _f32p), l.size, top, _p(ids, _u32p), _p(w, _f32p)):
        raise ValueError("invalid router scores or expert count")
    return ids[:top], w[:top]


def moe_sum(routed, weights, width: int, top: int) -> np.ndarray:
    r, w = _f32(routed).reshape(-1, width), _f32(weights).reshape(-1)
    tokens = r.shape[0] // top
    y = np.empty((tokens, width), dtype=np.float32)
    lib().oracle_moe_sum(_p(r, _f32p), _p(w, _f32p), width, top, tokens, _p(y, _f32p))
    return y


def combine(routed, shared, weights, shared_logit: float, width: int) -> np.ndarray:
    r, s, w = _f32(routed).reshape(-1, width), _f32(shared).reshape(-1), _f32(weights).reshape(-1)
    out = np.empty(width, dtype=np.float32)
    lib().oracle_combine(_p(r, _f32p), _p(s, _f32p), _p(w, _f32p), float(shared_logit), width,
                         w.size, _p(out, _f32p))
    return out


def expert_layout(ids, experts: int, tile_capacity: int):
    """(layout [experts,2], tiles [capacity,4], pairs [n], inverse [n], n_tiles)."""
    i = np.ascontiguousarray(np.asarray(ids, dtype=np.uint32).reshape(-1))
    layout = np.zeros((experts, 2), dtype=np.uint32)
    tiles = np.zeros((tile_capacity, 4), dtype=np.uint32)
    pairs = np.zeros(max(i.size, 1), dtype=np.uint32)
    inverse = np.zeros(max(i.size, 1), dtype=np.uint32)
    n = lib().oracle_expert_layout(_p(i, _u32p), i.size, experts, tile_capacity, _p(layout, _u32p),
                                   _p(tiles, _u32p), _p(pairs, _u32p), _p(inverse, _u32p))
    if n < 0:
        raise ValueError("expert id out of range or tile capacity exceeded")
    return layout, tiles, pairs[:i.size], inverse[:i.size], n


def combine_packed(routed, weights, inverse, width: int, top: int) -> np.ndarray:
    r, w = _f32(routed).reshape(-1, width), _f32(weights).reshape(-1)
    inv = np.ascontiguousarray(np.asarray(inverse, dtype=np.uint32).reshape(-1))
    tokens = inv.size // top
    out = np.empty((tokens, width), dtype=np.float32)
    lib().oracle_combine_packed(_p(r, _f32p), None, _p(w, _f32p), None, _p(inv, _u32p), width, top,
                                tokens, _p(out, _f32p))
    return out


def add_rms(a, b, w, eps: float, add: bool = True):
    """(s, y) per row: s = a + b, y = s * rsqrt(mean(s^2) + eps) * w."""
    av = _f32(a)
    width = av.shape[-1]
    a2 = av.reshape(-1, width)
    b2 = _f32(b).reshape(-1, width) if add else a2
    wv = None if w is None else _f32(w).reshape(-1)
    s = np.empty_like(a2)
    y = np.empty_like(a2)
    for r in range(a2.shape[0]):
        ar, br = np.ascontiguousarray(a2[r]), np.ascontiguousarray(b2[r])
        sr, yr = np.empty(width, np.float32), np.empty(width, np.float32)
        lib().oracle_add_rms(_p(ar, _f32p), _p(br, _f32p), None if wv is None else _p(wv, _f32p),
                             width, float(eps), int(add), _p(sr, _f32p), _p(yr, _f32p))
        s[r], y[r] = sr, yr
    return s.reshape(av.shape), y.reshape(av.shape)


def to_bf16_bits(x) -> np.ndarray:
    """float32 -> bf16 bit patterns (uint16), round to nearest even."""
    u = _f32(x).view(np.uint32).astype(np.uint64)
    r = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return r.astype(np.uint16).reshape(np.shape(x))


def from_bf16_bits(b) -> np.ndarray:
    return (np.asarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def to_f16_rounded(x) -> np.ndarray:
    return _f32(x).astype(np.float16).astype(np.float32)


# ---- the reference's own scalar decoders, compiled from its shader text ----

def ref_available() -> bool:
    return os.path.exists(_REF_PATH)


_ref = None


def ref_lib():
    """oracle/_ref/libref_decode.so (built by oracle/build_ref.sh where the
    reference tree is mounted); None when it has not been built."""
    global _ref
    if _ref is None and ref_available():
        _ref = C.CDLL(_REF_PATH)
        _ref.ref_weight_at.restype = C.c_float
        _ref.ref_weight_at.argtypes = [_u8p, C.c_uint32, C.c_uint32]
        _ref.ref_dequant_row.restype = None
        _ref.ref_dequant_row.argtypes = [_u8p, C.c_uint32, C.c_uint32, _f32p]
        _ref.ref_kquant_scale_min.restype = None
        _ref.ref_kquant_scale_min.argtypes = [_u8p, C.c_uint32, _u32p]
    return _ref


def ref_dequant(data, cols: int, rows: int, kind: int) -> np.ndarray:
    """Dequantise with the reference's weight_at itself."""
    r = ref_lib()
    if r is None:
        raise RuntimeError("oracle/_ref/libref_decode.so has not been built")
    raw = _bytes(data)
    stride = stride_of(kind, cols)
    out = np.empty((rows, cols), dtype=np.float32)
    for i in range(rows):
        row = np.ascontiguousarray(raw[i * stride:(i + 1) * stride])
        o = np.empty(cols, np.float32)
        r.ref_dequant_row(_p(row, _u8p), kind, cols, _p(o, _f32p))
        out[i] = o
    return out


# ---- the rest of a generic decode step ----

def embedding(data, ids, width: int, rows: int, kind: int) -> np.ndarray:
    raw = _bytes(data)
    i = np.ascontiguousarray(np.asarray(ids, dtype=np.uint32).reshape(-1))
    y = np.empty((i.size, width), dtype=np.float32)
    if lib().oracle_embedding(_p(raw, _u8p), _p(i, _u32p), width, rows, stride_of(kind, width), kind, i.size, _p(y, _f32p)):
        raise ValueError("token outside vocabulary")
    return y


def qk_rope_cache(q, k, v, kc, vc, *, head_dim, heads, kv_heads, rotated, position, base, tokens, neox=False, factors=None,
                  q_norm=None, k_norm=None, eps=1e-6, value_norm=False, q_scale=1.0):
    """Returns q_out [tokens, heads, D]; kc and vc (float32 [rows, kv_heads, D]) are updated in place."""
    qf, kf, vf = _f32(q).reshape(-1), _f32(k).reshape(-1), _f32(v).reshape(-1)
    qo = np.empty(tokens * heads * head_dim, np.float32)
    ptr = lambda a: None if a is None else _p(_f32(a).reshape(-1), _f32p)
    lib().oracle_qk_rope_cache(_p(qf, _f32p), _p(kf, _f32p), _p(vf, _f32p), ptr(q_norm), ptr(k_norm), ptr(factors), _p(qo, _f32p),
                               _p(kc, _f32p), _p(vc, _f32p), head_dim, heads, kv_heads, rotated, position, base, int(neox),
                               int(factors is not None), int(q_norm is not None), eps, int(value_norm), q_scale,
                               tokens)
    return qo.reshape(tokens, heads, head_dim)


def attention_decode(q, kc, vc, head_dim, heads, kv_heads, position, tokens, window=0) -> np.ndarray:
    qf = _f32(q).reshape(-1)
    out = np.empty(tokens * heads * head_dim, np.float32)
    lib().oracle_attention_decode(_p(qf, _f32p), _p(kc, _f32p), _p(vc, _f32p), _p(out, _f32p), head_dim, heads, kv_heads, position,
                                  window, tokens)
    return out.reshape(tokens, heads, head_dim)


def greedy(logits, vocab: int, mapping=None) -> np.ndarray:
    """uint32 [rows, 2]: (token, non-finite flag)."""
    l = _f32(logits).reshape(-1, vocab)
    m = None if mapping is None else np.ascontiguousarray(np.asarray(mapping, dtype=np.uint32))
    out = np.empty((l.shape[0], 2), np.uint32)
    lib().oracle_greedy(_p(l, _f32p), None if m is None else _p(m, _u32p), l.shape[0], vocab, _p(out, _u32p))
    return out


# ---- architecture glue of the generic path (kernels/generic_arch.metal:2-17), restated in numpy ----

def scale_rows(x, scale: float) -> np.ndarray:
    """y = x * scale in float32 (:2-3)."""
    return _f32(x) * np.float32(scale)


def softcap_rows(x, cap: float) -> np.ndarray:
    """y = c * tanh(x / c) (:4-5), evaluated in float64 and rounded once."""
    c = np.float64(np.float32(cap))
    return (c * np.tanh(_f32(x).astype(np.float64) / c)).astype(np.float32)


def swiglu_fused(x, tokens: int, ff: int) -> np.ndarray:
    """y[t][j] = silu(x[t][j]) * x[t][ff + j] over fused gate|up rows of width 2 ff (:11-15), in float64, rounded once."""
    rows = _f32(x).reshape(tokens, 2 * ff).astype(np.float64)
    g, u = rows[:, :ff], rows[:, ff:]
    return (g / (1.0 + np.exp(-g)) * u).astype(np.float32)


def copy_columns(x, rows: int, width: int, offset: int, stride: int) -> np.ndarray:
    """Columns [offset, offset + width) of rows of `stride` floats (:16-17)."""
    return np.ascontiguousarray(_f32(x).reshape(-1)[: rows * stride].reshape(rows, stride)[:, offset:offset + width])

