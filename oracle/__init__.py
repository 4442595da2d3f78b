"""ctypes front end of the CPU oracle (krea_oracle.c).  Test infrastructure, not product code.

PARITY UNPINNED: the reference has no tests, golden vectors or CPU code for this path; see the header of
krea_oracle.c for what the oracle is checked against instead.
"""
import ctypes

import numpy as np

from . import build as _build

_lib = None

_f32p = ctypes.POINTER(ctypes.c_float)
_u16p = ctypes.POINTER(ctypes.c_uint16)
_i32p = ctypes.POINTER(ctypes.c_int32)


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(_build.build())
        _lib.ko_num_threads.restype = ctypes.c_int
    return _lib


def _p(a, ty):
    if a is None:
        return ctypes.cast(None, ty)
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(ty)


def set_num_threads(n: int) -> None:
    """OpenMP threads the oracle may use from now on (a launcher may have exported OMP_NUM_THREADS=1)."""
    lib().ko_set_num_threads(int(n))


def num_threads() -> int:
    return int(lib().ko_num_threads())


def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().ko_f32_to_bf16(_p(x, _f32p), _p(out, _u16p), ctypes.c_int64(x.size))
    return out


def bf16_to_f32(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.uint16)
    out = np.empty(x.shape, dtype=np.float32)
    lib().ko_bf16_to_f32(_p(x, _u16p), _p(out, _f32p), ctypes.c_int64(x.size))
    return out


def gen_normal_bf16(seed: int, first: int, n: int) -> np.ndarray:
    out = np.empty(n, dtype=np.uint16)
    lib().ko_gen_normal_bf16(ctypes.c_uint64(seed), ctypes.c_uint64(first), _p(out, _u16p), ctypes.c_int64(n))
    return out


def gen_normal_f32(seed: int, first: int, n: int) -> np.ndarray:
    out = np.empty(n, dtype=np.float32)
    lib().ko_gen_normal_f32(ctypes.c_uint64(seed), ctypes.c_uint64(first), _p(out, _f32p), ctypes.c_int64(n))
    return out


def gen_uniform_f32(seed: int, first: int, lo: float, hi: float, n: int) -> np.ndarray:
    out = np.empty(n, dtype=np.float32)
    lib().ko_gen_uniform_f32(ctypes.c_uint64(seed), ctypes.c_uint64(first), ctypes.c_float(lo), ctypes.c_float(hi),
                             _p(out, _f32p), ctypes.c_int64(n))
    return out


def rope_tables_ref3axis(T: int, gh: int, gw: int):
    R = T + gh * gw
    c = np.empty((R, 64), dtype=np.float32)
    s = np.empty((R, 64), dtype=np.float32)
    lib().ko_rope_tables_ref3axis(_p(c, _f32p), _p(s, _f32p), T, gh, gw)
    return c, s


def rope_tables_axial2d(T: int, gh: int, gw: int, theta: float = 10000.0):
    R = T + gh * gw
    c = np.empty((R, 64), dtype=np.float32)
    s = np.empty((R, 64), dtype=np.float32)
    lib().ko_rope_tables_axial2d(_p(c, _f32p), _p(s, _f32p), T, gh, gw, ctypes.c_double(theta))
    return c, s


def qk_norm_rope(qkv, wq, wk, cos, sin, rows, ld, q_off, n_q, k_off, n_k, eps, rope_mode=0, big_dim=-1):
    """In place on the uint16 (bf16 bits) array `qkv` [rows, ld].  Returns (qbig, kbig) or (None, None)."""
    assert qkv.dtype == np.uint16
    qbig = kbig = None
    if big_dim >= 0:
        qbig = np.zeros((rows, max(n_q, 1)), dtype=np.float32)
        kbig = np.zeros((rows, max(n_k, 1)), dtype=np.float32)
    lib().ko_qk_norm_rope(_p(qkv, _u16p), _p(wq, _f32p), _p(wk, _f32p), _p(cos, _f32p), _p(sin, _f32p), rows, ld,
                          q_off, n_q, k_off, n_k, ctypes.c_float(eps), rope_mode, big_dim, _p(qbig, _f32p),
                          _p(kbig, _f32p))
    return qbig, kbig


def attention(Q, K, V, Lq, Lk, heads, ldq, ldk, ldv, group=1, causal=False, q_pos0=0, G=None, ldg=0, QB=None,
              KB=None, ref_rounding=False):
    """Q/K/V/G: uint16 arrays whose first element is row 0, head 0.  Returns fp32 [Lq, heads*128]."""
    O = np.zeros((Lq, heads * 128), dtype=np.float32)
    lib().ko_attention(_p(Q, _u16p), _p(K, _u16p), _p(V, _u16p), _p(O, _f32p), Lq, Lk, heads, ldq, ldk, ldv, group,
                       int(causal), q_pos0, _p(G, _u16p), ldg, _p(QB, _f32p), _p(KB, _f32p), int(ref_rounding))
    return O


def joint_attention(qkv, B, S, heads, wq, wk, cos, sin, eps=1e-6, rope_mode=0, text_len=None, text_slots=0,
                    heads_sel=None, ref_rounding=False, group=1):
    """qkv: uint16 [B, S, (heads + 2*heads/group)*128], fused q|k|v rows.  Returns fp32 [B, S, heads*128]."""
    kvh = heads // group
    ld = (heads + 2 * kvh) * 128
    assert qkv.dtype == np.uint16 and qkv.shape == (B, S, ld)
    flat = qkv.reshape(-1)
    O = np.zeros((B, S, heads * 128), dtype=np.float32)
    tl = None if text_len is None else np.ascontiguousarray(text_len, dtype=np.int32)
    hs = None if heads_sel is None else np.ascontiguousarray(heads_sel, dtype=np.int32)
    base = flat.ctypes.data
    q_ptr = ctypes.cast(base, _u16p)
    k_ptr = ctypes.cast(base + 2 * heads * 128, _u16p)
    v_ptr = ctypes.cast(base + 2 * (heads + kvh) * 128, _u16p)
    i64 = ctypes.c_int64
    lib().ko_joint_attention(q_ptr, k_ptr, v_ptr, _p(O, _f32p), B, S, heads, group, i64(ld), i64(ld), i64(ld),
                             i64(S * ld), i64(S * ld), i64(S * ld), _p(wq, _f32p), _p(wk, _f32p), _p(cos, _f32p),
                             _p(sin, _f32p), ctypes.c_float(eps), rope_mode, _p(tl, _i32p), text_slots,
                             _p(hs, _i32p), 0 if hs is None else len(hs), int(ref_rounding))
    return O


def joint_attention_rows(qkv_b, S, heads, h, wq, wk, cos, sin, rows_sel, eps=1e-6, rope_mode=0, text_len=-1,
                         text_slots=0, ref_rounding=False, group=1):
    """Selected query rows of head h of one sample.  qkv_b: uint16 [S, ld] fused rows.  fp32 [n, 128]."""
    kvh_n = heads // group
    ld = (heads + 2 * kvh_n) * 128
    assert qkv_b.dtype == np.uint16 and qkv_b.shape == (S, ld) and qkv_b.flags["C_CONTIGUOUS"]
    rs = np.ascontiguousarray(rows_sel, dtype=np.int32)
    out = np.zeros((len(rs), 128), dtype=np.float32)
    base = qkv_b.ctypes.data
    q_ptr = ctypes.cast(base, _u16p)
    k_ptr = ctypes.cast(base + 2 * heads * 128, _u16p)
    v_ptr = ctypes.cast(base + 2 * (heads + kvh_n) * 128, _u16p)
    i64 = ctypes.c_int64
    lib().ko_joint_attention_rows(q_ptr, k_ptr, v_ptr, _p(out, _f32p), S, h, h // group, i64(ld), i64(ld), i64(ld),
                                  _p(wq, _f32p), _p(wk, _f32p), _p(cos, _f32p), _p(sin, _f32p), ctypes.c_float(eps),
                                  rope_mode, text_len, text_slots, _p(rs, _i32p), len(rs), int(ref_rounding))
    return out


def layerwise_attn(qkvg, rows, ld, heads, q_off, k_off, v_off, g_off, ref_rounding=False):
    """The text fusion's 12-tap attention (norm.metal:136-178).  qkvg: uint16 [rows, ld]; fp32 [rows, heads*128]."""
    assert qkvg.dtype == np.uint16 and qkvg.flags["C_CONTIGUOUS"] and rows % 12 == 0
    out = np.zeros((rows, heads * 128), dtype=np.float32)
    lib().ko_layerwise_attn(_p(qkvg, _u16p), _p(out, _f32p), rows, ld, heads, q_off, k_off, v_off, g_off, int(ref_rounding))
    return out
