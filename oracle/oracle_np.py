"""Independent float64 numpy statement of the same formulas as krea_oracle.c (small shapes only).

Test infrastructure.  Written from the formulas, not from the C file, so that a slip in either shows up
as a disagreement: RMSNorm (norm.metal:102-103), interleaved-pair RoPE (norm.metal:105-113),
softmax(q.k/sqrt(128)) with masked keys removed (attention.metal:237-249,270-271), P V / l with an empty
row giving zeros (attention.metal:316), sigmoid gate (attention.metal:321-329).
"""
import numpy as np


def bf16_bits_to_f64(u16: np.ndarray) -> np.ndarray:
    return (u16.astype(np.uint32) << 16).view(np.float32).astype(np.float64)


def round_bf16(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even to bf16, returned as float64."""
    f = np.asarray(x, dtype=np.float32)
    u = f.view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32).astype(np.float64)


def norm_rope(x, w, cos, sin, eps, rope_mode=0):
    """x [..., S, 128] float64; cos/sin [S, 64]."""
    rrms = 1.0 / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)
    y = x * rrms * w
    if rope_mode == 2:
        return y
    out = np.empty_like(y)
    if rope_mode == 0:
        a, b = y[..., 0::2], y[..., 1::2]
        out[..., 0::2] = a * cos - b * sin
        out[..., 1::2] = a * sin + b * cos
    else:
        a, b = y[..., :64], y[..., 64:]
        out[..., :64] = a * cos - b * sin
        out[..., 64:] = b * cos + a * sin
    return out


def attention_core(q, k, v, key_ok=None, causal=False, q_pos0=0, round_p=False):
    """q [Lq,128], k/v [Lk,128] float64.  key_ok bool [Lk]."""
    s = (q @ k.T) / np.sqrt(128.0)
    ok = np.ones(s.shape, dtype=bool)
    if key_ok is not None:
        ok &= key_ok[None, :]
    if causal:
        ok &= np.arange(k.shape[0])[None, :] <= (np.arange(q.shape[0])[:, None] + q_pos0)
    s = np.where(ok, s, -np.inf)
    m = s.max(axis=1, keepdims=True)
    m = np.where(np.isfinite(m), m, 0.0)
    p = np.exp(s - m)
    l = p.sum(axis=1, keepdims=True)
    pv = round_bf16(p) if round_p else p
    o = pv @ v
    return np.where(l > 0, o / np.where(l > 0, l, 1.0), 0.0)


def joint_attention(qkv_bits, B, S, heads, wq, wk, cos, sin, eps=1e-6, rope_mode=0, text_len=None, text_slots=0,
                    ref_rounding=False):
    """qkv_bits uint16 [B, S, 3*heads*128] (group = 1).  Returns float64 [B, S, heads*128]."""
    x = bf16_bits_to_f64(qkv_bits).reshape(B, S, 3, heads, 128)
    cos = cos.astype(np.float64)
    sin = sin.astype(np.float64)
    out = np.zeros((B, S, heads, 128))
    for b in range(B):
        key_ok = None
        if text_len is not None:
            idx = np.arange(S)
            key_ok = ~((idx >= text_len[b]) & (idx < text_slots))
        for h in range(heads):
            q = norm_rope(x[b, :, 0, h], wq.astype(np.float64), cos, sin, eps, rope_mode)
            k = norm_rope(x[b, :, 1, h], wk.astype(np.float64), cos, sin, eps, rope_mode)
            if ref_rounding:
                q, k = round_bf16(q), round_bf16(k)
            o = attention_core(q, k, x[b, :, 2, h], key_ok, round_p=ref_rounding)
            if key_ok is not None:
                o[~key_ok] = 0.0
            out[b, :, h] = round_bf16(o) if ref_rounding else o
    return out.reshape(B, S, heads * 128)


def layerwise_attn(qkvg_bits, rows, ld, heads, q_off, k_off, v_off, g_off):
    """float64 statement of the 12-tap attention: each row attends over the 12 rows of its token."""
    x = bf16_bits_to_f64(qkvg_bits).reshape(rows // 12, 12, ld)

    def blk(off):
        return x[:, :, off:off + heads * 128].reshape(-1, 12, heads, 128)
    q, k, v, g = blk(q_off), blk(k_off), blk(v_off), blk(g_off)
    s = np.einsum("tihd,tjhd->thij", q, k) / np.sqrt(128.0)
    p = np.exp(s - s.max(axis=-1, keepdims=True))
    p /= p.sum(axis=-1, keepdims=True)
    o = np.einsum("thij,tjhd->tihd", p, v) / (1.0 + np.exp(-g))
    return o.reshape(rows, heads * 128)


def rms_norm(x, mul, add, eps):
    """Metal::rms_norm (norm.metal:28-55): x [rows, width] float64."""
    r = 1.0 / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)
    y = x * r * mul
    return y if add is None else y + add


def dit_block(x, mods, w_qkvg, w_o, w_gu, w_down, qn, kn, cos, sin, heads, kv_heads, ff, eps=1e-6, ref_rounding=False):
    """DiT::layer (model.mm:369-385) in float64.  x [rows, heads*128]; mods [6, dim]; weights [K, N] as float64
    (already widened from bf16).  ref_rounding rounds to bf16 wherever the reference stores bf16: the normalised
    rows, the projection, q and k after the norm, P inside P V, the attention output, the SwiGLU output."""
    R = round_bf16 if ref_rounding else (lambda a: a)
    D = heads * 128
    group = heads // kv_heads
    x = np.array(x, dtype=np.float64)
    h = R(rms_norm(x, mods[0], mods[1], eps))
    y = R(h @ w_qkvg)
    S = x.shape[0]
    q = y[:, :D].reshape(S, heads, 128).transpose(1, 0, 2)
    k = y[:, D:D + kv_heads * 128].reshape(S, kv_heads, 128).transpose(1, 0, 2)
    v = y[:, D + kv_heads * 128:D + 2 * kv_heads * 128].reshape(S, kv_heads, 128).transpose(1, 0, 2)
    g = y[:, D + 2 * kv_heads * 128:].reshape(S, heads, 128).transpose(1, 0, 2)
    q = R(norm_rope(q, qn, cos, sin, eps, 0))
    k = R(norm_rope(k, kn, cos, sin, eps, 0))
    ao = np.empty((S, heads, 128))
    for hh in range(heads):
        o = attention_core(q[hh], k[hh // group], v[hh // group], round_p=ref_rounding)
        ao[:, hh] = o / (1.0 + np.exp(-g[hh]))
    ao = R(ao.reshape(S, D))
    x = x + mods[2] * (ao @ w_o)
    h = R(rms_norm(x, mods[3], mods[4], eps))
    z = (h @ w_gu).reshape(S, 2 * ff // 64, 2, 32)              # groups of 64 columns: 32 gate, then 32 up
    mid = R((z[:, :, 0] / (1.0 + np.exp(-z[:, :, 0])) * z[:, :, 1]).reshape(S, ff))
    return x + mods[5] * (mid @ w_down)
