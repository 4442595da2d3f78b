"""Seeded synthetic inputs for the joint-attention benchmark configurations.

No dataset stands behind these: the configurations name shapes and distributions only (Q/K/V ~ N(0,1) as
bf16, QK-norm scale ~ U(0.5,1.5), text lengths ~ U{77..512}).  The normal generator restates the
reference's own seeded noise source (engine/src/pipeline.mm:108-122: a splitmix64 counter stream fed to
Box-Muller in double precision) in counter-based form, so any rank can produce any slice of a tensor
without communication; bf16 rounding is round-to-nearest-even (engine/src/model.mm:17-24).
"""
import os
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass

import numpy as np

_GOLD = np.uint64(0x9E3779B97F4A7C15)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)

HEAD_DIM = 128


def _mix(z: np.ndarray) -> np.ndarray:
    z = (z ^ (z >> np.uint64(30))) * _M1
    z = (z ^ (z >> np.uint64(27))) * _M2
    return z ^ (z >> np.uint64(31))


def _normal_pairs(seed: int, even: np.ndarray):
    """Box-Muller pairs driven by counters (even, even+1): the cos and the sin branch as float64."""
    with np.errstate(over="ignore"):
        base = np.uint64(seed) * _GOLD
        a = _mix(base + even)
        b = _mix(base + even + np.uint64(1))
    u1 = ((a >> np.uint64(11)).astype(np.float64) + 1.0) / 9007199254740993.0
    u2 = (b >> np.uint64(11)).astype(np.float64) / 9007199254740992.0
    r = np.sqrt(-2.0 * np.log(u1))
    t = 2.0 * np.pi * u2
    return r * np.cos(t), r * np.sin(t)


def normal_f32(seed: int, first: int, n: int) -> np.ndarray:
    """Elements [first, first+n) of stream `seed` as float32.  Elements (2i, 2i+1) are the cos and sin
    branch of one Box-Muller pair driven by counters 2i and 2i+1."""
    lo = first & ~1
    hi = (first + n + 1) & ~1
    c, sn = _normal_pairs(seed, np.arange(lo, hi, 2, dtype=np.uint64))
    out = np.empty(hi - lo, dtype=np.float32)
    out[0::2] = c
    out[1::2] = sn
    return out[first - lo:first - lo + n]


def normal_f32_rows(seed: int, first: int, row_stride: int, nrows: int, width: int) -> np.ndarray:
    """float32 [nrows, width]: row r holds elements [first + r*row_stride, +width) of the stream
    (first, row_stride and width even, so no Box-Muller pair straddles a row)."""
    assert first % 2 == 0 and row_stride % 2 == 0 and width % 2 == 0
    even = (np.uint64(first) + np.arange(nrows, dtype=np.uint64)[:, None] * np.uint64(row_stride)
            + np.arange(0, width, 2, dtype=np.uint64)[None, :])
    c, sn = _normal_pairs(seed, even)
    out = np.empty((nrows, width), dtype=np.float32)
    out[:, 0::2] = c
    out[:, 1::2] = sn
    return out


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    u = (u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)
    return u.astype(np.uint16)


def bf16_bits_to_f32(u: np.ndarray) -> np.ndarray:
    return (u.astype(np.uint32) << np.uint32(16)).view(np.float32)


def normal_bf16(seed: int, first: int, n: int, chunk: int = 1 << 20) -> np.ndarray:
    out = np.empty(n, dtype=np.uint16)

    def work(s):
        m = min(chunk, n - s)
        out[s:s + m] = f32_to_bf16_bits(normal_f32(seed, first + s, m))

    starts = range(0, n, chunk)
    if n > chunk:
        with ThreadPoolExecutor(max_workers=min(16, os.cpu_count() or 1)) as ex:
            list(ex.map(work, starts))
    else:
        for s in starts:
            work(s)
    return out


def uniform_f32(seed: int, first: int, lo: float, hi: float, n: int) -> np.ndarray:
    with np.errstate(over="ignore"):
        a = _mix(np.uint64(seed) * _GOLD + np.arange(first, first + n, dtype=np.uint64))
    return (lo + (hi - lo) * ((a >> np.uint64(11)).astype(np.float64) / 9007199254740992.0)).astype(np.float32)


def rope_tables_axial2d(T: int, gh: int, gw: int, theta: float = 10000.0):
    """f32 cos/sin [T + gh*gw, 64]: pairs 0-31 turn with the grid row, 32-63 with the grid column,
    frequency k = theta^(-2k/64); text rows sit at position 0.  Same table mechanism as the reference's
    DiT::set_grid (engine/src/model.mm:290-315), different axis split."""
    om = 1.0 / np.power(theta, 2.0 * np.arange(32, dtype=np.float64) / 64.0)
    R = T + gh * gw
    k = np.arange(R) - T
    pi = np.where(k < 0, 0, k // gw).astype(np.float64)
    pj = np.where(k < 0, 0, k % gw).astype(np.float64)
    ang = np.concatenate([pi[:, None] * om[None, :], pj[:, None] * om[None, :]], axis=1)
    return np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)


def rope_tables_ref3axis(T: int, gh: int, gw: int):
    """The reference model's own tables (engine/src/model.mm:290-315): pairs 0-15 frame (always 0),
    16-39 grid row, 40-63 grid column, theta 1000 over 32/48/48 dims."""
    om = np.empty(64)
    for p in range(64):
        ax = 0 if p < 16 else 1 if p < 40 else 2
        kk = p - (0 if ax == 0 else 16 if ax == 1 else 40)
        d = 32 if ax == 0 else 48
        om[p] = 1.0 / np.power(1000.0, (2.0 * kk) / d)
    R = T + gh * gw
    k = np.arange(R) - T
    pi = np.where(k < 0, 0, k // gw).astype(np.float64)
    pj = np.where(k < 0, 0, k % gw).astype(np.float64)
    pos = np.zeros((R, 64))
    pos[:, 16:40] = pi[:, None]
    pos[:, 40:] = pj[:, None]
    ang = pos * om[None, :]
    return np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)


@dataclass(frozen=True)
class Config:
    """One benchmark configuration (shapes only)."""
    cid: int
    name: str
    batch: int
    heads: int
    text: int
    grid: int          # image tokens = grid * grid
    masked: bool = False

    @property
    def seq(self) -> int:
        return self.text + self.grid * self.grid

    @property
    def seed(self) -> int:
        return 1234 + self.cid


CONFIGS = {
    0: Config(0, "c0-512sq", 1, 24, 512, 32),
    1: Config(1, "c1-1024sq", 1, 24, 512, 64),
    2: Config(2, "c2-1024sq-b4-textmask", 4, 24, 512, 64, masked=True),
    3: Config(3, "c3-2048sq", 1, 24, 512, 128),
    4: Config(4, "c4-4096sq-seqpar", 1, 24, 512, 256),
}


def text_lengths(cfg: Config) -> np.ndarray:
    """Valid text rows per sample, uniform on [77, 512]."""
    with np.errstate(over="ignore"):
        a = _mix(np.uint64(cfg.seed) * _GOLD + np.uint64(5 << 40) + np.arange(cfg.batch, dtype=np.uint64))
    return (77 + (a % np.uint64(436))).astype(np.int32)


def qk_weights(cfg: Config):
    """QK-norm scales, f32 [128] each, shared by all heads like the reference's L{l}.qn / L{l}.kn."""
    return (uniform_f32(cfg.seed, 3 << 40, 0.5, 1.5, HEAD_DIM), uniform_f32(cfg.seed, 4 << 40, 0.5, 1.5, HEAD_DIM))


def qkv_slice(cfg: Config, head0: int = 0, nheads: int = None, row0: int = 0, nrows: int = None,
              b0: int = 0, nb: int = None) -> np.ndarray:
    """bf16 bits of the fused q|k|v rows restricted to heads [head0, head0+nheads) and rows
    [row0, row0+nrows): uint16 [nb, nrows, 3*nheads*128].  Element (tensor t, sample b, row s, head h,
    channel d) is counter ((t*B + b)*S + s)*H*128 + h*128 + d of the config's stream, whatever the slice."""
    H, S, B = cfg.heads, cfg.seq, cfg.batch
    nheads = H - head0 if nheads is None else nheads
    nrows = S - row0 if nrows is None else nrows
    nb = B - b0 if nb is None else nb
    out = np.empty((nb, nrows, 3, nheads * HEAD_DIM), dtype=np.uint16)
    width = nheads * HEAD_DIM
    for t in range(3):
        for b in range(nb):
            if nheads == H:
                first = ((t * B + b0 + b) * S + row0) * H * HEAD_DIM
                out[b, :, t, :] = normal_bf16(cfg.seed, first, nrows * width).reshape(nrows, width)
            else:
                for s0 in range(0, nrows, 8192):
                    m = min(8192, nrows - s0)
                    first = ((t * B + b0 + b) * S + row0 + s0) * H * HEAD_DIM + head0 * HEAD_DIM
                    out[b, s0:s0 + m, t, :] = f32_to_bf16_bits(normal_f32_rows(cfg.seed, first, H * HEAD_DIM, m, width))
    return out.reshape(nb, nrows, 3 * width)


def attention_flops(cfg: Config, text_len=None) -> float:
    """Algorithmic FLOPs 4*D*H*sum_b Lq_b*Lk_b (QK^T and PV, 2 per multiply-add); valid rows only."""
    if text_len is None:
        return 4.0 * HEAD_DIM * cfg.heads * cfg.batch * float(cfg.seq) ** 2
    img = cfg.grid * cfg.grid
    return 4.0 * HEAD_DIM * cfg.heads * float(sum((int(t) + img) ** 2 for t in text_len))
