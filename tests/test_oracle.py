"""CPU tests of the oracle itself: closed-form cases, agreement with the independent float64 numpy
statement, committed golden fixtures, and the seeded input generator.  The reference has no tests for
this path to borrow; these follow the semantics its kernels state (file:line in each test)."""
import os
import zlib

import numpy as np
import pytest

import oracle
from krea_image_b200 import synth
from oracle import oracle_np

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _bits(x):
    return synth.f32_to_bf16_bits(np.asarray(x, dtype=np.float32))


def _rand_case(rng, B, S, H, T, gh, gw):
    qkv = _bits(rng.standard_normal((B, S, 3 * H * 128)))
    wq = rng.uniform(0.5, 1.5, 128).astype(np.float32)
    wk = rng.uniform(0.5, 1.5, 128).astype(np.float32)
    cos, sin = synth.rope_tables_axial2d(T, gh, gw)
    return qkv, wq, wk, cos, sin


def test_bf16_round_matches_reference_rule():
    # engine/src/model.mm:17-24: u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    x = np.array([1.0, 1.00390625, 1.005859375, -2.7182817, 3.1415927, 1e-30, 65504.0], dtype=np.float32)
    u = x.view(np.uint32).astype(np.uint64)
    want = (((u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000) >> 16).astype(np.uint16)
    assert np.array_equal(oracle.f32_to_bf16(x), want)
    assert np.array_equal(synth.f32_to_bf16_bits(x), want)


def test_generator_known_answers_and_slicing():
    kat = np.load(os.path.join(GOLD, "generator_kat.npz"))
    for sd, fi in ((1234, 0), (1235, 7), (1238, 1 << 33)):
        want = kat[f"normal_seed{sd}_first{fi}"]
        assert np.array_equal(oracle.gen_normal_bf16(sd, fi, 16), want)
        assert np.array_equal(synth.normal_bf16(sd, fi, 16), want)
    assert np.array_equal(oracle.gen_uniform_f32(1234, 3 << 40, 0.5, 1.5, 8), kat["uniform_1234"])
    assert np.array_equal(synth.uniform_f32(1234, 3 << 40, 0.5, 1.5, 8), kat["uniform_1234"])
    # counter-based: any slice of a stream equals the same range of a longer draw
    full = synth.normal_bf16(99, 0, 4099)
    assert np.array_equal(synth.normal_bf16(99, 1001, 777), full[1001:1778])
    f = synth.bf16_bits_to_f32(synth.normal_bf16(5, 0, 200000))
    assert abs(f.mean()) < 0.01 and abs(f.std() - 1.0) < 0.01


def test_rope_tables_match_reference_formula():
    # engine/src/model.mm:290-315
    c, s = oracle.rope_tables_ref3axis(5, 3, 4)
    assert np.all(c[:5] == 1.0) and np.all(s[:5] == 0.0)            # text rows at position 0
    assert np.all(c[:, :16] == 1.0) and np.all(s[:, :16] == 0.0)    # frame axis always 0
    r = 5 + 2 * 4 + 3                                               # image token (i=2, j=3)
    assert np.isclose(c[r, 16], np.cos(2.0)) and np.isclose(s[r, 40], np.sin(3.0))
    assert np.isclose(c[r, 17], np.cos(2.0 / 1000.0 ** (2.0 / 48.0)))
    c2, s2 = synth.rope_tables_ref3axis(5, 3, 4)
    assert np.allclose(c, c2, atol=1e-7) and np.allclose(s, s2, atol=1e-7)
    ca, sa = oracle.rope_tables_axial2d(7, 4, 6)
    r = 7 + 3 * 6 + 5
    assert np.isclose(ca[r, 0], np.cos(3.0)) and np.isclose(sa[r, 32], np.sin(5.0))
    assert np.isclose(ca[r, 33], np.cos(5.0 / 10000.0 ** (2.0 / 64.0)))
    cb, sb = synth.rope_tables_axial2d(7, 4, 6)
    assert np.allclose(ca, cb, atol=1e-7) and np.allclose(sa, sb, atol=1e-7)


def test_qk_norm_rope_closed_forms():
    # norm.metal:102-103: x * rsqrt(mean(x^2) + eps) * w; position 0 leaves the vector unrotated
    rows, heads = 3, 2
    x = np.zeros((rows, heads * 128), dtype=np.float32)
    x[:, :128] = 2.0
    x[:, 128:] = np.tile(np.arange(128, dtype=np.float32) - 64, (rows, 1))
    q = _bits(x)
    w = np.full(128, 1.5, dtype=np.float32)
    cos = np.ones((rows, 64), dtype=np.float32)
    sin = np.zeros((rows, 64), dtype=np.float32)
    oracle.qk_norm_rope(q, w, w, cos, sin, rows, heads * 128, 0, heads, 0, 0, 1e-6)
    got = synth.bf16_bits_to_f32(q)
    assert np.allclose(got[:, :128], 1.5, atol=1e-2)               # constant vector -> w
    # a zero row is dominated by eps and stays zero (no NaN)
    z = np.zeros((1, 128), dtype=np.uint16)
    oracle.qk_norm_rope(z, w, w, cos, sin, 1, 128, 0, 1, 0, 0, 1e-6)
    assert np.all(z == 0)
    # a quarter-turn swaps each pair: (a, b) -> (-b, a)   (norm.metal:105-113)
    y = _bits(np.arange(1, 129, dtype=np.float32).reshape(1, 128))
    y0 = synth.bf16_bits_to_f32(y).astype(np.float64)
    oracle.qk_norm_rope(y, np.ones(128, np.float32), np.ones(128, np.float32), np.zeros((1, 64), np.float32),
                        np.ones((1, 64), np.float32), 1, 128, 0, 1, 0, 0, 0.0)
    yn = y0 / np.sqrt((y0 * y0).mean())
    want = np.empty_like(yn)
    want[:, 0::2], want[:, 1::2] = -yn[:, 1::2], yn[:, 0::2]
    assert np.allclose(synth.bf16_bits_to_f32(y), want, rtol=1e-2)


def test_qk_norm_rope_modes_and_big_dim_vs_numpy():
    rng = np.random.default_rng(3)
    rows, n_q, n_k = 9, 3, 2
    ld = (n_q + n_k) * 128 + 64
    base = _bits(rng.standard_normal((rows, ld)))
    wq = rng.uniform(0.5, 1.5, 128).astype(np.float32)
    wk = rng.uniform(0.5, 1.5, 128).astype(np.float32)
    cos, sin = synth.rope_tables_axial2d(2, 1, 7)
    for mode in (0, 1, 2):
        q = base.copy()
        oracle.qk_norm_rope(q, wq, wk, cos, sin, rows, ld, 0, n_q, n_q * 128, n_k, 1e-5, mode)
        x = oracle_np.bf16_bits_to_f64(base)
        for hh in range(n_q + n_k):
            w = wq if hh < n_q else wk
            want = oracle_np.norm_rope(x[:, hh * 128:(hh + 1) * 128], w.astype(np.float64), cos.astype(np.float64),
                                       sin.astype(np.float64), 1e-5, mode)
            got = synth.bf16_bits_to_f32(q[:, hh * 128:(hh + 1) * 128])
            assert np.allclose(got, want, rtol=1e-2, atol=1e-3), (mode, hh)
        assert np.array_equal(q[:, (n_q + n_k) * 128:], base[:, (n_q + n_k) * 128:])   # untouched columns
    # big_dim: value extracted in fp32 and zeroed in the bf16 buffer (norm.metal:127-132)
    q = base.copy()
    plain = base.copy()
    oracle.qk_norm_rope(plain, wq, wk, cos, sin, rows, ld, 0, n_q, n_q * 128, n_k, 1e-5, 0)
    qbig, kbig = oracle.qk_norm_rope(q, wq, wk, cos, sin, rows, ld, 0, n_q, n_q * 128, n_k, 1e-5, 0, big_dim=37)
    assert np.all(q[:, 37::128][:, :n_q + n_k] == 0)
    assert np.allclose(qbig, synth.bf16_bits_to_f32(plain[:, 37:n_q * 128:128]), rtol=1e-2, atol=1e-3)
    assert np.allclose(kbig, synth.bf16_bits_to_f32(plain[:, n_q * 128 + 37:(n_q + n_k) * 128:128]), rtol=1e-2, atol=1e-3)


def test_attention_closed_forms():
    rng = np.random.default_rng(0)
    Lq, Lk, H = 5, 11, 2
    Q = _bits(rng.standard_normal((Lq, H * 128)))
    K = _bits(rng.standard_normal((Lk, H * 128)))
    # uniform V: every output row equals that V row, whatever the scores are
    vrow = rng.standard_normal(H * 128).astype(np.float32)
    V = _bits(np.tile(vrow, (Lk, 1)))
    o = oracle.attention(Q, K, V, Lq, Lk, H, H * 128, H * 128, H * 128)
    assert np.allclose(o, np.tile(synth.bf16_bits_to_f32(_bits(vrow)), (Lq, 1)), atol=1e-5)
    # one dominant key: output = that key's V row
    K2 = np.zeros((Lk, H * 128), dtype=np.float32)
    K2[4] = 40.0
    Q2 = np.full((Lq, H * 128), 1.0, dtype=np.float32)
    V2 = rng.standard_normal((Lk, H * 128)).astype(np.float32)
    o = oracle.attention(_bits(Q2), _bits(K2), _bits(V2), Lq, Lk, H, H * 128, H * 128, H * 128)
    assert np.allclose(o, np.tile(synth.bf16_bits_to_f32(_bits(V2[4])), (Lq, 1)), atol=1e-4)
    # causal with q_pos0 = -1: row 0 sees no key at all -> zeros, not NaN (attention.metal:316)
    o = oracle.attention(Q, K, V, Lq, Lk, H, H * 128, H * 128, H * 128, causal=True, q_pos0=-1)
    assert np.all(o[0] == 0) and np.all(np.isfinite(o))
    # causal row i with q_pos0 = 0 equals non-causal attention over the first i+1 keys (attention.metal:237-249)
    Vr = _bits(rng.standard_normal((Lk, H * 128)))
    oc = oracle.attention(Q, K, Vr, Lq, Lk, H, H * 128, H * 128, H * 128, causal=True)
    for i in range(Lq):
        oi = oracle.attention(Q[i:i + 1].copy(), K[:i + 1].copy(), Vr[:i + 1].copy(), 1, i + 1, H, H * 128, H * 128, H * 128)
        assert np.allclose(oc[i], oi[0], atol=1e-5)


def test_attention_gqa_gate_big_vs_numpy():
    rng = np.random.default_rng(5)
    Lq, Lk, H, group = 7, 19, 4, 2
    kvh = H // group
    Q = _bits(rng.standard_normal((Lq, H * 128)))
    K = _bits(rng.standard_normal((Lk, kvh * 128)))
    V = _bits(rng.standard_normal((Lk, kvh * 128)))
    G = _bits(rng.standard_normal((Lq, H * 128)))
    QB = rng.standard_normal((Lq, H)).astype(np.float32)
    KB = rng.standard_normal((Lk, kvh)).astype(np.float32)
    o = oracle.attention(Q, K, V, Lq, Lk, H, H * 128, kvh * 128, kvh * 128, group=group, G=G, ldg=H * 128, QB=QB, KB=KB)
    q64, k64, v64, g64 = (oracle_np.bf16_bits_to_f64(t) for t in (Q, K, V, G))
    for h in range(H):
        kh = h // group
        s = (q64[:, h * 128:(h + 1) * 128] @ k64[:, kh * 128:(kh + 1) * 128].T + np.outer(QB[:, h], KB[:, kh])) / np.sqrt(128.0)
        p = np.exp(s - s.max(axis=1, keepdims=True))
        want = (p / p.sum(axis=1, keepdims=True)) @ v64[:, kh * 128:(kh + 1) * 128]
        want = want / (1.0 + np.exp(-g64[:, h * 128:(h + 1) * 128]))      # attention.metal:321-329
        assert np.allclose(o[:, h * 128:(h + 1) * 128], want, rtol=2e-5, atol=2e-6)


@pytest.mark.parametrize("ref_rounding", [False, True])
def test_joint_matches_numpy_with_padding_mask(ref_rounding):
    rng = np.random.default_rng(11)
    B, H, T, gh, gw = 2, 3, 22, 6, 8
    S = T + gh * gw
    qkv, wq, wk, cos, sin = _rand_case(rng, B, S, H, T, gh, gw)
    tl = np.array([5, 22], dtype=np.int32)
    got = oracle.joint_attention(qkv, B, S, H, wq, wk, cos, sin, text_len=tl, text_slots=T, ref_rounding=ref_rounding)
    want = oracle_np.joint_attention(qkv, B, S, H, wq, wk, cos, sin, text_len=tl, text_slots=T, ref_rounding=ref_rounding)
    d = got - want
    if ref_rounding:   # a rounding tie may flip one bf16 ulp here and there
        assert np.linalg.norm(d) / np.linalg.norm(want) < 1e-3 and (d != 0).mean() < 0.01
    else:
        assert np.abs(d).max() < 5e-6
    assert np.all(got[0, 5:22] == 0) and np.any(got[0, :5] != 0)    # padded query rows are zero


def test_padding_mask_equals_compaction():
    """Masked attention over 512 text slots == the reference's behaviour of dropping padding rows before
    the engine (ui/krea.py:3-6): run unmasked on the compacted rows and scatter back."""
    rng = np.random.default_rng(12)
    H, T, gh, gw = 2, 16, 4, 5
    S = T + gh * gw
    qkv, wq, wk, cos, sin = _rand_case(rng, 1, S, H, T, gh, gw)
    tl = 6
    masked = oracle.joint_attention(qkv, 1, S, H, wq, wk, cos, sin, text_len=np.array([tl], np.int32), text_slots=T)
    keep = np.r_[0:tl, T:S]
    compact = oracle.joint_attention(np.ascontiguousarray(qkv[:, keep]), 1, len(keep), H, wq, wk,
                                     np.ascontiguousarray(cos[keep]), np.ascontiguousarray(sin[keep]))
    assert np.allclose(masked[0, keep], compact[0], atol=2e-6)
    assert np.all(masked[0, tl:T] == 0)


def test_rows_entry_point_matches_full():
    rng = np.random.default_rng(13)
    H, T, gh, gw = 3, 10, 5, 6
    S = T + gh * gw
    qkv, wq, wk, cos, sin = _rand_case(rng, 1, S, H, T, gh, gw)
    full = oracle.joint_attention(qkv, 1, S, H, wq, wk, cos, sin, text_len=np.array([4], np.int32), text_slots=T)
    rows = np.array([0, 3, 5, 9, 10, 39], dtype=np.int32)
    part = oracle.joint_attention_rows(qkv[0], S, H, 2, wq, wk, cos, sin, rows, text_len=4, text_slots=T)
    assert np.allclose(part, full[0, rows, 256:384], atol=1e-6)


@pytest.mark.parametrize("name", ["c0_rows", "c1_rows", "c2_rows"])
def test_golden_fixture_inputs_and_outputs(name):
    """The committed fixtures still describe what the generator and the oracle produce."""
    g = np.load(os.path.join(GOLD, name + ".npz"))
    cfg = synth.CONFIGS[int(g["cid"])]
    wq, wk = synth.qk_weights(cfg)
    cos, sin = synth.rope_tables_axial2d(cfg.text, cfg.grid, cfg.grid)
    assert zlib.crc32(wq.tobytes()) == int(g["wq_crc"]) and zlib.crc32(wk.tobytes()) == int(g["wk_crc"])
    if cfg.masked:
        assert np.array_equal(synth.text_lengths(cfg), g["text_len"])
    # recompute the first block only (keeps the CPU suite quick)
    b, h, rows = int(g["sample"][0]), int(g["head_of_block"][0]), g["rows"][0]
    qkv_b = synth.qkv_slice(cfg, b0=b, nb=1)[0]
    kw = dict(text_len=int(g["text_len"][b]), text_slots=cfg.text) if cfg.masked else {}
    got = oracle.joint_attention_rows(qkv_b, cfg.seq, cfg.heads, h, wq, wk, cos, sin, rows, **kw)
    assert np.allclose(got, g["fp32"][0], atol=1e-6)
    got = oracle.joint_attention_rows(qkv_b, cfg.seq, cfg.heads, h, wq, wk, cos, sin, rows, ref_rounding=True, **kw)
    assert (got != g["ref"][0]).mean() < 1e-3
    if cfg.batch == 1:
        assert zlib.crc32(qkv_b.tobytes()) == int(g["qkv_crc"])


@pytest.mark.parametrize("name", ["c3_rows", "c4_rows"])
def test_golden_fixture_long_sequences(name):
    """Fixtures of the long-sequence configurations, recomputed from a one-head slice of the inputs."""
    g = np.load(os.path.join(GOLD, name + ".npz"))
    cfg = synth.CONFIGS[int(g["cid"])]
    wq, wk = synth.qk_weights(cfg)
    cos, sin = synth.rope_tables_axial2d(cfg.text, cfg.grid, cfg.grid)
    assert zlib.crc32(wq.tobytes()) == int(g["wq_crc"]) and zlib.crc32(cos.tobytes()) == int(g["cos_crc"])
    h, rows = int(g["head_of_block"][0]), g["rows"][0]
    q1 = synth.qkv_slice(cfg, head0=h, nheads=1)[0]
    assert zlib.crc32(q1.tobytes()) == int(g["head_slice_crc"][0])
    got = oracle.joint_attention_rows(q1, cfg.seq, 1, 0, wq, wk, cos, sin, rows)
    assert np.allclose(got, g["fp32"][0], atol=1e-6)
    assert rows[0] == 0 and rows[-1] == cfg.seq - 1 and cfg.text - 1 in rows and cfg.text in rows


def test_head_slices_equal_columns_of_the_full_tensor():
    cfg = synth.CONFIGS[0]
    full = synth.qkv_slice(cfg).reshape(1, cfg.seq, 3, cfg.heads, 128)
    part = synth.qkv_slice(cfg, head0=3, nheads=2, row0=5, nrows=100)
    assert np.array_equal(full[:, 5:105, :, 3:5].reshape(1, 100, -1), part)


def test_layerwise_attn_vs_numpy_and_closed_form():
    """The text fusion's 12-tap attention (norm.metal:136-178) against the float64 statement, plus a closed
    form: identical taps give uniform weights, so the output is the tap's v row times sigmoid(gate)."""
    rng = np.random.default_rng(5)
    T, H = 7, 3
    rows, ld = T * 12, 4 * H * 128 + 16
    offs = (8, 8 + H * 128, 8 + 2 * H * 128, 16 + 3 * H * 128)
    x = synth.f32_to_bf16_bits(rng.standard_normal((rows, ld)).astype(np.float32))
    a = oracle.layerwise_attn(x, rows, ld, H, *offs)
    b = oracle_np.layerwise_attn(x, rows, ld, H, *offs)
    assert np.abs(a - b).max() < 2e-6
    r = oracle.layerwise_attn(x, rows, ld, H, *offs, ref_rounding=True)
    assert np.array_equal(r, oracle.bf16_to_f32(oracle.f32_to_bf16(a)))
    x[:] = x[0]                                            # every row the same
    a = oracle.layerwise_attn(x, rows, ld, H, *offs)
    xf = synth.bf16_bits_to_f32(x[0])
    want = xf[offs[2]:offs[2] + H * 128] / (1.0 + np.exp(-xf[offs[3]:offs[3] + H * 128]))
    assert np.allclose(a, want[None], atol=1e-6)


def test_flop_count():
    assert synth.attention_flops(synth.CONFIGS[1]) == pytest.approx(2.6092e11, rel=1e-4)
    assert synth.attention_flops(synth.CONFIGS[0]) == pytest.approx(2.899e10, rel=1e-3)
