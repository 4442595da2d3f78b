"""Property tests of the CPU oracle on small random shapes (hypothesis): the C restatement against the
independent float64 numpy statement, with Lq != Lk, ragged sizes, GQA groups, the gate, the causal mask with an
offset, the fp32 rank-1 term - and invariants that hold whatever the inputs: rows are convex combinations of V
rows, permuting the keys together with their values changes nothing, a fully masked row is zero."""
import numpy as np
from hypothesis import given, settings, strategies as st

import oracle
from krea_image_b200 import synth
from oracle import oracle_np

SET = settings(max_examples=25, deadline=None, derandomize=True)


def _bits(rng, shape, scale=1.0):
    return synth.f32_to_bf16_bits((scale * rng.standard_normal(shape)).astype(np.float32)).reshape(shape)


def _f64(b):
    return synth.bf16_bits_to_f32(b).astype(np.float64)


@SET
@given(seed=st.integers(0, 2 ** 31 - 1), Lq=st.integers(1, 40), Lk=st.integers(1, 70), kvh=st.integers(1, 2), group=st.sampled_from([1, 2, 4]),
       causal=st.booleans(), q_pos0=st.integers(-3, 30), gate=st.booleans(), big=st.booleans())
def test_attention_matches_numpy(seed, Lq, Lk, kvh, group, causal, q_pos0, gate, big):
    rng = np.random.default_rng(seed)
    H = kvh * group
    ldq, ldk, ldv, ldg = H * 128 + 8, kvh * 128, kvh * 128 + 16, H * 128
    Q, K, V, G = _bits(rng, (Lq, ldq)), _bits(rng, (Lk, ldk)), _bits(rng, (Lk, ldv)), _bits(rng, (Lq, ldg))
    QB = rng.standard_normal((Lq, H)).astype(np.float32) if big else None
    KB = rng.standard_normal((Lk, kvh)).astype(np.float32) if big else None
    got = oracle.attention(Q.reshape(-1), K.reshape(-1), V.reshape(-1), Lq, Lk, H, ldq, ldk, ldv, group=group, causal=causal, q_pos0=q_pos0,
                           G=G.reshape(-1) if gate else None, ldg=ldg if gate else 0, QB=QB, KB=KB)
    for h in range(H):
        q, k, v = _f64(Q[:, h * 128:(h + 1) * 128]), _f64(K[:, (h // group) * 128:(h // group + 1) * 128]), _f64(V[:, (h // group) * 128:(h // group + 1) * 128])
        s = (q @ k.T)
        if big:
            s = s + QB[:, h:h + 1].astype(np.float64) * KB[:, h // group][None, :].astype(np.float64)
        s = s / np.sqrt(128.0)
        ok = np.ones_like(s, dtype=bool)
        if causal:
            ok = np.arange(Lk)[None, :] <= (np.arange(Lq)[:, None] + q_pos0)
        s = np.where(ok, s, -np.inf)
        m = np.where(np.isfinite(s.max(axis=1, keepdims=True)), s.max(axis=1, keepdims=True), 0.0)
        p = np.exp(s - m)
        l = p.sum(axis=1, keepdims=True)
        want = np.where(l > 0, (p @ v) / np.where(l > 0, l, 1.0), 0.0)
        if gate:
            want = want / (1.0 + np.exp(-_f64(G[:, h * 128:(h + 1) * 128])))
        assert np.allclose(got[:, h * 128:(h + 1) * 128], want, rtol=2e-4, atol=2e-5)


@SET
@given(seed=st.integers(0, 2 ** 31 - 1), Lq=st.integers(1, 30), Lk=st.integers(2, 60), H=st.integers(1, 3))
def test_attention_invariants(seed, Lq, Lk, H):
    rng = np.random.default_rng(seed)
    ld = H * 128
    Q, K, V = _bits(rng, (Lq, ld)), _bits(rng, (Lk, ld)), _bits(rng, (Lk, ld))
    out = oracle.attention(Q.reshape(-1), K.reshape(-1), V.reshape(-1), Lq, Lk, H, ld, ld, ld)
    v = synth.bf16_bits_to_f32(V)
    assert np.all(out <= v.max(axis=0)[None] + 1e-5) and np.all(out >= v.min(axis=0)[None] - 1e-5)       # convex combinations
    perm = rng.permutation(Lk)
    out_p = oracle.attention(Q.reshape(-1), np.ascontiguousarray(K[perm]).reshape(-1), np.ascontiguousarray(V[perm]).reshape(-1), Lq, Lk, H, ld, ld, ld)
    assert np.allclose(out, out_p, rtol=1e-4, atol=1e-5)                                               # key order is irrelevant
    masked = oracle.attention(Q.reshape(-1), K.reshape(-1), V.reshape(-1), Lq, Lk, H, ld, ld, ld, causal=True, q_pos0=-Lq - 1)
    assert not masked.any()                                                                            # no visible key: zeros (attention.metal:316)


@SET
@given(seed=st.integers(0, 2 ** 31 - 1), rows=st.integers(1, 20), n_q=st.integers(0, 3), n_k=st.integers(0, 3), mode=st.sampled_from([0, 1, 2]))
def test_qk_norm_rope_matches_numpy(seed, rows, n_q, n_k, mode):
    rng = np.random.default_rng(seed)
    ld = (n_q + n_k) * 128 + 8
    x = _bits(rng, (rows, ld), 2.0)
    wq = rng.uniform(0.5, 1.5, 128).astype(np.float32)
    wk = rng.uniform(0.5, 1.5, 128).astype(np.float32)
    ang = rng.uniform(0, 6.28, (rows, 64))
    cos, sin = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
    got = x.copy()
    oracle.qk_norm_rope(got, wq, wk, cos, sin, rows, ld, 8, n_q, 8 + n_q * 128, n_k, 1e-6, mode)
    assert np.array_equal(got[:, :8], x[:, :8])
    for h in range(n_q + n_k):
        w = wq if h < n_q else wk
        src = _f64(x[:, 8 + h * 128:8 + (h + 1) * 128])
        want = oracle_np.norm_rope(src, w.astype(np.float64), cos.astype(np.float64), sin.astype(np.float64), 1e-6, mode)
        g = synth.bf16_bits_to_f32(got[:, 8 + h * 128:8 + (h + 1) * 128])
        assert np.allclose(g, want, rtol=2.0 ** -7, atol=1e-3)        # one bf16 rounding at the store
