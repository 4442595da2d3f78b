"""GPU parity of the projection GEMM next to the attention (Metal::gemm with Epi::BF16, engine/src/metal.h:64-67)
and of its fused QK-norm + RoPE epilogue (gemm followed by Metal::qk_norm_rope in the reference,
engine/src/model.mm:349-359, 376) against float64 / float32 numpy statements of the same math."""
import numpy as np
import pytest
import torch

from krea_image_b200 import binding, ops, synth
from oracle import oracle_np

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", params=["by-size", "cta-pair"])
def kc(request):
    """Every test of this module runs twice: with the library choosing the tile by problem size (small cases take
    the one-CTA tiles) and with the 256 x 256 tile on CTA pairs forced, so that its loads, products and every
    epilogue see the same ragged shapes."""
    import os
    if request.param == "cta-pair":
        os.environ["KREA_CUDA_GEMM_BN"] = "512"
    try:
        k = ops.KreaCuda(0)
    finally:
        os.environ.pop("KREA_CUDA_GEMM_BN", None)
    k.set_stream(torch.cuda.current_stream())
    yield k
    k.close()


def _bits(a):
    return synth.f32_to_bf16_bits(np.ascontiguousarray(a, dtype=np.float32)).reshape(a.shape)


def _dev(bits):
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).cuda().view(torch.bfloat16)


def _case(seed, M, N, K, lda, ldw):
    rng = np.random.default_rng(seed)
    a = _bits(rng.standard_normal((M, lda)))
    w = _bits(rng.standard_normal((K, ldw)) / np.sqrt(K))
    return a, w


def _rel(got, want):
    d = got.astype(np.float64) - want
    return np.linalg.norm(d) / max(np.linalg.norm(want), 1e-30), np.abs(d).max()


@pytest.mark.parametrize("M,N,K,pad", [(128, 256, 64, 0), (1, 8, 8, 0), (300, 520, 200, 8), (257, 1000, 72, 16), (1024, 768, 2048, 0)])
def test_gemm_bf16_shapes(kc, M, N, K, pad):
    lda, ldw, ldc = K + pad, N + pad, N + 2 * pad
    a, w = _case(M + N + K, M, N, K, lda, ldw)
    want = synth.bf16_bits_to_f32(a[:, :K]).astype(np.float64) @ synth.bf16_bits_to_f32(w[:, :N]).astype(np.float64)
    c = torch.full((M, ldc), float("nan"), dtype=torch.bfloat16, device="cuda")
    n0 = kc.launches
    kc.gemm(_dev(a), _dev(w), c, M, N, K, lda, ldw, ldc)
    kc.wait()
    assert kc.launches - n0 == 1
    got = c.float().cpu().numpy()
    rel, mx = _rel(got[:, :N], want)
    assert rel <= 3e-3, f"rel-L2 {rel:.3e} max-abs {mx:.3e}"          # one bf16 rounding of the output: ~1.7e-3
    assert np.all(np.isnan(got[:, N:]))                                # nothing written past column N


def test_gemm_fused_qk_norm_rope(kc):
    """q|k|v projection of a small model (4 heads, S = 400 with a 16 x 20 grid): Q and K blocks come out
    normalised and rotated, V plain; the result drives the attention operator and matches the oracle chain."""
    import oracle
    H, T, gh, gw, K = 4, 80, 16, 20, 320
    S = T + gh * gw
    N = 3 * H * 128
    a, w = _case(5, S, N, K, K, N)
    rng = np.random.default_rng(6)
    wq = rng.uniform(0.5, 1.5, 128).astype(np.float32)
    wk = rng.uniform(0.5, 1.5, 128).astype(np.float32)
    cos, sin = synth.rope_tables_axial2d(T, gh, gw)
    y = synth.bf16_bits_to_f32(a).astype(np.float64) @ synth.bf16_bits_to_f32(w).astype(np.float64)       # [S, N]
    want = y.copy()
    for h in range(H):
        want[:, h * 128:(h + 1) * 128] = oracle_np.norm_rope(y[:, h * 128:(h + 1) * 128], wq.astype(np.float64), cos, sin, 1e-6, 0)
        want[:, (H + h) * 128:(H + h + 1) * 128] = oracle_np.norm_rope(y[:, (H + h) * 128:(H + h + 1) * 128], wk.astype(np.float64), cos, sin, 1e-6, 0)
    dev = lambda x: torch.from_numpy(np.ascontiguousarray(x)).cuda()
    d_wq, d_wk, d_cos, d_sin = dev(wq), dev(wk), dev(cos), dev(sin)
    c = torch.zeros((S, N), dtype=torch.bfloat16, device="cuda")
    kc.gemm(_dev(a), _dev(w), c, S, N, K, K, N, N,
            qk_norm=dict(q_off=0, n_q=H, k_off=H * 128, n_k=H, wq=d_wq, wk=d_wk, cos=d_cos, sin=d_sin, row0=0, eps=1e-6, rope_mode=0))
    kc.wait()
    got = c.float().cpu().numpy()
    for name, lo, hi in (("Q", 0, H * 128), ("K", H * 128, 2 * H * 128), ("V", 2 * H * 128, N)):
        rel, mx = _rel(got[:, lo:hi], want[:, lo:hi])
        assert rel <= 3e-3, f"{name}: rel-L2 {rel:.3e} max-abs {mx:.3e}"
    # ... and the attention operator on the projected, already normalised rows against the oracle's attention on the same bits
    cb = c.view(torch.int16).cpu().numpy().view(np.uint16)
    o = torch.zeros((S, H * 128), dtype=torch.bfloat16, device="cuda")
    cf = c.view(-1)
    kc.attention(cf, cf[H * 128:], cf[2 * H * 128:], o, S, S, H, N, N, N, H * 128, 1)
    kc.wait()
    flat = cb.reshape(-1)
    want_o = oracle.attention(flat, flat[H * 128:], flat[2 * H * 128:], S, S, H, N, N, N)
    rel, mx = _rel(o.float().cpu().numpy(), want_o)
    assert rel <= 5e-3 and mx <= 2e-2
    # errors: rotate-half is not fused, head blocks must sit on 128-column boundaries
    with pytest.raises(ops.KreaCudaError) as e:
        kc.gemm(_dev(a), _dev(w), c, S, N, K, K, N, N, qk_norm=dict(q_off=0, n_q=H, k_off=H * 128, n_k=H, wq=d_wq, wk=d_wk, cos=d_cos, sin=d_sin, rope_mode=1))
    assert e.value.code == binding.E_UNSUPPORTED
    with pytest.raises(ops.KreaCudaError):
        kc.gemm(_dev(a), _dev(w), c, S, N, K, K, N, N, qk_norm=dict(q_off=64, n_q=H, k_off=H * 128, n_k=H, wq=d_wq, wk=d_wk, cos=d_cos, sin=d_sin))
    with pytest.raises(ops.KreaCudaError):
        kc.gemm(_dev(a), _dev(w), c, S, N + 4, K, K, N, N)


@pytest.mark.parametrize("with_gate", [True, False])
def test_gemm_gated_residual_epilogue(kc, with_gate):
    """Epi::ResidGate / Epi::Resid (gemm.metal:262-267): the fp32 residual stream receives += gate[n] * acc."""
    M, N, K = 333, 520, 264
    a, w = _case(21, M, N, K, K, N)
    rng = np.random.default_rng(22)
    x0 = rng.standard_normal((M, N + 8)).astype(np.float32)
    gate = np.tanh(rng.standard_normal(N)).astype(np.float32)
    acc = synth.bf16_bits_to_f32(a).astype(np.float64) @ synth.bf16_bits_to_f32(w).astype(np.float64)
    want = x0[:, :N] + (gate[None, :] if with_gate else 1.0) * acc
    x = torch.from_numpy(x0).cuda()
    kc.gemm(_dev(a), _dev(w), x, M, N, K, K, N, N + 8, epilogue=binding.EPI_RESID_GATE, vec=torch.from_numpy(gate).cuda() if with_gate else None)
    kc.wait()
    got = x.cpu().numpy()
    assert np.allclose(got[:, :N], want, rtol=1e-4, atol=1e-4)       # fp32 in, fp32 out: only accumulation order differs
    assert np.array_equal(got[:, N:], x0[:, N:])                       # columns past N untouched


def test_gemm_swiglu_epilogue(kc):
    """Epi::SwiGLU (gemm.metal:233-250): weight columns come in groups of 64 = 32 gate + 32 up columns."""
    M, H1, K = 200, 160, 136          # N = 2 * H1 = 320 = five groups of 64
    N = 2 * H1
    a, w = _case(31, M, N, K, K, N)
    acc = synth.bf16_bits_to_f32(a).astype(np.float64) @ synth.bf16_bits_to_f32(w).astype(np.float64)
    g = acc.reshape(M, N // 64, 2, 32)
    want = (g[:, :, 0] / (1.0 + np.exp(-g[:, :, 0])) * g[:, :, 1]).reshape(M, H1)
    c = torch.full((M, H1 + 8), float("nan"), dtype=torch.bfloat16, device="cuda")
    kc.gemm(_dev(a), _dev(w), c, M, N, K, K, N, H1 + 8, epilogue=binding.EPI_SWIGLU)
    kc.wait()
    got = c.float().cpu().numpy()
    rel, mx = _rel(got[:, :H1], want)
    assert rel <= 3e-3, f"rel-L2 {rel:.3e} max-abs {mx:.3e}"
    assert np.all(np.isnan(got[:, H1:]))
    with pytest.raises(ops.KreaCudaError):
        kc.gemm(_dev(a), _dev(w), c, M, N - 32, K, K, N, H1 + 8, epilogue=binding.EPI_SWIGLU)   # not a whole number of groups


def test_gemm_tile_width_variants(monkeypatch):
    """The three tiles (128 x 256, 128 x 128 and 256 x 256 on a CTA pair, chosen per problem by how the tiles fill
    the last wave) accumulate every output element in the same order: forced any way, the results are bit-identical."""
    M, N, K = 300, 1000, 328
    a, w = _case(41, M, N, K, K, N)
    outs = []
    for bn in ("128", "256", "512"):
        monkeypatch.setenv("KREA_CUDA_GEMM_BN", bn)
        k2 = ops.KreaCuda(0)
        try:
            k2.set_stream(torch.cuda.current_stream())
            c = torch.zeros((M, N), dtype=torch.bfloat16, device="cuda")
            k2.gemm(_dev(a), _dev(w), c, M, N, K, K, N, N)
            k2.wait()
            outs.append(c)
        finally:
            k2.close()
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    want = synth.bf16_bits_to_f32(a).astype(np.float64) @ synth.bf16_bits_to_f32(w).astype(np.float64)
    rel, _ = _rel(outs[0].float().cpu().numpy(), want)
    assert rel <= 3e-3


@pytest.mark.parametrize("epi", ["f32", "gelu", "bias_bf16", "bias_f32"])
def test_gemm_remaining_epilogues(kc, epi):
    """Epi::F32, Epi::GELU, Epi::BiasBF16, Epi::BiasF32 (gemm.metal:257-260, 268-277)."""
    M, N, K = 150, 264, 136
    a, w = _case(61, M, N, K, K, N)
    rng = np.random.default_rng(62)
    bias = rng.standard_normal(N).astype(np.float32)
    acc = synth.bf16_bits_to_f32(a).astype(np.float64) @ synth.bf16_bits_to_f32(w).astype(np.float64)
    code = {"f32": binding.EPI_F32, "gelu": binding.EPI_GELU, "bias_bf16": binding.EPI_BIAS_BF16, "bias_f32": binding.EPI_BIAS_F32}[epi]
    f32_out = epi in ("f32", "bias_f32")
    want = {"f32": acc, "gelu": 0.5 * acc * (1.0 + np.tanh(0.7978845608028654 * (acc + 0.044715 * acc ** 3))),
            "bias_bf16": acc + bias, "bias_f32": acc + bias}[epi]
    c = torch.full((M, N + 8), float("nan"), dtype=torch.float32 if f32_out else torch.bfloat16, device="cuda")
    kc.gemm(_dev(a), _dev(w), c, M, N, K, K, N, N + 8, epilogue=code, vec=torch.from_numpy(bias).cuda() if "bias" in epi else None)
    kc.wait()
    got = c.float().cpu().numpy()
    if f32_out:
        assert np.allclose(got[:, :N], want, rtol=1e-4, atol=1e-4)
    else:
        rel, mx = _rel(got[:, :N], want)
        assert rel <= 3e-3, f"rel-L2 {rel:.3e} max-abs {mx:.3e}"
    assert np.all(np.isnan(got[:, N:]))
    if "bias" in epi:
        with pytest.raises(ops.KreaCudaError):
            kc.gemm(_dev(a), _dev(w), c, M, N, K, K, N, N + 8, epilogue=code)          # bias vector missing


@pytest.mark.parametrize("rank,epi", [(16, "bf16"), (40, "swiglu"), (128, "resid")])
def test_gemm_second_product_lora_term(kc, rank, epi):
    """LoraTerm (metal.h:31-35, gemm.metal:46-50): acc += A2[M, K2] x W2[K2, N] before the epilogue, so the fused
    epilogues see the full result."""
    M, N, K = 260, 384, 200
    a, w = _case(71, M, N, K, K, N)
    rng = np.random.default_rng(72 + rank)
    a2 = _bits(rng.standard_normal((M, rank)))
    w2 = _bits(rng.standard_normal((rank, N)) / np.sqrt(rank))
    acc = (synth.bf16_bits_to_f32(a).astype(np.float64) @ synth.bf16_bits_to_f32(w).astype(np.float64)
           + synth.bf16_bits_to_f32(a2).astype(np.float64) @ synth.bf16_bits_to_f32(w2).astype(np.float64))
    lora = (_dev(a2), _dev(w2), rank, rank, N)
    if epi == "bf16":
        c = torch.zeros((M, N), dtype=torch.bfloat16, device="cuda")
        kc.gemm(_dev(a), _dev(w), c, M, N, K, K, N, N, lora=lora)
        want = acc
    elif epi == "swiglu":
        c = torch.zeros((M, N // 2), dtype=torch.bfloat16, device="cuda")
        kc.gemm(_dev(a), _dev(w), c, M, N, K, K, N, N // 2, epilogue=binding.EPI_SWIGLU, lora=lora)
        g = acc.reshape(M, N // 64, 2, 32)
        want = (g[:, :, 0] / (1.0 + np.exp(-g[:, :, 0])) * g[:, :, 1]).reshape(M, N // 2)
    else:
        x0 = rng.standard_normal((M, N)).astype(np.float32)
        c = torch.from_numpy(x0).cuda()
        kc.gemm(_dev(a), _dev(w), c, M, N, K, K, N, N, epilogue=binding.EPI_RESID_GATE, lora=lora)
        want = x0 + acc
    kc.wait()
    rel, mx = _rel(c.float().cpu().numpy(), want)
    assert rel <= 3e-3, f"rel-L2 {rel:.3e} max-abs {mx:.3e}"
    with pytest.raises(ops.KreaCudaError):
        kc.gemm(_dev(a), _dev(w), c, M, N, K, K, N, N, lora=(_dev(a2), None, rank, rank, N))


def test_gemm_column_remap(kc):
    """GemmParams::seg (gemm.metal:41-43): segments of `seg` output columns land `seg_stride` apart - the reference
    uses it to drop the GPU's slice of a head-split projection into a wider row."""
    M, N, K, seg, stride = 130, 384, 72, 128, 200
    a, w = _case(81, M, N, K, K, N)
    acc = synth.bf16_bits_to_f32(a).astype(np.float64) @ synth.bf16_bits_to_f32(w).astype(np.float64)
    ldc = 2 * stride + seg + 8
    c = torch.full((M, ldc), float("nan"), dtype=torch.bfloat16, device="cuda")
    kc.gemm(_dev(a), _dev(w), c, M, N, K, K, N, ldc, seg=seg, seg_stride=stride)
    kc.wait()
    got = c.float().cpu().numpy()
    touched = np.zeros(ldc, dtype=bool)
    for s0 in range(N // seg):
        rel, _ = _rel(got[:, s0 * stride:s0 * stride + seg], acc[:, s0 * seg:(s0 + 1) * seg])
        assert rel <= 3e-3
        touched[s0 * stride:s0 * stride + seg] = True
    assert np.all(np.isnan(got[:, ~touched]))
    with pytest.raises(ops.KreaCudaError):
        kc.gemm(_dev(a), _dev(w), c, M, N, K, K, N, 2 * stride, seg=seg, seg_stride=stride)      # ldc does not cover the last segment


def _q8(w):
    """tools/convert.py:92-99: symmetric int8 per output column and group of 128 input rows."""
    K, N = w.shape
    g = w.reshape(K // 128, 128, N)
    scale = np.maximum(np.abs(g).max(axis=1), 1e-12) / 127.0
    q = np.clip(np.rint(g / scale[:, None, :]), -127, 127).reshape(K, N)
    return q.astype(np.int8), scale.astype(np.float32)


def test_dequant_q8_bit_exact_and_feeds_the_gemm(kc):
    """Weight::q8 (gemm.metal:159-170): d = bf16(float(q) * s).  Integer and byte work: bit-exact against numpy."""
    rng = np.random.default_rng(51)
    K, N, M = 384, 272, 200
    q, sc = _q8((rng.standard_normal((K, N)) / np.sqrt(K)).astype(np.float32))
    want_bits = synth.f32_to_bf16_bits(q.astype(np.float32) * np.repeat(sc, 128, axis=0)).reshape(K, N)
    out = torch.zeros((K, N + 8), dtype=torch.bfloat16, device="cuda")
    kc.dequant_q8(torch.from_numpy(q).cuda(), torch.from_numpy(sc).cuda(), out, K, N, N, N, N + 8)
    kc.wait()
    got_bits = out.view(torch.int16).cpu().numpy().view(np.uint16)
    assert np.array_equal(got_bits[:, :N], want_bits) and not got_bits[:, N:].any()
    # ... and the product with the dequantised copy equals the product the reference forms tile by tile
    a = _bits(rng.standard_normal((M, K)))
    c = torch.zeros((M, N), dtype=torch.bfloat16, device="cuda")
    kc.gemm(_dev(a), out, c, M, N, K, K, N + 8, N)
    kc.wait()
    want = synth.bf16_bits_to_f32(a).astype(np.float64) @ synth.bf16_bits_to_f32(want_bits).astype(np.float64)
    rel, _ = _rel(c.float().cpu().numpy(), want)
    assert rel <= 3e-3
    with pytest.raises(ops.KreaCudaError):
        kc.dequant_q8(torch.from_numpy(q).cuda(), torch.from_numpy(sc).cuda(), out, K - 64, N, N, N, N + 8)    # not whole scale groups


def test_gemm_model_size_projection(kc):
    """The q|k|v projection at the headline configuration's size (4608 x 9216 x 3072) against float32 numpy."""
    M, N, K = 4608, 9216, 3072
    a, w = _case(11, M, N, K, K, N)
    c = torch.zeros((M, N), dtype=torch.bfloat16, device="cuda")
    kc.gemm(_dev(a), _dev(w), c, M, N, K, K, N, N)
    kc.wait()
    rows = np.arange(0, M, 37)
    want = synth.bf16_bits_to_f32(a[rows]) @ synth.bf16_bits_to_f32(w)
    got = c[torch.from_numpy(rows).cuda()].float().cpu().numpy()
    rel, mx = _rel(got, want)
    assert rel <= 3e-3, f"rel-L2 {rel:.3e} max-abs {mx:.3e}"
