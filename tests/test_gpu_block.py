"""GPU parity of Metal::rms_norm and of one whole DiT block (DiT::layer, engine/src/model.mm:369-385) against
the float64 numpy statement, at a reduced width (2 heads of 128, GQA 2:1) and at 8 heads."""
import numpy as np
import pytest
import torch

from krea_image_b200 import ops, synth
from oracle import oracle_np

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def kc():
    k = ops.KreaCuda(0)
    k.set_stream(torch.cuda.current_stream())
    yield k
    k.close()


def _bits(a):
    return synth.f32_to_bf16_bits(np.ascontiguousarray(a, dtype=np.float32)).reshape(a.shape)


def _dev_bf16(bits):
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).cuda().view(torch.bfloat16)


def _f64(bits):
    return synth.bf16_bits_to_f32(bits).astype(np.float64)


@pytest.mark.parametrize("rows,width,pad,with_add,f32_out", [(5, 256, 0, True, False), (33, 6144, 8, True, False), (7, 10240, 0, False, True), (1, 4, 4, True, True)])
def test_rms_norm_operator(kc, rows, width, pad, with_add, f32_out):
    rng = np.random.default_rng(rows + width)
    x = (3.0 * rng.standard_normal((rows, width + pad))).astype(np.float32)
    mul = (1.0 + 0.3 * rng.standard_normal(width)).astype(np.float32)
    add = (0.2 * rng.standard_normal(width)).astype(np.float32) if with_add else None
    want = oracle_np.rms_norm(x[:, :width].astype(np.float64), mul.astype(np.float64), None if add is None else add.astype(np.float64), 1e-6)
    ld_out = width + (8 if not f32_out else 4)
    y = torch.full((rows, ld_out), float("nan"), dtype=torch.float32 if f32_out else torch.bfloat16, device="cuda")
    kc.rms_norm(torch.from_numpy(x).cuda(), torch.from_numpy(mul).cuda(), None if add is None else torch.from_numpy(add).cuda(), y,
                rows, width, width + pad, ld_out, 1e-6, f32_out)
    kc.wait()
    got = y.float().cpu().numpy()
    tol = 2e-5 if f32_out else 6e-3          # bf16 output: half an ulp of 2^-8
    assert np.allclose(got[:, :width], want, rtol=tol, atol=tol)
    assert np.all(np.isnan(got[:, width:]))
    with pytest.raises(ops.KreaCudaError):
        kc.rms_norm(torch.from_numpy(x).cuda(), torch.from_numpy(mul).cuda(), None, y, rows, width + 2, width + pad, ld_out, 1e-6, f32_out)


@pytest.mark.parametrize("heads,kv_heads,ff,T,gh,gw", [(2, 1, 512, 24, 8, 10), (8, 2, 1024, 64, 12, 16)])
def test_dit_block_matches_oracle(kc, heads, kv_heads, ff, T, gh, gw):
    rng = np.random.default_rng(heads * 7 + ff)
    D, S = heads * 128, T + gh * gw
    QC = (2 * heads + 2 * kv_heads) * 128
    x0 = rng.standard_normal((S, D)).astype(np.float32)
    mods = np.stack([1.0 + 0.2 * rng.standard_normal(D), 0.1 * rng.standard_normal(D), np.tanh(rng.standard_normal(D)),
                     1.0 + 0.2 * rng.standard_normal(D), 0.1 * rng.standard_normal(D), np.tanh(rng.standard_normal(D))]).astype(np.float32)
    w_qkvg = _bits(rng.standard_normal((D, QC)) / np.sqrt(D))
    w_o = _bits(rng.standard_normal((D, D)) / np.sqrt(D))
    w_gu = _bits(rng.standard_normal((D, 2 * ff)) / np.sqrt(D))
    w_down = _bits(rng.standard_normal((ff, D)) / np.sqrt(ff))
    qn = rng.uniform(0.5, 1.5, 128).astype(np.float32)
    kn = rng.uniform(0.5, 1.5, 128).astype(np.float32)
    cos, sin = synth.rope_tables_axial2d(T, gh, gw)
    args = (x0, mods.astype(np.float64), _f64(w_qkvg), _f64(w_o), _f64(w_gu), _f64(w_down), qn.astype(np.float64), kn.astype(np.float64),
            cos.astype(np.float64), sin.astype(np.float64), heads, kv_heads, ff)
    want = oracle_np.dit_block(*args)
    want_r = oracle_np.dit_block(*args, ref_rounding=True)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    x = dev(x0)
    n0 = kc.launches
    kc.dit_block(x, dev(mods), _dev_bf16(w_qkvg), _dev_bf16(w_o), _dev_bf16(w_gu), _dev_bf16(w_down), dev(qn), dev(kn), dev(cos), dev(sin),
                 S, heads, kv_heads, ff)
    kc.wait()
    assert kc.launches - n0 == 7                      # two norms, four GEMMs, one attention
    got = x.cpu().numpy().astype(np.float64)
    # what the block added to the residual stream, against the two oracle modes
    upd, upd_w, upd_r = got - x0, want - x0, want_r - x0
    rel = np.linalg.norm(upd - upd_w) / np.linalg.norm(upd_w)
    rel_r = np.linalg.norm(upd - upd_r) / np.linalg.norm(upd_r)
    gap = np.linalg.norm(upd_r - upd_w) / np.linalg.norm(upd_w)       # the reference's own bf16 roundings
    print(f"block update: rel-L2 {rel:.3e} vs float64, {rel_r:.3e} vs reference rounding (the two oracles differ by {gap:.3e})")
    assert rel <= 6e-3 and rel_r <= 5e-3 and np.all(np.isfinite(got))
    # a caller-provided workspace gives the same bits
    a = ops.B.DitBlockArgs()
    a.rows, a.heads, a.kv_heads, a.ff = S, heads, kv_heads, ff
    nbytes = int(kc.lib.krea_cuda_dit_block_workspace_bytes(a))
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    x2 = dev(x0)
    kc.dit_block(x2, dev(mods), _dev_bf16(w_qkvg), _dev_bf16(w_o), _dev_bf16(w_gu), _dev_bf16(w_down), dev(qn), dev(kn), dev(cos), dev(sin),
                 S, heads, kv_heads, ff, workspace=ws)
    kc.wait()
    assert torch.equal(x2, x)
    with pytest.raises(ops.KreaCudaError):
        kc.dit_block(x2, dev(mods), _dev_bf16(w_qkvg), _dev_bf16(w_o), _dev_bf16(w_gu), _dev_bf16(w_down), dev(qn), dev(kn), dev(cos), dev(sin),
                     S, heads, kv_heads, ff, workspace=ws[:nbytes // 2])


def test_dit_block_with_the_big_gain_dimension(kc):
    """The reference's block 0 (model.mm:226-239, norm.metal:68-71): one head dimension carries a QK-norm gain of
    52.8 on both q and k, its q.k term dominates the logits, and it is routed through fp32 side buffers and the
    attention's rank-1 term.  With the split the block stays within 1e-2 of the float64 statement and is closer to it
    than without (here 7.2e-3 against 8.4e-3: near-hard softmax rows amplify every rounding of q and k)."""
    rng = np.random.default_rng(77)
    heads, kv_heads, ff, T, gh, gw = 4, 2, 512, 32, 10, 12
    D, S = heads * 128, T + gh * gw
    QC = (2 * heads + 2 * kv_heads) * 128
    x0 = rng.standard_normal((S, D)).astype(np.float32)
    mods = np.stack([np.ones(D), np.zeros(D), np.ones(D), np.ones(D), np.zeros(D), np.ones(D)]).astype(np.float32)
    w_qkvg = _bits(rng.standard_normal((D, QC)) / np.sqrt(D))
    w_o = _bits(rng.standard_normal((D, D)) / np.sqrt(D))
    w_gu = _bits(rng.standard_normal((D, 2 * ff)) / np.sqrt(D))
    w_down = _bits(rng.standard_normal((ff, D)) / np.sqrt(ff))
    qn = rng.uniform(0.5, 1.5, 128).astype(np.float32)
    kn = rng.uniform(0.5, 1.5, 128).astype(np.float32)
    big = 37
    qn[big] = kn[big] = 52.8
    from krea_image_b200 import weights
    assert weights.big_dim(qn, kn) == big
    cos, sin = synth.rope_tables_axial2d(T, gh, gw)
    want = oracle_np.dit_block(x0, mods.astype(np.float64), _f64(w_qkvg), _f64(w_o), _f64(w_gu), _f64(w_down), qn.astype(np.float64),
                               kn.astype(np.float64), cos.astype(np.float64), sin.astype(np.float64), heads, kv_heads, ff)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    rels = {}
    for bd in (big, -1):
        x = dev(x0)
        kc.dit_block(x, dev(mods), _dev_bf16(w_qkvg), _dev_bf16(w_o), _dev_bf16(w_gu), _dev_bf16(w_down), dev(qn), dev(kn), dev(cos), dev(sin),
                     S, heads, kv_heads, ff, big_dim=bd)
        kc.wait()
        got = x.cpu().numpy().astype(np.float64)
        rels[bd] = np.linalg.norm(got - want) / np.linalg.norm(want - x0)
    print(f"update error with the fp32 split {rels[big]:.3e}, without {rels[-1]:.3e}")
    assert rels[big] <= 1e-2 and rels[big] < rels[-1]
