"""The `.qw` reader, the int8 dequantisation and the SwiGLU column interleave against files that the
REFERENCE's own converter code wrote (tests/golden/qw_dit_bf16.qw, qw_dit_q8.qw; generator
tests/golden/make_qw_fixture.py imports tools/convert.py and uses its StreamWriter, dit_specs,
put_linear, q8 and interleave_gate_up on the seeded tensors of tests/qw_fixture_sources.py).

CPU: what the reader reports equals the writer's own header (tests/golden/qw_manifest.json); the tensor
bytes are what the converter makes of the sources (transposed to [in, out], bf16 by round-to-nearest-even,
norm weights stored as 1 + scale, gate/up rows interleaved per 64-column tile, int8 + per-128-row scales).
GPU: krea_cuda_dequant_q8 on the file's int8 + scales is bit-equal to bf16(float(q) * s) and within the
quantiser's bound of the source; the SwiGLU epilogue on the file's interleaved `gu` equals
silu(x gate^T) * (x up^T) computed from the un-interleaved source."""
import json
import os

import numpy as np
import pytest

import qw_fixture_sources as src
from krea_image_b200 import binding, synth, weights

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
MANIFEST = json.load(open(os.path.join(GOLD, "qw_manifest.json")))
BF16_FILE, Q8_FILE = "qw_dit_bf16.qw", "qw_dit_q8.qw"


def _bf16(a):
    return synth.f32_to_bf16_bits(np.ascontiguousarray(a, dtype=np.float32)).reshape(a.shape)


def _qkvg_t(L):
    return np.concatenate([L["wq"], L["wk"], L["wv"], L["gate"]]).T          # [in, out] = [D, 2D + 3072]


@pytest.mark.parametrize("fname", [BF16_FILE, Q8_FILE])
def test_reader_reports_what_the_reference_writer_planned(fname):
    m = MANIFEST["files"][fname]
    tensors, path = m["header"]["tensors"], os.path.join(GOLD, fname)
    assert os.path.getsize(path) == m["size"]
    with weights.WeightFile(path) as w:
        assert len(w) == len(tensors) and w.names() == sorted(tensors)
        assert w.meta() == m["header"]["meta"]
        assert w.data_bytes() == m["size"] - m["data_start"]
        for name, t in tensors.items():
            ti = w.info(name)
            assert (ti.dtype, list(ti.shape), ti.offset, ti.nbytes) == (t["dtype"], t["shape"], t["offset"], t["nbytes"]), name
            assert ti.offset % MANIFEST["constants"]["ALIGN"] == 0
        for l in range(src.LAYERS):                                        # a layer's tensors are one contiguous range
            mine = [t for n, t in tensors.items() if n.startswith(f"L{l}.")]
            lo, hi = min(t["offset"] for t in mine), max(t["offset"] + t["nbytes"] for t in mine)
            assert w.span(f"L{l}.") == (lo, hi - lo)
        assert w.has("L1.qkvg") and w.has("L1.qkvg.s") == (fname == Q8_FILE)   # Weight::q8's companion (weights.h:36-39)
        with pytest.raises(KeyError):
            w.info(f"L{src.LAYERS}.qn")


def test_bf16_file_holds_the_converters_view_of_the_sources():
    with weights.WeightFile(os.path.join(GOLD, BF16_FILE)) as w:
        for l in range(src.LAYERS):
            L, p = src.layer(l), f"L{l}."
            assert np.array_equal(w.get(p + "qkvg"), _bf16(_qkvg_t(L)))      # fused q|k|v|gate, transposed, RNE bf16
            assert np.array_equal(w.get(p + "o"), _bf16(L["wo"].T))
            assert np.array_equal(w.get(p + "down"), _bf16(L["mlp_down"].T))
            # tools/convert.py:102-106: per 64 output columns, 32 gate columns then the 32 up columns of the same units
            gu = w.get(p + "gu").reshape(src.D, src.F // 32, 2, 32)
            assert np.array_equal(gu[:, :, 0].reshape(src.D, src.F), _bf16(L["mlp_gate"].T))
            assert np.array_equal(gu[:, :, 1].reshape(src.D, src.F), _bf16(L["mlp_up"].T))
            assert np.array_equal(w.get(p + "qn"), L["qnorm_scale"] + np.float32(1))   # tools/convert.py:212-213
            assert np.array_equal(w.get(p + "kn"), L["knorm_scale"] + np.float32(1))
            assert np.array_equal(w.get(p + "mod"), L["mod"])
            assert weights.big_dim(w.get(p + "qn"), w.get(p + "kn")) == -1
        o = src.outer()
        assert np.array_equal(w.get("first.w"), o["first_w"].T) and np.array_equal(w.get("last.n"), o["last_n"] + np.float32(1))


def _group_scale_bound(wt, sc):
    """|w - q*s| <= s/2 for every element whose group maximum defined s (round to nearest, no clipping inside +-127)."""
    return np.repeat(sc, 128, axis=0).astype(np.float64) * 0.5 + np.abs(wt) * 1e-6        # + fp32 rounding of w / s


def test_q8_file_is_within_the_quantisers_bound_of_the_sources():
    with weights.WeightFile(os.path.join(GOLD, Q8_FILE)) as w:
        for l in range(src.LAYERS):
            L, p = src.layer(l), f"L{l}."
            for name, wt in (("qkvg", _qkvg_t(L)), ("o", L["wo"].T), ("down", L["mlp_down"].T)):
                q, sc = w.get(p + name), w.get(p + name + ".s")
                assert q.dtype == np.int8 and q.shape == wt.shape and sc.shape == (wt.shape[0] // 128, wt.shape[1])
                assert np.abs(q.astype(np.int32)).max() == 127             # every column group's maximum maps to +-127
                g = np.abs(wt.reshape(-1, 128, wt.shape[1])).max(axis=1)
                assert np.allclose(sc, g / 127.0, rtol=1e-6, atol=0)        # tools/convert.py:92-99
                deq = q.astype(np.float64) * np.repeat(sc, 128, axis=0)
                assert np.all(np.abs(deq - wt) <= _group_scale_bound(wt, sc))


# ---------------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def kc():
    import torch

    from krea_image_b200 import ops
    k = ops.KreaCuda(0)
    k.set_stream(torch.cuda.current_stream())
    yield k
    k.close()


@pytest.mark.gpu
def test_dequant_of_the_reference_made_int8_tensors(kc):
    import torch
    with weights.WeightFile(os.path.join(GOLD, Q8_FILE)) as w:
        for name, wt in (("L1.qkvg", _qkvg_t(src.layer(1))), ("L0.gu", None), ("L0.down", src.layer(0)["mlp_down"].T)):
            ti, si = w.info(name), w.info(name + ".s")
            K, N = ti.shape
            d_q = torch.empty((K, N), dtype=torch.int8, device="cuda")
            d_s = torch.empty(si.shape, dtype=torch.float32, device="cuda")
            w.upload_tensor(kc, name, d_q)
            w.upload_tensor(kc, name + ".s", d_s)
            out = torch.zeros((K, N), dtype=torch.bfloat16, device="cuda")
            kc.dequant_q8(d_q, d_s, out, K, N)
            kc.wait()
            got = out.view(torch.int16).cpu().numpy().view(np.uint16)
            q, sc = w.get(name), w.get(name + ".s")
            want = _bf16(q.astype(np.float32) * np.repeat(sc, 128, axis=0))          # gemm.metal:159-170: bf16(float(q) * s)
            assert np.array_equal(got, want), name
            if wt is not None:                                                        # ... and close to what was quantised
                err = np.abs(synth.bf16_bits_to_f32(got) - wt)
                assert np.all(err <= _group_scale_bound(wt, sc) + np.abs(wt) * 2.0 ** -8), name


@pytest.mark.gpu
def test_swiglu_epilogue_on_the_reference_made_interleave(kc):
    import torch
    rng = np.random.default_rng(5)
    M, K, F = 200, src.D, src.F
    a = _bf16(rng.standard_normal((M, K)))
    x = synth.bf16_bits_to_f32(a).astype(np.float64)
    with weights.WeightFile(os.path.join(GOLD, BF16_FILE)) as w:
        for l in range(src.LAYERS):
            L = src.layer(l)
            d_gu = torch.empty((K, 2 * F), dtype=torch.bfloat16, device="cuda")
            w.upload_tensor(kc, f"L{l}.gu", d_gu)
            c = torch.full((M, F), float("nan"), dtype=torch.bfloat16, device="cuda")
            kc.gemm(torch.from_numpy(a.view(np.int16)).cuda().view(torch.bfloat16), d_gu, c, M, 2 * F, K, K, 2 * F, F, epilogue=binding.EPI_SWIGLU)
            kc.wait()
            gate = synth.bf16_bits_to_f32(_bf16(L["mlp_gate"])).astype(np.float64)     # the un-interleaved source, as the file rounds it
            up = synth.bf16_bits_to_f32(_bf16(L["mlp_up"])).astype(np.float64)
            g, u = x @ gate.T, x @ up.T
            want = g / (1.0 + np.exp(-g)) * u                                         # gemm.metal:233-250
            got = c.float().cpu().numpy().astype(np.float64)
            rel = np.linalg.norm(got - want) / np.linalg.norm(want)
            assert rel <= 3e-3, f"layer {l}: rel-L2 {rel:.3e}"
