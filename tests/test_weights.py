"""The `.qw` weight-file reader (the format that supplies the attention path's QK-norm weights): CPU tests
of the parser on contents no converter writes (tests/qw_writer.py) and on damaged copies of a
converter-written file, and GPU tests that take qn / kn and whole layers from a file all the way into the
fused attention call and the DiT block.  tests/test_qw_reference_fixture.py pins the format itself."""
import json
import os
import struct

import numpy as np
import pytest

from krea_image_b200 import binding, synth, weights
from krea_image_b200.ops import KreaCudaError
from qw_writer import ALIGN, write_qw


def _model_like(rng, layers=3):
    """Tensors named and typed like the converter's DiT file (tools/convert.py:212-213: qn/kn = scale + 1, f32[128])."""
    ts = []
    for l in range(layers):
        ts.append((f"L{l}.qn", "f32", (rng.uniform(-0.5, 0.5, 128) + 1).astype(np.float32)))
        ts.append((f"L{l}.kn", "f32", (rng.uniform(-0.5, 0.5, 128) + 1).astype(np.float32)))
        ts.append((f"L{l}.qkvg", "i8", rng.integers(-127, 128, (256, 384), dtype=np.int8)))
        ts.append((f"L{l}.qkvg.s", "f32", rng.uniform(0.001, 0.01, (2, 384)).astype(np.float32)))
        ts.append((f"L{l}.o", "bf16", synth.f32_to_bf16_bits(rng.standard_normal((64, 96)).astype(np.float32)).reshape(64, 96)))
    ts.append(("E.emb", "f16", rng.standard_normal((5, 7)).astype(np.float16)))
    return ts


def test_reader_matches_writer(tmp_path):
    rng = np.random.default_rng(3)
    ts = _model_like(rng)
    path = tmp_path / "dit.qw"
    header, data_start = write_qw(path, ts, meta={"model": "krea-2-turbo", "units": 16384, "note": 'a "quoted" name\n'},
                                  extra_header={"ignored": [1, {"x": None}, True, "s"]})
    with weights.WeightFile(path) as w:
        assert len(w) == len(ts) and w.names() == sorted(n for n, _, _ in ts)
        assert w.meta() == header["meta"]
        assert w.data_bytes() == os.path.getsize(path) - data_start
        for name, dtype, a in ts:
            ti = w.info(name)
            assert (ti.dtype, ti.shape, ti.offset, ti.nbytes) == (dtype, a.shape, header["tensors"][name]["offset"], a.nbytes)
            assert ti.offset % ALIGN == 0
            assert np.array_equal(w.get(name), a)
        assert w.has("L1.qkvg.s") and not w.has("L1.qkvg.z")          # WeightFile::linear looks for the ".s" companion
        with pytest.raises(KeyError):
            w.info("L9.qn")
        off, ln = w.span("L1.")                                        # one layer's segment is contiguous
        lo = min(header["tensors"][n]["offset"] for n in header["tensors"] if n.startswith("L1."))
        hi = max(header["tensors"][n]["offset"] + header["tensors"][n]["nbytes"] for n in header["tensors"] if n.startswith("L1."))
        assert (off, ln) == (lo, hi - lo)
        with pytest.raises(KeyError):
            w.span("Z")


def test_reader_rejects_damaged_files(tmp_path):
    # the intact file is one the reference's converter code wrote (tests/golden/make_qw_fixture.py)
    raw = open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "qw_dit_bf16.qw"), "rb").read()

    def expect(name, data, needle):
        p = tmp_path / name
        p.write_bytes(data)
        with pytest.raises(KreaCudaError) as e:
            weights.WeightFile(p)
        assert needle in str(e.value), str(e.value)

    expect("magic.qw", b"QWTX" + raw[4:], "magic")
    expect("short.qw", raw[:10], "short")
    expect("hlen.qw", raw[:8] + struct.pack("<Q", len(raw)) + raw[16:], "header length")
    hlen = struct.unpack("<Q", raw[8:16])[0]
    expect("json.qw", raw[:16] + raw[16:16 + hlen].replace(b'"offset"', b'"offset', 1) + raw[16 + hlen:], "header")
    expect("eof.qw", raw[:len(raw) - ALIGN], "outside")                # the last tensor no longer fits
    hdr = json.loads(raw[16:16 + hlen])
    hdr["tensors"]["L0.qn"]["shape"] = [127]
    hj = json.dumps(hdr).encode().ljust(hlen)                           # same length: offsets stay valid
    expect("shape.qw", raw[:16] + hj + raw[16 + hlen:], "disagree")

    # numbers that are no sizes: negative, fractional, infinite, beyond any file; a shape whose product wraps around
    # 64 bits; a header nested deeper than any converter writes
    def with_header(mutate):
        h = json.loads(raw[16:16 + hlen])
        mutate(h)
        hj = json.dumps(h).encode()
        assert len(hj) <= hlen + ALIGN - 64
        body = b"QWTS" + struct.pack("<IQ", 1, len(hj)) + hj
        start = (len(body) + ALIGN - 1) // ALIGN * ALIGN
        old_start = (16 + hlen + ALIGN - 1) // ALIGN * ALIGN
        return body.ljust(start, b"\0") + raw[old_start:]

    def set_field(field, value):
        return lambda h: h["tensors"]["L0.qn"].__setitem__(field, value)

    expect("neg.qw", with_header(set_field("offset", -16384)), "whole number")
    expect("frac.qw", with_header(set_field("nbytes", 511.5)), "whole number")
    expect("huge.qw", with_header(set_field("offset", 1e300)), "whole number")
    expect("inf.qw", with_header(set_field("offset", 0)).replace(b'"offset": 0', b'"offset": inf', 1), "header")
    expect("wrap.qw", with_header(set_field("shape", [2 ** 32, 2 ** 32, 128])), "overflows")
    deep = json.loads("[" * 100 + "]" * 100)
    expect("deep.qw", with_header(lambda h: h.__setitem__("extra", deep)), "nested")
    with pytest.raises(KreaCudaError):
        weights.WeightFile(tmp_path / "absent.qw")


def test_big_dim_detection():
    """model.mm:226-239: the dimension with the largest |qn*kn| above the threshold, else -1."""
    qn = np.full(128, 1.2, np.float32)
    kn = np.full(128, 0.9, np.float32)
    assert weights.big_dim(qn, kn) == -1
    qn[37], kn[37] = 52.8, -52.8
    assert weights.big_dim(qn, kn) == 37
    qn[90], kn[90] = 60.0, 60.0
    assert weights.big_dim(qn, kn) == 90
    assert weights.big_dim(qn, kn, gain_threshold=1e9) == -1
    assert binding.load().krea_cuda_qw_big_dim(None, None, 256.0) == -1


@pytest.mark.gpu
def test_weights_from_file_feed_the_fused_attention(tmp_path):
    import torch

    import oracle
    from krea_image_b200 import ops
    rng = np.random.default_rng(8)
    ts = _model_like(rng, 2)
    big = rng.standard_normal(40 << 20 >> 2).astype(np.float32)         # 40 MB: several staging chunks
    ts.append(("Z.big", "f32", big))
    path = tmp_path / "dit.qw"
    write_qw(path, ts)
    kc = ops.KreaCuda(0)
    kc.set_stream(torch.cuda.current_stream())
    try:
        with weights.WeightFile(path) as w:
            d_qn = torch.empty(128, dtype=torch.float32, device="cuda")
            d_kn = torch.empty(128, dtype=torch.float32, device="cuda")
            w.upload_tensor(kc, "L1.qn", d_qn)
            w.upload_tensor(kc, "L1.kn", d_kn)
            qn, kn = w.get("L1.qn").copy(), w.get("L1.kn").copy()
            assert np.array_equal(d_qn.cpu().numpy(), qn) and np.array_equal(d_kn.cpu().numpy(), kn)
            d_big = torch.empty(big.size + 3, dtype=torch.float32, device="cuda").fill_(7.0)
            ti = w.upload_tensor(kc, "Z.big", d_big)
            assert ti.nbytes == big.nbytes
            assert np.array_equal(d_big[:big.size].cpu().numpy(), big) and bool((d_big[big.size:] == 7.0).all())
            off, ln = w.span("L0.")
            seg = torch.empty(ln, dtype=torch.uint8, device="cuda")
            w.upload(kc, off, ln, seg)                                   # a whole layer segment in one range
            ti = w.info("L0.kn")
            assert np.array_equal(seg[ti.offset - off:ti.offset - off + 512].cpu().numpy().view(np.float32), w.get("L0.kn"))
            with pytest.raises(KreaCudaError):
                w.upload(kc, w.data_bytes() - 4, 8, seg)                 # range past the end of the data section
        # the uploaded weights drive the fused call
        H, T, gh, gw = 2, 32, 8, 8
        S = T + gh * gw
        qkv = synth.f32_to_bf16_bits(rng.standard_normal((1, S, 3 * H * 128)).astype(np.float32))
        cos, sin = synth.rope_tables_axial2d(T, gh, gw)
        want = oracle.joint_attention(qkv, 1, S, H, qn, kn, cos, sin)
        x = torch.from_numpy(qkv.view(np.int16)).cuda().view(torch.bfloat16).view(-1)
        o = torch.zeros((S, H * 128), dtype=torch.bfloat16, device="cuda")
        ld = 3 * H * 128
        dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
        kc.joint_attention(x, x[H * 128:], x[2 * H * 128:], o, S, S, H, ld, ld, ld, H * 128, d_qn, d_kn, dev(cos), dev(sin))
        kc.wait()
        got = o.float().cpu().numpy()
        rel = np.linalg.norm(got - want[0]) / np.linalg.norm(want[0])
        assert rel <= 5e-3 and np.abs(got - want[0]).max() <= 2e-2
    finally:
        kc.close()


@pytest.mark.gpu
def test_block_weights_from_file_drive_the_dit_block(tmp_path):
    """A converter-style file (tools/convert.py:196-213: qkvg = q|k|v|gate, gu interleaved, all [K, N] bf16) ->
    one segment upload -> krea_cuda_dit_block: same bits as the block run on separately uploaded tensors."""
    import torch

    from krea_image_b200 import ops
    rng = np.random.default_rng(12)
    heads, kv, ff, T, gh, gw = 2, 1, 256, 16, 6, 8
    D, S = heads * 128, T + gh * gw
    QC = (2 * heads + 2 * kv) * 128
    bf = lambda a: synth.f32_to_bf16_bits(np.ascontiguousarray(a, dtype=np.float32)).reshape(a.shape)
    ts = []
    for l in range(2):
        ts += [(f"L{l}.qkvg", "bf16", bf(rng.standard_normal((D, QC)) / np.sqrt(D))), (f"L{l}.o", "bf16", bf(rng.standard_normal((D, D)) / np.sqrt(D))),
               (f"L{l}.gu", "bf16", bf(rng.standard_normal((D, 2 * ff)) / np.sqrt(D))), (f"L{l}.down", "bf16", bf(rng.standard_normal((ff, D)) / np.sqrt(ff))),
               (f"L{l}.qn", "f32", rng.uniform(0.5, 1.5, 128).astype(np.float32)), (f"L{l}.kn", "f32", rng.uniform(0.5, 1.5, 128).astype(np.float32)),
               (f"L{l}.n1", "f32", np.ones(D, np.float32))]
    path = tmp_path / "dit.qw"
    write_qw(path, ts, meta={"model": "krea2-turbo-dit", "layers": 2, "q8": False})
    x0 = rng.standard_normal((S, D)).astype(np.float32)
    mods = (1.0 + 0.1 * rng.standard_normal((6, D))).astype(np.float32)
    cos, sin = synth.rope_tables_axial2d(T, gh, gw)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    kc = ops.KreaCuda(0)
    kc.set_stream(torch.cuda.current_stream())
    try:
        with weights.WeightFile(path) as w:
            assert w.meta()["q8"] is False
            bw = weights.BlockWeights(kc, w, 1)
            x = dev(x0)
            bw.run(kc, x, dev(mods), dev(cos), dev(sin), S, heads, kv)
            kc.wait()
            t = {n: a for n, _, a in ts}
            tb = lambda n: torch.from_numpy(t[n].view(np.int16)).cuda().view(torch.bfloat16)
            x2 = dev(x0)
            kc.dit_block(x2, dev(mods), tb("L1.qkvg"), tb("L1.o"), tb("L1.gu"), tb("L1.down"), dev(t["L1.qn"]), dev(t["L1.kn"]), dev(cos), dev(sin),
                         S, heads, kv, ff)
            kc.wait()
            assert torch.equal(x, x2) and bool(torch.isfinite(x).all()) and not torch.equal(x, dev(x0))
        # the same layer stored as int8 + group scales (the converter's `dit_q8.qw` flavour): dequantised at load
        # time into the values the reference's GEMM would form, then the same block call
        def q8(wb):
            w = synth.bf16_bits_to_f32(wb)
            K, N = w.shape
            g = w.reshape(K // 128, 128, N)
            scale = np.maximum(np.abs(g).max(axis=1), 1e-12) / 127.0
            return np.clip(np.rint(g / scale[:, None, :]), -127, 127).reshape(K, N).astype(np.int8), scale.astype(np.float32)
        ts8 = []
        for n, dt, a in ts:
            if n.startswith("L1.") and dt == "bf16":
                q, sc = q8(a)
                ts8 += [(n, "i8", q), (n + ".s", "f32", sc)]
            elif n.startswith("L1."):
                ts8.append((n, dt, a))
        path8 = tmp_path / "dit_q8.qw"
        write_qw(path8, ts8, meta={"q8": True})
        with weights.WeightFile(path8) as w8:
            bw8 = weights.BlockWeights(kc, w8, 1)
            kc.wait()
            deq = bw8.qkvg.float().cpu().numpy()
            q, sc = q8(t["L1.qkvg"])
            want = synth.bf16_bits_to_f32(synth.f32_to_bf16_bits(q.astype(np.float32) * np.repeat(sc, 128, axis=0))).reshape(q.shape)
            assert np.array_equal(deq, want)
            x8 = dev(x0)
            bw8.run(kc, x8, dev(mods), dev(cos), dev(sin), S, heads, kv)
            kc.wait()
            upd, upd8 = (x - dev(x0)).double(), (x8 - dev(x0)).double()
            assert float((upd - upd8).norm() / upd.norm()) < 5e-2       # int8 weights: a percent-level change of the update
    finally:
        kc.close()
