"""Write tests/golden/qw_dit_bf16.qw, qw_dit_q8.qw and qw_manifest.json with the REFERENCE's converter code.

    python tests/golden/make_qw_fixture.py [path of the reference checkout, default /root/reference]

The reference's tools/convert.py is imported as it is (it is plain Python + torch; importing it reads no
checkpoint).  Its module constants are shrunk (LAYERS = 2, D = 128, the MLP width passed as H1 = 128) and its
own StreamWriter, dit_specs, linear_specs, put_linear, q8 and interleave_gate_up lay out and write one bf16
and one int8 DiT file from the seeded tensors of tests/qw_fixture_sources.py, following convert_dit's
sequence of writes (tools/convert.py:189-224).  The manifest is the writer's own header (tensor table,
meta, start of the data section).  These files pin the `.qw` reader, the int8 dequantisation and the
SwiGLU column interleave to the reference's code rather than to a restatement of it; they need the
reference checkout only when they are regenerated.
"""
import json
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import qw_fixture_sources as src  # noqa: E402


def main():
    ref = sys.argv[1] if len(sys.argv) > 1 else "/root/reference"
    sys.path.insert(0, os.path.join(ref, "tools"))
    import convert                                     # the reference's converter module
    convert.LAYERS, convert.D = src.LAYERS, src.D
    t = lambda a: torch.from_numpy(a)
    manifest = {"written_by": "tools/convert.py of the reference (StreamWriter, dit_specs, put_linear, q8, interleave_gate_up)",
                "constants": {"LAYERS": src.LAYERS, "D": src.D, "H1": src.F, "ALIGN": convert.ALIGN, "Q_GROUP": convert.Q_GROUP,
                              "GEMM_BN": convert.GEMM_BN}, "files": {}}
    for quant, fname in ((False, "qw_dit_bf16.qw"), (True, "qw_dit_q8.qw")):
        path = os.path.join(HERE, fname)
        w = convert.StreamWriter(path, convert.dit_specs(quant, src.F),
                                 {"model": "krea2-turbo-dit", "layers": src.LAYERS, "q8": quant, "gpu_units": src.F, "attn_split": None, "lora": None})
        cast = (lambda x: x) if quant else (lambda x: x.to(torch.bfloat16))
        for i in range(src.LAYERS):
            p, L = f"L{i}.", src.layer(i)
            qkvg = torch.cat([t(L[n]).float() for n in ("wq", "wk", "wv", "gate")])
            convert.put_linear(w, p + "qkvg", cast(qkvg.t()), quant)
            convert.put_linear(w, p + "o", cast(t(L["wo"]).float().t()), quant)
            gu = convert.interleave_gate_up(t(L["mlp_gate"]).float(), t(L["mlp_up"]).float())
            convert.put_linear(w, p + "gu", cast(gu.t()), quant)
            convert.put_linear(w, p + "down", cast(t(L["mlp_down"]).float().t()), quant)
            w.write(p + "qn", t(L["qnorm_scale"]).float() + 1)
            w.write(p + "kn", t(L["knorm_scale"]).float() + 1)
            w.write(p + "n1", t(L["prenorm_scale"]).float() + 1)
            w.write(p + "n2", t(L["postnorm_scale"]).float() + 1)
            w.write(p + "mod", t(L["mod"]).float().view(6, src.D))
        o = src.outer()
        w.write("first.w", t(o["first_w"]).float().t())
        w.write("first.b", t(o["first_b"]).float())
        w.write("last.w", t(o["last_w"]).float().t())
        w.write("last.b", t(o["last_b"]).float())
        w.write("last.n", t(o["last_n"]).float() + 1)
        w.write("last.mod", t(o["last_mod"]).float())
        w.close()
        manifest["files"][fname] = {"header": w.header, "data_start": w.data_start, "size": os.path.getsize(path)}
    with open(os.path.join(HERE, "qw_manifest.json"), "w") as f:
        json.dump(manifest, f, indent=1, sort_keys=True)
    for fname, m in manifest["files"].items():
        print(fname, m["size"], "bytes,", len(m["header"]["tensors"]), "tensors")


if __name__ == "__main__":
    main()
