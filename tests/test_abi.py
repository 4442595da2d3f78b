"""CPU tests of the drop-in boundary: the shared library builds, loads without a GPU, exports exactly
what include/krea_cuda.h declares, and its host-side pieces (RoPE table builders, argument checks that
need no device) behave like the reference's (engine/src/model.mm:290-315, engine/src/metal.mm:182-202)."""
import ctypes
import os
import re

import numpy as np

import oracle
from krea_image_b200 import binding, ops

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "krea_cuda.h")).read()
    return re.findall(r"KREA_CUDA_API\s+[\w\s\*]+?\b(krea_cuda_\w+)\s*\(", text)


def test_library_exports_every_declared_symbol():
    lib = binding.load()
    names = _declared_symbols()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), n
    assert set(names) == set(binding.SYMBOLS), set(names) ^ set(binding.SYMBOLS)


def test_library_is_built_in_tree():
    assert binding.library_path().startswith(ROOT)
    assert os.path.exists(binding.library_path())


def test_struct_layouts_match_header_field_order():
    text = open(os.path.join(ROOT, "include", "krea_cuda.h")).read()
    for cname, st in (("krea_cuda_qknorm_args", binding.QKNormArgs), ("krea_cuda_attn_args", binding.AttnArgs),
                      ("krea_cuda_joint_args", binding.JointArgs), ("krea_cuda_reshard_args", binding.ReshardArgs),
                      ("krea_cuda_layerwise_args", binding.LayerwiseArgs), ("krea_cuda_gemm_args", binding.GemmArgs), ("krea_cuda_rmsnorm_args", binding.RmsNormArgs), ("krea_cuda_dequant_args", binding.DequantArgs),
                      ("krea_cuda_dit_block_args", binding.DitBlockArgs), ("krea_cuda_a2a_args", binding.A2AArgs), ("krea_cuda_seqpar_args", binding.SeqParArgs)):
        end = text.index("} " + cname + ";")
        body = text[text.rindex("typedef struct {", 0, end) + len("typedef struct {"):end]
        body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
        fields = []
        for decl in body.split(";"):
            decl = decl.strip()
            if not decl:
                continue
            names = [re.sub(r"[\*\s]", "", n.split()[-1]) for n in decl.split(",")]
            fields += names
        assert fields == [f[0] for f in st._fields_], cname


_STRUCTS = (("krea_cuda_qknorm_args", "QKNormArgs"), ("krea_cuda_attn_args", "AttnArgs"), ("krea_cuda_joint_args", "JointArgs"),
            ("krea_cuda_reshard_args", "ReshardArgs"), ("krea_cuda_layerwise_args", "LayerwiseArgs"), ("krea_cuda_gemm_args", "GemmArgs"),
            ("krea_cuda_rmsnorm_args", "RmsNormArgs"), ("krea_cuda_dequant_args", "DequantArgs"), ("krea_cuda_dit_block_args", "DitBlockArgs"),
            ("krea_cuda_a2a_args", "A2AArgs"), ("krea_cuda_seqpar_args", "SeqParArgs"), ("krea_cuda_qw_info", "QwInfo"))


def test_struct_sizes_and_field_offsets_match_the_c_compiler(tmp_path):
    """Field names in the right order are not enough: a ctypes field one type too narrow shifts everything after it.
    A C program built from the header prints sizeof and every offsetof; the ctypes mirrors must agree byte for byte."""
    import ctypes
    import subprocess
    lines = ["#include <stddef.h>", "#include <stdio.h>", '#include "krea_cuda.h"', "int main(void) {"]
    for cname, pyname in _STRUCTS:
        st = getattr(binding, pyname)
        lines.append(f'  printf("{cname} %zu\\n", sizeof({cname}));')
        for field in st._fields_:
            lines.append(f'  printf("{cname}.{field[0]} %zu\\n", offsetof({cname}, {field[0]}));')
    lines += ["  return 0;", "}"]
    src = tmp_path / "layout.c"
    src.write_text("\n".join(lines) + "\n")
    exe = tmp_path / "layout"
    r = subprocess.run(["gcc", "-std=c11", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    got = dict(line.split() for line in subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.splitlines())
    for cname, pyname in _STRUCTS:
        st = getattr(binding, pyname)
        assert int(got[cname]) == ctypes.sizeof(st), cname
        for field in st._fields_:
            assert int(got[f"{cname}.{field[0]}"]) == getattr(st, field[0]).offset, f"{cname}.{field[0]}"


def test_rope_tables_match_oracle():
    for T, gh, gw in ((512, 32, 32), (7, 3, 5), (0, 2, 2), (4, 0, 0)):
        c, s = ops.rope_tables_axial2d(T, gh, gw)
        c2, s2 = oracle.rope_tables_axial2d(T, gh, gw)
        assert np.allclose(c, c2, atol=1e-7) and np.allclose(s, s2, atol=1e-7)
        c, s = ops.rope_tables_ref3axis(T, gh, gw)
        c2, s2 = oracle.rope_tables_ref3axis(T, gh, gw)
        assert np.allclose(c, c2, atol=1e-7) and np.allclose(s, s2, atol=1e-7)


def test_host_side_argument_errors():
    lib = binding.load()
    assert lib.krea_cuda_rope_tables_axial2d(None, None, 1, 1, 1, 10000.0) == binding.E_ARG
    assert lib.krea_cuda_rope_tables_ref3axis(None, None, 1, 1, 1) == binding.E_ARG
    # null handles are rejected, never dereferenced
    assert lib.krea_cuda_sync(None) == binding.E_ARG
    assert lib.krea_cuda_attention(None, None) == binding.E_ARG
    assert lib.krea_cuda_qk_norm_rope(None, None) == binding.E_ARG
    assert lib.krea_cuda_joint_attention(None, None) == binding.E_ARG
    assert lib.krea_cuda_layerwise_attn(None, None) == binding.E_ARG
    assert lib.krea_cuda_gemm(None, None) == binding.E_ARG
    assert lib.krea_cuda_rms_norm(None, None) == binding.E_ARG
    assert lib.krea_cuda_dequant_q8(None, None) == binding.E_ARG
    assert lib.krea_cuda_dit_block(None, None) == binding.E_ARG
    assert lib.krea_cuda_dit_block_workspace_bytes(None) == 0
    # the sequence-parallel entry points need a handle with a communicator
    assert lib.krea_cuda_dist_init(None, 0, 1, None) == binding.E_ARG
    assert lib.krea_cuda_dist_sync(None, 10) == binding.E_ARG
    assert lib.krea_cuda_seqpar_joint_attention(None, None) == binding.E_ARG
    assert lib.krea_cuda_reshard_seq_to_heads(None, None) == binding.E_ARG
    assert lib.krea_cuda_dist_rank(None) == -1 and lib.krea_cuda_dist_size(None) == 0
    assert lib.krea_cuda_dist_unique_id(None, None, 0) == binding.E_ARG
    a = binding.JointArgs()
    a.Lk, a.heads, a.group, a.batch = 4608, 24, 1, 1
    assert lib.krea_cuda_joint_scratch_bytes(ctypes.byref(a)) == 4608 * 24 * 128 * 2


def test_create_fails_loudly_without_a_device():
    import torch
    if torch.cuda.is_available():
        return
    try:
        ops.KreaCuda(0)
    except ops.KreaCudaError as e:
        assert "CUDA" in str(e) or "device" in str(e)
    else:
        raise AssertionError("krea_cuda_create must fail when there is no GPU (no CPU fallback)")


def test_header_compiles_as_c_and_a_c_program_links(tmp_path):
    """The boundary is a C ABI: a C11 translation unit including the header builds with -Wall -Werror -pedantic, links
    against the library and gets sensible answers from the entry points that need no GPU."""
    import subprocess
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from qw_writer import write_qw
    lib = binding.library_path()
    exe = tmp_path / "c_abi_smoke"
    src = os.path.join(ROOT, "tests", "c_abi_smoke.c")
    cmd = ["gcc", "-std=c11", "-Wall", "-Werror", "-pedantic", "-I", os.path.join(ROOT, "include"), src, "-o", str(exe),
           "-L", os.path.dirname(lib), "-lkrea_cuda", "-lm", "-Wl,-rpath," + os.path.dirname(lib)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    qw = tmp_path / "w.qw"
    write_qw(qw, [("L0.qn", "f32", np.full(128, 1.25, np.float32)), ("L0.kn", "f32", np.ones(128, np.float32))])
    r = subprocess.run([str(exe), str(qw)], capture_output=True, text=True)
    assert r.returncode == 0 and r.stdout.strip().endswith("OK"), r.stdout + r.stderr
    assert "L0.qn[0] = 1.250000, 2 tensors" in r.stdout
