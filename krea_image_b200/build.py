"""Build libkrea_cuda.so (sm_100a only) in-tree with nvcc.

    python -m krea_image_b200.build [--force]

nvcc cross-compiles without a GPU.  The CUDA runtime is linked statically and the one driver entry point
the library needs (cuTensorMapEncodeTiled) is resolved at run time, so the shared object loads - and its
exported symbols can be inspected - on a machine without a GPU driver.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT_DIR = os.path.join(HERE, "_build")
LIB = os.path.join(OUT_DIR, "libkrea_cuda.so")
SOURCES = ["krea_cuda.cu", "attention_sm100.cu", "attention_persist_sm100.cu", "qk_norm_rope.cu", "layerwise_attn.cu", "gemm_sm100.cu", "rms_norm.cu", "dequant_q8.cu", "dist_nccl.cu", "qw_file.cu"]
HEADERS = ["attention_sm100.h", "sm100_ptx.cuh", "handle.h", os.path.join("..", "..", "include", "krea_cuda.h")]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-fvisibility=hidden"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.sep not in cand or os.path.exists(cand)):
            return cand
    return "nvcc"


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in SOURCES + HEADERS] + [os.path.abspath(__file__)]
    return any(os.path.getmtime(d) > t for d in deps)


def _check_register_budget(ptxas_log: str) -> None:
    """The attention kernel re-balances registers between warpgroups with setmaxnreg: the softmax warps go
    up and the producer / MMA warpgroup goes down, which only adds up (and can only be granted) if the CTA
    starts with exactly the count the kernel's configuration assumes (168 per thread for the 384-thread
    variant, 96 for the 640-thread one).  A different launch count would leave the softmax warps waiting
    for registers that never come, so refuse to build such a library."""
    import re
    expect = {"1": 168, "2": 96}
    for m in re.finditer(r"Compiling entry function '(\w*attn_fwd_sm100ILi(\d)\w*)'.*?Used (\d+) registers", ptxas_log, re.S):
        want = expect.get(m.group(2))
        if want is not None and int(m.group(3)) != want:
            raise RuntimeError(f"{m.group(1)} starts with {m.group(3)} registers per thread; setmaxnreg needs {want}")
    # the persistent kernel: 512 threads, 128 registers each at launch
    for m in re.finditer(r"Compiling entry function '(\w*attn_persist_sm100\w*)'.*?Used (\d+) registers", ptxas_log, re.S):
        if int(m.group(2)) != 128:
            raise RuntimeError(f"{m.group(1)} starts with {m.group(2)} registers per thread; setmaxnreg needs 128")


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not _stale():
        return LIB
    os.makedirs(OUT_DIR, exist_ok=True)
    objs = []
    procs = []
    for src in SOURCES:
        obj = os.path.join(OUT_DIR, src.replace(".cu", ".o"))
        cmd = [_nvcc(), "-Xptxas", "-v", *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    for src, pr in procs:
        out, _ = pr.communicate()
        if verbose or pr.returncode:
            sys.stderr.write(out)
        if pr.returncode:
            raise RuntimeError(f"nvcc failed on {src}")
        _check_register_budget(out)
    cmd = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", LIB, *objs, "-cudart", "static", "-ldl"]
    subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
