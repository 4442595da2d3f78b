"""`.qw` weight files through libkrea_cuda's reader (the reference's WeightFile, engine/src/weights.h:26-75).

The file is mapped by the library; tensors come back as numpy views of that mapping (no copy) and byte
ranges can be uploaded to device memory through a KreaCuda handle.  Opening and querying need no GPU.
"""
import ctypes
import json

import numpy as np

from . import binding as B
from .ops import KreaCudaError, _ptr

_NP = {"f32": np.float32, "f16": np.float16, "i8": np.int8, "bf16": np.uint16}   # bf16 as raw bits


class TensorInfo:
    def __init__(self, info: B.QwInfo):
        self.name = info.name.decode()
        self.dtype = info.dtype.decode()
        self.shape = tuple(int(info.shape[i]) for i in range(info.rank))
        self.offset = int(info.offset)
        self.nbytes = int(info.nbytes)

    def __repr__(self):
        return f"TensorInfo({self.name!r}, {self.dtype}, {self.shape}, offset={self.offset}, nbytes={self.nbytes})"


class WeightFile:
    def __init__(self, path: str):
        self.lib = B.load()
        err = ctypes.create_string_buffer(512)
        self.q = self.lib.krea_cuda_qw_open(str(path).encode(), err, 512)
        if not self.q:
            raise KreaCudaError(B.E_ARG, err.value.decode())
        self.path = str(path)

    def close(self):
        if self.q:
            self.lib.krea_cuda_qw_close(self.q)
            self.q = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def __len__(self):
        return int(self.lib.krea_cuda_qw_count(self.q))

    def names(self):
        out, info = [], B.QwInfo()
        for i in range(len(self)):
            self.lib.krea_cuda_qw_info_at(self.q, i, ctypes.byref(info))
            out.append(info.name.decode())
        return out

    def has(self, name: str) -> bool:
        return self.lib.krea_cuda_qw_find(self.q, name.encode(), None) == B.OK

    def info(self, name: str) -> TensorInfo:
        info = B.QwInfo()
        if self.lib.krea_cuda_qw_find(self.q, name.encode(), ctypes.byref(info)) != B.OK:
            raise KeyError(f"missing tensor: {name} in {self.path}")    # weights.mm:88
        return TensorInfo(info)

    def get(self, name: str) -> np.ndarray:
        """numpy view of the mapping (read-only; bf16 tensors as uint16 bits).  Valid until close()."""
        ti = self.info(name)
        addr = self.lib.krea_cuda_qw_host_ptr(self.q, ti.offset)
        buf = (ctypes.c_char * ti.nbytes).from_address(addr)
        a = np.frombuffer(buf, dtype=_NP[ti.dtype]).reshape(ti.shape)
        a.flags.writeable = False
        return a

    def meta(self) -> dict:
        m = self.lib.krea_cuda_qw_meta(self.q).decode()
        return json.loads(m) if m else {}

    def data_bytes(self) -> int:
        return int(self.lib.krea_cuda_qw_data_bytes(self.q))

    def span(self, prefix: str):
        """(offset, length) of the data-section range covering every tensor whose name starts with prefix."""
        off, ln = ctypes.c_uint64(0), ctypes.c_uint64(0)
        if self.lib.krea_cuda_qw_span(self.q, prefix.encode(), ctypes.byref(off), ctypes.byref(ln)) != B.OK:
            raise KeyError(f"no tensor of {self.path} starts with {prefix!r}")
        return int(off.value), int(ln.value)

    def upload(self, kc, off: int, length: int, dst):
        """Copies data-section bytes [off, off+length) to the device tensor / pointer dst."""
        kc._check(self.lib.krea_cuda_qw_upload(kc.h, self.q, off, length, _ptr(dst)))

    def upload_tensor(self, kc, name: str, dst):
        ti = self.info(name)
        self.upload(kc, ti.offset, ti.nbytes, dst)
        return ti


def big_dim(qn: np.ndarray, kn: np.ndarray, gain_threshold: float = 256.0) -> int:
    """The head dimension the reference routes through fp32 side buffers (model.mm:226-239), or -1."""
    qn = np.ascontiguousarray(qn, dtype=np.float32)
    kn = np.ascontiguousarray(kn, dtype=np.float32)
    assert qn.size == 128 and kn.size == 128
    return int(B.load().krea_cuda_qw_big_dim(qn.ctypes.data, kn.ctypes.data, ctypes.c_float(gain_threshold)))


class BlockWeights:
    """One DiT layer's tensors (`L<l>.qkvg`, `.o`, `.gu`, `.down` bf16 [K, N]; `.qn`, `.kn` f32 [128]) on the
    device: the layer's whole segment of the file is uploaded as one byte range (its tensors are contiguous
    in the file, weights.h:17-22) and the tensors are views into that buffer."""

    NAMES = ("qkvg", "o", "gu", "down", "qn", "kn")

    def __init__(self, kc, wf: WeightFile, layer: int):
        import torch
        prefix = f"L{layer}."
        off, length = wf.span(prefix)
        self.segment = torch.empty(length, dtype=torch.uint8, device=f"cuda:{kc.device}")
        wf.upload(kc, off, length, self.segment)
        self.info = {}
        tdt = {"bf16": torch.bfloat16, "f32": torch.float32, "i8": torch.int8, "f16": torch.float16}

        def view(name):
            ti = wf.info(name)
            raw = self.segment[ti.offset - off:ti.offset - off + ti.nbytes]
            return ti, raw.view(tdt[ti.dtype]).view(ti.shape)
        for n in self.NAMES:
            ti, t = view(prefix + n)
            self.info[n] = ti
            if ti.dtype == "i8":
                # Weight::q8 (weights.h:36-39: companion `<name>.s`): dequantised once into a bf16 copy - the values the
                # reference's GEMM forms tile by tile - because 180 GB of HBM have room for it
                _, sc = view(prefix + n + ".s")
                K, N = ti.shape
                full = torch.empty((K, N), dtype=torch.bfloat16, device=t.device)
                kc.dequant_q8(t, sc, full, K, N)
                t = full
            setattr(self, n, t)

    def run(self, kc, x, mods, cos, sin, rows, heads, kv_heads, eps=1e-6):
        """DiT::layer on the residual stream x with this layer's weights."""
        ff = self.info["down"].shape[0]
        kc.dit_block(x, mods, self.qkvg, self.o, self.gu, self.down, self.qn, self.kn, cos, sin, rows, heads, kv_heads, ff, eps)
