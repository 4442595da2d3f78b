"""Writes small `.qw` files for the tests, following the layout the reference's converter produces
(tools/convert.py:49-89): "QWTS", u32 version = 1, u64 header length, JSON header with tensor offsets
relative to a data section that starts at the next multiple of 16 KiB; every tensor 16 KiB aligned."""
import json
import struct

import numpy as np

ALIGN = 16384
_DT = {"bf16": (np.uint16, 2), "f32": (np.float32, 4), "f16": (np.float16, 2), "i8": (np.int8, 1)}


def write_qw(path, tensors, meta=None, extra_header=None):
    """tensors: list of (name, dtype string, numpy array); bf16 arrays are uint16 bit patterns."""
    header = {"tensors": {}, "meta": meta or {}}
    if extra_header:
        header.update(extra_header)
    off = 0
    for name, dtype, a in tensors:
        nbytes = int(np.prod(a.shape, dtype=np.int64)) * _DT[dtype][1]
        header["tensors"][name] = {"dtype": dtype, "shape": list(a.shape), "offset": off, "nbytes": nbytes}
        off = (off + nbytes + ALIGN - 1) // ALIGN * ALIGN
    hj = json.dumps(header).encode()
    data_start = (16 + len(hj) + ALIGN - 1) // ALIGN * ALIGN
    with open(path, "wb") as f:
        f.write(b"QWTS" + struct.pack("<IQ", 1, len(hj)) + hj)
        f.truncate(data_start + off)
        for name, dtype, a in tensors:
            f.seek(data_start + header["tensors"][name]["offset"])
            f.write(np.ascontiguousarray(a, dtype=_DT[dtype][0]).tobytes())
    return header, data_start
