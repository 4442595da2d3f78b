"""Builds small `.qw` files in memory for the tests that need contents no converter writes (a half-precision
tensor, unknown header keys, a 40 MB tensor, block-shaped layers).  Container layout as engine/src/weights.mm:16-81
reads it: 4 bytes "QWTS", little-endian u32 version, u64 JSON length, the JSON, then a data section that starts
on a 16 KiB boundary and holds every tensor at a 16 KiB-aligned offset relative to that start.  The tests that
pin the format to the reference use the converter-written files under tests/golden instead."""
import json
import struct

import numpy as np

ALIGN = 16384
_ITEM = {"bf16": np.uint16, "f32": np.float32, "f16": np.float16, "i8": np.int8}


def _up(n):
    return -(-n // ALIGN) * ALIGN


def write_qw(path, tensors, meta=None, extra_header=None):
    """tensors: list of (name, dtype string, numpy array); bf16 arrays are uint16 bit patterns.
    Returns (header dict, byte position of the data section)."""
    blobs = [np.ascontiguousarray(a, dtype=_ITEM[dt]).tobytes() for _, dt, a in tensors]
    starts = np.concatenate([[0], np.cumsum([_up(len(b)) for b in blobs])]).astype(np.int64)
    table = {name: {"dtype": dt, "shape": list(a.shape), "offset": int(o), "nbytes": len(b)}
             for (name, dt, a), b, o in zip(tensors, blobs, starts)}
    header = dict(extra_header or {}, tensors=table, meta=meta or {})
    text = json.dumps(header).encode()
    data_start = _up(16 + len(text))
    image = bytearray(data_start + int(starts[-1]))
    image[:16 + len(text)] = b"QWTS" + struct.pack("<IQ", 1, len(text)) + text
    for b, o in zip(blobs, starts):
        image[data_start + int(o):data_start + int(o) + len(b)] = b
    with open(path, "wb") as f:
        f.write(image)
    return header, data_start
