"""Seeded source tensors behind tests/golden/qw_dit_bf16.qw and qw_dit_q8.qw.

Those two files were written by the reference's own converter code (tools/convert.py: StreamWriter,
dit_specs, linear_specs, put_linear, q8, interleave_gate_up) from the arrays below - see
tests/golden/make_qw_fixture.py - so the tests can compare what the library reads, dequantises and
multiplies with the values the converter was given, without the fixture having to carry them: the
counter-based generator reproduces them bit for bit anywhere.

Shapes are the checkpoint's ([out, in] for linear weights), shrunk: model width D = 128, MLP width F = 128,
two layers; the k and v projections keep the converter's fixed 1536 rows each.
"""
import numpy as np

from krea_image_b200 import synth

D, F, LAYERS, KV = 128, 128, 2, 1536
SEED = 777


def _normal(stream, shape, scale):
    n = int(np.prod(shape))
    n2 = n + (n & 1)
    return (synth.normal_f32(SEED, stream << 32, n2)[:n] * np.float32(scale)).reshape(shape)


def layer(i):
    """The tensors of block i as the checkpoint would hold them (float32)."""
    s = 100 * (i + 1)
    return {
        "wq": _normal(s + 0, (D, D), D ** -0.5), "wk": _normal(s + 1, (KV, D), D ** -0.5), "wv": _normal(s + 2, (KV, D), D ** -0.5),
        "gate": _normal(s + 3, (D, D), D ** -0.5), "wo": _normal(s + 4, (D, D), D ** -0.5),
        "mlp_gate": _normal(s + 5, (F, D), D ** -0.5), "mlp_up": _normal(s + 6, (F, D), D ** -0.5), "mlp_down": _normal(s + 7, (D, F), F ** -0.5),
        "qnorm_scale": _normal(s + 8, (128,), 0.2), "knorm_scale": _normal(s + 9, (128,), 0.2),
        "prenorm_scale": _normal(s + 10, (D,), 0.1), "postnorm_scale": _normal(s + 11, (D,), 0.1), "mod": _normal(s + 12, (6, D), 0.1),
    }


def outer():
    """first / last tensors of the DiT file."""
    return {"first_w": _normal(1, (D, 64), 0.125), "first_b": _normal(2, (D,), 0.1), "last_w": _normal(3, (64, D), D ** -0.5),
            "last_b": _normal(4, (64,), 0.1), "last_n": _normal(5, (D,), 0.1), "last_mod": _normal(6, (2, D), 0.1)}
