"""ctypes binding of libkrea_cuda (include/krea_cuda.h), in the style of the reference's own binding of
its C ABI (ui/krea.py:120-145): load the shared object, declare argtypes/restypes, mirror the structs.

The library is looked up in-tree (krea_image_b200/_build); if it is missing this module raises - there
is no fallback implementation.
"""
import ctypes
import os

from . import build as _build

PART_FIRST, PART_MID, PART_LAST = 0, 1, 2
OK, E_ARG, E_UNSUPPORTED, E_CUDA, E_DEVICE, E_NOMEM, E_COMM, E_TIMEOUT = 0, -1, -2, -3, -4, -5, -6, -7
ROPE_PAIRS, ROPE_HALF, ROPE_NONE = 0, 1, 2
EPI_BF16, EPI_QKNORM_ROPE, EPI_RESID_GATE, EPI_SWIGLU, EPI_F32, EPI_GELU, EPI_BIAS_BF16, EPI_BIAS_F32 = 0, 1, 2, 3, 4, 5, 6, 7
STATIC_SCRATCH_BYTES = 32 << 20   # KREA_CUDA_STATIC_SCRATCH_BYTES
DIST_ID_BYTES = 128                # KREA_CUDA_DIST_ID_BYTES

_vp = ctypes.c_void_p
_int = ctypes.c_int
_i64 = ctypes.c_int64


class QKNormArgs(ctypes.Structure):
    _fields_ = [("qkv", _vp), ("wq", _vp), ("wk", _vp), ("cos", _vp), ("sin", _vp),
                ("rows", _int), ("ld", _int), ("q_off", _int), ("n_q", _int), ("k_off", _int), ("n_k", _int),
                ("eps", ctypes.c_float), ("rope_mode", _int), ("big_dim", _int), ("qbig", _vp), ("kbig", _vp)]


class AttnArgs(ctypes.Structure):
    _fields_ = [("Q", _vp), ("K", _vp), ("V", _vp), ("O", _vp),
                ("Lq", _int), ("Lk", _int), ("heads", _int),
                ("ldq", _int), ("ldk", _int), ("ldv", _int), ("ldo", _int),
                ("group", _int), ("causal", _int), ("q_pos0", _int),
                ("G", _vp), ("ldg", _int), ("QB", _vp), ("KB", _vp),
                ("batch", _int), ("bsq", _i64), ("bsk", _i64), ("bsv", _i64), ("bso", _i64), ("bsg", _i64),
                ("text_len", _vp), ("text_slots", _int), ("q_row0", _int)]


class JointArgs(ctypes.Structure):
    _fields_ = [("Q", _vp), ("K", _vp), ("V", _vp), ("O", _vp),
                ("batch", _int), ("Lq", _int), ("Lk", _int), ("q_row0", _int), ("heads", _int), ("group", _int),
                ("ldq", _int), ("ldk", _int), ("ldv", _int), ("ldo", _int),
                ("bsq", _i64), ("bsk", _i64), ("bsv", _i64), ("bso", _i64),
                ("wq", _vp), ("wk", _vp), ("cos", _vp), ("sin", _vp), ("eps", ctypes.c_float), ("rope_mode", _int),
                ("text_len", _vp), ("text_slots", _int), ("G", _vp), ("ldg", _int), ("bsg", _i64),
                ("k_scratch", _vp), ("k_scratch_bytes", ctypes.c_size_t)]


class ReshardArgs(ctypes.Structure):
    _fields_ = [("src", _vp), ("dst", _vp), ("nranks", _int), ("rows", _int), ("cols_per_rank", _int),
                ("src_ld", _int), ("dst_ld", _int), ("src_col0", _int), ("dst_col0", _int)]


class LayerwiseArgs(ctypes.Structure):
    _fields_ = [("qkvg", _vp), ("out", _vp), ("rows", _int), ("ld", _int), ("ldo", _int), ("heads", _int),
                ("q_off", _int), ("k_off", _int), ("v_off", _int), ("g_off", _int)]


class GemmArgs(ctypes.Structure):
    _fields_ = [("A", _vp), ("W", _vp), ("C", _vp), ("M", _int), ("N", _int), ("K", _int),
                ("lda", _int), ("ldw", _int), ("ldc", _int), ("epilogue", _int),
                ("q_off", _int), ("n_q", _int), ("k_off", _int), ("n_k", _int),
                ("wq", _vp), ("wk", _vp), ("cos", _vp), ("sin", _vp), ("row0", _int), ("eps", ctypes.c_float), ("rope_mode", _int), ("vec", _vp),
                ("big_dim", _int), ("qbig", _vp), ("kbig", _vp),
                ("lora_A", _vp), ("lora_W", _vp), ("lora_K", _int), ("lora_lda", _int), ("lora_ldw", _int),
                ("seg", _int), ("seg_stride", _int)]


class DequantArgs(ctypes.Structure):
    _fields_ = [("wq", _vp), ("scales", _vp), ("out", _vp), ("K", _int), ("N", _int), ("ldq", _int), ("lds", _int), ("ldo", _int)]


class RmsNormArgs(ctypes.Structure):
    _fields_ = [("x", _vp), ("mul", _vp), ("add", _vp), ("y", _vp), ("rows", _int), ("width", _int), ("ld_in", _int),
                ("ld_out", _int), ("eps", ctypes.c_float), ("f32_out", _int)]


class DitBlockArgs(ctypes.Structure):
    _fields_ = [("x", _vp), ("mods", _vp), ("w_qkvg", _vp), ("w_o", _vp), ("w_gu", _vp), ("w_down", _vp),
                ("qn", _vp), ("kn", _vp), ("cos", _vp), ("sin", _vp),
                ("rows", _int), ("heads", _int), ("kv_heads", _int), ("ff", _int), ("eps", ctypes.c_float),
                ("workspace", _vp), ("workspace_bytes", ctypes.c_size_t), ("use_big_dim", _int), ("big_dim", _int)]


class QwInfo(ctypes.Structure):
    _fields_ = [("name", ctypes.c_char_p), ("dtype", ctypes.c_char_p), ("rank", _int), ("shape", _i64 * 8),
                ("offset", ctypes.c_uint64), ("nbytes", ctypes.c_uint64)]


class A2AArgs(ctypes.Structure):
    _fields_ = [("src", _vp), ("dst", _vp), ("rows_local", _int), ("cols_per_rank", _int),
                ("src_ld", _int), ("dst_ld", _int), ("src_col0", _int), ("dst_col0", _int)]


class SeqParArgs(ctypes.Structure):
    _fields_ = [("Q", _vp), ("K", _vp), ("V", _vp), ("O", _vp),
                ("seq", _int), ("heads", _int), ("group", _int),
                ("ldq", _int), ("ldk", _int), ("ldv", _int), ("ldo", _int),
                ("wq", _vp), ("wk", _vp), ("cos", _vp), ("sin", _vp), ("eps", ctypes.c_float), ("rope_mode", _int)]


# every symbol include/krea_cuda.h declares: name -> (restype, argtypes)
SYMBOLS = {
    "krea_cuda_create": (_vp, [_int, ctypes.c_char_p, _int]),
    "krea_cuda_destroy": (None, [_vp]),
    "krea_cuda_last_error": (ctypes.c_char_p, [_vp]),
    "krea_cuda_set_stream": (_int, [_vp, _vp]),
    "krea_cuda_sync": (_int, [_vp]),
    "krea_cuda_launch_count": (ctypes.c_uint64, [_vp]),
    "krea_cuda_set_wait_limit": (_int, [_vp, ctypes.c_uint64]),
    "krea_cuda_test_drop_one_load": (_int, [_vp, _int]),
    "krea_cuda_profile_enable": (_int, [_vp, _int]),
    "krea_cuda_profile_read": (_int, [_vp, _int, ctypes.POINTER(ctypes.c_double), ctypes.POINTER(_int)]),
    "krea_cuda_profile_trace": (_int, [_vp, ctypes.c_char_p]),
    "krea_cuda_qk_norm_rope": (_int, [_vp, ctypes.POINTER(QKNormArgs)]),
    "krea_cuda_attention": (_int, [_vp, ctypes.POINTER(AttnArgs)]),
    "krea_cuda_attention_partial": (_int, [_vp, ctypes.POINTER(AttnArgs), _int, _vp, _vp, _vp]),
    "krea_cuda_joint_scratch_bytes": (ctypes.c_size_t, [ctypes.POINTER(JointArgs)]),
    "krea_cuda_joint_attention": (_int, [_vp, ctypes.POINTER(JointArgs)]),
    "krea_cuda_joint_attention_host": (_int, [_vp, ctypes.POINTER(JointArgs)]),
    "krea_cuda_joint_attention_static": (_int, [_vp, ctypes.POINTER(JointArgs)]),
    "krea_cuda_rope_tables_ref3axis": (_int, [_vp, _vp, _int, _int, _int]),
    "krea_cuda_rope_tables_axial2d": (_int, [_vp, _vp, _int, _int, _int, ctypes.c_double]),
    "krea_cuda_gemm": (_int, [_vp, ctypes.POINTER(GemmArgs)]),
    "krea_cuda_dequant_q8": (_int, [_vp, ctypes.POINTER(DequantArgs)]),
    "krea_cuda_rms_norm": (_int, [_vp, ctypes.POINTER(RmsNormArgs)]),
    "krea_cuda_dit_block_workspace_bytes": (ctypes.c_size_t, [ctypes.POINTER(DitBlockArgs)]),
    "krea_cuda_dit_block": (_int, [_vp, ctypes.POINTER(DitBlockArgs)]),
    "krea_cuda_layerwise_attn": (_int, [_vp, ctypes.POINTER(LayerwiseArgs)]),
    "krea_cuda_qw_open": (_vp, [ctypes.c_char_p, ctypes.c_char_p, _int]),
    "krea_cuda_qw_close": (None, [_vp]),
    "krea_cuda_qw_count": (_int, [_vp]),
    "krea_cuda_qw_info_at": (_int, [_vp, _int, ctypes.POINTER(QwInfo)]),
    "krea_cuda_qw_find": (_int, [_vp, ctypes.c_char_p, ctypes.POINTER(QwInfo)]),
    "krea_cuda_qw_host_ptr": (_vp, [_vp, ctypes.c_uint64]),
    "krea_cuda_qw_meta": (ctypes.c_char_p, [_vp]),
    "krea_cuda_qw_data_bytes": (ctypes.c_uint64, [_vp]),
    "krea_cuda_qw_span": (_int, [_vp, ctypes.c_char_p, ctypes.POINTER(ctypes.c_uint64), ctypes.POINTER(ctypes.c_uint64)]),
    "krea_cuda_qw_upload": (_int, [_vp, _vp, ctypes.c_uint64, ctypes.c_uint64, _vp]),
    "krea_cuda_qw_big_dim": (_int, [_vp, _vp, ctypes.c_float]),
    "krea_cuda_reshard_pack": (_int, [_vp, ctypes.POINTER(ReshardArgs)]),
    "krea_cuda_reshard_unpack": (_int, [_vp, ctypes.POINTER(ReshardArgs)]),
    "krea_cuda_dist_unique_id": (_int, [_vp, ctypes.c_char_p, _int]),
    "krea_cuda_dist_init": (_int, [_vp, _int, _int, _vp]),
    "krea_cuda_dist_exchange_mode": (_int, [_vp]),
    "krea_cuda_dist_rank": (_int, [_vp]),
    "krea_cuda_dist_size": (_int, [_vp]),
    "krea_cuda_dist_sync": (_int, [_vp, _int]),
    "krea_cuda_dist_shutdown": (_int, [_vp]),
    "krea_cuda_reshard_seq_to_heads": (_int, [_vp, ctypes.POINTER(A2AArgs)]),
    "krea_cuda_reshard_heads_to_seq": (_int, [_vp, ctypes.POINTER(A2AArgs)]),
    "krea_cuda_seqpar_joint_attention": (_int, [_vp, ctypes.POINTER(SeqParArgs)]),
}

_lib = None


def library_path() -> str:
    """The in-tree build, unless KREA_CUDA_LIB names another build of the same library (A/B measurements)."""
    return os.environ.get("KREA_CUDA_LIB") or _build.LIB


def load(build_if_missing: bool = True) -> ctypes.CDLL:
    """Load libkrea_cuda.so and declare every prototype.  Raises if the library cannot be found or built."""
    global _lib
    if _lib is not None:
        return _lib
    path = library_path()
    if not os.path.exists(path):
        if not build_if_missing:
            raise FileNotFoundError(f"{path} is missing: run `python -m krea_image_b200.build`")
        _build.build()
    lib = ctypes.CDLL(path)
    for name, (res, args) in SYMBOLS.items():
        fn = getattr(lib, name)   # AttributeError if the library does not export it
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib
