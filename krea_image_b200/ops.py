"""Host-side mirror of the reference's operator API for the attention path.

`KreaCuda` plays the role of the reference's `class Metal` (engine/src/metal.h:46-165) for its two
attention-path methods, with the same names, argument order, units (elements) and layouts:

    Metal::qk_norm_rope(qkv, wq, wk, cos, sin, rows, ld, q_off, n_q, k_off, n_k, eps, mode, big_dim, qbig, kbig)
    Metal::attention(Q, K, V, O, Lq, Lk, heads, ldq, ldk, ldv, ldo, group, causal, q_pos0, G, ldg, QB, KB)

A "Tensor" here is a torch CUDA tensor (or an int device address): only its data pointer crosses the C
ABI; torch supplies device memory and streams, nothing else.  Like the reference, the operators enqueue
work and return; `wait()` is the counterpart of Metal::wait.  Errors raise `KreaCudaError` (the
reference throws std::runtime_error inside and returns -1 + message at its C ABI).
"""
import ctypes

from . import binding as B


class KreaCudaError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"[{code}] {msg}")
        self.code = code


def _ptr(t):
    """Device (or host) address of a tensor-like: torch tensor, numpy array, int, or None."""
    if t is None:
        return None
    if isinstance(t, int):
        return t
    if hasattr(t, "data_ptr"):
        return t.data_ptr()
    if hasattr(t, "ctypes"):
        return t.ctypes.data
    raise TypeError(f"cannot take the address of {type(t)}")


class KreaCuda:
    def __init__(self, device: int = 0):
        self.lib = B.load()
        err = ctypes.create_string_buffer(1024)
        self.h = self.lib.krea_cuda_create(device, err, 1024)
        if not self.h:
            raise KreaCudaError(B.E_CUDA, err.value.decode() or "krea_cuda_create failed")
        self.device = device

    def close(self):
        if getattr(self, "h", None):
            self.lib.krea_cuda_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc):
        if rc != B.OK:
            raise KreaCudaError(rc, self.lib.krea_cuda_last_error(self.h).decode())

    # ---- stream handling --------------------------------------------------------------------------
    def set_stream(self, stream):
        """stream: a torch.cuda.Stream or a raw cudaStream_t address (0 / None = the CUDA default stream)."""
        s = None if stream is None else (getattr(stream, "cuda_stream", stream) or None)
        self._check(self.lib.krea_cuda_set_stream(self.h, s))

    def wait(self):
        """Block until the stream is idle; raises if a kernel reported a timed-out wait."""
        self._check(self.lib.krea_cuda_sync(self.h))

    def set_wait_limit(self, seconds: float):
        """Bound on every wait inside the attention kernel (default 2 s); a wait that runs out makes wait() raise E_DEVICE."""
        self._check(self.lib.krea_cuda_set_wait_limit(self.h, int(seconds * 1e9)))

    def test_drop_one_load(self, on: bool):
        """Test hook: attention launches never request their last K tile, so that a bounded wait runs out."""
        self._check(self.lib.krea_cuda_test_drop_one_load(self.h, int(on)))

    @property
    def launches(self) -> int:
        return int(self.lib.krea_cuda_launch_count(self.h))

    def profile(self, on: bool):
        """Per-kernel GPU timing like the reference's KREA_PROFILE marks (engine/src/metal.h:126-145)."""
        self._check(self.lib.krea_cuda_profile_enable(self.h, int(on)))

    def profile_read(self, which: int):
        """(total device ms, launches) of the prologue (0) or attention (1) kernel since profile(True)."""
        ms, n = ctypes.c_double(0), ctypes.c_int(0)
        self._check(self.lib.krea_cuda_profile_read(self.h, which, ctypes.byref(ms), ctypes.byref(n)))
        return ms.value, n.value

    def profile_trace(self, path):
        """Chrome-trace JSON of the marks recorded since profile(True) (the reference's KREA_TRACE)."""
        self._check(self.lib.krea_cuda_profile_trace(self.h, str(path).encode()))

    # ---- Metal::qk_norm_rope (engine/src/metal.h:80-82) ---------------------------------------------
    def qk_norm_rope(self, qkv, wq, wk, cos, sin, rows, ld, q_off, n_q, k_off, n_k, eps, mode=B.ROPE_PAIRS, big_dim=-1,
                     qbig=None, kbig=None):
        a = B.QKNormArgs(_ptr(qkv), _ptr(wq), _ptr(wk), _ptr(cos), _ptr(sin), rows, ld, q_off, n_q, k_off, n_k, eps,
                         int(mode), big_dim, _ptr(qbig), _ptr(kbig))
        self._check(self.lib.krea_cuda_qk_norm_rope(self.h, ctypes.byref(a)))

    # ---- Metal::attention (engine/src/metal.h:83-88) ------------------------------------------------
    def attention(self, Q, K, V, O, Lq, Lk, heads, ldq, ldk, ldv, ldo, group=1, causal=False, q_pos0=0, G=None, ldg=0,
                  QB=None, KB=None, *, batch=1, bsq=0, bsk=0, bsv=0, bso=0, bsg=0, text_len=None, text_slots=0, q_row0=0):
        a = B.AttnArgs(_ptr(Q), _ptr(K), _ptr(V), _ptr(O), Lq, Lk, heads, ldq, ldk, ldv, ldo, group, int(bool(causal)),
                       q_pos0, _ptr(G), ldg, _ptr(QB), _ptr(KB), batch, bsq, bsk, bsv, bso, bsg, _ptr(text_len),
                       text_slots, q_row0)
        self._check(self.lib.krea_cuda_attention(self.h, ctypes.byref(a)))

    def attention_partial(self, part, Q, K, V, O, Lq, Lk, heads, ldq, ldk, ldv, ldo, So, Sm, Sl, group=1, G=None, ldg=0, QB=None, KB=None):
        """attention_d128_first / _mid / _last (engine/kernels/attention.metal:353-370): part = 0 / 1 / 2; K, V, Lk describe
        one block of keys; So f32 [Lq, heads*128], Sm f32 [Lq, heads], Sl f32 [Lq, heads, 8] carry the loop state."""
        a = B.AttnArgs(_ptr(Q), _ptr(K), _ptr(V), _ptr(O), Lq, Lk, heads, ldq, ldk, ldv, ldo, group, 0, 0, _ptr(G), ldg,
                       _ptr(QB), _ptr(KB), 1, 0, 0, 0, 0, 0, None, 0, 0)
        self._check(self.lib.krea_cuda_attention_partial(self.h, ctypes.byref(a), int(part), _ptr(So), _ptr(Sm), _ptr(Sl)))

    # ---- DiT::qk_rope + DiT::attend in one call (engine/src/model.mm:271-288) -----------------------
    def _joint_args(self, Q, K, V, O, Lq, Lk, heads, ldq, ldk, ldv, ldo, wq, wk, cos, sin, eps, group, rope_mode, q_row0,
                    batch, bsq, bsk, bsv, bso, text_len, text_slots, G, ldg, bsg, k_scratch, k_scratch_bytes):
        return B.JointArgs(_ptr(Q), _ptr(K), _ptr(V), _ptr(O), batch, Lq, Lk, q_row0, heads, group, ldq, ldk, ldv, ldo,
                           bsq, bsk, bsv, bso, _ptr(wq), _ptr(wk), _ptr(cos), _ptr(sin), eps, int(rope_mode),
                           _ptr(text_len), text_slots, _ptr(G), ldg, bsg, _ptr(k_scratch), k_scratch_bytes)

    def joint_attention(self, Q, K, V, O, Lq, Lk, heads, ldq, ldk, ldv, ldo, wq, wk, cos, sin, eps=1e-6, group=1,
                        rope_mode=B.ROPE_PAIRS, q_row0=0, *, batch=1, bsq=0, bsk=0, bsv=0, bso=0, text_len=None,
                        text_slots=0, G=None, ldg=0, bsg=0, k_scratch=None, k_scratch_bytes=0):
        a = self._joint_args(Q, K, V, O, Lq, Lk, heads, ldq, ldk, ldv, ldo, wq, wk, cos, sin, eps, group, rope_mode,
                             q_row0, batch, bsq, bsk, bsv, bso, text_len, text_slots, G, ldg, bsg, k_scratch,
                             k_scratch_bytes)
        self._check(self.lib.krea_cuda_joint_attention(self.h, ctypes.byref(a)))

    def joint_attention_static(self, Q, K, V, O, Lq, Lk, heads, ldq, ldk, ldv, ldo, wq, wk, cos, sin, eps=1e-6, group=1,
                               rope_mode=B.ROPE_PAIRS, q_row0=0, *, batch=1, bsq=0, bsk=0, bsv=0, bso=0, text_len=None,
                               text_slots=0, G=None, ldg=0, bsg=0):
        """joint_attention for callers that may not allocate device memory: the normalised K goes to the
        library's built-in 32 MiB device array (shared by every call on the device - do not overlap calls),
        so problems with batch * Lk * kv_heads * 256 bytes above that size are refused with E_NOMEM."""
        a = self._joint_args(Q, K, V, O, Lq, Lk, heads, ldq, ldk, ldv, ldo, wq, wk, cos, sin, eps, group, rope_mode,
                             q_row0, batch, bsq, bsk, bsv, bso, text_len, text_slots, G, ldg, bsg, None, 0)
        self._check(self.lib.krea_cuda_joint_attention_static(self.h, ctypes.byref(a)))

    def joint_attention_host(self, Q, K, V, O, Lq, Lk, heads, ldq, ldk, ldv, ldo, wq, wk, cos, sin, eps=1e-6, group=1,
                             rope_mode=B.ROPE_PAIRS, q_row0=0, *, batch=1, bsq=0, bsk=0, bsv=0, bso=0, text_len=None,
                             text_slots=0):
        """Every argument lives in host memory (numpy arrays or pinned torch tensors); returns after O is back."""
        a = self._joint_args(Q, K, V, O, Lq, Lk, heads, ldq, ldk, ldv, ldo, wq, wk, cos, sin, eps, group, rope_mode,
                             q_row0, batch, bsq, bsk, bsv, bso, text_len, text_slots, None, 0, 0, None, 0)
        self._check(self.lib.krea_cuda_joint_attention_host(self.h, ctypes.byref(a)))

    def joint_scratch_bytes(self, Lk, heads, group=1, batch=1) -> int:
        a = B.JointArgs()
        a.Lk, a.heads, a.group, a.batch = Lk, heads, group, batch
        return int(self.lib.krea_cuda_joint_scratch_bytes(ctypes.byref(a)))

    def gemm(self, A, W, C, M, N, K, lda, ldw, ldc, *, qk_norm=None, epilogue=B.EPI_BF16, vec=None, lora=None, seg=0, seg_stride=0):
        """Metal::gemm with Epi::BF16 (engine/src/metal.h:64-67): C[M,N] = A[M,K] x Wt[K,N], bf16.
        qk_norm = dict(q_off, n_q, k_off, n_k, wq, wk, cos, sin, row0, eps, rope_mode) fuses Metal::qk_norm_rope
        on those head blocks into the store.  epilogue = B.EPI_RESID_GATE: C is f32 and receives += vec[n] * acc
        (vec None: += acc); B.EPI_SWIGLU: C is bf16 [M, N/2] = silu(gate) * up on tile-interleaved weights."""
        a = B.GemmArgs()
        a.A, a.W, a.C = _ptr(A), _ptr(W), _ptr(C)
        a.M, a.N, a.K, a.lda, a.ldw, a.ldc = M, N, K, lda, ldw, ldc
        a.epilogue, a.vec = epilogue, _ptr(vec)
        a.seg, a.seg_stride = seg, seg_stride
        if lora is not None:      # (A2, W2, K2, lda2, ldw2): acc += A2 x W2 before the epilogue (metal.h:31-35 LoraTerm)
            a.lora_A, a.lora_W, a.lora_K, a.lora_lda, a.lora_ldw = _ptr(lora[0]), _ptr(lora[1]), lora[2], lora[3], lora[4]
        if qk_norm is not None:
            a.epilogue = B.EPI_QKNORM_ROPE
            a.q_off, a.n_q, a.k_off, a.n_k = qk_norm["q_off"], qk_norm["n_q"], qk_norm["k_off"], qk_norm["n_k"]
            a.wq, a.wk = _ptr(qk_norm.get("wq")), _ptr(qk_norm.get("wk"))
            a.cos, a.sin = _ptr(qk_norm.get("cos")), _ptr(qk_norm.get("sin"))
            a.row0, a.eps, a.rope_mode = qk_norm.get("row0", 0), qk_norm.get("eps", 1e-6), qk_norm.get("rope_mode", B.ROPE_PAIRS)
            a.big_dim, a.qbig, a.kbig = qk_norm.get("big_dim", 0), _ptr(qk_norm.get("qbig")), _ptr(qk_norm.get("kbig"))
        self._check(self.lib.krea_cuda_gemm(self.h, ctypes.byref(a)))

    def dequant_q8(self, wq, scales, out, K, N, ldq=None, lds=None, ldo=None):
        """int8 [K, N] + f32 scales [K/128, N] -> bf16 [K, N], bf16(float(q) * s) (gemm.metal:159-170)."""
        a = B.DequantArgs(_ptr(wq), _ptr(scales), _ptr(out), K, N, N if ldq is None else ldq, N if lds is None else lds, N if ldo is None else ldo)
        self._check(self.lib.krea_cuda_dequant_q8(self.h, ctypes.byref(a)))

    def rms_norm(self, x, mul, add, y, rows, width, ld_in, ld_out, eps, f32_out=False):
        """Metal::rms_norm (engine/src/metal.h:75-77): same argument order."""
        a = B.RmsNormArgs(_ptr(x), _ptr(mul), _ptr(add), _ptr(y), rows, width, ld_in, ld_out, eps, int(bool(f32_out)))
        self._check(self.lib.krea_cuda_rms_norm(self.h, ctypes.byref(a)))

    def dit_block(self, x, mods, w_qkvg, w_o, w_gu, w_down, qn, kn, cos, sin, rows, heads, kv_heads, ff, eps=1e-6, workspace=None,
                  big_dim=-1):
        """DiT::layer (engine/src/model.mm:369-385) on the fp32 residual stream x [rows, heads*128], in place."""
        a = B.DitBlockArgs(_ptr(x), _ptr(mods), _ptr(w_qkvg), _ptr(w_o), _ptr(w_gu), _ptr(w_down), _ptr(qn), _ptr(kn),
                           _ptr(cos), _ptr(sin), rows, heads, kv_heads, ff, eps, _ptr(workspace),
                           0 if workspace is None else workspace.numel() * workspace.element_size(),
                           int(big_dim >= 0), max(big_dim, 0))
        self._check(self.lib.krea_cuda_dit_block(self.h, ctypes.byref(a)))

    def layerwise_attn(self, qkvg, out, rows, ld, ldo, heads, q_off, k_off, v_off, g_off):
        """Metal::layerwise_attn (engine/src/metal.h:90-91): same argument order."""
        a = B.LayerwiseArgs(_ptr(qkvg), _ptr(out), rows, ld, ldo, heads, q_off, k_off, v_off, g_off)
        self._check(self.lib.krea_cuda_layerwise_attn(self.h, ctypes.byref(a)))

    # ---- sequence <-> head resharding ---------------------------------------------------------------
    def reshard_pack(self, src, dst, nranks, rows, cols_per_rank, src_ld, src_col0=0):
        a = B.ReshardArgs(_ptr(src), _ptr(dst), nranks, rows, cols_per_rank, src_ld, 0, src_col0, 0)
        self._check(self.lib.krea_cuda_reshard_pack(self.h, ctypes.byref(a)))

    def reshard_unpack(self, src, dst, nranks, rows, cols_per_rank, dst_ld, dst_col0=0):
        a = B.ReshardArgs(_ptr(src), _ptr(dst), nranks, rows, cols_per_rank, 0, dst_ld, 0, dst_col0)
        self._check(self.lib.krea_cuda_reshard_unpack(self.h, ctypes.byref(a)))


    # ---- sequence-parallel execution over NCCL -------------------------------------------------------
    @staticmethod
    def dist_unique_id() -> bytes:
        """128 bytes that rank 0 creates and every rank passes to dist_init."""
        lib = B.load()
        buf = ctypes.create_string_buffer(B.DIST_ID_BYTES)
        err = ctypes.create_string_buffer(512)
        rc = lib.krea_cuda_dist_unique_id(ctypes.cast(buf, ctypes.c_void_p), err, 512)
        if rc:
            raise KreaCudaError(rc, err.value.decode() or "dist_unique_id failed")
        return buf.raw

    def dist_init(self, rank: int, nranks: int, uid: bytes):
        """Collective over the nranks handles (one process and one handle per GPU)."""
        if len(uid) != B.DIST_ID_BYTES:
            raise ValueError(f"the id must be {B.DIST_ID_BYTES} bytes")
        buf = ctypes.create_string_buffer(uid, B.DIST_ID_BYTES)
        self._check(self.lib.krea_cuda_dist_init(self.h, rank, nranks, ctypes.cast(buf, ctypes.c_void_p)))

    def dist_exchange_mode(self) -> str:
        """'p2p' (peer stores over NVLink, NCCL only for barriers), 'nccl' (ncclSend/ncclRecv) or 'none'."""
        return {1: "p2p", 0: "nccl"}.get(int(self.lib.krea_cuda_dist_exchange_mode(self.h)), "none")

    def dist_rank(self) -> int:
        return int(self.lib.krea_cuda_dist_rank(self.h))

    def dist_size(self) -> int:
        return int(self.lib.krea_cuda_dist_size(self.h))

    def dist_sync(self, timeout_ms: int = 0):
        self._check(self.lib.krea_cuda_dist_sync(self.h, timeout_ms))

    def dist_shutdown(self):
        self._check(self.lib.krea_cuda_dist_shutdown(self.h))

    def reshard_seq_to_heads(self, src, dst, rows_local, cols_per_rank, src_ld, src_col0=0):
        a = B.A2AArgs(_ptr(src), _ptr(dst), rows_local, cols_per_rank, src_ld, 0, src_col0, 0)
        self._check(self.lib.krea_cuda_reshard_seq_to_heads(self.h, ctypes.byref(a)))

    def reshard_heads_to_seq(self, src, dst, rows_local, cols_per_rank, dst_ld, dst_col0=0):
        a = B.A2AArgs(_ptr(src), _ptr(dst), rows_local, cols_per_rank, 0, dst_ld, 0, dst_col0)
        self._check(self.lib.krea_cuda_reshard_heads_to_seq(self.h, ctypes.byref(a)))

    def seqpar_joint_attention(self, Q, K, V, O, seq, heads, ldq, ldk, ldv, ldo, wq, wk, cos, sin, eps=1e-6, group=1,
                               rope_mode=B.ROPE_PAIRS):
        """Q, K, V, O: this rank's rows [seq / nranks] of every head; cos/sin: the global tables."""
        a = B.SeqParArgs(_ptr(Q), _ptr(K), _ptr(V), _ptr(O), seq, heads, group, ldq, ldk, ldv, ldo,
                         _ptr(wq), _ptr(wk), _ptr(cos), _ptr(sin), eps, rope_mode)
        self._check(self.lib.krea_cuda_seqpar_joint_attention(self.h, ctypes.byref(a)))


def rope_tables_ref3axis(T, gh, gw):
    """DiT::set_grid (engine/src/model.mm:290-315): numpy f32 cos/sin [T + gh*gw, 64] built by the library."""
    import numpy as np
    lib = B.load()
    c = np.empty((T + gh * gw, 64), dtype=np.float32)
    s = np.empty_like(c)
    rc = lib.krea_cuda_rope_tables_ref3axis(c.ctypes.data, s.ctypes.data, T, gh, gw)
    if rc:
        raise KreaCudaError(rc, "rope_tables_ref3axis: bad arguments")
    return c, s


def rope_tables_axial2d(T, gh, gw, theta=10000.0):
    import numpy as np
    lib = B.load()
    c = np.empty((T + gh * gw, 64), dtype=np.float32)
    s = np.empty_like(c)
    rc = lib.krea_cuda_rope_tables_axial2d(c.ctypes.data, s.ctypes.data, T, gh, gw, theta)
    if rc:
        raise KreaCudaError(rc, "rope_tables_axial2d: bad arguments")
    return c, s
