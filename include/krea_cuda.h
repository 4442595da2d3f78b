/*
 * libkrea_cuda - C ABI of the B200 (sm_100a) implementation of the Krea 2 Turbo DiT joint text+image
 * attention path: per-head QK-RMSNorm + RoPE prologue and flash attention with head_dim 128.
 *
 * The two operator entry points take the same arguments, in the same units (elements, not bytes) and
 * with the same row layouts as the reference engine's operator API, so a caller of
 *     Metal::qk_norm_rope   (engine/src/metal.h:80-82,  engine/src/metal.mm:182-191)
 *     Metal::attention      (engine/src/metal.h:83-88,  engine/src/metal.mm:193-202)
 * can switch to them by replacing its buffers with CUDA device pointers.  Conventions follow the
 * reference's only C ABI (engine/src/krea.h): opaque handle, plain structs, `char* err, int errlen`
 * at creation, integer status returns, no exceptions across the boundary.
 *
 * Execution model: every call validates its arguments on the host, then enqueues kernels on the
 * handle's CUDA stream and returns without synchronising (the reference's operators likewise only
 * encode into the current command buffer, engine/src/metal.mm:130-135).  One caller per handle at a
 * time, like the reference (ui/krea.py:140,223 holds a lock around each engine call).  There is no CPU
 * fallback: without a CUDA device krea_cuda_create fails.
 *
 * Pointer alignment: every tensor pointer and every row start must be 16-byte aligned (ld, column
 * offsets and batch strides multiples of 8 bf16 elements) - the reference's kernels make the same
 * assumption with their 16-byte vector loads (engine/kernels/attention.metal:102).
 */
#ifndef KREA_CUDA_H
#define KREA_CUDA_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define KREA_CUDA_API __attribute__((visibility("default")))
#else
#define KREA_CUDA_API
#endif

typedef struct krea_cuda krea_cuda;

/* Status codes.  0 = ok, negative = error (the reference's C ABI returns -1 on error, krea.h:66-69). */
enum {
  KREA_CUDA_OK = 0,
  KREA_CUDA_E_ARG = -1,         /* invalid argument; nothing was launched */
  KREA_CUDA_E_UNSUPPORTED = -2, /* valid in the reference's API but not built here; nothing was launched */
  KREA_CUDA_E_CUDA = -3,        /* a CUDA runtime / driver call failed */
  KREA_CUDA_E_DEVICE = -4,      /* a kernel gave up on a bounded wait and reported it (see krea_cuda_sync) */
  KREA_CUDA_E_NOMEM = -5,       /* workspace allocation failed or caller-provided scratch too small */
  KREA_CUDA_E_COMM = -6,        /* NCCL could not be loaded, or a communicator call failed */
  KREA_CUDA_E_TIMEOUT = -7      /* krea_cuda_dist_sync gave up waiting and aborted the communicator */
};

/* RoPE modes of qk_norm_rope: enum RopeMode, engine/src/metal.h:44; engine/kernels/norm.metal:64-66. */
enum { KREA_CUDA_ROPE_PAIRS = 0, KREA_CUDA_ROPE_HALF = 1, KREA_CUDA_ROPE_NONE = 2 };

/* ---- lifetime (pattern of krea_create / krea_destroy, engine/src/krea.h:54-55) ---- */
KREA_CUDA_API krea_cuda* krea_cuda_create(int device, char* err, int errlen);
KREA_CUDA_API void krea_cuda_destroy(krea_cuda* h);
/* Message of the last failing call on this handle ("" if none). */
KREA_CUDA_API const char* krea_cuda_last_error(krea_cuda* h);
/* Enqueue on the caller's cudaStream_t from now on (NULL = the CUDA default stream).  A new handle
 * starts on a private non-blocking stream of its own.  Changing the stream first waits for the work the
 * handle queued on the previous one (its workspaces belong to one stream at a time). */
KREA_CUDA_API int krea_cuda_set_stream(krea_cuda* h, void* cuda_stream);
/* Wait for the stream (the counterpart of Metal::wait, engine/src/metal.h:57-58) and return
 * KREA_CUDA_E_DEVICE if any kernel since the last sync reported a timed-out wait. */
KREA_CUDA_API int krea_cuda_sync(krea_cuda* h);
/* Number of kernels this handle has launched so far. */
KREA_CUDA_API uint64_t krea_cuda_launch_count(krea_cuda* h);
/* Every wait inside the attention kernel (on a TMA load, a tensor-core product, another warp) gives up after
 * this much device time, records where in a status word and lets the CTA run to its normal exit; krea_cuda_sync
 * then returns KREA_CUDA_E_DEVICE.  Default 2 s; accepted range 1 ms .. 60 s.  No counterpart in the reference
 * (Metal command buffers are bounded by the system's GPU watchdog instead). */
KREA_CUDA_API int krea_cuda_set_wait_limit(krea_cuda* h, uint64_t nanoseconds);
/* Test hook for that path: while on, the attention kernel's producer never requests the last K tile of a CTA,
 * so the wait for it runs out after the limit above.  Nothing faults and nothing waits longer than the limit;
 * the output of such a launch is meaningless.  Use with a limit of a few milliseconds. */
KREA_CUDA_API int krea_cuda_test_drop_one_load(krea_cuda* h, int on);
/* Per-operator GPU timing, the counterpart of the reference's KREA_PROFILE marks (Metal::mark,
 * engine/src/metal.h:126-145): while enabled, every kernel launch is bracketed by CUDA events on the
 * stream.  krea_cuda_profile_read synchronises the stream and returns the accumulated device time and
 * launch count of the prologue kernel (which = 0), the attention kernel (which = 1), the exchange
 * kernels and copies of the sequence-parallel step (which = 2) or its rank barriers (which = 3) since the
 * last krea_cuda_profile_enable(h, 1), then clears them. */
KREA_CUDA_API int krea_cuda_profile_enable(krea_cuda* h, int on);
KREA_CUDA_API int krea_cuda_profile_read(krea_cuda* h, int which, double* total_ms, int* launches);
/* The reference's KREA_TRACE=path (engine/src/metal.mm:284-294): writes the marks recorded since the last
 * krea_cuda_profile_enable(h, 1) - not yet consumed by krea_cuda_profile_read - as Chrome-trace JSON (one
 * complete event per bracketed launch, microseconds since the enable call), for chrome://tracing / Perfetto. */
KREA_CUDA_API int krea_cuda_profile_trace(krea_cuda* h, const char* path);

/* ---- Metal::qk_norm_rope (engine/src/metal.h:80-82; kernel engine/kernels/norm.metal:81-134) ----
 * In place on bf16 rows [rows, ld]: for every row and head, x <- bf16(rope(x * rsqrt(mean(x^2) + eps) * w)).
 * q heads at column q_off + h*128 (n_q of them, weight wq), k heads at k_off + h*128 (n_k, weight wk);
 * n_q or n_k may be 0.  cos/sin: f32 [rows, 64] per-row tables (ignored for KREA_CUDA_ROPE_NONE).
 * big_dim >= 0: that channel's value goes to qbig [rows, n_q] / kbig [rows, n_k] (fp32) and is stored as 0. */
typedef struct {
  void* qkv;
  const float* wq;
  const float* wk;
  const float* cos;
  const float* sin;
  int rows, ld;
  int q_off, n_q;
  int k_off, n_k;
  float eps;
  int rope_mode;
  int big_dim; /* -1 = none */
  float* qbig;
  float* kbig;
} krea_cuda_qknorm_args;
KREA_CUDA_API int krea_cuda_qk_norm_rope(krea_cuda* h, const krea_cuda_qknorm_args* a);

/* ---- Metal::attention (engine/src/metal.h:83-88; kernel engine/kernels/attention.metal:131-351) ----
 * O[q, h*128 + d] = sum_k softmax_k(Q[q,h] . K[k,h/group] / sqrt(128)) V[k, h/group, d]  (x sigmoid(G) if G).
 * Q [Lq, ldq], K [Lk, ldk], V [Lk, ldv], O [Lq, ldo], G [Lq, ldg]: bf16, head h at column h*128 (K/V: (h/group)*128).
 * Operands are used as they are (Q and K already normalised and rotated).  fp32 scores, softmax and
 * accumulation; P is rounded to bf16 for the PV product, the row sum stays fp32; a row without any
 * visible key gives zeros.  QB [Lq, heads] / KB [Lk, heads/group]: optional fp32 rank-1 score term.
 * Extensions beyond the reference (all-zero = reference behaviour): a batch dimension with per-tensor
 * batch strides, and a text key-padding mask (see krea_cuda_joint_args). */
typedef struct {
  const void* Q;
  const void* K;
  const void* V;
  void* O;
  int Lq, Lk, heads;
  int ldq, ldk, ldv, ldo;
  int group;
  int causal;
  int q_pos0;
  const void* G;
  int ldg;
  const float* QB;
  const float* KB;
  /* extensions */
  int batch;                  /* 0 or 1 = single sample */
  int64_t bsq, bsk, bsv, bso, bsg; /* batch strides in elements */
  const int32_t* text_len;    /* device pointer, int32 [batch], or NULL */
  int text_slots;
  int q_row0;                 /* sequence position of query row 0 (for the padding test of query rows) */
} krea_cuda_attn_args;
KREA_CUDA_API int krea_cuda_attention(krea_cuda* h, const krea_cuda_attn_args* a);

/* Split-K forms of krea_cuda_attention: the reference's attention_d128_first / _mid / _last
 * (engine/kernels/attention.metal:14-19, 353-370; state at :164-179 and :288-306).  The same loop over ONE block
 * of keys (K, V and Lk describe the block), with the loop state carried between calls in fp32:
 *   So [Lq][heads*128] un-normalised output, Sm [Lq][heads] running max (log2 units),
 *   Sl [Lq][heads][8] partial row sums (their sum is the row sum; this library keeps it in the first of the eight).
 * FIRST starts from the empty state and stores it, MID loads and stores, LAST loads and writes the normalised
 * bf16 output (with the gate, if any) like krea_cuda_attention.  Non-causal, one sample, no padding mask.  When
 * every block but the last holds a multiple of 128 keys the result is bit-identical to one call over all keys.
 * Q must be the same rows in every call; O (and G) are only used by LAST. */
#define KREA_CUDA_PART_FIRST 0
#define KREA_CUDA_PART_MID 1
#define KREA_CUDA_PART_LAST 2
KREA_CUDA_API int krea_cuda_attention_partial(krea_cuda* h, const krea_cuda_attn_args* a, int part, float* So, float* Sm, float* Sl);

/* ---- The whole path in one call: DiT::qk_rope + DiT::attend (engine/src/model.mm:271-288) ----
 * Q, K, V are the raw projections (e.g. column blocks of one fused q|k|v row buffer).  Neither input is
 * modified: Q is normalised and rotated inside the attention kernel as it is staged; K is normalised
 * and rotated once into scratch memory by a pre-pass.  Query row i sits at sequence position
 * q_row0 + i (the reference's row0, model.mm:271-288); key row j at position j; cos/sin: f32 [>= max(q_row0+Lq, Lk), 64].
 * text_len (device, int32 [batch]) with text_slots > 0: keys at positions [text_len[b], text_slots) are
 * padding and contribute nothing; query rows at those positions are written as zeros.
 * k_scratch: caller-owned device scratch of k_scratch_bytes >= krea_cuda_joint_scratch_bytes(a), or
 * NULL to let the handle allocate (and keep, growing on demand) its own. */
typedef struct {
  const void* Q;
  const void* K;
  const void* V;
  void* O;
  int batch;
  int Lq, Lk, q_row0;
  int heads, group;
  int ldq, ldk, ldv, ldo;
  int64_t bsq, bsk, bsv, bso;
  const float* wq;
  const float* wk;
  const float* cos;
  const float* sin;
  float eps;
  int rope_mode;
  const int32_t* text_len;
  int text_slots;
  const void* G;
  int ldg;
  int64_t bsg;
  void* k_scratch;
  size_t k_scratch_bytes;
} krea_cuda_joint_args;
KREA_CUDA_API size_t krea_cuda_joint_scratch_bytes(const krea_cuda_joint_args* a);
KREA_CUDA_API int krea_cuda_joint_attention(krea_cuda* h, const krea_cuda_joint_args* a);

/* The fused call for callers that cannot allocate device memory.  No counterpart in the reference (its
 * operators never allocate either, but they also need no scratch: the reference normalises K in place).
 * Who needs it: code that runs after all device memory has been handed to another owner (a framework's
 * caching allocator, a fixed-partition inference server), code on a latency-critical path where
 * cudaMalloc's implicit device-wide synchronisation is not acceptable, and hosts whose rules forbid
 * allocation after start-up.  Those callers cannot give krea_cuda_joint_attention a k_scratch of their own
 * and must not let the handle grow one.
 * Same arguments and results as krea_cuda_joint_attention (k_scratch / k_scratch_bytes are ignored), but the
 * normalised K goes to a fixed KREA_CUDA_STATIC_SCRATCH_BYTES array that is part of the library's device
 * image: every GPU on which the library is used keeps those 32 MiB reserved until the process exits.
 *  - Limit: batch * Lk * (heads/group) * 256 bytes must fit in the array (e.g. one sample of 24 heads x
 *    5461 keys); larger problems return KREA_CUDA_E_NOMEM with a message and launch nothing.
 *  - The call performs no cudaMalloc / cudaFree and calls no allocating library routine, and it does no
 *    per-device set-up either: krea_cuda_create looks up the array's device address (cudaGetSymbolAddress,
 *    with the handle's device current - this is the moment the CUDA runtime loads the library's device image
 *    and the driver sets the 32 MiB aside), loads the two kernels' code and opts the attention kernel in to
 *    its shared memory (cudaFuncSetAttribute).  So create the handle at start-up, while device memory is
 *    still to be had and before any stream capture begins; krea_cuda_create fails if that set-up fails.
 *  - All calls, from every handle on the same device, share the one array: it keeps the previous call's
 *    contents (nothing needs clearing - each call overwrites what it reads), and two calls whose kernels
 *    can overlap on the GPU (different streams without ordering) race on it.  Serialise them. */
#define KREA_CUDA_STATIC_SCRATCH_BYTES (32u << 20)
KREA_CUDA_API int krea_cuda_joint_attention_static(krea_cuda* h, const krea_cuda_joint_args* a);

/* Same call with every pointer in HOST memory (the reference's Tensor is CPU-visible unified memory,
 * engine/src/metal.h:14-23): copies the operands to device buffers owned by the handle, runs
 * krea_cuda_joint_attention, copies O back and synchronises.  Pinned host memory makes the copies
 * asynchronous DMA; pageable memory works too.  k_scratch is ignored. */
KREA_CUDA_API int krea_cuda_joint_attention_host(krea_cuda* h, const krea_cuda_joint_args* a);

/* ---- RoPE tables, built on the host like DiT::set_grid (engine/src/model.mm:290-315) ----
 * cos/sin: host f32 [T + gh*gw, 64]; text rows (the first T) sit at position 0.
 * ref3axis: the reference model's split (pairs 0-15 frame = 0, 16-39 grid row, 40-63 grid column, theta 1000).
 * axial2d: two axes of 32 pairs (row, then column), frequency k = theta^(-2k/64). */
KREA_CUDA_API int krea_cuda_rope_tables_ref3axis(float* cos, float* sin, int T, int gh, int gw);
KREA_CUDA_API int krea_cuda_rope_tables_axial2d(float* cos, float* sin, int T, int gh, int gw, double theta);

/* ---- Metal::layerwise_attn (engine/src/metal.h:90-91, metal.mm:204-209; kernel norm.metal:136-178) ----
 * The text fusion's attention across the 12 tapped encoder states of each token.  Rows are token-major
 * (row = t*12 + j) in a fused bf16 [q | k | v | gate] buffer with `ld` columns, heads of 128 channels at
 * the four column offsets; out[row, h*128 + d] = softmax_j(q[row] . k[base+j] / sqrt(128)) v[base+j] *
 * sigmoid(gate[row]), fp32 inside, bf16 store.  Same argument order and units as the reference's method;
 * rows must be a multiple of 12 (the reference would read past the buffer otherwise). */
typedef struct {
  const void* qkvg;
  void* out;
  int rows, ld, ldo, heads;
  int q_off, k_off, v_off, g_off;
} krea_cuda_layerwise_args;
KREA_CUDA_API int krea_cuda_layerwise_attn(krea_cuda* h, const krea_cuda_layerwise_args* a);

/* ---- Metal::gemm, bf16 weights, EPI_BF16 (engine/src/metal.h:64-67; kernels/gemm.metal:29-30, 251-279) ----
 * C[M, N] (bf16, row stride ldc) = A[M, K] (bf16, row stride lda) x Wt[K, N] (bf16, row stride ldw): the
 * reference's operand layouts, weights "input-major" as tools/convert.py lays them out.  This is the
 * projection either side of the attention (the fused q|k|v|gate product, engine/src/model.mm:349-359).
 * KREA_CUDA_EPI_QKNORM_ROPE additionally applies Metal::qk_norm_rope (norm.metal:81-134) to the n_q head
 * blocks of 128 output columns starting at q_off and the n_k blocks starting at k_off before the store, so
 * the projection writes Q and K already normalised and rotated (rope_mode 0 or 2; cos/sin row = row0 + output
 * row); the attention is then called through krea_cuda_attention on the result.
 * KREA_CUDA_EPI_RESID_GATE / _SWIGLU are the epilogues of the O-projection and of the MLP (model.mm:357-366).
 * int8 weights (Weight::q8) are dequantised once with krea_cuda_dequant_q8 and then used as bf16.  Every
 * epilogue, the LoRA term and the column remap of the reference's kernel have a field here.  Pointers 16-byte aligned; lda, ldw, ldc, N, q_off and
 * k_off multiples of 8 (q_off, k_off of 128 with the fused epilogue). */
#define KREA_CUDA_EPI_BF16 0
#define KREA_CUDA_EPI_QKNORM_ROPE 1
#define KREA_CUDA_EPI_RESID_GATE 2 /* C is f32 [M, N]: C += vec[n] * acc (gemm.metal:262-264); vec NULL: C += acc (Epi::Resid) */
#define KREA_CUDA_EPI_SWIGLU 3     /* C is bf16 [M, N/2]: silu(gate) * up on tile-interleaved weights (gemm.metal:233-250); N % 64 == 0 */
#define KREA_CUDA_EPI_F32 4        /* C is f32: C = acc (Epi::F32) */
#define KREA_CUDA_EPI_GELU 5       /* C is bf16: gelu_tanh(acc) (Epi::GELU, common.h:26-29) */
#define KREA_CUDA_EPI_BIAS_BF16 6  /* C is bf16: acc + vec[n] (Epi::BiasBF16) */
#define KREA_CUDA_EPI_BIAS_F32 7   /* C is f32: acc + vec[n] (Epi::BiasF32) */
typedef struct {
  const void* A;
  const void* W;
  void* C;
  int M, N, K;
  int lda, ldw, ldc;
  int epilogue;
  int q_off, n_q, k_off, n_k;
  const float* wq;
  const float* wk;
  const float* cos;
  const float* sin;
  int row0;
  float eps;
  int rope_mode;
  const float* vec;   /* RESID_GATE: per-column gate; BIAS_*: per-column bias; f32 [N] (the reference's `vec` argument) */
  /* QKNORM_ROPE, optional (qk_norm_rope's big_dim, norm.metal:127-132): when qbig and kbig are given, head
   * dimension big_dim of every Q / K head is written to qbig [M, n_q] / kbig [M, n_k] in fp32 and stored as
   * zero in C, for the attention's QB / KB term.  NULL = off (big_dim ignored). */
  int big_dim;
  float* qbig;
  float* kbig;
  /* optional second product accumulated before the epilogue (the reference's LoraTerm, engine/src/metal.h:31-35,
   * gemm.metal:46-50): acc += lora_A[M, lora_K] x lora_W[lora_K, N], both bf16; NULL = none.  lora_K, lora_lda and
   * lora_ldw multiples of 8. */
  const void* lora_A;
  const void* lora_W;
  int lora_K, lora_lda, lora_ldw;
  /* EPI_BF16 only, optional column remap (GemmParams::seg, gemm.metal:41-43): output column n is stored at column
   * (n / seg) * seg_stride + n % seg; seg and seg_stride multiples of 8, 0 = off.  ldc must cover the last segment. */
  int seg, seg_stride;
} krea_cuda_gemm_args;
KREA_CUDA_API int krea_cuda_gemm(krea_cuda* h, const krea_cuda_gemm_args* a);

/* ---- int8 weights (the reference's Weight::q8, engine/src/metal.h:25-29) ----
 * Wq int8 [K, N] with f32 scales [K / 128, N] (tools/convert.py:92-99) -> bf16 [K, N], every value
 * bf16(float(q) * s) exactly as the reference's GEMM dequantises it on the fly (gemm.metal:159-170).  Done once
 * per matrix at load time; krea_cuda_gemm then runs on the bf16 copy.  K a multiple of 128 (metal.mm:151), N of
 * 16; leading dimensions in elements; pointers 16-byte aligned. */
typedef struct {
  const void* wq;
  const float* scales;
  void* out;
  int K, N;
  int ldq, lds, ldo;
} krea_cuda_dequant_args;
KREA_CUDA_API int krea_cuda_dequant_q8(krea_cuda* h, const krea_cuda_dequant_args* a);

/* ---- Metal::rms_norm (engine/src/metal.h:75-77; kernel norm.metal:28-55) ----
 * y[row, c] = x[row, c] * rsqrt(mean_c(x[row]^2) + eps) * mul[c] (+ add[c]); x f32 [rows, ld_in], y bf16 (or f32
 * when f32_out) [rows, ld_out]; width, ld_in, ld_out multiples of 4 (8 for bf16 output); add may be NULL. */
typedef struct {
  const float* x;
  const float* mul;
  const float* add;
  void* y;
  int rows, width, ld_in, ld_out;
  float eps;
  int f32_out;
} krea_cuda_rmsnorm_args;
KREA_CUDA_API int krea_cuda_rms_norm(krea_cuda* h, const krea_cuda_rmsnorm_args* a);

/* ---- one DiT block, DiT::layer (engine/src/model.mm:369-385) ----
 * x (the fp32 residual stream [rows, dim], dim = heads * 128) is updated in place:
 *   h = rms_norm(x, mul1, add1);  q|k|v|gate = h Wqkvg with per-head QK-norm + RoPE on q and k;
 *   ao = attention(q, k, v) * sigmoid(gate);  x += gate1 * (ao Wo);
 *   h = rms_norm(x, mul2, add2);  mid = swiglu(h Wgu);  x += gate2 * (mid Wdown).
 * mods: the six modulation vectors of `dim` floats in that order (mul1, add1, gate1, mul2, add2, gate2), as
 * the reference lays them out per layer (model.mm:371-372).  Weights are bf16, input-major ([K, N]), Wgu with
 * gate / up columns interleaved in groups of 32 (tools/convert.py); column layout of the fused projection:
 * q [heads*128] | k [kv_heads*128] | v [kv_heads*128] | gate [heads*128] (model.mm:282-288).  The rows are
 * [text ; image] tokens; cos / sin are their [rows, 64] tables.  Seven kernels: two norms, four GEMMs (the
 * first with the fused QK-norm epilogue) and the attention.  Not handled here: int8 weights, the GPU/ANE
 * hybrid schedule.
 * Workspace: krea_cuda_dit_block_workspace_bytes; pass a buffer or let the handle own one. */
typedef struct {
  float* x;
  const float* mods;
  const void* w_qkvg;
  const void* w_o;
  const void* w_gu;
  const void* w_down;
  const float* qn;
  const float* kn;
  const float* cos;
  const float* sin;
  int rows, heads, kv_heads, ff;
  float eps;
  void* workspace;
  size_t workspace_bytes;
  /* the reference's block 0 (model.mm:226-239): use_big_dim != 0 routes head dimension big_dim of q and k
   * through fp32 side buffers (in the workspace) and the attention's QB / KB term */
  int use_big_dim;
  int big_dim;
} krea_cuda_dit_block_args;
KREA_CUDA_API size_t krea_cuda_dit_block_workspace_bytes(const krea_cuda_dit_block_args* a);
KREA_CUDA_API int krea_cuda_dit_block(krea_cuda* h, const krea_cuda_dit_block_args* a);

/* ---- `.qw` weight files (the reference's WeightFile, engine/src/weights.h:26-75, weights.mm:16-81; format
 * written by tools/convert.py:49-89) ----
 * The on-disk format that supplies the path's QK-norm weights `L<l>.qn` / `L<l>.kn` (f32[128]):
 * "QWTS", u32 version, u64 header length, JSON header {"tensors": {name: {dtype, shape, offset, nbytes}},
 * "meta": {...}}, data section at the next multiple of 16 KiB.  dtype is one of "bf16", "f16", "f32", "i8".
 * The file is mapped read-only; queries need no GPU.  krea_cuda_qw_upload copies a byte range of the data
 * section to device memory on the handle's stream (staged through pinned memory) and returns when the
 * bytes are on the device.  Strings returned here live as long as the file object. */
typedef struct krea_qw krea_qw;
typedef struct {
  const char* name;
  const char* dtype;
  int rank;
  int64_t shape[8];
  uint64_t offset;   /* relative to the data section (TensorInfo::offset) */
  uint64_t nbytes;
} krea_cuda_qw_info;
KREA_CUDA_API krea_qw* krea_cuda_qw_open(const char* path, char* err, int errlen);   /* WeightFile::WeightFile */
KREA_CUDA_API void krea_cuda_qw_close(krea_qw* q);
KREA_CUDA_API int krea_cuda_qw_count(const krea_qw* q);
KREA_CUDA_API int krea_cuda_qw_info_at(const krea_qw* q, int index, krea_cuda_qw_info* out);       /* sorted by name */
KREA_CUDA_API int krea_cuda_qw_find(const krea_qw* q, const char* name, krea_cuda_qw_info* out);   /* WeightFile::info / has */
KREA_CUDA_API const void* krea_cuda_qw_host_ptr(const krea_qw* q, uint64_t offset);                /* WeightFile::host_ptr */
KREA_CUDA_API const char* krea_cuda_qw_meta(const krea_qw* q);                                     /* WeightFile::meta_json */
KREA_CUDA_API uint64_t krea_cuda_qw_data_bytes(const krea_qw* q);
KREA_CUDA_API int krea_cuda_qw_span(const krea_qw* q, const char* prefix, uint64_t* off, uint64_t* len); /* WeightFile::span */
KREA_CUDA_API int krea_cuda_qw_upload(krea_cuda* h, const krea_qw* q, uint64_t off, uint64_t len, void* dst_device);
/* The head dimension whose |qn[d]*kn[d]| is the largest one above gain_threshold (the reference uses 256), or
 * -1: the dimension DiT::DiT routes through the fp32 side buffers (engine/src/model.mm:226-239). */
KREA_CUDA_API int krea_cuda_qw_big_dim(const float* qn, const float* kn, float gain_threshold);

/* ---- sequence-parallel resharding helpers (no counterpart in the reference, which is single-device) ----
 * Pack / unpack kernels either side of an all-to-all that turns sequence-sharded rows (all heads, rows
 * [r*S/P, (r+1)*S/P)) into head-sharded rows (all S rows, heads [r*H/P, (r+1)*H/P)) and back.
 *   pack:   dst[peer][row][c] = src[row][src_col0 + peer*cols_per_rank + c]     (one block per destination)
 *   unpack: dst[row][dst_col0 + peer*cols_per_rank + c] = src[peer][row][c]     (the inverse)
 * Forward: pack the local rows by destination head block, all-to-all; the received blocks, in peer
 * order, already are the S rows of the local heads.  Backward: send the output rows as they are
 * (row blocks are contiguous), all-to-all, unpack merges the per-peer head blocks into full rows.
 * bf16 elements; cols_per_rank, the leading dimensions and column offsets are multiples of 8. */
typedef struct {
  const void* src;
  void* dst;
  int nranks;
  int rows;          /* rows held locally */
  int cols_per_rank; /* bf16 elements per row per peer */
  int src_ld, dst_ld;
  int src_col0, dst_col0;
} krea_cuda_reshard_args;
KREA_CUDA_API int krea_cuda_reshard_pack(krea_cuda* h, const krea_cuda_reshard_args* a);
KREA_CUDA_API int krea_cuda_reshard_unpack(krea_cuda* h, const krea_cuda_reshard_args* a);

/* ---- sequence-parallel execution over NCCL (no counterpart in the reference, which is single-device) ----
 * One process and one handle per GPU.  The library loads NCCL at run time (dlopen of "libnccl.so.2", or of
 * the path in the environment variable KREA_CUDA_NCCL_LIB), so nothing here is needed to use the
 * single-GPU entry points.  Rank 0 obtains an id with krea_cuda_dist_unique_id and hands the 128 bytes to
 * every rank by whatever means the host program has (a file, a socket, MPI, torch.distributed);
 * krea_cuda_dist_init is collective over the nranks handles.  Everything is enqueued on the handle's
 * stream; remote rows always land in local memory (through NCCL, or through the sending rank's own stores in
 * peer-store mode) before a kernel of this library reads them.
 *
 * Layout: with S rows and H heads over P ranks (S and H multiples of P), rank r starts with rows
 * [r*S/P, (r+1)*S/P) of every head ("sequence-sharded") and the exchange gives it every row of heads
 * [r*H/P, (r+1)*H/P) ("head-sharded"), where the single-GPU kernel runs unchanged - the RoPE position
 * of a row depends only on its global index, so the prologue runs after the exchange with the global
 * tables. */
#define KREA_CUDA_DIST_ID_BYTES 128
KREA_CUDA_API int krea_cuda_dist_unique_id(void* id_out /* KREA_CUDA_DIST_ID_BYTES */, char* err, int errlen);
KREA_CUDA_API int krea_cuda_dist_init(krea_cuda* h, int rank, int nranks, const void* id);
/* How krea_cuda_seqpar_joint_attention moves rows between ranks: 1 = peer stores (every rank's workspace is
 * mapped into every process with CUDA IPC; the pack kernels and the attention epilogue store straight into
 * the destination GPU's memory over NVLink and NCCL only provides the barriers in between), 0 = NCCL
 * transfers (ncclSend/ncclRecv between staging buffers), -1 = no communicator.  Peer stores are the
 * default for 2 to 8 ranks; set the environment variable KREA_CUDA_SEQPAR_EXCHANGE=nccl (identically on
 * every rank) to force NCCL transfers, which are also used when a mapping cannot be made. */
KREA_CUDA_API int krea_cuda_dist_exchange_mode(krea_cuda* h);
KREA_CUDA_API int krea_cuda_dist_rank(krea_cuda* h);    /* -1 before krea_cuda_dist_init */
KREA_CUDA_API int krea_cuda_dist_size(krea_cuda* h);    /* 0 before krea_cuda_dist_init */
/* Waits for the handle's stream for at most timeout_ms (<= 0: no limit), polling the communicator for
 * asynchronous errors.  On an error or a timeout the communicator is aborted, so that no collective is
 * left waiting for a peer that will not come, and KREA_CUDA_E_COMM / KREA_CUDA_E_TIMEOUT is returned;
 * the handle then accepts single-GPU calls only, until krea_cuda_dist_init is called again. */
KREA_CUDA_API int krea_cuda_dist_sync(krea_cuda* h, int timeout_ms);
KREA_CUDA_API int krea_cuda_dist_shutdown(krea_cuda* h); /* collective; also done by krea_cuda_destroy */

typedef struct {
  const void* src;   /* seq_to_heads: local rows [rows_local][src_ld]; heads_to_seq: [nranks*rows_local][cols_per_rank] */
  void* dst;         /* seq_to_heads: [nranks*rows_local][cols_per_rank] contiguous; heads_to_seq: local rows [rows_local][dst_ld] */
  int rows_local;    /* S / nranks */
  int cols_per_rank; /* (H / nranks) * 128 */
  int src_ld, dst_ld;     /* leading dimension of the sequence-sharded side (the other side is contiguous) */
  int src_col0, dst_col0; /* first column of the head block on the sequence-sharded side */
} krea_cuda_a2a_args;
/* dst[p*rows_local + i][c] = (rank p's src)[i][src_col0 + rank*cols_per_rank + c] */
KREA_CUDA_API int krea_cuda_reshard_seq_to_heads(krea_cuda* h, const krea_cuda_a2a_args* a);
/* dst[i][dst_col0 + p*cols_per_rank + c] = (rank p's src)[rank*rows_local + i][c] */
KREA_CUDA_API int krea_cuda_reshard_heads_to_seq(krea_cuda* h, const krea_cuda_a2a_args* a);

/* The fused call on sequence-sharded rows: Q, K and V rows travel to the ranks that own their heads, the
 * joint attention runs on the local heads, and the output rows travel home.  With peer stores the
 * attention kernel's epilogue itself writes every output row into its home rank's memory; with NCCL
 * transfers K travels first, so that its normalisation pass overlaps the exchange of V and Q on a second
 * stream.  Q, K, V: local rows [rows_local][ld*] holding all `heads` (K, V:
 * heads/group) heads; O: local rows [rows_local][ldo], all heads.  cos/sin: the global tables
 * [seq][64].  batch, the padding mask and the gate are not supported here.  Workspace (about six
 * times seq * heads/nranks * 256 bytes) is owned by the handle and grown on demand. */
typedef struct {
  const void* Q; const void* K; const void* V; void* O;
  int seq, heads, group;
  int ldq, ldk, ldv, ldo;
  const float* wq; const float* wk; const float* cos; const float* sin;
  float eps;
  int rope_mode;
} krea_cuda_seqpar_args;
KREA_CUDA_API int krea_cuda_seqpar_joint_attention(krea_cuda* h, const krea_cuda_seqpar_args* a);

#ifdef __cplusplus
}
#endif
#endif
