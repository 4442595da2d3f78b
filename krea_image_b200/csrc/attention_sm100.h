// Host-visible parameter block and launcher of the sm_100a attention kernel (attention_sm100.cu).
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace krea {

// Strides are in bf16 elements.  Field meanings follow the reference's AttnParams
// (engine/kernels/attention.metal:65-75) plus the batch / padding-mask / fused-prologue extensions.
struct AttnParams {
  const __nv_bfloat16* Q;
  __nv_bfloat16* O;
  const __nv_bfloat16* G;      // optional output gate, nullptr = none
  int64_t ldq, ldo, ldg;
  int64_t bsq, bso, bsg;
  int Lq, Lk, heads, group, batch;
  float scale_log2;            // softmax scale * log2(e)
  int causal, q_pos0;          // causal: key k visible to query row i iff k <= i + q_pos0
  const float* QB;             // optional fp32 rank-1 score term QB[q, heads] * KB[k, heads/group] (no batch)
  const float* KB;
  int ldqb, ldkb;
  // fused Q prologue (nullptr wq = Q is used as it is)
  const float* wq;
  const float* cos;
  const float* sin;
  float eps;
  int rope_mode;
  int q_row0;                  // sequence position of query row 0
  // optional device float: an upper bound (log2 units, scale included) on every |logit|, written by the
  // K pre-pass from the QK-norm weights; nullptr = unknown (plain operator on already-normalised input)
  const float* logit_bound;
  // text key-padding: keys / query rows at positions [text_len[b], text_slots) are padding
  const int32_t* text_len;
  int text_slots;
  // Row-block scatter of the output (the sequence-parallel return path): when o_blk_rows > 0, query row r
  // is stored at O_blk[r / o_blk_rows] + (r % o_blk_rows) * ldo + head * 128 instead of O + r * ldo + head * 128.
  // The bases may point into other GPUs' memory (plain peer stores); batch must be 1.
  __nv_bfloat16* O_blk[8];
  int o_blk_rows;
  int o_tma;                   // 1: the output tiles leave shared memory as TMA stores through the O tensor map
  int q_tma;                   // 1 (only without a Q prologue): the Q tiles are TMA loads through the Q tensor map
  // 1: launch with programmatic stream serialisation, so that barrier set-up, TMEM allocation and Q staging
  // overlap the tail of the previous kernel in the stream (the K pre-pass).  Only for callers whose Q,
  // tables and weights do not come from that previous kernel: K, V and the logit bound are read after
  // griddepcontrol.wait, everything else before it.
  int pdl;
  uint32_t* status;            // device word: 0 = ok, else (site | qblk << 8 | head << 20) of a timed-out wait
  // K normalised inside the persistent kernel (an option of the fused call; Kraw == nullptr: K was normalised by an
  // earlier kernel).  Every work item whose head is the first of its group normalises and rotates one slice of the
  // key rows of its (sample, kv head) - rows [query block * k_slice_rows, + k_slice_rows) - from Kraw into Kn, the
  // array the K tensor map describes, and adds 16 to kcount[sample * kv heads + kv head]; a CTA asks for the keys of
  // a (sample, kv head) once that counter has reached 16 * k_slices.  kcount is zero at launch; the launch also
  // zeroes kcount_clear (the next launch's counters).
  const __nv_bfloat16* Kraw;
  int64_t ldkr, bskr;          // raw K: row stride, sample stride (elements)
  const float* wk;
  __nv_bfloat16* Kn;           // [batch][Lk][kv heads * 128]
  uint32_t* kcount;
  uint32_t* kcount_clear;
  int kcount_clear_n;
  int k_slices, k_slice_rows;
  int bound_in_kernel;         // the kernel works the logit bound out of wq and wk itself (else: online softmax)
  // Split-K state (attention.metal:14-19): fp32 So [Lq][heads*128] un-normalised output, Sm [Lq][heads] running max
  // (log2 units), Sl [Lq][heads][8] partial row sums (their sum is the row sum).  state_load: start from it instead
  // of the empty state; state_store: leave it instead of the normalised bf16 output.  One-item kernel only.
  float* So;
  float* Sm;
  float* Sl;
  int state_load, state_store;
  uint64_t wait_limit_ns;      // bound on every wait inside the kernel (device wall time); 2 s unless a test shortens it
  int test_drop_last_k;        // test hook: the producer never requests the last K tile, so that a bounded wait runs out
  long long* trace;            // tuning builds only (KREA_ATTN_TRACE): clock64 samples of CTA 0, else nullptr
};

// K and V are described by 3-D tensor maps (column, row, sample) with 64-column x 128-row boxes and
// 128-byte swizzle.  split = threads per query row in the softmax (1 or 2); emu = 1 lets one of every four
// element pairs evaluate exp2 with the FMA-pipe polynomial instead of the special-function unit.
// O is described the same way when p.o_tma is set (its rows past Lq are clipped by the map).
// ... and Q when p.q_tma is set.
cudaError_t launch_attention_sm100(const CUtensorMap& tmK, const CUtensorMap& tmV, const CUtensorMap& tmO, const CUtensorMap& tmQ, const AttnParams& p,
                                   int split, int emu, cudaStream_t stream);

// The persistent form of the same kernel (attention_persist_sm100.cu): one CTA per SM walks over the (query block,
// head, sample) items, a fourth warpgroup stages the next item's Q and writes the previous item's output while the
// tensor pipe keeps running.  Same parameters and results; `sms` = SMs of the device (the grid never exceeds it).
// p.o_tma is ignored (the output rows are stored straight from registers), tmQ is used when p.q_tma is set.
cudaError_t launch_attention_persist_sm100(const CUtensorMap& tmK, const CUtensorMap& tmV, const CUtensorMap& tmQ, const AttnParams& p, int emu,
                                           int sms, cudaStream_t stream);
cudaError_t prepare_attention_persist_sm100(int emu, bool keys_inside);

// The per-device set-up the first launch of that variant would otherwise do (shared-memory opt-in, loading of
// the device code), for the current device: lets a handle pay for it when it is created.
cudaError_t prepare_attention_sm100(int split, int emu);

// Out-of-place / in-place per-head RMSNorm + RoPE (qk_norm_rope.cu).
struct NormRopeParams {
  const __nv_bfloat16* src;
  __nv_bfloat16* dst;          // may equal src
  int64_t ld_src, ld_dst, bs_src, bs_dst;
  int rows, batch;
  int q_off, n_q, k_off, n_k;  // column offsets (in src) / head counts
  int q_off_dst, k_off_dst;    // column offsets in dst
  const float* wq;
  const float* wk;
  const float* cos;
  const float* sin;
  int row0;                    // table row of local row 0
  float eps;
  int rope_mode;
  int big_dim;
  float* qbig;
  float* kbig;
  // joint call only: the pre-pass also derives the a-priori logit bound from both weight vectors
  int pdl;                     // 1: launch with programmatic stream serialisation (the kernel waits for its predecessors first thing)
  const float* bound_wq;       // nullptr = do not compute
  float* bound_out;
  float bound_scale_log2;      // softmax scale * log2(e)
};
cudaError_t launch_qk_norm_rope(const NormRopeParams& p, cudaStream_t stream);
// Loads the norm kernels' device code on the current device (what their first launch would otherwise do).
cudaError_t prepare_qk_norm_rope();

struct ReshardParams {
  const __nv_bfloat16* src;
  __nv_bfloat16* dst;
  // pack only: when dst_peer[0] != nullptr, block `peer` is written to dst_peer[peer] (which may be another
  // GPU's memory) at rows [dst_row0, dst_row0 + rows) of a contiguous [.., cols_per_rank] array, instead of
  // to block `peer` of dst.
  __nv_bfloat16* dst_peer[8];
  int dst_row0;
  int nranks, rows, cols_per_rank;
  int64_t src_ld, dst_ld;
  int src_col0, dst_col0;
};
cudaError_t launch_reshard_pack(const ReshardParams& p, cudaStream_t stream);
cudaError_t launch_reshard_unpack(const ReshardParams& p, cudaStream_t stream);

// The text fusion's 12-tap attention (norm.metal:141-145 LayerAttnParams): rows = tokens * 12.
struct LayerwiseParams {
  const __nv_bfloat16* qkvg;
  __nv_bfloat16* out;
  int rows, heads;
  int64_t ld, ldo;
  int q_off, k_off, v_off, g_off;
  float scale;
};
cudaError_t launch_layerwise_attn(const LayerwiseParams& p, cudaStream_t stream);

// Row-wise RMSNorm of fp32 rows with per-column multiplier / addend (rms_norm.cu).
struct RmsNormParams {
  const float* x;
  const float* mul;
  const float* add;   // nullptr = none
  void* y;            // bf16 or fp32
  int rows, width;
  int64_t ld_in, ld_out;
  float eps;
  int f32_out;
};
cudaError_t launch_rms_norm(const RmsNormParams& p, cudaStream_t stream);

// int8 weights [K, N] with f32 group scales [K / 128, N] -> bf16 [K, N] (dequant_q8.cu).  Strides in elements.
struct DequantParams {
  const int8_t* wq;
  const float* scales;
  __nv_bfloat16* out;
  int K, N;
  int64_t ldq, lds, ldo;
};
cudaError_t launch_dequant_q8(const DequantParams& p, cudaStream_t stream);

// bf16 GEMM C = A x Wt with optional fused QK-norm + RoPE epilogue (gemm_sm100.cu).  Strides in elements.
struct GemmParams {
  __nv_bfloat16* C;
  int64_t ldc;
  int M, N, K;
  int seg, seg_stride;          // epi 0, seg > 0: output column n is stored at (n / seg) * seg_stride + n % seg
  int K2;                       // > 0: a second product A2[M, K2] x W2[K2, N] is accumulated before the epilogue
  int epi;                      // 0: bf16 store; 1: Q / K head blocks are RMS-normalised, weighted and rotated first;
                                // 2: C is fp32 and receives += vec[col] * acc (vec nullptr: += acc); 3: SwiGLU, C has N / 2 columns;
                                // 4: fp32 store; 5: gelu_tanh, bf16; 6: + vec[col], bf16; 7: + vec[col], fp32
  const float* vec;             // epi 2: per-column gate; epi 6, 7: per-column bias
  int q_off, n_q, k_off, n_k;   // epi 1: output columns of the Q and K heads (multiples of 128) and head counts
  const float* wq;
  const float* wk;
  const float* cos;
  const float* sin;
  int row0;                     // table row of output row 0
  float eps;
  int rope_mode;                // 0 interleaved pairs, 2 none
  // epi 1, optional: one CTA also writes the a-priori bound on |q'.k'| * scale * log2(e) that the QK-norm
  // weights imply (128 * max|wq| * max|wk|, 2 % head-room), for the attention kernel's bounded softmax
  float* bound_out;
  float bound_scale_log2;
  // epi 1, optional (norm.metal:127-132): head dimension big_dim of every Q / K head goes to qbig [M, n_q] /
  // kbig [M, n_k] in fp32 and is stored as zero in C; big_dim < 0 = off
  int big_dim;
  float* qbig;
  float* kbig;
  uint32_t* status;
  int group_m;                  // set by the launcher: row blocks per group of the tile order
};
// A: 3-D map (k, row, 1) with 64 x 128 boxes; Wt: (n, k, 1) with 64 x 64 boxes; both 128-byte swizzled.
// force_bn: 0 = choose the tile (128 x 128, 128 x 256, or 256 x 256 on a CTA pair) by how well the tiles fill the
// last wave; 128 / 256 = one-CTA tile of that width, 512 = the CTA-pair tile
// tmA2 / tmW2 describe the second product the same way (ignored when p.K2 == 0)
cudaError_t launch_gemm_bf16_sm100(const CUtensorMap& tmA, const CUtensorMap& tmW, const CUtensorMap& tmA2, const CUtensorMap& tmW2, const GemmParams& p,
                                   int sms, int force_bn, cudaStream_t stream);

}  // namespace krea
