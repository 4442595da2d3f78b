// Per-head RMSNorm (f32 weight [128]) + rotary embedding on bf16 rows: the operator
// Metal::qk_norm_rope of the reference (engine/kernels/norm.metal:81-134), plus an out-of-place form
// with batch strides used as the K pre-pass of the fused joint-attention call.
//
// HBM-bound elementwise pass: one warp per (row, head), each lane owns 4 consecutive channels (one
// 8-byte load and one 8-byte store per lane, 256 contiguous bytes per warp); sums of squares are
// reduced with shuffles; all math in fp32; the result is rounded to bf16 once, at the store.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "attention_sm100.h"
#include "sm100_ptx.cuh"

namespace krea {

__global__ void __launch_bounds__(256) qk_norm_rope_kernel(const NormRopeParams p) {
  const int lane = threadIdx.x & 31;
  if (p.bound_wq != nullptr && blockIdx.x == 0 && threadIdx.x < 32) {
    // After RMSNorm every head vector has norm <= sqrt(128) * max|w| (RoPE is a rotation), so
    // |q'.k'| <= 128 * max|wq| * max|wk|.  2% head-room covers the bf16 rounding of q' and k'
    // (2^-8 each) and the approximate rsqrt.
    const float4 a = __ldg((const float4*)p.bound_wq + lane), c = __ldg((const float4*)p.wk + lane);
    float mq = fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(a.z), fabsf(a.w)));
    float mk = fmaxf(fmaxf(fabsf(c.x), fabsf(c.y)), fmaxf(fabsf(c.z), fabsf(c.w)));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      mq = fmaxf(mq, __shfl_xor_sync(0xffffffffu, mq, o));
      mk = fmaxf(mk, __shfl_xor_sync(0xffffffffu, mk, o));
    }
    if (lane == 0) *p.bound_out = 128.0f * mq * mk * p.bound_scale_log2 * 1.02f;
  }
  const int heads = p.n_q + p.n_k;
  const long long units = (long long)p.batch * p.rows * heads;
  const long long stride = (long long)gridDim.x * (blockDim.x >> 5);
  for (long long unit = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); unit < units; unit += stride) {
    const int hh = (int)(unit % heads);
    const long long rb = unit / heads;
    const int row = (int)(rb % p.rows);
    const int b = (int)(rb / p.rows);
    const bool is_q = hh < p.n_q;
    const int hl = is_q ? hh : hh - p.n_q;
    const size_t src_col = (size_t)(is_q ? p.q_off : p.k_off) + (size_t)hl * 128;
    const size_t dst_col = (size_t)(is_q ? p.q_off_dst : p.k_off_dst) + (size_t)hl * 128;
    const uint2 raw = __ldg((const uint2*)(p.src + (size_t)b * p.bs_src + (size_t)row * p.ld_src + src_col) + lane);
    float x0 = bf16lo_to_f32(raw.x), x1 = bf16hi_to_f32(raw.x), x2 = bf16lo_to_f32(raw.y), x3 = bf16hi_to_f32(raw.y);
    float ss = x0 * x0 + x1 * x1 + x2 * x2 + x3 * x3;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float rrms = rsqrtf(ss * (1.0f / 128.0f) + p.eps);
    const float4 w = __ldg((const float4*)(is_q ? p.wq : p.wk) + lane);
    x0 *= rrms * w.x; x1 *= rrms * w.y; x2 *= rrms * w.z; x3 *= rrms * w.w;
    float o0 = x0, o1 = x1, o2 = x2, o3 = x3;
    const size_t trow = (size_t)(p.row0 + row) * 64;
    if (p.rope_mode == 0) {
      // interleaved pairs (2i, 2i+1) share frequency i: this lane holds pairs 2*lane and 2*lane+1
      const float2 c = __ldg((const float2*)(p.cos + trow) + lane), s = __ldg((const float2*)(p.sin + trow) + lane);
      o0 = x0 * c.x - x1 * s.x;
      o1 = x0 * s.x + x1 * c.x;
      o2 = x2 * c.y - x3 * s.y;
      o3 = x2 * s.y + x3 * c.y;
    } else if (p.rope_mode == 1) {
      // rotate-half: channel i pairs with i + 64, whose owner is lane ^ 16
      const float y0 = __shfl_xor_sync(0xffffffffu, x0, 16), y1 = __shfl_xor_sync(0xffffffffu, x1, 16);
      const float y2 = __shfl_xor_sync(0xffffffffu, x2, 16), y3 = __shfl_xor_sync(0xffffffffu, x3, 16);
      const float4 c = __ldg((const float4*)(p.cos + trow) + (lane & 15)), s = __ldg((const float4*)(p.sin + trow) + (lane & 15));
      const float sg = lane < 16 ? -1.f : 1.f;
      o0 = x0 * c.x + sg * y0 * s.x;
      o1 = x1 * c.y + sg * y1 * s.y;
      o2 = x2 * c.z + sg * y2 * s.z;
      o3 = x3 * c.w + sg * y3 * s.w;
    }
    if (p.big_dim >= 0 && lane == (p.big_dim >> 2)) {
      const int e = p.big_dim & 3;
      const float v = e == 0 ? o0 : e == 1 ? o1 : e == 2 ? o2 : o3;
      if (is_q) p.qbig[((size_t)b * p.rows + row) * p.n_q + hl] = v;
      else p.kbig[((size_t)b * p.rows + row) * p.n_k + hl] = v;
      if (e == 0) o0 = 0.f; else if (e == 1) o1 = 0.f; else if (e == 2) o2 = 0.f; else o3 = 0.f;
    }
    uint2 out;
    out.x = pack_bf16x2(o0, o1);
    out.y = pack_bf16x2(o2, o3);
    *((uint2*)(p.dst + (size_t)b * p.bs_dst + (size_t)row * p.ld_dst + dst_col) + lane) = out;
  }
}

cudaError_t launch_qk_norm_rope(const NormRopeParams& p, cudaStream_t stream) {
  const long long units = (long long)p.batch * p.rows * (p.n_q + p.n_k);
  if (units <= 0) return cudaSuccess;
  long long blocks = (units + 7) / 8;
  const long long cap = 148LL * 8 * 4;   // a few waves of 8 resident CTAs per SM; the loop strides over the rest
  if (blocks > cap) blocks = cap;
  qk_norm_rope_kernel<<<(unsigned)blocks, 256, 0, stream>>>(p);
  return cudaGetLastError();
}

// ---- sequence <-> head resharding (pack / unpack around an all-to-all) -------------------------------
// pack:   dst[peer][row][c] = src[row][src_col0 + peer*cols_per_rank + c]
// unpack: dst[row][dst_col0 + peer*cols_per_rank + c] = src[peer][row][c]      (the inverse of pack)
// Sequence-sharded rows [rows, all heads] are packed into one block per destination rank; after the
// all-to-all the received blocks are already the rows of the local heads in sequence order.  On the way
// back the output rows are sent as they are and unpack merges the received per-rank head blocks.
// 16-byte vectors; cols_per_rank is a multiple of 8.
__global__ void __launch_bounds__(256) reshard_kernel(const ReshardParams p, int unpack) {
  const int vec_per_row = p.cols_per_rank >> 3;
  const long long total = (long long)p.nranks * p.rows * vec_per_row;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int v = (int)(i % vec_per_row);
    const long long t = i / vec_per_row;
    const int row = (int)(t % p.rows);
    const int peer = (int)(t / p.rows);
    if (!unpack) {
      const uint4 x = __ldg((const uint4*)(p.src + (size_t)row * p.src_ld + p.src_col0 + (size_t)peer * p.cols_per_rank) + v);
      *((uint4*)(p.dst + ((size_t)peer * p.rows + row) * p.cols_per_rank) + v) = x;
    } else {
      const uint4 x = __ldg((const uint4*)(p.src + ((size_t)peer * p.rows + row) * p.cols_per_rank) + v);
      *((uint4*)(p.dst + (size_t)row * p.dst_ld + p.dst_col0 + (size_t)peer * p.cols_per_rank) + v) = x;
    }
  }
}

static cudaError_t launch_reshard(const ReshardParams& p, int unpack, cudaStream_t stream) {
  const long long total = (long long)p.nranks * p.rows * (p.cols_per_rank >> 3);
  if (total <= 0) return cudaSuccess;
  long long blocks = (total + 255) / 256;
  if (blocks > 148LL * 16) blocks = 148LL * 16;
  reshard_kernel<<<(unsigned)blocks, 256, 0, stream>>>(p, unpack);
  return cudaGetLastError();
}
cudaError_t launch_reshard_pack(const ReshardParams& p, cudaStream_t stream) { return launch_reshard(p, 0, stream); }
cudaError_t launch_reshard_unpack(const ReshardParams& p, cudaStream_t stream) { return launch_reshard(p, 1, stream); }

}  // namespace krea
