// Per-head RMSNorm (f32 weight [128]) + rotary embedding on bf16 rows: the operator
// Metal::qk_norm_rope of the reference (engine/kernels/norm.metal:81-134), plus an out-of-place form
// with batch strides used as the K pre-pass of the fused joint-attention call.
//
// HBM-bound elementwise pass; sums of squares are reduced with shuffles; all math in fp32; the result is
// rounded to bf16 once, at the store.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "attention_sm100.h"
#include "sm100_ptx.cuh"

namespace krea {

// One warp per (row, eight heads) unit, two heads per step: 16 lanes cover one head with 16 bytes (8
// channels) each, so a warp load is 512 contiguous bytes.  The row's cos/sin entries and the weights depend
// only on the lane's channels, not on the head, and are loaded once per unit.
// MODE is the rope mode as a compile-time constant (dead branches cost registers, and registers decide
// how many warps cover the memory latency).  KONLY is the shape of the fused call's pre-pass - K heads
// only, no fp32 side buffer, fewer than 2^31 units - without the per-step query / key selection and with
// 32-bit unit arithmetic: the kernel is bound by instruction issue, so every instruction off the step counts.
template <int MODE, bool KONLY>
__global__ void __launch_bounds__(256, 3) qk_norm_rope_kernel(const NormRopeParams p) {
  const int lane = threadIdx.x & 31;
  griddep_wait();      // with a programmatic launch this kernel may start while its predecessor drains
  griddep_launch();    // ... and the kernel after it may set itself up while this one runs
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
  const int sub = lane >> 4, c = lane & 15;     // which of the two heads of a step, which 8-channel chunk
  const int heads = p.n_q + p.n_k;
  // weights of this lane's 8 channels as four packed pairs
  uint64_t wq2[4], wk2[4];
#pragma unroll
  for (int e = 0; e < 4; e++) wq2[e] = wk2[e] = pack_f32x2(0.f, 0.f);
  if (!KONLY && p.n_q > 0) {
    const float4 a = __ldg((const float4*)p.wq + 2 * c), bq = __ldg((const float4*)p.wq + 2 * c + 1);
    wq2[0] = pack_f32x2(a.x, a.y); wq2[1] = pack_f32x2(a.z, a.w); wq2[2] = pack_f32x2(bq.x, bq.y); wq2[3] = pack_f32x2(bq.z, bq.w);
  }
  if (p.n_k > 0) {
    const float4 a = __ldg((const float4*)p.wk + 2 * c), bk = __ldg((const float4*)p.wk + 2 * c + 1);
    wk2[0] = pack_f32x2(a.x, a.y); wk2[1] = pack_f32x2(a.z, a.w); wk2[2] = pack_f32x2(bk.x, bk.y); wk2[3] = pack_f32x2(bk.z, bk.w);
  }
  // work unit = (row, batch of up to eight heads): short dependent chains (weights, tables, one batch of
  // loads) and enough warps in flight to cover the memory latency even for a few thousand rows
  const int nhb = (heads + 7) >> 3;
  const long long nunits = (long long)p.batch * p.rows * nhb;
  const long long wstride = (long long)gridDim.x * (blockDim.x >> 5);
  for (long long u = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); u < nunits; u += wstride) {
    int rb, hb;
    if constexpr (KONLY) {
      rb = (int)((unsigned)u / (unsigned)nhb);
      hb = (int)((unsigned)u - (unsigned)rb * (unsigned)nhb) * 8;
    } else {
      rb = (int)(u / nhb);
      hb = (int)(u - (long long)rb * nhb) * 8;
    }
    const int b = rb / p.rows, row = rb - b * p.rows;
    const __nv_bfloat16* srow = p.src + (size_t)b * p.bs_src + (size_t)row * p.ld_src;
    __nv_bfloat16* drow = p.dst + (size_t)b * p.bs_dst + (size_t)row * p.ld_dst;
    const size_t trow = (size_t)(p.row0 + row) * 64;
    float cf[8], sf[8];
    if (MODE == 0) {
      // interleaved pairs (2i, 2i+1) share frequency i: this chunk holds pairs 4c .. 4c+3
      const float4 cc = __ldg((const float4*)(p.cos + trow) + c), sc = __ldg((const float4*)(p.sin + trow) + c);
      cf[0] = cc.x; cf[1] = cc.y; cf[2] = cc.z; cf[3] = cc.w;
      sf[0] = sc.x; sf[1] = sc.y; sf[2] = sc.z; sf[3] = sc.w;
    } else if (MODE == 1) {
      // rotate-half: channel i pairs with i + 64 (the lane 8 chunks away); both use frequency i mod 64
      const int f = (c & 7) * 2;
      const float4 c0 = __ldg((const float4*)(p.cos + trow) + f), c1 = __ldg((const float4*)(p.cos + trow) + f + 1);
      const float4 s0 = __ldg((const float4*)(p.sin + trow) + f), s1 = __ldg((const float4*)(p.sin + trow) + f + 1);
      cf[0] = c0.x; cf[1] = c0.y; cf[2] = c0.z; cf[3] = c0.w; cf[4] = c1.x; cf[5] = c1.y; cf[6] = c1.z; cf[7] = c1.w;
      sf[0] = s0.x; sf[1] = s0.y; sf[2] = s0.z; sf[3] = s0.w; sf[4] = s1.x; sf[5] = s1.y; sf[6] = s1.z; sf[7] = s1.w;
    }
    // four steps (eight heads): their loads are all issued before the first one is used
    {
      uint4 raw[4];
      int dcol[4], hl[4];
      bool live[4], isq[4];
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const int hh = hb + 2 * i + sub;
        live[i] = hh < heads;                      // ragged head count: idle lanes re-read the last head
        const int hc = live[i] ? hh : heads - 1;
        isq[i] = !KONLY && hc < p.n_q;
        hl[i] = isq[i] ? hc : hc - p.n_q;
        const int scol = (isq[i] ? p.q_off : p.k_off) + hl[i] * 128 + 8 * c;
        dcol[i] = (isq[i] ? p.q_off_dst : p.k_off_dst) + hl[i] * 128 + 8 * c;
        raw[i] = __ldg((const uint4*)(srow + scol));
      }
#pragma unroll
      for (int i = 0; i < 4; i++) {
        if (hb + 2 * i >= heads) break;            // warp-uniform
        const uint32_t w4[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
        // packed fp32 pairs: the sum of squares and the scaling take half the instructions
        uint64_t y2[4];
        uint64_t acc2 = pack_f32x2(0.f, 0.f);
#pragma unroll
        for (int e = 0; e < 4; e++) {
          y2[e] = pack_f32x2(bf16lo_to_f32(w4[e]), bf16hi_to_f32(w4[e]));
          acc2 = fma_f32x2(y2[e], y2[e], acc2);
        }
        float s0, s1;
        unpack_f32x2(acc2, s0, s1);
        float ss = s0 + s1;
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float rrms = rsqrtf(ss * (1.0f / 128.0f) + p.eps);
        const uint64_t r2 = pack_f32x2(rrms, rrms);
        float y[8], z[8];
#pragma unroll
        for (int e = 0; e < 4; e++) {
          const uint64_t w2 = isq[i] ? wq2[e] : wk2[e];
          unpack_f32x2(mul_f32x2(y2[e], mul_f32x2(r2, w2)), y[2 * e], y[2 * e + 1]);
        }
        if (MODE == 0) {
#pragma unroll
          for (int e = 0; e < 4; e++) {
            z[2 * e] = y[2 * e] * cf[e] - y[2 * e + 1] * sf[e];
            z[2 * e + 1] = y[2 * e] * sf[e] + y[2 * e + 1] * cf[e];
          }
        } else if (MODE == 1) {
          const float sg = c < 8 ? -1.f : 1.f;
#pragma unroll
          for (int e = 0; e < 8; e++) {
            const float other = __shfl_xor_sync(0xffffffffu, y[e], 8);
            z[e] = y[e] * cf[e] + sg * other * sf[e];
          }
        } else {
#pragma unroll
          for (int e = 0; e < 8; e++) z[e] = y[e];
        }
        if (!KONLY && p.big_dim >= 0 && c == (p.big_dim >> 3)) {
          // that channel goes to the fp32 side buffer and is stored as zero (norm.metal:127-132)
          const int e = p.big_dim & 7;
          float v = 0.f;
#pragma unroll
          for (int k = 0; k < 8; k++)
            if (k == e) { v = z[k]; z[k] = 0.f; }
          if (live[i]) {
            if (isq[i]) p.qbig[((size_t)b * p.rows + row) * p.n_q + hl[i]] = v;
            else p.kbig[((size_t)b * p.rows + row) * p.n_k + hl[i]] = v;
          }
        }
        if (live[i]) *(uint4*)(drow + dcol[i]) = make_uint4(pack_bf16x2(z[0], z[1]), pack_bf16x2(z[2], z[3]), pack_bf16x2(z[4], z[5]), pack_bf16x2(z[6], z[7]));
      }
    }
  }
}

template <int MODE, bool KONLY>
static cudaError_t launch_norm_variant(const cudaLaunchConfig_t& cfg, const NormRopeParams& p) {
  return cudaLaunchKernelEx(&cfg, qk_norm_rope_kernel<MODE, KONLY>, p);
}

cudaError_t launch_qk_norm_rope(const NormRopeParams& p, cudaStream_t stream) {
  const long long nrows = (long long)p.batch * p.rows;
  if (nrows <= 0 || p.n_q + p.n_k <= 0) return cudaSuccess;
  const long long nunits = nrows * ((p.n_q + p.n_k + 7) / 8);
  long long blocks = (nunits + 7) / 8;   // 8 warps per CTA, one (row, eight heads) unit per warp and step
  const long long cap = 148LL * 3;       // all resident at once; the loop strides over the rest
  if (blocks > cap) blocks = cap;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)blocks);
  cfg.blockDim = dim3(256);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = p.pdl ? 1 : 0;
  const bool konly = p.n_q == 0 && p.big_dim < 0 && nunits < (1LL << 31);
  if (konly) {
    if (p.rope_mode == 0) return launch_norm_variant<0, true>(cfg, p);
    if (p.rope_mode == 1) return launch_norm_variant<1, true>(cfg, p);
    return launch_norm_variant<2, true>(cfg, p);
  }
  if (p.rope_mode == 0) return launch_norm_variant<0, false>(cfg, p);
  if (p.rope_mode == 1) return launch_norm_variant<1, false>(cfg, p);
  return launch_norm_variant<2, false>(cfg, p);
}

cudaError_t prepare_qk_norm_rope() {
  // the three forms the fused call's K pre-pass can take (one per rope mode)
  cudaFuncAttributes fa;
  cudaError_t e = cudaFuncGetAttributes(&fa, qk_norm_rope_kernel<0, true>);
  if (e == cudaSuccess) e = cudaFuncGetAttributes(&fa, qk_norm_rope_kernel<1, true>);
  if (e == cudaSuccess) e = cudaFuncGetAttributes(&fa, qk_norm_rope_kernel<2, true>);
  return e;
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
      if (p.dst_peer[0] != nullptr) {
        __nv_bfloat16* base = p.dst_peer[0];   // parameter space wants compile-time indices: selects
#pragma unroll
        for (int k = 1; k < 8; k++) base = peer == k ? p.dst_peer[k] : base;
        *((uint4*)(base + ((size_t)p.dst_row0 + row) * p.cols_per_rank) + v) = x;
      } else {
        *((uint4*)(p.dst + ((size_t)peer * p.rows + row) * p.cols_per_rank) + v) = x;
      }
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
