// The text fusion's layerwise attention (engine/kernels/norm.metal:136-178, dispatched by
// Metal::layerwise_attn, engine/src/metal.mm:204-209): rows are token-major (row = t*12 + j) and every row
// attends over the 12 tapped states of its own token,
//   out[row, h*128 + d] = softmax_j(q[row] . k[base + j] / sqrt(128)) v[base + j] * sigmoid(gate[row]),
// scores, softmax and the weighted sum in fp32, one bf16 rounding at the store.
//
// HBM-bound: per (token, head) 48 rows of 256 B are read and 12 written (15 KB), against ~37 K
// multiply-adds.  One warp owns a (token, head) unit: it loads the 12 q, k and v rows once (coalesced 16-byte
// accesses, 512 B per warp instruction) into shared memory, so every byte crosses HBM exactly once - the
// reference re-reads the k and v rows for each of the 12 query rows of a token.  The 12 x 12 scores are one
// 16 x 16 x 128 product on the warp-level tensor-core path (mma.sync m16n8k16, bf16 in, fp32 accumulate;
// rows and columns 12-15 are padding whose results are dropped): a 12-key problem is far too small for a
// tcgen05 tile, and on CUDA cores the bf16 -> fp32 conversions of the score phase made the kernel
// issue-bound at a third of the HBM rate.  The weighted sum runs on packed two-wide fp32 multiply-adds (the taps in
// order, so the values are those of a scalar sum).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "attention_sm100.h"
#include "sm100_ptx.cuh"

namespace krea {

constexpr int TAPS = 12;
constexpr int LW_WARPS = 4;                       // units per CTA
constexpr int LW_ROW_BYTES = 256 + 16;            // one head row of bf16, padded: rows start in different banks
constexpr int LW_TILE = 16 * LW_ROW_BYTES;        // q, k or v of one unit, padded to the 16 rows of an MMA tile

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem_row) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(smem_row)));
}
// d (16 x 8, fp32) += a (16 x 16, bf16, row-major) * b (16 x 8, bf16, "column-major": 8 rows of 16 k-values)
__device__ __forceinline__ void mma_m16n8k16_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(LW_WARPS * 32) layerwise_attn_kernel(const LayerwiseParams p) {
  __shared__ __align__(16) uint8_t tiles[LW_WARPS][2][LW_TILE];
  // probabilities, each stored twice in a row (p, p): a 16-byte load then yields two ready operands of the packed
  // two-wide multiply-add
  __shared__ __align__(16) float probs[LW_WARPS][TAPS][2 * TAPS];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tokens = p.rows / TAPS;
  const long long units = (long long)tokens * p.heads;
  uint8_t* tq = tiles[warp][0];
  uint8_t* tk = tiles[warp][1];
  for (long long u = (long long)blockIdx.x * LW_WARPS + warp; u < units; u += (long long)gridDim.x * LW_WARPS) {
    const int t = (int)(u / p.heads), h = (int)(u - (long long)t * p.heads);
    const __nv_bfloat16* base = p.qkvg + (size_t)t * TAPS * p.ld + (size_t)h * 128;
    // ---- load: q and k rows go to shared memory for the tensor-core product (16 lanes x 16 bytes per row,
    // two rows per instruction); v and the gate stay in registers, each lane holding its own 4 channels of
    // all 12 rows.  All 36 loads of a lane are issued before the first is used. ----
    uint2 vraw[TAPS], gate[TAPS];
    {
      const int sub = lane >> 4, c = lane & 15;
      uint4 r[12];
#pragma unroll
      for (int i = 0; i < 6; i++) {
        const __nv_bfloat16* row = base + (size_t)(2 * i + sub) * p.ld + 8 * c;
        r[2 * i] = __ldg((const uint4*)(row + p.q_off));
        r[2 * i + 1] = __ldg((const uint4*)(row + p.k_off));
      }
#pragma unroll
      for (int j = 0; j < TAPS; j++) {
        vraw[j] = __ldg((const uint2*)(base + (size_t)j * p.ld + p.v_off + 4 * lane));
        gate[j] = __ldg((const uint2*)(base + (size_t)j * p.ld + p.g_off + 4 * lane));
      }
      __syncwarp();     // the previous unit's readers are done with the tiles
#pragma unroll
      for (int i = 0; i < 6; i++) {
        const int off = (2 * i + sub) * LW_ROW_BYTES + 16 * c;
        *(uint4*)(tq + off) = r[2 * i];
        *(uint4*)(tk + off) = r[2 * i + 1];
      }
      __syncwarp();
    }
    // ---- scores: S[16 x 16] = Q[16 x 128] K^T on mma.sync; lane (g = lane / 4, t = lane % 4) ends up with
    // rows g and g + 8, columns 2t, 2t + 1 of the key blocks 0-7 (c_lo) and 8-15 (c_hi) ----
    float c_lo[4] = {0.f, 0.f, 0.f, 0.f}, c_hi[4] = {0.f, 0.f, 0.f, 0.f};
    {
      // ldmatrix row addresses.  A: matrices (rows 0-7, k 0-7), (rows 8-15, k 0-7), (rows 0-7, k 8-15), (rows 8-15, k 8-15);
      // B: (keys 0-7, k 0-7), (keys 0-7, k 8-15), (keys 8-15, k 0-7), (keys 8-15, k 8-15)
      const uint8_t* qa = tq + ((lane & 7) + ((lane >> 3) & 1) * 8) * LW_ROW_BYTES + ((lane >> 4) & 1) * 16;
      const uint8_t* kb = tk + ((lane & 7) + ((lane >> 4) & 1) * 8) * LW_ROW_BYTES + ((lane >> 3) & 1) * 16;
#pragma unroll
      for (int kk = 0; kk < 8; kk++) {
        uint32_t a[4], bq[4];
        ldmatrix_x4(a, qa + kk * 32);
        ldmatrix_x4(bq, kb + kk * 32);
        mma_m16n8k16_bf16(c_lo, a, bq[0], bq[1]);
        mma_m16n8k16_bf16(c_hi, a, bq[2], bq[3]);
      }
    }
    // ---- softmax over the 12 taps: a row's scores sit in the four lanes of a quad ----
    {
      const int g = lane >> 2, t = lane & 3;
      const bool hi_ok = t < 2;                       // key columns 8 + 2t, 9 + 2t exist only for t < 2
#pragma unroll
      for (int half = 0; half < 2; half++) {          // rows g and g + 8
        const float s0 = c_lo[2 * half] * p.scale, s1 = c_lo[2 * half + 1] * p.scale;
        const float s2 = hi_ok ? c_hi[2 * half] * p.scale : -INFINITY, s3 = hi_ok ? c_hi[2 * half + 1] * p.scale : -INFINITY;
        float mx = fmaxf(fmaxf(s0, s1), fmaxf(s2, s3));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float e0 = __expf(s0 - mx), e1 = __expf(s1 - mx), e2 = __expf(s2 - mx), e3 = __expf(s3 - mx);
        float l = (e0 + e1) + (e2 + e3);
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        const float inv = rcp_approx(l);
        const int row = g + 8 * half;
        if (row < TAPS) {
          float4* prow = (float4*)&probs[warp][row][0];
          const float p0 = e0 * inv, p1 = e1 * inv;
          prow[t] = make_float4(p0, p0, p1, p1);                        // key columns 2t, 2t + 1
          if (hi_ok) {
            const float p2 = e2 * inv, p3 = e3 * inv;
            prow[4 + t] = make_float4(p2, p2, p3, p3);                  // key columns 8 + 2t, 9 + 2t
          }
        }
      }
    }
    __syncwarp();
    // ---- weighted sum, gate, store: lane owns channels 4*lane .. 4*lane+3 of every row ----
    {
      uint64_t v2[TAPS][2];                             // channels (0, 1) and (2, 3) of every value row as fp32 pairs
#pragma unroll
      for (int j = 0; j < TAPS; j++) {
        v2[j][0] = pack_f32x2(bf16lo_to_f32(vraw[j].x), bf16hi_to_f32(vraw[j].x));
        v2[j][1] = pack_f32x2(bf16lo_to_f32(vraw[j].y), bf16hi_to_f32(vraw[j].y));
      }
      __nv_bfloat16* obase = p.out + (size_t)t * TAPS * p.ldo + (size_t)h * 128 + 4 * lane;
#pragma unroll
      for (int i = 0; i < TAPS; i++) {
        uint64_t acc0 = pack_f32x2(0.f, 0.f), acc1 = acc0;
        const ulonglong2* prow = (const ulonglong2*)&probs[warp][i][0];
#pragma unroll
        for (int jj = 0; jj < TAPS / 2; jj++) {         // taps in order, as the scalar sum would take them
          const ulonglong2 pp = prow[jj];               // (p_2jj, p_2jj), (p_2jj+1, p_2jj+1)
          acc0 = fma_f32x2(pp.x, v2[2 * jj][0], acc0);
          acc1 = fma_f32x2(pp.x, v2[2 * jj][1], acc1);
          acc0 = fma_f32x2(pp.y, v2[2 * jj + 1][0], acc0);
          acc1 = fma_f32x2(pp.y, v2[2 * jj + 1][1], acc1);
        }
        float o[4];
        unpack_f32x2(acc0, o[0], o[1]);
        unpack_f32x2(acc1, o[2], o[3]);
        const float g4[4] = {bf16lo_to_f32(gate[i].x), bf16hi_to_f32(gate[i].x), bf16lo_to_f32(gate[i].y), bf16hi_to_f32(gate[i].y)};
#pragma unroll
        for (int e = 0; e < 4; e++) o[e] *= sigmoid_approx(g4[e]);
        *(uint2*)(obase + (size_t)i * p.ldo) = make_uint2(pack_bf16x2(o[0], o[1]), pack_bf16x2(o[2], o[3]));
      }
    }
  }
}

cudaError_t launch_layerwise_attn(const LayerwiseParams& p, cudaStream_t stream) {
  const long long units = (long long)(p.rows / TAPS) * p.heads;
  if (units <= 0) return cudaSuccess;
  long long blocks = (units + LW_WARPS - 1) / LW_WARPS;
  const long long cap = 148LL * 8;
  if (blocks > cap) blocks = cap;
  layerwise_attn_kernel<<<(unsigned)blocks, LW_WARPS * 32, 0, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace krea
