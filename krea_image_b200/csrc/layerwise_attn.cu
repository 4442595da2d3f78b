// The text fusion's layerwise attention (engine/kernels/norm.metal:136-178, dispatched by
// Metal::layerwise_attn, engine/src/metal.mm:204-209): rows are token-major (row = t*12 + j) and every row
// attends over the 12 tapped states of its own token,
//   out[row, h*128 + d] = softmax_j(q[row] . k[base + j] / sqrt(128)) v[base + j] * sigmoid(gate[row]),
// scores, softmax and the weighted sum in fp32, one bf16 rounding at the store.
//
// HBM-bound: per (token, head) 48 rows of 256 B are read and 12 written (15 KB), against ~37 K
// multiply-adds.  One warp owns a (token, head) unit: it loads the 12 q, k and v rows once (coalesced 16-byte
// accesses, 512 B per warp instruction) into shared memory, so every byte crosses HBM exactly once - the
// reference re-reads the k and v rows for each of the 12 query rows of a token.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "attention_sm100.h"
#include "sm100_ptx.cuh"

namespace krea {

constexpr int TAPS = 12;
constexpr int LW_WARPS = 4;                       // units per CTA
constexpr int LW_ROW_BYTES = 256 + 16;            // one head row of bf16, padded: rows start in different banks
constexpr int LW_TILE = TAPS * LW_ROW_BYTES;      // q, k or v of one unit

__global__ void __launch_bounds__(LW_WARPS * 32) layerwise_attn_kernel(const LayerwiseParams p) {
  __shared__ __align__(16) uint8_t tiles[LW_WARPS][3][LW_TILE];
  __shared__ float probs[LW_WARPS][TAPS][TAPS + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tokens = p.rows / TAPS;
  const long long units = (long long)tokens * p.heads;
  uint8_t* tq = tiles[warp][0];
  uint8_t* tk = tiles[warp][1];
  uint8_t* tv = tiles[warp][2];
  for (long long u = (long long)blockIdx.x * LW_WARPS + warp; u < units; u += (long long)gridDim.x * LW_WARPS) {
    const int t = (int)(u / p.heads), h = (int)(u - (long long)t * p.heads);
    const __nv_bfloat16* base = p.qkvg + (size_t)t * TAPS * p.ld + (size_t)h * 128;
    // ---- load: 16 lanes x 16 bytes per row, two rows per instruction, all 18 loads issued up front ----
    {
      const int sub = lane >> 4, c = lane & 15;
      uint4 r[18];
#pragma unroll
      for (int i = 0; i < 6; i++) {
        const __nv_bfloat16* row = base + (size_t)(2 * i + sub) * p.ld + 8 * c;
        r[3 * i] = __ldg((const uint4*)(row + p.q_off));
        r[3 * i + 1] = __ldg((const uint4*)(row + p.k_off));
        r[3 * i + 2] = __ldg((const uint4*)(row + p.v_off));
      }
      __syncwarp();     // the previous unit's readers are done with the tiles
#pragma unroll
      for (int i = 0; i < 6; i++) {
        const int off = (2 * i + sub) * LW_ROW_BYTES + 16 * c;
        *(uint4*)(tq + off) = r[3 * i];
        *(uint4*)(tk + off) = r[3 * i + 1];
        *(uint4*)(tv + off) = r[3 * i + 2];
      }
      __syncwarp();
    }
    // ---- scores: the 144 (query tap, key tap) pairs are dealt to the lanes, 4 or 5 each ----
    for (int pr = lane; pr < TAPS * TAPS; pr += 32) {
      const int i = pr / TAPS, j = pr - i * TAPS;
      const uint4* qa = (const uint4*)(tq + i * LW_ROW_BYTES);
      const uint4* kb = (const uint4*)(tk + j * LW_ROW_BYTES);
      float acc = 0.f;
#pragma unroll
      for (int c = 0; c < 16; c++) {
        const uint4 a = qa[c], b = kb[c];
        const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
        for (int e = 0; e < 4; e++) {
          acc = fmaf(bf16lo_to_f32(aw[e]), bf16lo_to_f32(bw[e]), acc);
          acc = fmaf(bf16hi_to_f32(aw[e]), bf16hi_to_f32(bw[e]), acc);
        }
      }
      probs[warp][i][j] = acc * p.scale;
    }
    __syncwarp();
    // ---- softmax over the 12 taps of each query row (lanes 0-11), normalised in place ----
    if (lane < TAPS) {
      float* s = probs[warp][lane];
      float mx = s[0];
#pragma unroll
      for (int j = 1; j < TAPS; j++) mx = fmaxf(mx, s[j]);
      float e[TAPS], l = 0.f;
#pragma unroll
      for (int j = 0; j < TAPS; j++) {
        e[j] = __expf(s[j] - mx);
        l += e[j];
      }
      const float inv = 1.0f / l;
#pragma unroll
      for (int j = 0; j < TAPS; j++) s[j] = e[j] * inv;
    }
    __syncwarp();
    // ---- weighted sum, gate, store: lane owns channels 4*lane .. 4*lane+3 of every row ----
    {
      float v[TAPS][4];
#pragma unroll
      for (int j = 0; j < TAPS; j++) {
        const uint2 w = *(const uint2*)(tv + j * LW_ROW_BYTES + 8 * lane);
        v[j][0] = bf16lo_to_f32(w.x); v[j][1] = bf16hi_to_f32(w.x);
        v[j][2] = bf16lo_to_f32(w.y); v[j][3] = bf16hi_to_f32(w.y);
      }
      const __nv_bfloat16* gbase = base + p.g_off + 4 * lane;
      __nv_bfloat16* obase = p.out + (size_t)t * TAPS * p.ldo + (size_t)h * 128 + 4 * lane;
      uint2 gate[TAPS];
#pragma unroll
      for (int i = 0; i < TAPS; i++) gate[i] = __ldg((const uint2*)(gbase + (size_t)i * p.ld));
#pragma unroll
      for (int i = 0; i < TAPS; i++) {
        float o[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int j = 0; j < TAPS; j++) {
          const float pij = probs[warp][i][j];
#pragma unroll
          for (int e = 0; e < 4; e++) o[e] = fmaf(pij, v[j][e], o[e]);
        }
        const float g4[4] = {bf16lo_to_f32(gate[i].x), bf16hi_to_f32(gate[i].x), bf16lo_to_f32(gate[i].y), bf16hi_to_f32(gate[i].y)};
#pragma unroll
        for (int e = 0; e < 4; e++) o[e] *= 1.0f / (1.0f + __expf(-g4[e]));   // common.h:24
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
