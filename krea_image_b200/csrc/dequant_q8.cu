// int8 weights with group scales -> bf16 weights, once, at load time.
//
// The reference keeps `Weight::q8` matrices as int8 Wq[K, N] with f32 scales S[K / 128, N] (symmetric, per
// output column and group of 128 input rows; tools/convert.py:92-99) and dequantises every tile to bf16 on its
// way into threadgroup memory, d = bf16(float(q) * s) (engine/kernels/gemm.metal:55-58, 159-170): on a machine
// whose whole memory is 36 GB that halves the weight footprint.  A B200 has 180 GB of its own: the same
// arithmetic is done once per matrix into a bf16 copy in HBM - bit-identical values - and the tensor-core GEMM
// then runs on bf16 operands with nothing extra in its inner loop.  HBM-bound: 1 byte read, 2 written per weight.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "attention_sm100.h"
#include "sm100_ptx.cuh"

namespace krea {

__global__ void __launch_bounds__(256) dequant_q8_kernel(const DequantParams p) {
  const int vec_per_row = p.N >> 4;                       // 16 weights per thread step
  const long long total = (long long)p.K * vec_per_row;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int k = (int)(i / vec_per_row), n = (int)(i - (long long)k * vec_per_row) << 4;
    const uint4 q = __ldg((const uint4*)(p.wq + (size_t)k * p.ldq + n));
    const float4* sp = (const float4*)(p.scales + (size_t)(k >> 7) * p.lds + n);
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
    uint32_t out[8];
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const float4 s = __ldg(sp + j);
      const float f0 = (float)(int8_t)(w[j] & 0xffu) * s.x, f1 = (float)(int8_t)((w[j] >> 8) & 0xffu) * s.y;
      const float f2 = (float)(int8_t)((w[j] >> 16) & 0xffu) * s.z, f3 = (float)(int8_t)(w[j] >> 24) * s.w;
      out[2 * j] = pack_bf16x2(f0, f1);
      out[2 * j + 1] = pack_bf16x2(f2, f3);
    }
    uint4* dst = (uint4*)(p.out + (size_t)k * p.ldo + n);
    dst[0] = make_uint4(out[0], out[1], out[2], out[3]);
    dst[1] = make_uint4(out[4], out[5], out[6], out[7]);
  }
}

cudaError_t launch_dequant_q8(const DequantParams& p, cudaStream_t stream) {
  const long long total = (long long)p.K * (p.N >> 4);
  if (total <= 0) return cudaSuccess;
  long long blocks = (total + 255) / 256;
  if (blocks > 148LL * 16) blocks = 148LL * 16;
  dequant_q8_kernel<<<(unsigned)blocks, 256, 0, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace krea
