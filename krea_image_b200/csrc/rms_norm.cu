// Row-wise RMSNorm of the fp32 residual stream with a per-column multiplier and optional addend:
//   y[row, c] = x[row, c] * rsqrt(mean_c(x^2) + eps) * mul[c] (+ add[c]),  bf16 or fp32 output
// (Metal::rms_norm, engine/src/metal.h:75-77; kernel engine/kernels/norm.metal:28-55).  In the DiT block mul
// and add carry the timestep modulation (engine/src/model.mm:371-373).
//
// HBM-bound: one CTA per row keeps the row in registers between the sum of squares and the scaling, so x is
// read once (the reference reads it twice); rows wider than the register budget fall back to a second read,
// which L2 serves.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "attention_sm100.h"
#include "sm100_ptx.cuh"

namespace krea {

constexpr int RN_THREADS = 256;
constexpr int RN_HOLD = 8;   // float4 per thread kept in registers: rows up to 8192 columns

template <bool F32_OUT>
__global__ void __launch_bounds__(RN_THREADS) rms_norm_kernel(const RmsNormParams p) {
  __shared__ float part[RN_THREADS / 32];
  const int row = blockIdx.x, tid = threadIdx.x;
  const float4* xr = (const float4*)(p.x + (size_t)row * p.ld_in);
  const int n4 = p.width >> 2;
  float4 hold[RN_HOLD];
  float q = 0.f;
#pragma unroll
  for (int k = 0; k < RN_HOLD; k++) {
    const int i = tid + k * RN_THREADS;
    hold[k] = i < n4 ? __ldg(xr + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    q += hold[k].x * hold[k].x + hold[k].y * hold[k].y + hold[k].z * hold[k].z + hold[k].w * hold[k].w;
  }
  for (int i = tid + RN_HOLD * RN_THREADS; i < n4; i += RN_THREADS) {
    const float4 v = __ldg(xr + i);
    q += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) q += __shfl_xor_sync(0xffffffffu, q, o);
  if ((tid & 31) == 0) part[tid >> 5] = q;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int w = 0; w < RN_THREADS / 32; w++) tot += part[w];
  const float rrms = rsqrtf(tot / (float)p.width + p.eps);            // norm.metal:46
  const float4* mv = (const float4*)p.mul;
  const float4* av = (const float4*)p.add;
  auto emit = [&](int i, float4 v) {
    const float4 m = __ldg(mv + i);
    float4 o = make_float4(v.x * rrms * m.x, v.y * rrms * m.y, v.z * rrms * m.z, v.w * rrms * m.w);
    if (av) {
      const float4 a = __ldg(av + i);
      o.x += a.x; o.y += a.y; o.z += a.z; o.w += a.w;
    }
    if (F32_OUT) ((float4*)((float*)p.y + (size_t)row * p.ld_out))[i] = o;
    else ((uint2*)((__nv_bfloat16*)p.y + (size_t)row * p.ld_out))[i] = make_uint2(pack_bf16x2(o.x, o.y), pack_bf16x2(o.z, o.w));
  };
#pragma unroll
  for (int k = 0; k < RN_HOLD; k++) {
    const int i = tid + k * RN_THREADS;
    if (i < n4) emit(i, hold[k]);
  }
  for (int i = tid + RN_HOLD * RN_THREADS; i < n4; i += RN_THREADS) emit(i, __ldg(xr + i));
}

cudaError_t launch_rms_norm(const RmsNormParams& p, cudaStream_t stream) {
  if (p.rows <= 0 || p.width <= 0) return cudaSuccess;
  if (p.f32_out) rms_norm_kernel<true><<<p.rows, RN_THREADS, 0, stream>>>(p);
  else rms_norm_kernel<false><<<p.rows, RN_THREADS, 0, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace krea
