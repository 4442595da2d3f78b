// bf16 GEMM for B200 (sm_100a) with the epilogues the attention path's neighbours need:
//   C[M, N] = A[M, K] (bf16, row stride lda) x Wt[K, N] (bf16, row stride ldw, "input-major" weights)
// the operand layouts of the reference's Metal::gemm (engine/src/metal.h:64-67, kernels/gemm.metal:1-6).
// EPI_BF16 stores the product as bf16 (gemm.metal:29-30); EPI_QKNORM additionally applies, to the head
// blocks of 128 output columns that hold Q and K, the per-head RMSNorm x weight + RoPE of
// engine/kernels/norm.metal:81-134 before the store - the projection that feeds the attention
// (engine/src/model.mm:349-359, 376) then writes Q and K already normalised and rotated, and the separate
// pass over them disappears.
//
// Shares nothing with the reference's simdgroup kernels:
//   * persistent CTAs walk 128 x 256 output tiles (128 x 128 when that fills the last wave of CTAs better); one warp issues TMA loads of A (K-major) and Wt (N-major,
//     exactly as it lies in memory) into a 4-stage ring of 128B-swizzled shared memory, one warp issues
//     tcgen05.mma (M128 N256 K16) into one of two 256-column accumulators in tensor memory, four warps
//     drain the other accumulator - the epilogue of tile i overlaps the main loop of tile i + 1;
//   * a thread of the epilogue owns one output row (= one TMEM lane), so a head's 128 columns - its sum of
//     squares, its rotation pairs - are all in that thread's registers: the fused norm needs no exchange;
//   * every wait is bounded (status word, normal exit) as in the attention kernel;
//   * PAIR: the same kernel on clusters of two CTAs (tcgen05 cta_group::2): a pair works on a 256 x 256 tile, each
//     CTA loads its own 128 rows of A and HALF of the Wt tile (128 columns) - 32 KB instead of 48 KB into shared
//     memory per 512 tensor-pipe clocks - the leader CTA's MMA warp issues M256 N256 K16 products that read both
//     CTAs' shared memory and write both CTAs' tensor memory, and every CTA drains its own 128 accumulator rows.
//     All loads signal the leader's barriers; stage releases and accumulator hand-overs are committed to both
//     CTAs (two plain commits, no multicast anywhere).  Measured at 4608 x 9216 x 3072: 1503-1534 TFLOP/s against
//     1402-1434 for the one-CTA tile and 1505 for the library GEMM on the same box.
#include <mutex>
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include "attention_sm100.h"
#include "sm100_ptx.cuh"

namespace krea {

namespace gemm {
constexpr int BM = 128, BK = 64;
constexpr int A_BYTES = BM * BK * 2;          // 16 KB: [128 rows][64 k], K-major
constexpr int B_BLOCK = BK * 64 * 2;          // 8 KB: [64 k][64 n], N-major
constexpr int THREADS = 256;                  // warp 0 TMA, warp 1 MMA, warps 4-7 epilogue
enum : uint32_t { SITE_FULL = 11, SITE_EMPTY = 12, SITE_ACC_FULL = 13, SITE_ACC_EMPTY = 14 };
// Tile width: 256 columns halve the A traffic per flop; 128 columns give twice as many tiles, which only pays
// when the 256-wide tiles would leave most of the 148 CTAs idle (small problems).
// ---- the CTA-pair forms of the instructions (cluster of two CTAs, rank 0 = leader) ----
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same shared-memory offset in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa(uint32_t saddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA tile load into this CTA's shared memory; the bytes are counted on an mbarrier that may sit in the peer CTA
__device__ __forceinline__ void tma_load_3d_pair(void* smem_dst, const void* tmap, uint32_t bar_cluster_addr, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"((uint64_t)tmap), "r"(bar_cluster_addr), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t* smem_slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
template <bool ACC>
__device__ __forceinline__ void umma_ss2(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "n"(ACC ? 1 : 0)
      : "memory");
}
// one arrival on the mbarrier at this shared::cluster address once every MMA issued so far has finished
__device__ __forceinline__ void umma_commit2(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr) : "memory");
}

template <int BN_, bool PAIR_ = false>
struct Cfg {
  static constexpr int BN = BN_;
  static constexpr int BN_CTA = PAIR_ ? BN / 2 : BN;          // columns of Wt this CTA stages
  static constexpr int B_BYTES = BK * BN_CTA * 2;             // BN_CTA / 64 blocks
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;       // 48 KB or 32 KB
  static constexpr int STAGES = STAGE_BYTES == 48 * 1024 ? 4 : 6;
  static constexpr int SMEM = STAGES * STAGE_BYTES + 256 + 1024;
};
}  // namespace gemm

template <int BN, bool PAIR>
__global__ void __launch_bounds__(gemm::THREADS, 1)
gemm_bf16_sm100(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmA2,
                const __grid_constant__ CUtensorMap tmW2, const GemmParams p) {
  using namespace gemm;
  using C = Cfg<BN, PAIR>;
  constexpr int STAGES = C::STAGES, STAGE_BYTES = C::STAGE_BYTES;
  constexpr int TILE_M = PAIR ? 2 * BM : BM;             // rows of an output tile (of the pair's)
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* bars = (uint64_t*)(smem + STAGES * STAGE_BYTES);
  uint64_t* full = bars;                 // [STAGES] TMA landed (PAIR: the leader's count both CTAs' bytes)
  uint64_t* empty = bars + STAGES;       // [STAGES] MMAs that read the stage have finished
  uint64_t* acc_full = empty + STAGES;   // [2] accumulator complete
  uint64_t* acc_empty = acc_full + 2;    // [2] accumulator drained by the epilogue warps (PAIR: the leader's, by both CTAs')
  uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
  volatile uint32_t* abort_word = (volatile uint32_t*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;     // 0 = leader
  const int worker = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x, workers = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  const int mt = (p.M + TILE_M - 1) / TILE_M, nt = (p.N + BN - 1) / BN;
  // the optional second product (A2 x W2, the reference's LoRA term, gemm.metal:46-50) is just more k-blocks
  // accumulated into the same tile before the epilogue
  const int kb1 = (p.K + BK - 1) / BK, kblocks = kb1 + (p.K2 + BK - 1) / BK;
  const int tiles = mt * nt;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; a++) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], PAIR ? 256 : 128);
    }
    abort_word[0] = (p.status != nullptr && *p.status != 0u) ? 0xFFu : 0u;
    fence_mbar_init();
  }
  if (warp == 1) {
    if constexpr (PAIR) {
      tmem_alloc2(tmem_slot, 2 * BN);      // one warp of each CTA of the pair
      tmem_relinquish2();
    } else {
      tmem_alloc(tmem_slot, 2 * BN);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (PAIR) cluster_sync_all();  // the peer's barriers are initialised, both allocations are done
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // tile t -> (m tile, n tile): tiles are dealt out in groups of GROUP_M row blocks x all column blocks, row
  // block fastest inside a group.  The CTAs running together then share GROUP_M row blocks of A and a few column
  // blocks of Wt; the host sizes the group so that its slice of A (tens of MB at most) stays in L2 while the group
  // sweeps the columns: Wt is then streamed from HBM once per group and A once.
  const int GROUP_M = p.group_m;
  auto tile_origin = [&](int t, int& m0, int& n0) {
    const int per_group = GROUP_M * nt;
    const int g = t / per_group, first = g * GROUP_M;
    const int gm = min(GROUP_M, mt - first);
    const int local = t - g * per_group;
    m0 = (first + local % gm) * TILE_M + (int)rank * BM;      // this CTA's rows of the tile
    n0 = (local / gm) * BN;
  };
  if (warp == 0) {
    // ======================================= TMA producer =======================================
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmW);
      if (p.K2 > 0) {
        tma_prefetch_desc(&tmA2);
        tma_prefetch_desc(&tmW2);
      }
      uint32_t n = 0;     // k-blocks issued so far
      for (int t = worker; t < tiles && *abort_word == 0u; t += workers) {
        int m0, n0;
        tile_origin(t, m0, n0);
        for (int kb = 0; kb < kblocks; kb++, n++) {
          const int s = n % STAGES;
          if (!mbar_wait(&empty[s], ((n / STAGES) & 1) ^ 1, abort_word, SITE_EMPTY)) break;
          uint8_t* a_dst = smem + s * STAGE_BYTES;
          uint8_t* b_dst = a_dst + A_BYTES;
          const CUtensorMap* ma = kb < kb1 ? &tmA : &tmA2;
          const CUtensorMap* mw = kb < kb1 ? &tmW : &tmW2;
          const int k0 = (kb < kb1 ? kb : kb - kb1) * BK;
          if constexpr (PAIR) {
            // both CTAs' bytes are counted on the leader's barrier, which the leader arms for both
            if (rank == 0) mbar_arrive_expect_tx(&full[s], 2 * STAGE_BYTES);
            const uint32_t bar = mapa(smem_u32(&full[s]), 0);
            tma_load_3d_pair(a_dst, ma, bar, k0, m0, 0);
#pragma unroll
            for (int j = 0; j < C::BN_CTA / 64; j++)
              tma_load_3d_pair(b_dst + j * B_BLOCK, mw, bar, n0 + (int)rank * C::BN_CTA + j * 64, k0, 0);
          } else {
            mbar_arrive_expect_tx(&full[s], STAGE_BYTES);
            tma_load_3d(a_dst, ma, &full[s], k0, m0, 0);
#pragma unroll
            for (int j = 0; j < BN / 64; j++) tma_load_3d(b_dst + j * B_BLOCK, mw, &full[s], n0 + j * 64, k0, 0);
          }
        }
      }
      // nothing may still be in flight into this CTA's shared memory when it exits
      if (*abort_word != 0u && (!PAIR || rank == 0)) {
        for (uint32_t i = (n > STAGES ? n - STAGES : 0); i < n; i++)
          mbar_wait_slow(&full[i % STAGES], (i / STAGES) & 1, abort_word + 1, SITE_FULL);
      }
    }
  } else if (warp == 1 && rank == 0) {
    // ======================================== MMA issuer ========================================
    // (PAIR: the leader CTA's only; A rows 0-127 and Wt columns 0-127 of a product come from its shared memory, the
    // others from the same offsets of the peer's; accumulator rows 128-255 live in the peer's tensor memory)
    const bool leader = elect_one();
    constexpr uint32_t idesc = umma_idesc_bf16(TILE_M, BN, true);
    constexpr uint32_t HI = desc_hi(1024);
    constexpr uint32_t LBO_A = (16u >> 4) << 16;                       // K-major: unused
    constexpr uint32_t LBO_B = ((uint32_t)B_BLOCK >> 4) << 16;         // N-major: next 64 columns 8 KB away
    const uint32_t smem_lo = smem_u32(smem) >> 4;
    uint32_t n = 0;
    int it = 0;
    for (int t = worker; t < tiles; t += workers, it++) {
      const int a = it & 1;
      if (it >= 2) {
        if (!mbar_wait(&acc_empty[a], ((it >> 1) - 1) & 1, abort_word, SITE_ACC_EMPTY)) break;
        tc_fence_after();
      }
      const uint32_t d_tmem = tmem_base + a * BN;
      for (int kb = 0; kb < kblocks; kb++, n++) {
        const int s = n % STAGES;
        if (!mbar_wait(&full[s], (n / STAGES) & 1, abort_word, SITE_FULL)) break;
        tc_fence_after();
        const uint32_t a_lo = (smem_lo + s * (STAGE_BYTES >> 4)) | LBO_A;
        const uint32_t b_lo = (smem_lo + s * (STAGE_BYTES >> 4) + (A_BYTES >> 4)) | LBO_B;
#pragma unroll
        for (int k = 0; k < BK / 16; k++) {
          const uint64_t da = make_desc(a_lo + k * 2, HI), db = make_desc(b_lo + k * 128, HI);   // 32 B / 2048 B per 16 k
          if (leader) {
            if constexpr (PAIR) {
              if (kb == 0 && k == 0) umma_ss2<false>(d_tmem, da, db, idesc);
              else umma_ss2<true>(d_tmem, da, db, idesc);
            } else {
              if (kb == 0 && k == 0) umma_ss<false>(d_tmem, da, db, idesc);
              else umma_ss<true>(d_tmem, da, db, idesc);
            }
          }
        }
        if (leader) {
          if constexpr (PAIR) {
            umma_commit2(mapa(smem_u32(&empty[s]), 0));
            umma_commit2(mapa(smem_u32(&empty[s]), 1));
          } else {
            umma_commit(&empty[s]);
          }
        }
        __syncwarp();
      }
      if (leader) {
        if constexpr (PAIR) {
          umma_commit2(mapa(smem_u32(&acc_full[a]), 0));
          umma_commit2(mapa(smem_u32(&acc_full[a]), 1));
        } else {
          umma_commit(&acc_full[a]);
        }
      }
      __syncwarp();
      if (*abort_word != 0u) break;
    }
  } else if (warp == 2) {
    // an otherwise idle warp of CTA 0: the logit bound that the normalised Q and K of this product obey
    if (p.epi == 1 && p.bound_out != nullptr && blockIdx.x == 0) {
      const float4 a = __ldg((const float4*)p.wq + lane), c = __ldg((const float4*)p.wk + lane);
      float mq = fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(a.z), fabsf(a.w)));
      float mk = fmaxf(fmaxf(fabsf(c.x), fabsf(c.y)), fmaxf(fabsf(c.z), fabsf(c.w)));
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        mq = fmaxf(mq, __shfl_xor_sync(0xffffffffu, mq, o));
        mk = fmaxf(mk, __shfl_xor_sync(0xffffffffu, mk, o));
      }
      if (lane == 0) *p.bound_out = 128.0f * mq * mk * p.bound_scale_log2 * 1.02f;
    }
  } else if (warp >= 4) {
    // ========================================= epilogue =========================================
    const int r = (warp & 3) * 32 + lane;                 // row of the tile = TMEM lane
    const uint32_t lane_addr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
    int it = 0;
    for (int t = worker; t < tiles; t += workers, it++) {
      const int a = it & 1;
      int m0, n0;
      tile_origin(t, m0, n0);
      if (!mbar_wait(&acc_full[a], (it >> 1) & 1, abort_word, SITE_ACC_FULL)) break;
      tc_fence_after();
      const int row = m0 + r;
      __nv_bfloat16* crow = p.C + (size_t)min(row, p.M - 1) * p.ldc;
      if (p.epi == 2) {
        // X(f32)[row, col] += vec[col] * acc (gated residual, gemm.metal:262-264); vec == nullptr: X += acc (:265-267)
        float* xrow = (float*)p.C + (size_t)min(row, p.M - 1) * p.ldc;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          const int col0 = n0 + c0;
          if (col0 >= p.N) break;
          uint32_t v[32];
          tmem_ld32(lane_addr + a * BN + c0, v);
          tmem_wait_ld();
          if (row < p.M) {
#pragma unroll
            for (int q4 = 0; q4 < 8; q4++) {
              const int col = col0 + q4 * 4;
              if (col + 4 <= p.N) {
                float4 x = *(float4*)(xrow + col);
                const float4 gt = p.vec ? __ldg((const float4*)(p.vec + col)) : make_float4(1.f, 1.f, 1.f, 1.f);
                x.x = fmaf(gt.x, __uint_as_float(v[q4 * 4]), x.x);
                x.y = fmaf(gt.y, __uint_as_float(v[q4 * 4 + 1]), x.y);
                x.z = fmaf(gt.z, __uint_as_float(v[q4 * 4 + 2]), x.z);
                x.w = fmaf(gt.w, __uint_as_float(v[q4 * 4 + 3]), x.w);
                *(float4*)(xrow + col) = x;
              }
            }
          }
        }
      } else if (p.epi == 3) {
        // SwiGLU on tile-interleaved weights (gemm.metal:233-250): every 64 weight columns hold 32 gate columns,
        // then the 32 matching up columns; output column (n / 64) * 32 + i = silu(gate_i) * up_i, bf16
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 64) {
          const int col0 = n0 + c0;
          if (col0 >= p.N) break;
          uint32_t g[32], u[32];
          tmem_ld32(lane_addr + a * BN + c0, g);
          tmem_ld32(lane_addr + a * BN + c0 + 32, u);
          tmem_wait_ld();
          if (row < p.M) {
            const int ocol0 = (col0 >> 6) * 32;
            uint32_t pk[16];
#pragma unroll
            for (int q4 = 0; q4 < 4; q4++) {
              float f[8];
#pragma unroll
              for (int e = 0; e < 8; e++) {
                const float gv = __uint_as_float(g[q4 * 8 + e]);
                f[e] = gv * sigmoid_approx(gv) * __uint_as_float(u[q4 * 8 + e]);      // common.h silu
              }
#pragma unroll
              for (int e = 0; e < 4; e++) pk[q4 * 4 + e] = pack_bf16x2(f[2 * e], f[2 * e + 1]);
            }
            if ((((uintptr_t)(crow + ocol0)) & 31u) == 0) {     // whole 32-byte sectors per store when the row allows it
              st_global_32B(crow + ocol0, pk);
              st_global_32B(crow + ocol0 + 16, pk + 8);
            } else {
#pragma unroll
              for (int q4 = 0; q4 < 4; q4++) *(uint4*)(crow + ocol0 + q4 * 8) = make_uint4(pk[q4 * 4], pk[q4 * 4 + 1], pk[q4 * 4 + 2], pk[q4 * 4 + 3]);
            }
          }
        }
      } else if (p.epi >= 4) {
        // Epi::F32 (4), Epi::GELU (5), Epi::BiasBF16 (6), Epi::BiasF32 (7): gemm.metal:257-260, 268-277
        const bool f32_out = p.epi == 4 || p.epi == 7;
        float* xrow = (float*)p.C + (size_t)min(row, p.M - 1) * p.ldc;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          const int col0 = n0 + c0;
          if (col0 >= p.N) break;
          uint32_t v[32];
          tmem_ld32(lane_addr + a * BN + c0, v);
          tmem_wait_ld();
          if (row < p.M) {
#pragma unroll
            for (int q4 = 0; q4 < 4; q4++) {
              const int col = col0 + q4 * 8;
              if (col + 8 > p.N) continue;
              float f[8];
#pragma unroll
              for (int e = 0; e < 8; e++) f[e] = __uint_as_float(v[q4 * 8 + e]);
              if (p.epi >= 6) {
                const float4 b0 = __ldg((const float4*)(p.vec + col)), b1 = __ldg((const float4*)(p.vec + col) + 1);
                f[0] += b0.x; f[1] += b0.y; f[2] += b0.z; f[3] += b0.w; f[4] += b1.x; f[5] += b1.y; f[6] += b1.z; f[7] += b1.w;
              } else if (p.epi == 5) {
#pragma unroll
                for (int e = 0; e < 8; e++) {          // common.h:26-29 gelu_tanh
                  const float x = f[e];
                  f[e] = 0.5f * x * (1.0f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
                }
              }
              if (f32_out) {
                *(float4*)(xrow + col) = make_float4(f[0], f[1], f[2], f[3]);
                *(float4*)(xrow + col + 4) = make_float4(f[4], f[5], f[6], f[7]);
              } else {
                *(uint4*)(crow + col) = make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
              }
            }
          }
        }
      } else
#pragma unroll 1
      for (int hb = 0; hb < BN / 128; hb++) {             // one block of 128 columns (one head) at a time
        const int col0 = n0 + hb * 128;
        if (col0 >= p.N) break;
        // which treatment this block of columns gets: 0 plain, 1 Q head, 2 K head
        int kind = 0, head = 0;
        if (p.epi == 1) {
          if (col0 >= p.q_off && col0 < p.q_off + p.n_q * 128) { kind = 1; head = (col0 - p.q_off) >> 7; }
          else if (col0 >= p.k_off && col0 < p.k_off + p.n_k * 128) { kind = 2; head = (col0 - p.k_off) >> 7; }
        }
        float rrms = 1.f;
        if (kind != 0) {
          // pass 1 over the accumulator: sum of squares of the row's 128 values of this head
          float ss = 0.f;
#pragma unroll 1
          for (int c0 = 0; c0 < 128; c0 += 32) {
            uint32_t v[32];
            tmem_ld32(lane_addr + a * BN + hb * 128 + c0, v);
            tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < 32; e++) ss = fmaf(__uint_as_float(v[e]), __uint_as_float(v[e]), ss);
          }
          rrms = rsqrtf(ss * (1.0f / 128.0f) + p.eps);                       // norm.metal:102
        }
        const float* w = kind == 1 ? p.wq : p.wk;
        const size_t trow = (size_t)(p.row0 + min(row, p.M - 1)) * 64;
#pragma unroll 1
        for (int c0 = 0; c0 < 128; c0 += 32) {
          uint32_t v[32];
          tmem_ld32(lane_addr + a * BN + hb * 128 + c0, v);
          tmem_wait_ld();
          float f[32];
#pragma unroll
          for (int e = 0; e < 32; e++) f[e] = __uint_as_float(v[e]);
          if (kind != 0) {
#pragma unroll
            for (int e4 = 0; e4 < 8; e4++) {
              const float4 wv = __ldg((const float4*)(w + c0) + e4);
              f[4 * e4] *= rrms * wv.x; f[4 * e4 + 1] *= rrms * wv.y; f[4 * e4 + 2] *= rrms * wv.z; f[4 * e4 + 3] *= rrms * wv.w;
            }
            if (p.rope_mode == 0) {
              // interleaved pairs (2i, 2i+1) turn by the row's entry i (norm.metal:105-113): pairs c0/2 .. c0/2+15
#pragma unroll
              for (int e4 = 0; e4 < 4; e4++) {
                const float4 cc = __ldg((const float4*)(p.cos + trow + (c0 >> 1)) + e4), sc = __ldg((const float4*)(p.sin + trow + (c0 >> 1)) + e4);
                const float cf[4] = {cc.x, cc.y, cc.z, cc.w}, sf[4] = {sc.x, sc.y, sc.z, sc.w};
#pragma unroll
                for (int q = 0; q < 4; q++) {
                  const float x0 = f[8 * e4 + 2 * q], x1 = f[8 * e4 + 2 * q + 1];
                  f[8 * e4 + 2 * q] = x0 * cf[q] - x1 * sf[q];
                  f[8 * e4 + 2 * q + 1] = x0 * sf[q] + x1 * cf[q];
                }
              }
            }
          }
          if (kind != 0 && p.big_dim >= 0 && (p.big_dim >> 5) == (c0 >> 5)) {
            // this head's big dimension: fp32 side buffer, zero in the bf16 row (norm.metal:127-132)
            const int e = p.big_dim & 31;
            float v = 0.f;
#pragma unroll
            for (int k = 0; k < 32; k++)
              if (k == e) { v = f[k]; f[k] = 0.f; }
            if (row < p.M) {
              if (kind == 1) p.qbig[(size_t)row * p.n_q + head] = v;
              else p.kbig[(size_t)row * p.n_k + head] = v;
            }
          }
          // 64 contiguous bytes of the row: two stores of a whole 32-byte sector each when the row allows it (a
          // 16-byte store to 32 different rows fills every sector in two halves)
          if (row < p.M && p.seg <= 0 && col0 + c0 + 32 <= p.N && (((uintptr_t)(crow + col0 + c0)) & 31u) == 0) {
            uint32_t pk[16];
#pragma unroll
            for (int e = 0; e < 16; e++) pk[e] = pack_bf16x2(f[2 * e], f[2 * e + 1]);
            st_global_32B(crow + col0 + c0, pk);
            st_global_32B(crow + col0 + c0 + 16, pk + 8);
          } else if (row < p.M) {
#pragma unroll
            for (int q4 = 0; q4 < 4; q4++) {
              const int col = col0 + c0 + q4 * 8;
              // optional column remap of the plain store (gemm.metal:41-43, 255-256): segments of `seg` columns land
              // seg_stride apart; seg is a multiple of 8, so an 8-column chunk never straddles two segments
              const int ocol = p.seg > 0 ? (col / p.seg) * p.seg_stride + col % p.seg : col;
              if (col + 8 <= p.N)
                *(uint4*)(crow + ocol) = make_uint4(pack_bf16x2(f[q4 * 8], f[q4 * 8 + 1]), pack_bf16x2(f[q4 * 8 + 2], f[q4 * 8 + 3]),
                                                   pack_bf16x2(f[q4 * 8 + 4], f[q4 * 8 + 5]), pack_bf16x2(f[q4 * 8 + 6], f[q4 * 8 + 7]));
            }
          }
        }
      }
      tc_fence_before();
      if constexpr (PAIR) mbar_arrive_cluster(mapa(smem_u32(&acc_empty[a]), 0));   // the leader's barrier counts both CTAs' threads
      else mbar_arrive(&acc_empty[a]);
    }
  }

  // (PAIR) nobody leaves or frees tensor memory while the peer may still read this CTA's shared memory, signal its
  // barriers or write its accumulator
  tc_fence_before();
  __syncthreads();
  if constexpr (PAIR) cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    if constexpr (PAIR) tmem_dealloc2(tmem_base, 2 * BN);
    else tmem_dealloc(tmem_base, 2 * BN);
  }
  if (threadIdx.x == 0 && p.status != nullptr) {
    const uint32_t a = *abort_word;
    if (a != 0u && a != 0xFFu) atomicCAS(p.status, 0u, a | ((uint32_t)blockIdx.x << 8));
  }
}

template <int BN, bool PAIR>
static cudaError_t launch_gemm_variant(const CUtensorMap& tmA, const CUtensorMap& tmW, const CUtensorMap& tmA2, const CUtensorMap& tmW2, GemmParams p,
                                       int sms, cudaStream_t stream) {
  using namespace gemm;
  static bool configured[64] = {};
  static std::mutex configure_mutex;       // handles on several threads may launch at the same time
  int dev = 0;
  cudaGetDevice(&dev);
  {
    std::lock_guard<std::mutex> lock(configure_mutex);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
      cudaError_t e = cudaFuncSetAttribute(gemm_bf16_sm100<BN, PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<BN, PAIR>::SMEM);
      if (e != cudaSuccess) return e;
      configured[dev] = true;
    }
  }
  constexpr int TILE_M = PAIR ? 2 * BM : BM;
  const int tiles = ((p.M + TILE_M - 1) / TILE_M) * ((p.N + BN - 1) / BN);
  // as many workers (CTAs, or CTA pairs) as the waves need: 1080 tiles on 74 pairs take 15 waves, and so they do on 72
  // pairs, with four SMs' worth of power left to the others' clocks
  int workers = PAIR ? sms / 2 : sms;
  if (tiles < workers) workers = tiles;
  const int waves = (tiles + workers - 1) / workers;
  workers = (tiles + waves - 1) / waves;
  const int grid = workers * (PAIR ? 2 : 1);
  // row blocks per group: the group's slice of A (rows x K, 32 MB at most) should stay in L2 while the group sweeps
  // the columns; groups of equal size (measured at 4608 x 15360 x 6144: groups of 8-9 row blocks of 256 rows 1512-1528
  // TFLOP/s, of 4: 1468, of 18: 1490; at K = 3072 all 18 in one group 1511, two groups of 16 + 2: 1494)
  const long long k_all = (long long)p.K + p.K2;
  const int mt = (p.M + TILE_M - 1) / TILE_M;
  long long gmax = (32ll << 20) / (k_all * 2 * TILE_M);
  if (gmax < 1) gmax = 1;
  const int groups = (int)((mt + gmax - 1) / gmax);
  p.group_m = (mt + groups - 1) / groups;
  static const int group_m_knob = [] { const char* e = getenv("KREA_CUDA_GEMM_GROUP_M"); return e ? atoi(e) : 0; }();   // tuning knob
  if (group_m_knob > 0) p.group_m = group_m_knob;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = Cfg<BN, PAIR>::SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = PAIR ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, gemm_bf16_sm100<BN, PAIR>, tmA, tmW, tmA2, tmW2, (const GemmParams)p);
}

cudaError_t launch_gemm_bf16_sm100(const CUtensorMap& tmA, const CUtensorMap& tmW, const CUtensorMap& tmA2, const CUtensorMap& tmW2, const GemmParams& p,
                                   int sms, int force_bn, cudaStream_t stream) {
  using namespace gemm;
  if (p.M <= 0 || p.N <= 0 || p.K <= 0) return cudaSuccess;
  // share of the CTAs' time slots that do work when the tiles are dealt out in waves of `sms`
  auto wave_eff = [&](int bn) {
    const long long tiles = (long long)((p.M + BM - 1) / BM) * ((p.N + bn - 1) / bn);
    const long long waves = (tiles + sms - 1) / sms;
    return (double)tiles / (double)(waves * sms);
  };
  // the narrow tile moves a third more bytes through shared memory per flop and measures ~20 % slower per tile
  // (1100 against 1340 TFLOP/s on full waves), so it has to fill the waves a good deal better to win
  const bool narrow = force_bn == 128 || (force_bn == 0 && wave_eff(128) > wave_eff(256) * 1.3);
  if (narrow) return launch_gemm_variant<128, false>(tmA, tmW, tmA2, tmW2, p, sms, stream);
  // 256 x 256 tiles on CTA pairs: 7 % faster per tile (a third fewer bytes into shared memory), with half as many,
  // twice as large units of work to fill the last wave with
  const int pairs = sms / 2;
  const long long ptiles = (long long)((p.M + 2 * BM - 1) / (2 * BM)) * ((p.N + 255) / 256);
  const double pair_eff = pairs > 0 ? (double)ptiles / (double)(((ptiles + pairs - 1) / pairs) * pairs) : 0.0;
  const bool pair = pairs > 0 && (force_bn == 512 || (force_bn == 0 && pair_eff * 1.07 >= wave_eff(256)));
  return pair ? launch_gemm_variant<256, true>(tmA, tmW, tmA2, tmW2, p, sms, stream) : launch_gemm_variant<256, false>(tmA, tmW, tmA2, tmW2, p, sms, stream);
}

}  // namespace krea
