// Private to the library: the handle behind `krea_cuda*` and the error helpers shared by its source files.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>

#include <string>
#include <utility>
#include <vector>

#include "../../include/krea_cuda.h"

struct KreaDist;   // NCCL state of the sequence-parallel entry points (dist_nccl.cu)

typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                    const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct krea_cuda {
  int device = 0;
  cudaStream_t own_stream = nullptr;
  cudaStream_t stream = nullptr;
  std::string err;
  uint32_t* status_dev = nullptr;   // kernels report timed-out waits here; words [64, 64 + 2 * kKeyCounters) are the
                                    // two sets of key-slice counters of the fused call (see AttnParams::kcount)
  static constexpr int kKeyCounters = 1024;
  uint64_t kfuse_seq = 0;           // launches that used the counters so far: launch n counts in set n & 1
  bool kfuse = false;               // fused call: K is normalised inside the persistent attention kernel instead of by
                                    // a kernel of its own (measured slower at every benchmark shape: off by default)
  uint32_t* status_host = nullptr;  // pinned mirror
  void* ws = nullptr;               // scratch for the normalised K of the joint call
  size_t ws_bytes = 0;
  void* stage[8] = {};              // device copies for the host-pointer entry point
  size_t stage_bytes[8] = {};
  uint64_t launches = 0;
  PFN_encodeTiled encode = nullptr;
  int split = 1;                    // softmax threads per query row
  int emu = 0;                      // 1: one of every 4 element pairs takes the polynomial exp2
  int persist = 1;                  // persistent attention kernel (one CTA per SM walking over the work items):
                                    // 0 never, 1 when there are more items than SMs, 2 always
  bool pdl = true;                  // fused call: pre-pass and attention use programmatic dependent launch
  bool q_tma = true;                // plain attention operator: Q tiles arrive as TMA loads
  bool o_tma = true;                // attention output tiles leave shared memory as TMA stores
  bool static_bound = true;         // let the fused call replace the running max by the QK-norm logit bound
  cudaStream_t copy_in = nullptr, copy_out = nullptr;   // host entry point: H2D and D2H streams
  cudaEvent_t pipe_ev[18] = {};                   // [0,8) group in, [8,16) group out, 16 start, 17 bounce
  void* bounce = nullptr;           // pinned host staging for the small operands of the host entry point
  size_t bounce_bytes = 0;
  bool profiling = false;
  std::vector<std::pair<cudaEvent_t, cudaEvent_t>> marks[4];   // pending (start, stop) pairs per kind of work
  std::vector<cudaEvent_t> event_pool;
  cudaEvent_t trace_base = nullptr;   // recorded by krea_cuda_profile_enable(h, 1): time zero of the trace file
  KreaDist* dist = nullptr;         // set by krea_cuda_dist_init
  int gemm_bn = 0;                  // GEMM tile: 0 = chosen per problem; 128 or 256 = one-CTA tile of that width,
                                    // 512 = 256 x 256 tile on a CTA pair
  int sm_count = 0;                 // SMs of the device (persistent kernels size their grid by it)
  void* block_ws = nullptr;         // intermediates of krea_cuda_dit_block when the caller passes no workspace
  size_t block_ws_bytes = 0;
  void* qw_stage = nullptr;         // pinned staging of krea_cuda_qw_upload (two 8 MiB halves)
  uint64_t wait_limit_ns = 2000000000ull;   // bound on every wait inside the attention kernel (krea_cuda_set_wait_limit)
  int test_drop_last_k = 0;         // krea_cuda_test_drop_one_load: the next attention launches never request their last K tile
};

static inline int fail(krea_cuda* h, int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  if (h) h->err = buf;
  return code;
}
#define CUDA_TRY(h, expr)                                                                       \
  do {                                                                                          \
    cudaError_t e_ = (expr);                                                                    \
    if (e_ != cudaSuccess) return fail(h, KREA_CUDA_E_CUDA, "%s: %s", #expr, cudaGetErrorString(e_)); \
  } while (0)

static inline bool aligned16(const void* p) { return ((uintptr_t)p & 15u) == 0; }


// Brackets one kernel launch with events while profiling is on (kind 0 = prologue,
// 1 = attention, 2 = exchange kernels and copies of the sequence-parallel step, 3 = its rank barriers).
struct ProfileMark {
  krea_cuda* h;
  int kind;
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  static cudaEvent_t get(krea_cuda* h) {
    if (!h->event_pool.empty()) {
      cudaEvent_t e = h->event_pool.back();
      h->event_pool.pop_back();
      return e;
    }
    cudaEvent_t e = nullptr;
    cudaEventCreate(&e);
    return e;
  }
  ProfileMark(krea_cuda* h_, int kind_) : h(h_), kind(kind_) {
    if (!h->profiling) return;
    e0 = get(h);
    e1 = get(h);
    if (e0) cudaEventRecord(e0, h->stream);
  }
  ~ProfileMark() {
    if (!e0 || !e1) return;
    cudaEventRecord(e1, h->stream);
    h->marks[kind].push_back({e0, e1});
  }
};

// Implemented in krea_cuda.cu for the other source files of the library.
// the fused call in two steps: K normalisation pass (+ logit bound), then the attention kernel
int krea_joint_prepass(krea_cuda* h, const krea_cuda_joint_args* a, void* k_scratch);
int krea_joint_attend(krea_cuda* h, const krea_cuda_joint_args* a, void* k_scratch);
// ... with output row r stored under o_blk[r / rows] (n bases, possibly in other GPUs' memory) instead of a->O
int krea_joint_attend_scatter(krea_cuda* h, const krea_cuda_joint_args* a, void* k_scratch, void* const* o_blk, int n, int rows);
int krea_validate_joint(krea_cuda* h, const krea_cuda_joint_args* a);
// Implemented in dist_nccl.cu: releases the communicator and its workspace (called by krea_cuda_destroy).
void krea_dist_release(krea_cuda* h);
