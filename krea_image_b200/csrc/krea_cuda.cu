// libkrea_cuda: the C ABI declared in include/krea_cuda.h.  Host side only: argument validation (so a bad
// call can never reach the GPU), tensor-map construction, stream handling, error strings.  The entry
// points mirror the reference's operator dispatch (engine/src/metal.mm:182-202) and its C ABI
// conventions (engine/src/pipeline.mm:594-630: catch everything, return a status, copy a message).
#include <cuda.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <mutex>
#include <string>
#include <utility>
#include <vector>

#include "../../include/krea_cuda.h"
#include "attention_sm100.h"
#include "handle.h"

using namespace krea;

// Scratch of krea_cuda_joint_attention_static (the normalised and rotated K that the pre-pass hands to the
// attention kernel): a fixed array in the library's device image instead of memory obtained at run time.
// In host code the array's name is only a stand-in for the device symbol - it is not a device address - so
// the address is looked up per device with cudaGetSymbolAddress (with that device current) and that pointer
// is what the kernels get.  The lookup is where the CUDA runtime loads this file's device image, i.e. where
// the driver sets the array's 32 MiB aside on that GPU, so it happens in krea_cuda_create - at start-up, when
// memory is still there to be had - and never inside a call of the entry point itself.
static __device__ __align__(256) unsigned char g_static_k_scratch[KREA_CUDA_STATIC_SCRATCH_BYTES];
static void* g_static_k_scratch_ptr[64] = {};
static std::mutex g_static_k_scratch_mutex;

// Device address of the array on `device`, which must be the current device.  nullptr + *e on failure.
static void* static_scratch_on(int device, cudaError_t* e) {
  *e = cudaSuccess;
  if (device < 0 || device >= 64) {
    *e = cudaErrorInvalidDevice;
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_static_k_scratch_mutex);
  if (g_static_k_scratch_ptr[device] == nullptr) {
    void* ptr = nullptr;
    *e = cudaGetSymbolAddress(&ptr, g_static_k_scratch);
    if (*e != cudaSuccess || ptr == nullptr) {
      if (*e == cudaSuccess) *e = cudaErrorInvalidSymbol;
      return nullptr;
    }
    g_static_k_scratch_ptr[device] = ptr;
  }
  return g_static_k_scratch_ptr[device];
}

extern "C" {

krea_cuda* krea_cuda_create(int device, char* err, int errlen) {
  auto say = [&](const char* m, const char* d) {
    if (err && errlen > 0) snprintf(err, (size_t)errlen, "%s%s", m, d ? d : "");
  };
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess || n <= 0) {
    say("krea_cuda_create: no CUDA device: ", cudaGetErrorString(e));
    return nullptr;
  }
  if (device < 0 || device >= n) {
    say("krea_cuda_create: device index out of range", nullptr);
    return nullptr;
  }
  cudaDeviceProp prop;
  if ((e = cudaGetDeviceProperties(&prop, device)) != cudaSuccess) {
    say("krea_cuda_create: ", cudaGetErrorString(e));
    return nullptr;
  }
  if (prop.major != 10) {
    say("krea_cuda_create: this library contains sm_100a code only (Blackwell B200 required)", nullptr);
    return nullptr;
  }
  krea_cuda* h = new krea_cuda();
  h->device = device;
  bool ok = cudaSetDevice(device) == cudaSuccess;
  ok = ok && cudaStreamCreateWithFlags(&h->own_stream, cudaStreamNonBlocking) == cudaSuccess;
  const size_t status_bytes = 256 + 2 * (size_t)krea_cuda::kKeyCounters * 4;
  ok = ok && cudaMalloc((void**)&h->status_dev, status_bytes) == cudaSuccess;
  ok = ok && cudaMemset(h->status_dev, 0, status_bytes) == cudaSuccess;
  ok = ok && cudaMallocHost((void**)&h->status_host, 256) == cudaSuccess;
  if (ok) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    ok = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess && fn != nullptr;
    h->encode = (PFN_encodeTiled)fn;
  }
  if (ok && device < 64) {
    // resolve the built-in scratch of krea_cuda_joint_attention_static now (see g_static_k_scratch)
    cudaError_t se;
    ok = static_scratch_on(device, &se) != nullptr;
  }
  if (!ok) {
    say("krea_cuda_create: CUDA initialisation failed: ", cudaGetErrorString(cudaGetLastError()));
    krea_cuda_destroy(h);
    return nullptr;
  }
  h->stream = h->own_stream;
  if (const char* s = getenv("KREA_CUDA_SPLIT")) {  // tuning knob: 1 or 2 softmax threads per query row
    const int v = atoi(s);
    if (v == 1 || v == 2) h->split = v;
  }
  if (const char* s = getenv("KREA_CUDA_STATIC_BOUND")) h->static_bound = atoi(s) != 0;   // tuning knob
  if (const char* s = getenv("KREA_CUDA_PERSIST")) {  // tuning knob: persistent attention kernel never / by problem size / always
    const int v = atoi(s);
    if (v >= 0 && v <= 2) h->persist = v;
  }
  if (const char* s = getenv("KREA_CUDA_KFUSE")) h->kfuse = atoi(s) != 0;                 // option: K normalised inside the attention kernel
  if (const char* s = getenv("KREA_CUDA_PDL")) h->pdl = atoi(s) != 0;                     // tuning knob
  if (const char* s = getenv("KREA_CUDA_O_TMA")) h->o_tma = atoi(s) != 0;                 // tuning knob
  if (const char* s = getenv("KREA_CUDA_Q_TMA")) h->q_tma = atoi(s) != 0;                 // tuning knob
  if (const char* s = getenv("KREA_CUDA_GEMM_BN")) {                                      // tuning knob: GEMM tile width
    const int v = atoi(s);
    if (v == 128 || v == 256 || v == 512) h->gemm_bn = v;     // 512: 256 x 256 tiles on CTA pairs
  }
  if (const char* s = getenv("KREA_CUDA_EMU")) {  // tuning knob: share of exp2 evaluated on the FMA pipe (0-3 of 4)
    const int v = atoi(s);
    if (v >= 0 && v <= 1) h->emu = v;
  }
  // Load the device code of the fused call's two kernels and opt the attention kernel in to its shared memory
  // now, so that the first call on this device does no set-up of its own (krea_cuda_joint_attention_static
  // relies on this: nothing may be reserved on the device once its callers have given all memory away).
  if (h->split != 1) h->persist = 0;       // the persistent kernel has one softmax thread per row
  {
    cudaDeviceProp prop2;
    if (cudaGetDeviceProperties(&prop2, device) == cudaSuccess) h->sm_count = prop2.multiProcessorCount;
  }
  if ((h->persist ? prepare_attention_persist_sm100(h->emu, false) : cudaSuccess) != cudaSuccess ||
      (h->persist && h->kfuse ? prepare_attention_persist_sm100(h->emu, true) : cudaSuccess) != cudaSuccess || prepare_attention_sm100(h->split, h->emu) != cudaSuccess ||
      prepare_qk_norm_rope() != cudaSuccess) {
    say("krea_cuda_create: kernel set-up failed: ", cudaGetErrorString(cudaGetLastError()));
    krea_cuda_destroy(h);
    return nullptr;
  }
  return h;
}

void krea_cuda_destroy(krea_cuda* h) {
  if (!h) return;
  cudaSetDevice(h->device);
  if (h->own_stream) cudaStreamSynchronize(h->own_stream);
  krea_dist_release(h);
  if (h->status_dev) cudaFree(h->status_dev);
  if (h->status_host) cudaFreeHost(h->status_host);
  if (h->ws) cudaFree(h->ws);
  for (int i = 0; i < 8; i++)
    if (h->stage[i]) cudaFree(h->stage[i]);
  for (int k = 0; k < 4; k++)
    for (auto& m : h->marks[k]) {
      cudaEventDestroy(m.first);
      cudaEventDestroy(m.second);
    }
  for (cudaEvent_t e : h->event_pool) cudaEventDestroy(e);
  if (h->trace_base) cudaEventDestroy(h->trace_base);
  for (int i = 0; i < 18; i++)
    if (h->pipe_ev[i]) cudaEventDestroy(h->pipe_ev[i]);
  if (h->bounce) cudaFreeHost(h->bounce);
  if (h->qw_stage) cudaFreeHost(h->qw_stage);
  if (h->block_ws) cudaFree(h->block_ws);
  if (h->copy_in) cudaStreamDestroy(h->copy_in);
  if (h->copy_out) cudaStreamDestroy(h->copy_out);
  if (h->own_stream) cudaStreamDestroy(h->own_stream);
  delete h;
}

const char* krea_cuda_last_error(krea_cuda* h) { return h ? h->err.c_str() : "null handle"; }

int krea_cuda_set_stream(krea_cuda* h, void* cuda_stream) {
  if (!h) return KREA_CUDA_E_ARG;
  cudaStream_t next = (cudaStream_t)cuda_stream;
  if (next != h->stream) {
    // Kernels queued on the old stream may still use the handle's workspaces, which later calls on the new
    // stream may free and re-allocate: let them finish first (the handle's buffers know one stream at a time).
    CUDA_TRY(h, cudaSetDevice(h->device));
    CUDA_TRY(h, cudaStreamSynchronize(h->stream));
  }
  h->stream = next;
  return KREA_CUDA_OK;
}

uint64_t krea_cuda_launch_count(krea_cuda* h) { return h ? h->launches : 0; }

int krea_cuda_set_wait_limit(krea_cuda* h, uint64_t ns) {
  if (!h) return KREA_CUDA_E_ARG;
  if (ns < 1000000ull || ns > 60000000000ull) return fail(h, KREA_CUDA_E_ARG, "set_wait_limit: the limit must lie between 1 ms and 60 s");
  h->wait_limit_ns = ns;
  return KREA_CUDA_OK;
}

int krea_cuda_test_drop_one_load(krea_cuda* h, int on) {
  if (!h) return KREA_CUDA_E_ARG;
  h->test_drop_last_k = on ? 1 : 0;
  return KREA_CUDA_OK;
}

int krea_cuda_profile_enable(krea_cuda* h, int on) {
  if (!h) return KREA_CUDA_E_ARG;
  CUDA_TRY(h, cudaSetDevice(h->device));
  CUDA_TRY(h, cudaStreamSynchronize(h->stream));
  for (int k = 0; k < 4; k++) {
    for (auto& m : h->marks[k]) {
      h->event_pool.push_back(m.first);
      h->event_pool.push_back(m.second);
    }
    h->marks[k].clear();
  }
  h->profiling = on != 0;
  if (h->profiling) {
    // time zero of krea_cuda_profile_trace
    if (!h->trace_base) CUDA_TRY(h, cudaEventCreate(&h->trace_base));
    CUDA_TRY(h, cudaEventRecord(h->trace_base, h->stream));
  }
  return KREA_CUDA_OK;
}

int krea_cuda_profile_trace(krea_cuda* h, const char* path) {
  if (!h || !path) return fail(h, KREA_CUDA_E_ARG, "profile_trace: null handle or path");
  if (!h->trace_base) return fail(h, KREA_CUDA_E_ARG, "profile_trace: profiling was never enabled");
  CUDA_TRY(h, cudaSetDevice(h->device));
  CUDA_TRY(h, cudaStreamSynchronize(h->stream));
  FILE* f = fopen(path, "w");
  if (!f) return fail(h, KREA_CUDA_E_ARG, "profile_trace: cannot open %s", path);
  static const char* names[4] = {"qk_norm_rope", "attention", "exchange", "rank_barrier"};
  fprintf(f, "{\"traceEvents\":[");
  bool first = true;
  for (int k = 0; k < 4; k++) {
    for (auto& m : h->marks[k]) {
      float t0 = 0.f, dt = 0.f;
      if (cudaEventElapsedTime(&t0, h->trace_base, m.first) != cudaSuccess || cudaEventElapsedTime(&dt, m.first, m.second) != cudaSuccess) {
        cudaGetLastError();
        continue;
      }
      fprintf(f, "%s\n{\"name\":\"%s\",\"ph\":\"X\",\"pid\":%d,\"tid\":%d,\"ts\":%.3f,\"dur\":%.3f}", first ? "" : ",", names[k], h->device, k,
              t0 * 1e3, dt * 1e3);
      first = false;
    }
  }
  fprintf(f, "\n]}\n");
  fclose(f);
  return KREA_CUDA_OK;
}

int krea_cuda_profile_read(krea_cuda* h, int which, double* total_ms, int* launches) {
  if (!h || which < 0 || which > 3 || !total_ms || !launches) return fail(h, KREA_CUDA_E_ARG, "profile_read: bad arguments");
  CUDA_TRY(h, cudaSetDevice(h->device));
  CUDA_TRY(h, cudaStreamSynchronize(h->stream));
  double sum = 0.0;
  for (auto& m : h->marks[which]) {
    float ms = 0.f;
    CUDA_TRY(h, cudaEventElapsedTime(&ms, m.first, m.second));
    sum += ms;
    h->event_pool.push_back(m.first);
    h->event_pool.push_back(m.second);
  }
  *total_ms = sum;
  *launches = (int)h->marks[which].size();
  h->marks[which].clear();
  return KREA_CUDA_OK;
}

int krea_cuda_sync(krea_cuda* h) {
  if (!h) return KREA_CUDA_E_ARG;
  CUDA_TRY(h, cudaSetDevice(h->device));
  CUDA_TRY(h, cudaMemcpyAsync(h->status_host, h->status_dev, 4, cudaMemcpyDeviceToHost, h->stream));
  CUDA_TRY(h, cudaStreamSynchronize(h->stream));
  const uint32_t st = h->status_host[0];
  if (st != 0) {
    cudaMemsetAsync(h->status_dev, 0, 4, h->stream);
    cudaStreamSynchronize(h->stream);
    return fail(h, KREA_CUDA_E_DEVICE, "attention kernel gave up on a bounded wait: site %u, query block %u, head %u",
                st & 0xFFu, (st >> 8) & 0xFFFu, st >> 20);
  }
  return KREA_CUDA_OK;
}

// ---------------------------------------------------------------------------------------------------
int krea_cuda_qk_norm_rope(krea_cuda* h, const krea_cuda_qknorm_args* a) {
  if (!h || !a) return fail(h, KREA_CUDA_E_ARG, "qk_norm_rope: null handle or arguments");
  if (a->rows < 0 || a->n_q < 0 || a->n_k < 0) return fail(h, KREA_CUDA_E_ARG, "qk_norm_rope: negative size");
  if (a->rows == 0 || a->n_q + a->n_k == 0) return KREA_CUDA_OK;
  if (!a->qkv || (a->n_q > 0 && !a->wq) || (a->n_k > 0 && !a->wk)) return fail(h, KREA_CUDA_E_ARG, "qk_norm_rope: null tensor");
  if (a->rope_mode < 0 || a->rope_mode > 2) return fail(h, KREA_CUDA_E_ARG, "qk_norm_rope: rope_mode must be 0, 1 or 2");
  if (a->rope_mode != KREA_CUDA_ROPE_NONE && (!a->cos || !a->sin)) return fail(h, KREA_CUDA_E_ARG, "qk_norm_rope: cos/sin tables missing");
  if (a->ld % 8 || a->q_off % 8 || a->k_off % 8 || !aligned16(a->qkv))
    return fail(h, KREA_CUDA_E_ARG, "qk_norm_rope: ld, q_off, k_off must be multiples of 8 and qkv 16-byte aligned");
  if (a->q_off < 0 || a->k_off < 0 || (a->n_q > 0 && a->q_off + a->n_q * 128 > a->ld) || (a->n_k > 0 && a->k_off + a->n_k * 128 > a->ld))
    return fail(h, KREA_CUDA_E_ARG, "qk_norm_rope: heads do not fit in a row of ld elements");
  if (!aligned16(a->wq) || !aligned16(a->wk) || !aligned16(a->cos) || !aligned16(a->sin))
    return fail(h, KREA_CUDA_E_ARG, "qk_norm_rope: weights and tables must be 16-byte aligned");
  if (a->big_dim >= 128) return fail(h, KREA_CUDA_E_ARG, "qk_norm_rope: big_dim out of range");
  // the reference throws here too (engine/src/metal.mm:185)
  if (a->big_dim >= 0 && (!a->qbig || !a->kbig)) return fail(h, KREA_CUDA_E_ARG, "qk_norm_rope: big_dim needs qbig / kbig");
  NormRopeParams p{};
  p.src = (const __nv_bfloat16*)a->qkv;
  p.dst = (__nv_bfloat16*)a->qkv;
  p.ld_src = p.ld_dst = a->ld;
  p.bs_src = p.bs_dst = 0;
  p.rows = a->rows;
  p.batch = 1;
  p.q_off = p.q_off_dst = a->q_off;
  p.k_off = p.k_off_dst = a->k_off;
  p.n_q = a->n_q;
  p.n_k = a->n_k;
  p.wq = a->wq;
  p.wk = a->wk;
  p.cos = a->cos;
  p.sin = a->sin;
  p.row0 = 0;
  p.eps = a->eps;
  p.rope_mode = a->rope_mode;
  p.big_dim = a->big_dim < 0 ? -1 : a->big_dim;
  p.qbig = a->qbig;
  p.kbig = a->kbig;
  CUDA_TRY(h, cudaSetDevice(h->device));
  {
    ProfileMark pm(h, 0);
    CUDA_TRY(h, launch_qk_norm_rope(p, h->stream));
  }
  h->launches++;
  return KREA_CUDA_OK;
}

// ---------------------------------------------------------------------------------------------------
static int make_kv_map(krea_cuda* h, CUtensorMap* tm, const void* base, int cols, int rows, int batch, int64_t ld, int64_t bs,
                       const char* what, int box_rows = 128) {
  // (column, row, sample) view; boxes of 64 columns x box_rows rows; rows past `rows` read as zero
  cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)batch};
  cuuint64_t strides[2] = {(cuuint64_t)ld * 2, (cuuint64_t)(batch > 1 ? bs : (int64_t)rows * ld) * 2};
  cuuint32_t box[3] = {64, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = h->encode(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(h, KREA_CUDA_E_CUDA, "attention: cuTensorMapEncodeTiled(%s) failed with %d", what, (int)r);
  return KREA_CUDA_OK;
}

struct AttnCall {
  const void *Q, *K, *V, *G;
  void* O;
  int batch, Lq, Lk, heads, group;
  int64_t ldq, ldk, ldv, ldo, ldg, bsq, bsk, bsv, bso, bsg;
  const float *wq, *cos, *sin;
  float eps;
  int rope_mode, q_row0;
  const int32_t* text_len;
  int text_slots;
  const float* logit_bound;
  int causal, q_pos0;
  const float *QB, *KB;
  bool pdl;             // programmatic dependent launch after the K pre-pass (fused call only)
  bool bound_given;     // logit_bound holds for Q and K as they are (normalised by an earlier kernel)
  void* const* o_blk;   // row-block scatter of the output (see AttnParams::O_blk), nullptr = none
  int o_blk_n, o_blk_rows;
  float *So, *Sm, *Sl;  // split-K state (krea_cuda_attention_partial), nullptr = none
  bool state_load, state_store;
  // fused call with K normalised inside the attention kernel: the caller's K (K above is then the scratch that
  // receives the normalised keys), nullptr = K is final as it is
  const void* Kraw;
  int64_t ldkr, bskr;
  const float* wk;
};

// Query blocks (work items per head) of the attention kernels, and the key rows each of them normalises when K is
// normalised inside the persistent kernel.
static inline int attn_query_blocks(int Lq) { return (Lq + 255) / 256; }
static inline int key_slice_rows(int Lq, int Lk) { const int n = attn_query_blocks(Lq); return (Lk + n - 1) / n; }
// whether a problem runs as the persistent kernel: one CTA per SM walking over its work items pays when there is
// more than one item per CTA; a problem that fits the SMs in one wave runs the one-item kernel (measured at 120
// items: 4 % faster)
static inline bool runs_persistent(const krea_cuda* h, int batch, int heads, int Lq) {
  const long long items = (long long)attn_query_blocks(Lq) * heads * batch;
  return h->persist != 0 && h->sm_count > 0 && (h->persist == 2 || items > h->sm_count);
}

// Whether the fused call normalises K inside the persistent kernel (the handle's option, and a shape that allows
// it).  The keys of a (sample, kv head) are spread over the query blocks of one head; a CTA that waits for them must
// find every such block among the items that its neighbours have already passed or hold now, which is so when a
// head has no more blocks than there are CTAs.
static bool fuse_keys(const krea_cuda* h, const krea_cuda_joint_args* a) {
  if (!h->kfuse || a->Lk <= 0) return false;
  const int batch = a->batch <= 0 ? 1 : a->batch;
  if (!runs_persistent(h, batch, a->heads, a->Lq)) return false;
  const int nqb = attn_query_blocks(a->Lq);
  if (nqb > h->sm_count) return false;
  // a CTA with three or more items leaves the later key slices to two of its warps, which keep up with the
  // attention only when a head has enough query blocks to share its keys among
  if ((int64_t)batch * a->heads * nqb > 2 * (int64_t)h->sm_count && nqb < 13) return false;
  if ((int64_t)batch * (a->heads / a->group) > krea_cuda::kKeyCounters) return false;
  if (key_slice_rows(a->Lq, a->Lk) > 2048) return false;          // few queries, many keys: the separate pass is faster
  if (a->text_len && a->text_slots >= a->Lk) return false;        // every work item must have keys to visit
  return true;
}

static int run_attention(krea_cuda* h, const AttnCall& c) {
  if (c.Lq < 0 || c.Lk < 0 || c.heads < 0 || c.batch < 0) return fail(h, KREA_CUDA_E_ARG, "attention: negative size");
  if (c.Lq == 0 || c.heads == 0 || c.batch == 0) return KREA_CUDA_OK;
  if (c.group < 1 || c.heads % c.group) return fail(h, KREA_CUDA_E_ARG, "attention: heads must be a multiple of group");
  if (!c.Q || !c.O || (c.Lk > 0 && (!c.K || !c.V))) return fail(h, KREA_CUDA_E_ARG, "attention: null tensor");
  const int kvheads = c.heads / c.group;
  if (c.ldq < (int64_t)c.heads * 128 || c.ldo < (int64_t)c.heads * 128 || c.ldk < (int64_t)kvheads * 128 || c.ldv < (int64_t)kvheads * 128)
    return fail(h, KREA_CUDA_E_ARG, "attention: a leading dimension is smaller than heads*128");
  if (c.G && c.ldg < (int64_t)c.heads * 128) return fail(h, KREA_CUDA_E_ARG, "attention: ldg smaller than heads*128");
  if ((c.ldq | c.ldk | c.ldv | c.ldo | c.ldg | c.bsq | c.bsk | c.bsv | c.bso | c.bsg) % 8)
    return fail(h, KREA_CUDA_E_ARG, "attention: leading dimensions and batch strides must be multiples of 8 elements");
  if (!aligned16(c.Q) || !aligned16(c.K) || !aligned16(c.V) || !aligned16(c.O) || !aligned16(c.G))
    return fail(h, KREA_CUDA_E_ARG, "attention: tensor pointers must be 16-byte aligned");
  if (c.batch > 65535 || c.heads > 65535) return fail(h, KREA_CUDA_E_ARG, "attention: batch and heads are limited to 65535");
  if (c.text_len && (c.text_slots <= 0 || c.text_slots > c.Lk)) return fail(h, KREA_CUDA_E_ARG, "attention: text_slots must be in (0, Lk]");
  if (c.wq && c.rope_mode != KREA_CUDA_ROPE_NONE && (!c.cos || !c.sin)) return fail(h, KREA_CUDA_E_ARG, "attention: cos/sin tables missing");
  if (c.wq && (((uintptr_t)c.wq | (uintptr_t)c.cos | (uintptr_t)c.sin) & 15u)) return fail(h, KREA_CUDA_E_ARG, "attention: wq/cos/sin must be 16-byte aligned");
  CUDA_TRY(h, cudaSetDevice(h->device));

  AttnParams p{};
  p.Q = (const __nv_bfloat16*)c.Q;
  p.O = (__nv_bfloat16*)c.O;
  p.G = (const __nv_bfloat16*)c.G;
  p.ldq = c.ldq; p.ldo = c.ldo; p.ldg = c.ldg;
  p.bsq = c.bsq; p.bso = c.bso; p.bsg = c.bsg;
  p.Lq = c.Lq; p.Lk = c.Lk; p.heads = c.heads; p.group = c.group; p.batch = c.batch;
  p.scale_log2 = (float)(1.0 / sqrt(128.0) * 1.4426950408889634);   // engine/src/metal.mm:198
  p.causal = c.causal ? 1 : 0; p.q_pos0 = c.q_pos0;
  p.QB = c.QB; p.KB = c.KB; p.ldqb = c.heads; p.ldkb = kvheads;      // row strides = heads and heads / group (metal.h:85)
  p.wq = c.wq; p.cos = c.cos; p.sin = c.sin; p.eps = c.eps; p.rope_mode = c.rope_mode; p.q_row0 = c.q_row0;
  p.text_len = c.text_len; p.text_slots = c.text_len ? c.text_slots : 0;
  p.logit_bound = (h->static_bound && (c.wq || c.bound_given)) ? c.logit_bound : nullptr;
  p.So = c.So; p.Sm = c.Sm; p.Sl = c.Sl;
  p.state_load = c.state_load ? 1 : 0; p.state_store = c.state_store ? 1 : 0;
  const bool partial = c.state_load || c.state_store;     // the split-K forms live in the one-item kernel
  p.status = h->status_dev;
  p.wait_limit_ns = h->wait_limit_ns;
  p.test_drop_last_k = h->test_drop_last_k;
  p.pdl = c.pdl ? 1 : 0;
  const bool persist = !partial && runs_persistent(h, c.batch, c.heads, c.Lq);
  if (c.Kraw != nullptr) {
    if (!persist) return fail(h, KREA_CUDA_E_ARG, "attention: K can only be normalised inside the persistent kernel");
    p.Kraw = (const __nv_bfloat16*)c.Kraw;
    p.ldkr = c.ldkr; p.bskr = c.bskr;
    p.wk = c.wk;
    p.Kn = (__nv_bfloat16*)const_cast<void*>(c.K);
    uint32_t* counters = h->status_dev + 64;
    p.kcount = counters + (h->kfuse_seq & 1) * krea_cuda::kKeyCounters;
    p.kcount_clear = counters + ((h->kfuse_seq + 1) & 1) * krea_cuda::kKeyCounters;
    p.kcount_clear_n = krea_cuda::kKeyCounters;
    p.k_slices = attn_query_blocks(c.Lq);
    p.k_slice_rows = key_slice_rows(c.Lq, c.Lk);
    p.bound_in_kernel = h->static_bound ? 1 : 0;
    p.logit_bound = nullptr;
    p.pdl = 0;      // the kernel reads the caller's K: it must not start before the stream's previous kernel has ended
  }
  if (c.o_blk != nullptr) {
    if (c.batch != 1 || c.o_blk_rows <= 0 || c.o_blk_n < 1 || c.o_blk_n > 8 || (int64_t)c.o_blk_n * c.o_blk_rows < c.Lq)
      return fail(h, KREA_CUDA_E_ARG, "attention: bad output row-block table");
    for (int k = 0; k < 8; k++) {
      p.O_blk[k] = (__nv_bfloat16*)c.o_blk[k < c.o_blk_n ? k : c.o_blk_n - 1];
      if (!p.O_blk[k] || !aligned16(p.O_blk[k])) return fail(h, KREA_CUDA_E_ARG, "attention: null or misaligned output block");
    }
    p.o_blk_rows = c.o_blk_rows;
  }

  CUtensorMap tmK, tmV, tmO, tmQ;
  memset(&tmK, 0, sizeof(tmK));
  memset(&tmV, 0, sizeof(tmV));
  memset(&tmO, 0, sizeof(tmO));
  memset(&tmQ, 0, sizeof(tmQ));
  if (h->q_tma && c.wq == nullptr && c.Lk > 0 && !partial) {
    // no prologue: Q goes from global to the MMA's shared-memory layout by TMA, no thread touches it
    int rc = make_kv_map(h, &tmQ, c.Q, c.heads * 128, c.Lq, c.batch, c.ldq, c.bsq, "Q");
    if (rc) return rc;
    p.q_tma = 1;
  }
  if (h->o_tma && c.o_blk == nullptr && c.Lk > 0) {
    // the output leaves shared memory as TMA tile stores (not with the row-block scatter, whose rows have several bases)
    int rc = make_kv_map(h, &tmO, c.O, c.heads * 128, c.Lq, c.batch, c.ldo, c.bso, "O");
    if (rc) return rc;
    p.o_tma = 1;
  }
  if (c.Lk > 0) {
    int rc = make_kv_map(h, &tmK, c.K, kvheads * 128, c.Lk, c.batch, c.ldk, c.bsk, "K");
    if (rc) return rc;
    rc = make_kv_map(h, &tmV, c.V, kvheads * 128, c.Lk, c.batch, c.ldv, c.bsv, "V");
    if (rc) return rc;
  }
  {
    ProfileMark pm(h, 1);
    if (persist) CUDA_TRY(h, launch_attention_persist_sm100(tmK, tmV, tmQ, p, h->emu, h->sm_count, h->stream));
    else CUDA_TRY(h, launch_attention_sm100(tmK, tmV, tmO, tmQ, p, partial ? 1 : h->split, h->emu, h->stream));
  }
  h->launches++;
  if (c.Kraw != nullptr) h->kfuse_seq++;
  return KREA_CUDA_OK;
}

int krea_cuda_attention(krea_cuda* h, const krea_cuda_attn_args* a) {
  if (!h || !a) return fail(h, KREA_CUDA_E_ARG, "attention: null handle or arguments");
  const bool big = a->QB && a->KB;                                     // engine/src/metal.mm:196
  if (big && a->batch > 1) return fail(h, KREA_CUDA_E_UNSUPPORTED, "attention: QB/KB have no batch dimension");
  if (a->causal && a->text_len) return fail(h, KREA_CUDA_E_UNSUPPORTED, "attention: causal masking and the text padding mask are not combined");
  AttnCall c{};
  c.Q = a->Q; c.K = a->K; c.V = a->V; c.O = a->O;
  c.G = (a->G && a->ldg > 0) ? a->G : nullptr;
  c.batch = a->batch <= 0 ? 1 : a->batch;
  c.Lq = a->Lq; c.Lk = a->Lk; c.heads = a->heads; c.group = a->group;
  c.ldq = a->ldq; c.ldk = a->ldk; c.ldv = a->ldv; c.ldo = a->ldo; c.ldg = c.G ? a->ldg : 0;
  c.bsq = a->bsq; c.bsk = a->bsk; c.bsv = a->bsv; c.bso = a->bso; c.bsg = c.G ? a->bsg : 0;
  c.wq = nullptr; c.cos = c.sin = nullptr; c.eps = 0.f; c.rope_mode = KREA_CUDA_ROPE_NONE;
  c.q_row0 = a->q_row0;
  c.text_len = a->text_len; c.text_slots = a->text_slots;
  c.causal = a->causal; c.q_pos0 = a->q_pos0;
  c.QB = big ? a->QB : nullptr; c.KB = big ? a->KB : nullptr;
  return run_attention(h, c);
}

int krea_cuda_attention_partial(krea_cuda* h, const krea_cuda_attn_args* a, int part, float* So, float* Sm, float* Sl) {
  if (!h || !a) return fail(h, KREA_CUDA_E_ARG, "attention_partial: null handle or arguments");
  if (part < KREA_CUDA_PART_FIRST || part > KREA_CUDA_PART_LAST) return fail(h, KREA_CUDA_E_ARG, "attention_partial: part must be FIRST, MID or LAST");
  if (!So || !Sm || !Sl || !aligned16(So) || !aligned16(Sl) || ((uintptr_t)Sm & 3u)) return fail(h, KREA_CUDA_E_ARG, "attention_partial: null or misaligned state");
  // the reference's split kernels are non-causal (attention.metal:14) and, like every operator of it, unbatched
  if (a->causal) return fail(h, KREA_CUDA_E_UNSUPPORTED, "attention_partial: the split-K forms are non-causal");
  if (a->batch > 1 || a->text_len) return fail(h, KREA_CUDA_E_UNSUPPORTED, "attention_partial: no batch and no padding mask");
  if (a->Lk <= 0) return fail(h, KREA_CUDA_E_ARG, "attention_partial: a key block must hold at least one key");
  const bool big = a->QB && a->KB;
  AttnCall c{};
  c.Q = a->Q; c.K = a->K; c.V = a->V; c.O = a->O;
  c.G = (part == KREA_CUDA_PART_LAST && a->G && a->ldg > 0) ? a->G : nullptr;   // the gate belongs to the store of the output
  c.batch = 1;
  c.Lq = a->Lq; c.Lk = a->Lk; c.heads = a->heads; c.group = a->group;
  c.ldq = a->ldq; c.ldk = a->ldk; c.ldv = a->ldv; c.ldo = a->ldo; c.ldg = c.G ? a->ldg : 0;
  c.rope_mode = KREA_CUDA_ROPE_NONE;
  c.QB = big ? a->QB : nullptr; c.KB = big ? a->KB : nullptr;
  c.So = So; c.Sm = Sm; c.Sl = Sl;
  c.state_load = part != KREA_CUDA_PART_FIRST;
  c.state_store = part != KREA_CUDA_PART_LAST;
  if (part != KREA_CUDA_PART_LAST && !c.O) c.O = So;   // never written by these parts; run_attention wants a pointer
  return run_attention(h, c);
}

// ---------------------------------------------------------------------------------------------------
size_t krea_cuda_joint_scratch_bytes(const krea_cuda_joint_args* a) {
  if (!a || a->group < 1 || a->Lk <= 0 || a->heads <= 0) return 0;
  const size_t batch = a->batch <= 0 ? 1 : (size_t)a->batch;
  return batch * (size_t)a->Lk * (size_t)(a->heads / a->group) * 128 * 2;
}

// The fused call in two steps, so that a caller inside the library can put other work between them:
// joint_prepass writes the normalised + rotated K and the logit bound, joint_attend runs the attention kernel.
static int joint_prepass(krea_cuda* h, const krea_cuda_joint_args* a, void* kscr) {
  const int batch = a->batch <= 0 ? 1 : a->batch;
  const int kvheads = a->heads / a->group;
  // K pre-pass: normalised + rotated K, written once to scratch [batch, Lk, kvheads*128]
  NormRopeParams n{};
  n.src = (const __nv_bfloat16*)a->K;
  n.dst = (__nv_bfloat16*)kscr;
  n.ld_src = a->ldk;
  n.ld_dst = (int64_t)kvheads * 128;
  n.bs_src = a->bsk;
  n.bs_dst = (int64_t)a->Lk * kvheads * 128;
  n.rows = a->Lk;
  n.batch = batch;
  n.q_off = n.q_off_dst = 0;
  n.n_q = 0;
  n.k_off = n.k_off_dst = 0;
  n.n_k = kvheads;
  n.wq = n.wk = a->wk;
  n.cos = a->cos;
  n.sin = a->sin;
  n.row0 = 0;
  n.eps = a->eps;
  n.rope_mode = a->rope_mode;
  n.big_dim = -1;
  n.bound_wq = a->wq;
  n.bound_out = (float*)(h->status_dev + 8);   // a device float next to the status word
  n.bound_scale_log2 = (float)(1.0 / sqrt(128.0) * 1.4426950408889634);
  n.pdl = h->pdl ? 1 : 0;
  CUDA_TRY(h, cudaSetDevice(h->device));
  {
    ProfileMark pm(h, 0);
    CUDA_TRY(h, launch_qk_norm_rope(n, h->stream));
  }
  h->launches++;
  return KREA_CUDA_OK;
}

static int joint_attend(krea_cuda* h, const krea_cuda_joint_args* a, void* kscr, void* const* o_blk = nullptr, int o_blk_n = 0,
                        int o_blk_rows = 0, bool keys_inside = false) {
  const int batch = a->batch <= 0 ? 1 : a->batch;
  const int kvheads = a->heads / a->group;
  AttnCall c{};
  c.Q = a->Q; c.K = kscr; c.V = a->V; c.O = a->O;
  c.G = (a->G && a->ldg > 0) ? a->G : nullptr;
  c.batch = batch; c.Lq = a->Lq; c.Lk = a->Lk; c.heads = a->heads; c.group = a->group;
  c.ldq = a->ldq; c.ldk = (int64_t)kvheads * 128; c.ldv = a->ldv; c.ldo = a->ldo; c.ldg = c.G ? a->ldg : 0;
  c.bsq = a->bsq; c.bsk = (int64_t)a->Lk * kvheads * 128; c.bsv = a->bsv; c.bso = a->bso; c.bsg = c.G ? a->bsg : 0;
  c.wq = a->wq; c.cos = a->cos; c.sin = a->sin; c.eps = a->eps; c.rope_mode = a->rope_mode; c.q_row0 = a->q_row0;
  c.text_len = a->text_len; c.text_slots = a->text_slots;
  c.logit_bound = (float*)(h->status_dev + 8);
  c.o_blk = o_blk; c.o_blk_n = o_blk_n; c.o_blk_rows = o_blk_rows;
  c.pdl = h->pdl;          // the kernel right before this one in the stream is the K pre-pass
  if (keys_inside) {
    // no pre-pass: the attention kernel normalises the caller's K into the scratch itself (and works out the bound)
    c.Kraw = a->K; c.ldkr = a->ldk; c.bskr = a->bsk; c.wk = a->wk;
    c.logit_bound = nullptr;
  }
  return run_attention(h, c);
}

static int joint_on_device(krea_cuda* h, const krea_cuda_joint_args* a, void* kscr) {
  if (fuse_keys(h, a)) return joint_attend(h, a, kscr, nullptr, 0, 0, true);
  const int rc = joint_prepass(h, a, kscr);
  return rc ? rc : joint_attend(h, a, kscr);
}

static int validate_joint(krea_cuda* h, const krea_cuda_joint_args* a) {
  if (!h || !a) return fail(h, KREA_CUDA_E_ARG, "joint_attention: null handle or arguments");
  if (a->Lq < 0 || a->Lk < 0 || a->heads < 0 || a->q_row0 < 0) return fail(h, KREA_CUDA_E_ARG, "joint_attention: negative size");
  if (a->group < 1 || a->heads % a->group) return fail(h, KREA_CUDA_E_ARG, "joint_attention: heads must be a multiple of group");
  if (!a->wq || !a->wk) return fail(h, KREA_CUDA_E_ARG, "joint_attention: QK-norm weights missing");
  if (a->rope_mode < 0 || a->rope_mode > 2) return fail(h, KREA_CUDA_E_ARG, "joint_attention: rope_mode must be 0, 1 or 2");
  if (a->rope_mode != KREA_CUDA_ROPE_NONE && (!a->cos || !a->sin)) return fail(h, KREA_CUDA_E_ARG, "joint_attention: cos/sin tables missing");
  if (a->Lk > 0 && (!a->K || !a->V)) return fail(h, KREA_CUDA_E_ARG, "joint_attention: null tensor");
  if (!aligned16(a->wq) || !aligned16(a->wk) || !aligned16(a->cos) || !aligned16(a->sin))
    return fail(h, KREA_CUDA_E_ARG, "joint_attention: weights and tables must be 16-byte aligned");
  if (a->ldk % 8 || a->bsk % 8 || !aligned16(a->K)) return fail(h, KREA_CUDA_E_ARG, "joint_attention: K must be 16-byte aligned with ld, batch stride multiples of 8");
  if (a->ldk < (int64_t)(a->heads / a->group) * 128) return fail(h, KREA_CUDA_E_ARG, "joint_attention: ldk smaller than kv heads*128");
  return KREA_CUDA_OK;
}

int krea_cuda_joint_attention(krea_cuda* h, const krea_cuda_joint_args* a) {
  int rc = validate_joint(h, a);
  if (rc) return rc;
  if (a->Lq == 0 || a->heads == 0) return KREA_CUDA_OK;
  const size_t need = krea_cuda_joint_scratch_bytes(a);
  void* kscr = a->k_scratch;
  if (kscr) {
    if (a->k_scratch_bytes < need) return fail(h, KREA_CUDA_E_NOMEM, "joint_attention: k_scratch holds %zu bytes, %zu needed", a->k_scratch_bytes, need);
    if (!aligned16(kscr)) return fail(h, KREA_CUDA_E_ARG, "joint_attention: k_scratch must be 16-byte aligned");
  } else if (need > 0) {
    CUDA_TRY(h, cudaSetDevice(h->device));
    if (h->ws_bytes < need) {
      // growing the workspace: earlier kernels may still be reading the old one
      CUDA_TRY(h, cudaStreamSynchronize(h->stream));
      if (h->ws) cudaFree(h->ws);
      h->ws = nullptr;
      h->ws_bytes = 0;
      if (cudaMalloc(&h->ws, need) != cudaSuccess) {
        cudaGetLastError();
        return fail(h, KREA_CUDA_E_NOMEM, "joint_attention: cannot allocate %zu bytes of scratch", need);
      }
      h->ws_bytes = need;
    }
    kscr = h->ws;
  }
  if (a->Lk == 0) {
    AttnCall c{};
    c.Q = a->Q; c.O = a->O; c.batch = a->batch <= 0 ? 1 : a->batch; c.Lq = a->Lq; c.Lk = 0; c.heads = a->heads; c.group = a->group;
    c.ldq = a->ldq; c.ldk = c.ldv = (int64_t)(a->heads / a->group) * 128; c.ldo = a->ldo; c.bsq = a->bsq; c.bso = a->bso;
    c.K = c.V = a->Q;
    return run_attention(h, c);
  }
  return joint_on_device(h, a, kscr);
}

// ---------------------------------------------------------------------------------------------------
// The fused call for callers that must not allocate device memory: its scratch is g_static_k_scratch (top of
// this file), whose device address krea_cuda_create has already resolved for the handle's device.
int krea_cuda_joint_attention_static(krea_cuda* h, const krea_cuda_joint_args* a) {
  int rc = validate_joint(h, a);
  if (rc) return rc;
  if (a->Lq == 0 || a->heads == 0) return KREA_CUDA_OK;
  const size_t need = krea_cuda_joint_scratch_bytes(a);
  if (need > (size_t)KREA_CUDA_STATIC_SCRATCH_BYTES)
    return fail(h, KREA_CUDA_E_NOMEM,
                "joint_attention_static: batch * Lk * kv_heads * 256 = %zu bytes of normalised K exceed the built-in %zu-byte "
                "scratch; use krea_cuda_joint_attention with caller-provided k_scratch for this size",
                need, (size_t)KREA_CUDA_STATIC_SCRATCH_BYTES);
  if (h->device < 0 || h->device >= 64) return fail(h, KREA_CUDA_E_ARG, "joint_attention_static: device index above 63");
  CUDA_TRY(h, cudaSetDevice(h->device));
  // already resolved by krea_cuda_create for this device: a table look-up, no CUDA call
  cudaError_t se;
  void* scratch = static_scratch_on(h->device, &se);
  if (scratch == nullptr) return fail(h, KREA_CUDA_E_CUDA, "joint_attention_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(se));
  if (a->Lk == 0) {
    AttnCall c{};
    c.Q = a->Q; c.O = a->O; c.batch = a->batch <= 0 ? 1 : a->batch; c.Lq = a->Lq; c.Lk = 0; c.heads = a->heads; c.group = a->group;
    c.ldq = a->ldq; c.ldk = c.ldv = (int64_t)(a->heads / a->group) * 128; c.ldo = a->ldo; c.bsq = a->bsq; c.bso = a->bso;
    c.K = c.V = a->Q;
    return run_attention(h, c);
  }
  // Every element of the scratch that the attention kernel reads is written by the pre-pass of this same
  // call, so nothing has to be cleared between calls.
  return joint_on_device(h, a, scratch);
}

static int stage_buf(krea_cuda* h, int slot, size_t bytes, void** out) {
  if (h->stage_bytes[slot] < bytes) {
    CUDA_TRY(h, cudaStreamSynchronize(h->stream));
    if (h->stage[slot]) cudaFree(h->stage[slot]);
    h->stage[slot] = nullptr;
    h->stage_bytes[slot] = 0;
    if (cudaMalloc(&h->stage[slot], bytes) != cudaSuccess) {
      cudaGetLastError();
      return fail(h, KREA_CUDA_E_NOMEM, "joint_attention_host: cannot allocate %zu bytes", bytes);
    }
    h->stage_bytes[slot] = bytes;
  }
  *out = h->stage[slot];
  return KREA_CUDA_OK;
}

static int host_pipeline(krea_cuda* h, const krea_cuda_joint_args* a);

int krea_cuda_joint_attention_host(krea_cuda* h, const krea_cuda_joint_args* a) {
  const int rc = host_pipeline(h, a);
  if (rc != KREA_CUDA_OK && h) {
    // A failure part-way leaves copies from and to the caller's buffers in flight: let them finish before the
    // caller gets its buffers back.  The error already recorded in the handle stays the one reported.
    if (h->copy_in) cudaStreamSynchronize(h->copy_in);
    cudaStreamSynchronize(h->stream);
    if (h->copy_out) cudaStreamSynchronize(h->copy_out);
    cudaGetLastError();
  }
  return rc;
}

static int host_pipeline(krea_cuda* h, const krea_cuda_joint_args* a) {
  int rc = validate_joint(h, a);
  if (rc) return rc;
  if (!a->Q || !a->O) return fail(h, KREA_CUDA_E_ARG, "joint_attention_host: null tensor");
  if (a->Lq == 0 || a->heads == 0 || a->Lk == 0) return fail(h, KREA_CUDA_E_ARG, "joint_attention_host: empty problem");
  if (a->G) return fail(h, KREA_CUDA_E_UNSUPPORTED, "joint_attention_host: the gate is only available through device pointers");
  CUDA_TRY(h, cudaSetDevice(h->device));
  const int batch = a->batch <= 0 ? 1 : a->batch;
  const int kvheads = a->heads / a->group;
  const size_t qw = (size_t)a->heads * 128, kw = (size_t)kvheads * 128;
  const int trows = a->q_row0 + a->Lq > a->Lk ? a->q_row0 + a->Lq : a->Lk;
  void *dQ, *dK, *dV, *dO, *dT, *dW, *dL;
  if ((rc = stage_buf(h, 0, (size_t)batch * a->Lq * qw * 2, &dQ))) return rc;
  if ((rc = stage_buf(h, 1, (size_t)batch * a->Lk * kw * 2, &dK))) return rc;
  if ((rc = stage_buf(h, 2, (size_t)batch * a->Lk * kw * 2, &dV))) return rc;
  if ((rc = stage_buf(h, 3, (size_t)batch * a->Lq * qw * 2, &dO))) return rc;
  if ((rc = stage_buf(h, 4, (size_t)trows * 64 * 4 * 2, &dT))) return rc;
  if ((rc = stage_buf(h, 5, 1024, &dW))) return rc;
  if ((rc = stage_buf(h, 6, (size_t)batch * 4 + 16, &dL))) return rc;
  // Heads are independent, so the call is pipelined over groups of heads: while one group is being
  // computed, the next group's columns of Q, K and V are still arriving over PCIe on a second stream and
  // the previous group's output is already on its way back on a third (the two copy directions use
  // different DMA engines).  The results are the same as one call over all heads.
  int ngroups = 1;
  const size_t total_in = (size_t)batch * ((size_t)a->Lq * qw + 2 * (size_t)a->Lk * kw) * 2;
  if (total_in >= ((size_t)8 << 20)) {
    for (int cand : {6, 4, 3, 2})   // narrower column blocks than about 1 KB per row slow the DMA down
      if (kvheads % cand == 0) { ngroups = cand; break; }
  }
  // kv heads per group and the first kv head of every group (uniform unless the list knob below says otherwise)
  int gheads[8], gfirst[9];
  if (!h->copy_in) {
    CUDA_TRY(h, cudaStreamCreateWithFlags(&h->copy_in, cudaStreamNonBlocking));
    CUDA_TRY(h, cudaStreamCreateWithFlags(&h->copy_out, cudaStreamNonBlocking));
    for (int i = 0; i < 18; i++) CUDA_TRY(h, cudaEventCreateWithFlags(&h->pipe_ev[i], cudaEventDisableTiming));
  }
  if (const char* e = getenv("KREA_CUDA_HOST_GROUPS")) {   // tuning knob
    const int v = atoi(e);
    if (v >= 1 && v <= 8 && kvheads % v == 0) ngroups = v;
  }
  const bool ttrace = getenv("KREA_CUDA_HOST_TRACE") != nullptr;   // tuning aid: print the pipeline's timeline
  cudaEvent_t tev[32] = {};
  if (ttrace) for (int i = 0; i < 32; i++) cudaEventCreate(&tev[i]);
  for (int gi = 0; gi < ngroups; gi++) gheads[gi] = kvheads / ngroups;
  if (const char* e = getenv("KREA_CUDA_HOST_GROUP_HEADS")) {   // tuning knob: kv heads per group, e.g. "8,8,6,2"
    int n = 0, sum = 0, list[8];
    for (const char* c = e; *c && n < 8;) {
      char* end = nullptr;
      const long v = strtol(c, &end, 10);
      if (end == c || v < 1) { n = 0; break; }
      list[n++] = (int)v;
      sum += (int)v;
      c = (*end == ',') ? end + 1 : end;
      if (*end && *end != ',') { n = 0; break; }
    }
    if (n >= 1 && sum == kvheads) {
      ngroups = n;
      for (int gi = 0; gi < n; gi++) gheads[gi] = list[gi];
    }
  }
  gfirst[0] = 0;
  for (int gi = 0; gi < ngroups; gi++) gfirst[gi + 1] = gfirst[gi] + gheads[gi];
  // byte offset / width of group gi's column block in a row of K or V (kv heads) and of Q or O (group query heads per kv head)
  auto kc0 = [&](int gi) { return (size_t)gfirst[gi] * 128 * 2; };
  auto kcwf = [&](int gi) { return (size_t)gheads[gi] * 128 * 2; };
  auto qc0 = [&](int gi) { return (size_t)gfirst[gi] * a->group * 128 * 2; };
  auto qcwf = [&](int gi) { return (size_t)gheads[gi] * a->group * 128 * 2; };
  // order the copy streams after whatever the caller enqueued on the compute stream
  CUDA_TRY(h, cudaEventRecord(h->pipe_ev[16], h->stream));
  CUDA_TRY(h, cudaStreamWaitEvent(h->copy_in, h->pipe_ev[16], 0));
  CUDA_TRY(h, cudaStreamWaitEvent(h->copy_out, h->pipe_ev[16], 0));
  if (ttrace) cudaEventRecord(tev[0], h->copy_in);
  for (int gi = 0; gi < ngroups; gi++) {
    for (int b = 0; b < batch; b++) {
      CUDA_TRY(h, cudaMemcpy2DAsync((char*)dQ + (size_t)b * a->Lq * qw * 2 + qc0(gi), qw * 2,
                                    (const char*)a->Q + (size_t)b * a->bsq * 2 + qc0(gi), (size_t)a->ldq * 2, qcwf(gi), a->Lq,
                                    cudaMemcpyHostToDevice, h->copy_in));
      CUDA_TRY(h, cudaMemcpy2DAsync((char*)dK + (size_t)b * a->Lk * kw * 2 + kc0(gi), kw * 2,
                                    (const char*)a->K + (size_t)b * a->bsk * 2 + kc0(gi), (size_t)a->ldk * 2, kcwf(gi), a->Lk,
                                    cudaMemcpyHostToDevice, h->copy_in));
      CUDA_TRY(h, cudaMemcpy2DAsync((char*)dV + (size_t)b * a->Lk * kw * 2 + kc0(gi), kw * 2,
                                    (const char*)a->V + (size_t)b * a->bsv * 2 + kc0(gi), (size_t)a->ldv * 2, kcwf(gi), a->Lk,
                                    cudaMemcpyHostToDevice, h->copy_in));
    }
    if (gi == 0) {
    // The small operands (tables, weights, lengths) go right after the first group of heads and through a pinned bounce buffer: a copy from
    // pageable memory would block the calling thread until the copy engine reaches it - behind the large
    // transfers - and nothing could be launched meanwhile.
    {
      const size_t tbytes = a->rope_mode != KREA_CUDA_ROPE_NONE ? (size_t)trows * 64 * 4 : 0;
      const size_t need = 2 * tbytes + 1024 + (size_t)batch * 4;
      if (h->bounce_bytes < need) {
        CUDA_TRY(h, cudaStreamSynchronize(h->copy_in));
        if (h->bounce) cudaFreeHost(h->bounce);
        h->bounce = nullptr;
        h->bounce_bytes = 0;
        if (cudaMallocHost(&h->bounce, need) != cudaSuccess) {
          cudaGetLastError();
          return fail(h, KREA_CUDA_E_NOMEM, "joint_attention_host: cannot allocate %zu bytes of pinned memory", need);
        }
        h->bounce_bytes = need;
      } else {
        CUDA_TRY(h, cudaEventSynchronize(h->pipe_ev[17]));   // the previous call's copies out of the bounce buffer
      }
      char* bb = (char*)h->bounce;
      if (tbytes) {
        memcpy(bb, a->cos, tbytes);
        memcpy(bb + tbytes, a->sin, tbytes);
        CUDA_TRY(h, cudaMemcpyAsync(dT, bb, 2 * tbytes, cudaMemcpyHostToDevice, h->copy_in));
      }
      memcpy(bb + 2 * tbytes, a->wq, 512);
      memcpy(bb + 2 * tbytes + 512, a->wk, 512);
      CUDA_TRY(h, cudaMemcpyAsync(dW, bb + 2 * tbytes, 1024, cudaMemcpyHostToDevice, h->copy_in));
      if (a->text_len) {
        memcpy(bb + 2 * tbytes + 1024, a->text_len, (size_t)batch * 4);
        CUDA_TRY(h, cudaMemcpyAsync(dL, bb + 2 * tbytes + 1024, (size_t)batch * 4, cudaMemcpyHostToDevice, h->copy_in));
      }
      CUDA_TRY(h, cudaEventRecord(h->pipe_ev[17], h->copy_in));
    }
    }
    CUDA_TRY(h, cudaEventRecord(h->pipe_ev[gi], h->copy_in));
    if (ttrace) cudaEventRecord(tev[1 + gi], h->copy_in);
  }
  float* dcos = (float*)dT;
  float* dsin = dcos + (size_t)trows * 64;
  for (int gi = 0; gi < ngroups; gi++) {
    CUDA_TRY(h, cudaStreamWaitEvent(h->stream, h->pipe_ev[gi], 0));
    krea_cuda_joint_args d = *a;
    d.Q = (char*)dQ + qc0(gi); d.K = (char*)dK + kc0(gi); d.V = (char*)dV + kc0(gi); d.O = (char*)dO + qc0(gi);
    d.batch = batch;
    d.heads = gheads[gi] * a->group;
    d.ldq = d.ldo = (int)qw; d.ldk = d.ldv = (int)kw;
    d.bsq = d.bso = (int64_t)a->Lq * qw; d.bsk = d.bsv = (int64_t)a->Lk * kw;
    d.wq = (const float*)dW; d.wk = (const float*)dW + 128;
    d.cos = dcos; d.sin = dsin;
    d.text_len = a->text_len ? (const int32_t*)dL : nullptr;
    d.G = nullptr; d.ldg = 0; d.bsg = 0;
    d.k_scratch = nullptr; d.k_scratch_bytes = 0;
    if ((rc = krea_cuda_joint_attention(h, &d))) return rc;
    CUDA_TRY(h, cudaEventRecord(h->pipe_ev[8 + gi], h->stream));
    if (ttrace) cudaEventRecord(tev[10 + gi], h->stream);
    CUDA_TRY(h, cudaStreamWaitEvent(h->copy_out, h->pipe_ev[8 + gi], 0));
    for (int b = 0; b < batch; b++)
      CUDA_TRY(h, cudaMemcpy2DAsync((char*)a->O + (size_t)b * a->bso * 2 + qc0(gi), (size_t)a->ldo * 2,
                                    (const char*)dO + (size_t)b * a->Lq * qw * 2 + qc0(gi), qw * 2, qcwf(gi), a->Lq,
                                    cudaMemcpyDeviceToHost, h->copy_out));
    if (ttrace) cudaEventRecord(tev[20 + gi], h->copy_out);
  }
  CUDA_TRY(h, cudaStreamSynchronize(h->copy_out));
  if (ttrace) {
    cudaDeviceSynchronize();
    fprintf(stderr, "[krea_cuda host pipeline] groups=%d, ms since first copy:", ngroups);
    for (int gi = 0; gi < ngroups; gi++) {
      float t1 = 0, t2 = 0, t3 = 0;
      cudaEventElapsedTime(&t1, tev[0], tev[1 + gi]);
      cudaEventElapsedTime(&t2, tev[0], tev[10 + gi]);
      cudaEventElapsedTime(&t3, tev[0], tev[20 + gi]);
      fprintf(stderr, "  g%d in %.3f compute %.3f out %.3f;", gi, t1, t2, t3);
    }
    fprintf(stderr, "\n");
    for (int i = 0; i < 32; i++) cudaEventDestroy(tev[i]);
  }
  return krea_cuda_sync(h);
}

// ---------------------------------------------------------------------------------------------------
// RoPE tables on the host, like DiT::set_grid (engine/src/model.mm:290-315): frequencies in double,
// tables stored as f32 [T + gh*gw, 64]; text rows at position 0, image token k at (k / gw, k % gw).
static void fill_tables(float* c, float* s, int T, int gh, int gw, const double* om, const int* axis) {
  const int R = T + gh * gw;
  for (int r = 0; r < R; r++) {
    const int k = r - T;
    const double pos[3] = {0.0, r < T ? 0.0 : (double)(k / gw), r < T ? 0.0 : (double)(k % gw)};
    for (int pr = 0; pr < 64; pr++) {
      const double ang = pos[axis[pr]] * om[pr];
      c[(size_t)r * 64 + pr] = (float)cos(ang);
      s[(size_t)r * 64 + pr] = (float)sin(ang);
    }
  }
}

int krea_cuda_rope_tables_ref3axis(float* c, float* s, int T, int gh, int gw) {
  if (!c || !s || T < 0 || gh < 0 || gw < 0 || (gh > 0 && gw == 0)) return KREA_CUDA_E_ARG;
  double om[64];
  int axis[64];
  for (int pr = 0; pr < 64; pr++) {
    axis[pr] = pr < 16 ? 0 : pr < 40 ? 1 : 2;
    const int first = axis[pr] == 0 ? 0 : axis[pr] == 1 ? 16 : 40;
    const int dims = axis[pr] == 0 ? 32 : 48;
    om[pr] = 1.0 / pow(1000.0, (2.0 * (pr - first)) / dims);
  }
  fill_tables(c, s, T, gh, gw, om, axis);
  return KREA_CUDA_OK;
}

int krea_cuda_rope_tables_axial2d(float* c, float* s, int T, int gh, int gw, double theta) {
  if (!c || !s || T < 0 || gh < 0 || gw < 0 || (gh > 0 && gw == 0) || !(theta > 0)) return KREA_CUDA_E_ARG;
  double om[64];
  int axis[64];
  for (int pr = 0; pr < 64; pr++) {
    axis[pr] = pr < 32 ? 1 : 2;
    om[pr] = 1.0 / pow(theta, (2.0 * (pr & 31)) / 64.0);
  }
  fill_tables(c, s, T, gh, gw, om, axis);
  return KREA_CUDA_OK;
}

// ---------------------------------------------------------------------------------------------------
static int reshard(krea_cuda* h, const krea_cuda_reshard_args* a, bool unpack) {
  if (!h || !a) return fail(h, KREA_CUDA_E_ARG, "reshard: null handle or arguments");
  if (a->nranks < 1 || a->rows < 0 || a->cols_per_rank < 0) return fail(h, KREA_CUDA_E_ARG, "reshard: bad sizes");
  if (a->rows == 0 || a->cols_per_rank == 0) return KREA_CUDA_OK;
  if (!a->src || !a->dst || !aligned16(a->src) || !aligned16(a->dst)) return fail(h, KREA_CUDA_E_ARG, "reshard: null or misaligned pointer");
  const int ld = unpack ? a->dst_ld : a->src_ld, col0 = unpack ? a->dst_col0 : a->src_col0;
  if (a->cols_per_rank % 8 || ld % 8 || col0 % 8 || col0 < 0) return fail(h, KREA_CUDA_E_ARG, "reshard: columns and leading dimension must be multiples of 8");
  if ((int64_t)col0 + (int64_t)a->nranks * a->cols_per_rank > ld) return fail(h, KREA_CUDA_E_ARG, "reshard: column blocks exceed the leading dimension");
  ReshardParams p{};
  p.src = (const __nv_bfloat16*)a->src;
  p.dst = (__nv_bfloat16*)a->dst;
  p.nranks = a->nranks;
  p.rows = a->rows;
  p.cols_per_rank = a->cols_per_rank;
  p.src_ld = a->src_ld;
  p.dst_ld = a->dst_ld;
  p.src_col0 = a->src_col0;
  p.dst_col0 = a->dst_col0;
  CUDA_TRY(h, cudaSetDevice(h->device));
  CUDA_TRY(h, unpack ? launch_reshard_unpack(p, h->stream) : launch_reshard_pack(p, h->stream));
  h->launches++;
  return KREA_CUDA_OK;
}
// bound_out: with the fused QK-norm epilogue, where the kernel leaves the logit bound its weights imply (or nullptr)
static int gemm_impl(krea_cuda* h, const krea_cuda_gemm_args* a, float* bound_out) {
  if (!h || !a) return fail(h, KREA_CUDA_E_ARG, "gemm: null handle or arguments");
  if (a->M < 0 || a->N < 0 || a->K < 0) return fail(h, KREA_CUDA_E_ARG, "gemm: negative size");
  if (a->M == 0 || a->N == 0) return KREA_CUDA_OK;
  if (a->K == 0) return fail(h, KREA_CUDA_E_ARG, "gemm: K must be positive");
  if (!a->A || !a->W || !a->C || !aligned16(a->A) || !aligned16(a->W) || !aligned16(a->C)) return fail(h, KREA_CUDA_E_ARG, "gemm: null or misaligned pointer");
  if (a->lda % 8 || a->ldw % 8 || a->ldc % 8 || a->N % 8 || a->K % 8) return fail(h, KREA_CUDA_E_ARG, "gemm: lda, ldw, ldc, N and K must be multiples of 8");
  if (a->epilogue < KREA_CUDA_EPI_BF16 || a->epilogue > KREA_CUDA_EPI_BIAS_F32) return fail(h, KREA_CUDA_E_UNSUPPORTED, "gemm: epilogue %d is not built", a->epilogue);
  const bool has_bias = a->epilogue == KREA_CUDA_EPI_BIAS_BF16 || a->epilogue == KREA_CUDA_EPI_BIAS_F32;
  if (has_bias && (!a->vec || !aligned16(a->vec))) return fail(h, KREA_CUDA_E_ARG, "gemm: the bias vector is missing or misaligned");
  const int out_cols = a->epilogue == KREA_CUDA_EPI_SWIGLU ? a->N / 2 : a->N;
  if (a->seg < 0 || a->seg_stride < 0 || a->seg % 8 || a->seg_stride % 8 || (a->seg > 0 && (a->epilogue != KREA_CUDA_EPI_BF16 || a->seg_stride < a->seg)))
    return fail(h, KREA_CUDA_E_ARG, "gemm: the column remap needs the bf16 epilogue, seg and seg_stride multiples of 8 and seg_stride >= seg");
  const int out_span = a->seg > 0 ? ((a->N - 1) / a->seg) * a->seg_stride + (a->N - 1) % a->seg + 1 : out_cols;
  if (a->lda < a->K || a->ldw < a->N || a->ldc < out_span) return fail(h, KREA_CUDA_E_ARG, "gemm: a leading dimension is smaller than its row");
  if (a->epilogue == KREA_CUDA_EPI_SWIGLU && a->N % 64) return fail(h, KREA_CUDA_E_ARG, "gemm: SwiGLU needs N to be a multiple of 64 (32 gate + 32 up columns per group)");
  if (a->epilogue == KREA_CUDA_EPI_RESID_GATE && !aligned16(a->vec)) return fail(h, KREA_CUDA_E_ARG, "gemm: the gate vector must be 16-byte aligned");
  GemmParams p{};
  p.C = (__nv_bfloat16*)a->C;
  p.ldc = a->ldc;
  p.M = a->M; p.N = a->N; p.K = a->K;
  p.status = h->status_dev;
  p.epi = a->epilogue;
  p.seg = a->seg; p.seg_stride = a->seg_stride;
  p.vec = (a->epilogue == KREA_CUDA_EPI_RESID_GATE || has_bias) ? a->vec : nullptr;
  if (a->epilogue == KREA_CUDA_EPI_QKNORM_ROPE) {
    if (a->rope_mode == KREA_CUDA_ROPE_HALF) return fail(h, KREA_CUDA_E_UNSUPPORTED, "gemm: the fused epilogue rotates interleaved pairs only (rope_mode 0 or 2)");
    if (a->rope_mode != KREA_CUDA_ROPE_PAIRS && a->rope_mode != KREA_CUDA_ROPE_NONE) return fail(h, KREA_CUDA_E_ARG, "gemm: bad rope_mode");
    if (a->n_q < 0 || a->n_k < 0 || a->q_off < 0 || a->k_off < 0 || a->q_off % 128 || a->k_off % 128) return fail(h, KREA_CUDA_E_ARG, "gemm: head blocks must start at multiples of 128 columns");
    if ((int64_t)a->q_off + (int64_t)a->n_q * 128 > a->N || (int64_t)a->k_off + (int64_t)a->n_k * 128 > a->N) return fail(h, KREA_CUDA_E_ARG, "gemm: head blocks exceed N");
    if ((a->n_q > 0 && !a->wq) || (a->n_k > 0 && !a->wk)) return fail(h, KREA_CUDA_E_ARG, "gemm: QK-norm weights missing");
    if (a->rope_mode == KREA_CUDA_ROPE_PAIRS && (!a->cos || !a->sin)) return fail(h, KREA_CUDA_E_ARG, "gemm: cos/sin tables missing");
    if (!aligned16(a->wq) || !aligned16(a->wk) || !aligned16(a->cos) || !aligned16(a->sin) || a->row0 < 0) return fail(h, KREA_CUDA_E_ARG, "gemm: weights / tables must be 16-byte aligned, row0 >= 0");
    p.epi = 1;
    p.q_off = a->q_off; p.n_q = a->n_q; p.k_off = a->k_off; p.n_k = a->n_k;
    p.wq = a->wq ? a->wq : a->wk; p.wk = a->wk ? a->wk : a->wq;
    p.cos = a->cos; p.sin = a->sin; p.row0 = a->row0; p.eps = a->eps; p.rope_mode = a->rope_mode;
    p.big_dim = -1;
    if (a->qbig || a->kbig) {
      if (!a->qbig || !a->kbig || a->big_dim < 0 || a->big_dim >= 128) return fail(h, KREA_CUDA_E_ARG, "gemm: big_dim needs both side buffers and 0 <= big_dim < 128");
      p.big_dim = a->big_dim; p.qbig = a->qbig; p.kbig = a->kbig;
    }
    if (bound_out && a->n_q > 0 && a->n_k > 0) {
      p.bound_out = bound_out;
      p.bound_scale_log2 = (float)(1.0 / sqrt(128.0) * 1.4426950408889634);
    }
  }
  CUDA_TRY(h, cudaSetDevice(h->device));
  CUtensorMap tmA, tmW, tmA2, tmW2;
  memset(&tmA2, 0, sizeof(tmA2));
  memset(&tmW2, 0, sizeof(tmW2));
  int rc = make_kv_map(h, &tmA, a->A, a->K, a->M, 1, a->lda, 0, "A", 128);
  if (rc) return rc;
  if ((rc = make_kv_map(h, &tmW, a->W, a->N, a->K, 1, a->ldw, 0, "W", 64))) return rc;
  if (a->lora_A || a->lora_W) {
    if (!a->lora_A || !a->lora_W || !aligned16(a->lora_A) || !aligned16(a->lora_W) || a->lora_K <= 0 || a->lora_K % 8 || a->lora_lda % 8 || a->lora_ldw % 8 ||
        a->lora_lda < a->lora_K || a->lora_ldw < a->N)
      return fail(h, KREA_CUDA_E_ARG, "gemm: bad second (LoRA) product");
    if ((rc = make_kv_map(h, &tmA2, a->lora_A, a->lora_K, a->M, 1, a->lora_lda, 0, "lora A", 128))) return rc;
    if ((rc = make_kv_map(h, &tmW2, a->lora_W, a->N, a->lora_K, 1, a->lora_ldw, 0, "lora W", 64))) return rc;
    p.K2 = a->lora_K;
  }
  if (h->sm_count == 0) {
    cudaDeviceProp prop;
    CUDA_TRY(h, cudaGetDeviceProperties(&prop, h->device));
    h->sm_count = prop.multiProcessorCount;
  }
  CUDA_TRY(h, launch_gemm_bf16_sm100(tmA, tmW, tmA2, tmW2, p, h->sm_count, h->gemm_bn, h->stream));
  h->launches++;
  return KREA_CUDA_OK;
}

int krea_cuda_gemm(krea_cuda* h, const krea_cuda_gemm_args* a) { return gemm_impl(h, a, nullptr); }

int krea_cuda_dequant_q8(krea_cuda* h, const krea_cuda_dequant_args* a) {
  if (!h || !a) return fail(h, KREA_CUDA_E_ARG, "dequant_q8: null handle or arguments");
  if (a->K < 0 || a->N < 0) return fail(h, KREA_CUDA_E_ARG, "dequant_q8: negative size");
  if (a->K == 0 || a->N == 0) return KREA_CUDA_OK;
  if (a->K % 128 || a->N % 16) return fail(h, KREA_CUDA_E_ARG, "dequant_q8: K must be a multiple of 128 (the scale group) and N of 16");
  if (!a->wq || !a->scales || !a->out || !aligned16(a->wq) || !aligned16(a->scales) || !aligned16(a->out)) return fail(h, KREA_CUDA_E_ARG, "dequant_q8: null or misaligned pointer");
  if (a->ldq % 16 || a->lds % 4 || a->ldo % 8 || a->ldq < a->N || a->lds < a->N || a->ldo < a->N) return fail(h, KREA_CUDA_E_ARG, "dequant_q8: bad leading dimension");
  DequantParams p{};
  p.wq = (const int8_t*)a->wq; p.scales = a->scales; p.out = (__nv_bfloat16*)a->out;
  p.K = a->K; p.N = a->N; p.ldq = a->ldq; p.lds = a->lds; p.ldo = a->ldo;
  CUDA_TRY(h, cudaSetDevice(h->device));
  CUDA_TRY(h, launch_dequant_q8(p, h->stream));
  h->launches++;
  return KREA_CUDA_OK;
}

int krea_cuda_rms_norm(krea_cuda* h, const krea_cuda_rmsnorm_args* a) {
  if (!h || !a) return fail(h, KREA_CUDA_E_ARG, "rms_norm: null handle or arguments");
  if (a->rows < 0 || a->width < 0) return fail(h, KREA_CUDA_E_ARG, "rms_norm: negative size");
  if (a->rows == 0 || a->width == 0) return KREA_CUDA_OK;
  if (!a->x || !a->mul || !a->y || !aligned16(a->x) || !aligned16(a->mul) || !aligned16(a->add) || !aligned16(a->y))
    return fail(h, KREA_CUDA_E_ARG, "rms_norm: null or misaligned pointer");
  const int m = a->f32_out ? 4 : 8;
  if (a->width % 4 || a->ld_in % 4 || a->ld_out % m || a->ld_in < a->width || a->ld_out < a->width)
    return fail(h, KREA_CUDA_E_ARG, "rms_norm: width and leading dimensions must be multiples of 4 (8 for the bf16 output) and cover the row");
  RmsNormParams p{};
  p.x = a->x; p.mul = a->mul; p.add = a->add; p.y = a->y;
  p.rows = a->rows; p.width = a->width; p.ld_in = a->ld_in; p.ld_out = a->ld_out;
  p.eps = a->eps; p.f32_out = a->f32_out ? 1 : 0;
  CUDA_TRY(h, cudaSetDevice(h->device));
  CUDA_TRY(h, launch_rms_norm(p, h->stream));
  h->launches++;
  return KREA_CUDA_OK;
}

// byte offsets of the block's intermediates inside its workspace: h | qkvg | ao | mid
struct BlockLayout {
  size_t h, qkvg, ao, mid, qbig, kbig, total;
  int dim, qkvg_cols;
};
static BlockLayout block_layout(const krea_cuda_dit_block_args* a) {
  BlockLayout l{};
  l.dim = a->heads * 128;
  l.qkvg_cols = (2 * a->heads + 2 * a->kv_heads) * 128;
  auto up = [](size_t b) { return (b + 255) & ~(size_t)255; };
  const size_t rows = (size_t)(a->rows > 0 ? a->rows : 0);
  l.h = 0;
  l.qkvg = l.h + up(rows * l.dim * 2);
  l.ao = l.qkvg + up(rows * l.qkvg_cols * 2);
  l.mid = l.ao + up(rows * l.dim * 2);
  l.qbig = l.mid + up(rows * (size_t)(a->ff > 0 ? a->ff : 0) * 2);
  l.kbig = l.qbig + up(rows * (size_t)a->heads * 4);
  l.total = l.kbig + up(rows * (size_t)a->kv_heads * 4);
  return l;
}

size_t krea_cuda_dit_block_workspace_bytes(const krea_cuda_dit_block_args* a) {
  if (!a || a->rows <= 0 || a->heads <= 0 || a->kv_heads <= 0 || a->ff <= 0) return 0;
  return block_layout(a).total;
}

int krea_cuda_dit_block(krea_cuda* h, const krea_cuda_dit_block_args* a) {
  if (!h || !a) return fail(h, KREA_CUDA_E_ARG, "dit_block: null handle or arguments");
  if (a->rows < 0 || a->heads <= 0 || a->kv_heads <= 0 || a->ff <= 0 || a->heads % a->kv_heads) return fail(h, KREA_CUDA_E_ARG, "dit_block: bad sizes");
  if (a->ff % 32) return fail(h, KREA_CUDA_E_ARG, "dit_block: ff must be a multiple of 32 (gate / up interleave)");
  if (a->rows == 0) return KREA_CUDA_OK;
  if (!a->x || !a->mods || !a->w_qkvg || !a->w_o || !a->w_gu || !a->w_down || !a->qn || !a->kn || !a->cos || !a->sin)
    return fail(h, KREA_CUDA_E_ARG, "dit_block: null tensor");
  const BlockLayout l = block_layout(a);
  char* ws = (char*)a->workspace;
  if (ws) {
    if (a->workspace_bytes < l.total || !aligned16(ws)) return fail(h, KREA_CUDA_E_NOMEM, "dit_block: workspace too small (%zu < %zu) or misaligned", a->workspace_bytes, l.total);
  } else {
    CUDA_TRY(h, cudaSetDevice(h->device));
    if (h->block_ws_bytes < l.total) {
      CUDA_TRY(h, cudaStreamSynchronize(h->stream));
      if (h->block_ws) cudaFree(h->block_ws);
      h->block_ws = nullptr;
      h->block_ws_bytes = 0;
      if (cudaMalloc(&h->block_ws, l.total) != cudaSuccess) {
        cudaGetLastError();
        return fail(h, KREA_CUDA_E_NOMEM, "dit_block: cannot allocate %zu bytes of workspace", l.total);
      }
      h->block_ws_bytes = l.total;
    }
    ws = (char*)h->block_ws;
  }
  const int D = l.dim, QC = l.qkvg_cols, R = a->rows, H = a->heads, KV = a->kv_heads;
  const float* mod = a->mods;
  void* hb = ws + l.h;
  char* qkvg = ws + l.qkvg;
  void* ao = ws + l.ao;
  void* mid = ws + l.mid;
  int rc;
  // 1. h = rms_norm(x) * mul1 + add1                                           (model.mm:373)
  krea_cuda_rmsnorm_args n1 = {a->x, mod, mod + D, hb, R, D, D, D, a->eps, 0};
  if ((rc = krea_cuda_rms_norm(h, &n1))) return rc;
  // 2. q | k | v | gate = h Wqkvg, q and k normalised and rotated in the epilogue  (model.mm:374-375)
  krea_cuda_gemm_args g1 = {};
  g1.A = hb; g1.W = a->w_qkvg; g1.C = qkvg; g1.M = R; g1.N = QC; g1.K = D; g1.lda = D; g1.ldw = QC; g1.ldc = QC;
  g1.epilogue = KREA_CUDA_EPI_QKNORM_ROPE;
  g1.q_off = 0; g1.n_q = H; g1.k_off = D; g1.n_k = KV;
  g1.wq = a->qn; g1.wk = a->kn; g1.cos = a->cos; g1.sin = a->sin; g1.row0 = 0; g1.eps = a->eps; g1.rope_mode = KREA_CUDA_ROPE_PAIRS;
  if (a->use_big_dim) {
    if (a->big_dim < 0 || a->big_dim >= 128) return fail(h, KREA_CUDA_E_ARG, "dit_block: big_dim must be in [0, 128)");
    g1.big_dim = a->big_dim; g1.qbig = (float*)(ws + l.qbig); g1.kbig = (float*)(ws + l.kbig);
  }
  float* bound = (float*)(h->status_dev + 8);         // the device float the fused call's pre-pass uses too
  if ((rc = gemm_impl(h, &g1, bound))) return rc;
  // 3. ao = attention(q, k, v) * sigmoid(gate)                                  (model.mm:282-288, 377)
  // Q and K arrive normalised, so the operator runs without its prologue - but with the logit bound the
  // projection's epilogue derived from the QK-norm weights, i.e. with the bounded form of the softmax.
  AttnCall at{};
  at.Q = qkvg; at.K = qkvg + (size_t)D * 2; at.V = qkvg + (size_t)(D + KV * 128) * 2; at.O = ao;
  at.G = qkvg + (size_t)(D + 2 * KV * 128) * 2;
  at.batch = 1; at.Lq = R; at.Lk = R; at.heads = H; at.group = H / KV;
  at.ldq = QC; at.ldk = QC; at.ldv = QC; at.ldo = D; at.ldg = QC;
  at.logit_bound = bound;
  at.bound_given = true;
  if (a->use_big_dim) { at.QB = (const float*)(ws + l.qbig); at.KB = (const float*)(ws + l.kbig); }
  if ((rc = run_attention(h, at))) return rc;
  // 4. x += gate1 * (ao Wo)                                                     (model.mm:357-359, 379)
  krea_cuda_gemm_args g2 = {};
  g2.A = ao; g2.W = a->w_o; g2.C = a->x; g2.M = R; g2.N = D; g2.K = D; g2.lda = D; g2.ldw = D; g2.ldc = D;
  g2.epilogue = KREA_CUDA_EPI_RESID_GATE; g2.vec = mod + 2 * (size_t)D;
  if ((rc = krea_cuda_gemm(h, &g2))) return rc;
  // 5. h = rms_norm(x) * mul2 + add2                                           (model.mm:381)
  krea_cuda_rmsnorm_args n2 = {a->x, mod + 3 * (size_t)D, mod + 4 * (size_t)D, hb, R, D, D, D, a->eps, 0};
  if ((rc = krea_cuda_rms_norm(h, &n2))) return rc;
  // 6. mid = swiglu(h Wgu);  7. x += gate2 * (mid Wdown)                       (model.mm:361-366, 382)
  krea_cuda_gemm_args g3 = {};
  g3.A = hb; g3.W = a->w_gu; g3.C = mid; g3.M = R; g3.N = 2 * a->ff; g3.K = D; g3.lda = D; g3.ldw = 2 * a->ff; g3.ldc = a->ff;
  g3.epilogue = KREA_CUDA_EPI_SWIGLU;
  if ((rc = krea_cuda_gemm(h, &g3))) return rc;
  krea_cuda_gemm_args g4 = {};
  g4.A = mid; g4.W = a->w_down; g4.C = a->x; g4.M = R; g4.N = D; g4.K = a->ff; g4.lda = a->ff; g4.ldw = D; g4.ldc = D;
  g4.epilogue = KREA_CUDA_EPI_RESID_GATE; g4.vec = mod + 5 * (size_t)D;
  return krea_cuda_gemm(h, &g4);
}

int krea_cuda_layerwise_attn(krea_cuda* h, const krea_cuda_layerwise_args* a) {
  if (!h || !a) return fail(h, KREA_CUDA_E_ARG, "layerwise_attn: null handle or arguments");
  if (a->rows < 0 || a->heads < 0 || a->rows % 12) return fail(h, KREA_CUDA_E_ARG, "layerwise_attn: rows (%d) must be a non-negative multiple of 12", a->rows);
  if (a->rows == 0 || a->heads == 0) return KREA_CUDA_OK;
  if (!a->qkvg || !a->out || !aligned16(a->qkvg) || !aligned16(a->out)) return fail(h, KREA_CUDA_E_ARG, "layerwise_attn: null or misaligned pointer");
  const int offs[4] = {a->q_off, a->k_off, a->v_off, a->g_off};
  for (int o : offs)
    if (o < 0 || o % 8 || (int64_t)o + (int64_t)a->heads * 128 > a->ld) return fail(h, KREA_CUDA_E_ARG, "layerwise_attn: column offset %d does not fit %d heads inside ld %d (offsets are multiples of 8)", o, a->heads, a->ld);
  if (a->ld % 8 || a->ldo % 8 || a->ldo < a->heads * 128) return fail(h, KREA_CUDA_E_ARG, "layerwise_attn: leading dimensions must be multiples of 8 and ldo must cover all heads");
  LayerwiseParams p{};
  p.qkvg = (const __nv_bfloat16*)a->qkvg;
  p.out = (__nv_bfloat16*)a->out;
  p.rows = a->rows;
  p.heads = a->heads;
  p.ld = a->ld;
  p.ldo = a->ldo;
  p.q_off = a->q_off; p.k_off = a->k_off; p.v_off = a->v_off; p.g_off = a->g_off;
  p.scale = (float)(1.0 / sqrt(128.0));   // metal.mm:206
  CUDA_TRY(h, cudaSetDevice(h->device));
  CUDA_TRY(h, launch_layerwise_attn(p, h->stream));
  h->launches++;
  return KREA_CUDA_OK;
}

int krea_cuda_reshard_pack(krea_cuda* h, const krea_cuda_reshard_args* a) { return reshard(h, a, false); }
int krea_cuda_reshard_unpack(krea_cuda* h, const krea_cuda_reshard_args* a) { return reshard(h, a, true); }

}  // extern "C"

int krea_joint_prepass(krea_cuda* h, const krea_cuda_joint_args* a, void* k_scratch) { return joint_prepass(h, a, k_scratch); }
int krea_joint_attend(krea_cuda* h, const krea_cuda_joint_args* a, void* k_scratch) { return joint_attend(h, a, k_scratch); }
int krea_joint_attend_scatter(krea_cuda* h, const krea_cuda_joint_args* a, void* k_scratch, void* const* o_blk, int n, int rows) {
  return joint_attend(h, a, k_scratch, o_blk, n, rows);
}
int krea_validate_joint(krea_cuda* h, const krea_cuda_joint_args* a) { return validate_joint(h, a); }
