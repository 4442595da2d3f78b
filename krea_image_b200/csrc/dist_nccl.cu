// Sequence-parallel entry points of libkrea_cuda: an all-to-all over NCCL either side of the single-GPU
// joint attention (Ulysses-style reshard: sequence-sharded rows <-> head-sharded rows).  The reference is
// single-device (one MTLCommandQueue, engine/src/metal.mm:56-59), so nothing here has a counterpart in it;
// what is kept from it is that heads are independent units of work (grid.y = heads, metal.mm:199-201).
//
// NCCL is loaded at run time, so the library has no link-time dependency on it and the single-GPU entry
// points work on a machine without NCCL.  Remote rows always land in local memory before a kernel reads
// them: by ncclSend/ncclRecv, or - in peer-store mode - by the sending rank's own kernels, which write the
// destination GPU's mapped workspace with plain 16-byte stores.  No kernel of this library ever reads a
// peer's memory, and no TMA operation touches it.
#include <dlfcn.h>
#include <nccl.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

#include <mutex>

#include "attention_sm100.h"
#include "handle.h"

using namespace krea;

namespace {

struct NcclApi {
  void* lib = nullptr;
  decltype(&ncclGetUniqueId) GetUniqueId = nullptr;
  decltype(&ncclCommInitRank) CommInitRank = nullptr;
  decltype(&ncclCommDestroy) CommDestroy = nullptr;
  decltype(&ncclCommAbort) CommAbort = nullptr;
  decltype(&ncclCommGetAsyncError) CommGetAsyncError = nullptr;
  decltype(&ncclGetErrorString) GetErrorString = nullptr;
  decltype(&ncclGroupStart) GroupStart = nullptr;
  decltype(&ncclGroupEnd) GroupEnd = nullptr;
  decltype(&ncclSend) Send = nullptr;
  decltype(&ncclRecv) Recv = nullptr;
  decltype(&ncclAllReduce) AllReduce = nullptr;
  decltype(&ncclAllGather) AllGather = nullptr;
  std::string why;   // why loading failed
};

std::mutex g_nccl_mutex;
NcclApi g_nccl;

// Loads NCCL once per process.  Returns nullptr (with g_nccl.why set) if the library or a symbol is missing.
const NcclApi* nccl_api() {
  std::lock_guard<std::mutex> lock(g_nccl_mutex);
  if (g_nccl.lib) return &g_nccl;
  const char* name = getenv("KREA_CUDA_NCCL_LIB");
  if (!name || !*name) name = "libnccl.so.2";
  void* lib = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
  if (!lib) {
    const char* e = dlerror();
    g_nccl.why = std::string("cannot load ") + name + ": " + (e ? e : "unknown error");
    return nullptr;
  }
  bool ok = true;
  auto sym = [&](const char* s) {
    void* p = dlsym(lib, s);
    if (!p) {
      ok = false;
      g_nccl.why = std::string("NCCL symbol missing: ") + s;
    }
    return p;
  };
  NcclApi a;
  a.GetUniqueId = (decltype(a.GetUniqueId))sym("ncclGetUniqueId");
  a.CommInitRank = (decltype(a.CommInitRank))sym("ncclCommInitRank");
  a.CommDestroy = (decltype(a.CommDestroy))sym("ncclCommDestroy");
  a.CommAbort = (decltype(a.CommAbort))sym("ncclCommAbort");
  a.CommGetAsyncError = (decltype(a.CommGetAsyncError))sym("ncclCommGetAsyncError");
  a.GetErrorString = (decltype(a.GetErrorString))sym("ncclGetErrorString");
  a.GroupStart = (decltype(a.GroupStart))sym("ncclGroupStart");
  a.GroupEnd = (decltype(a.GroupEnd))sym("ncclGroupEnd");
  a.Send = (decltype(a.Send))sym("ncclSend");
  a.Recv = (decltype(a.Recv))sym("ncclRecv");
  a.AllReduce = (decltype(a.AllReduce))sym("ncclAllReduce");
  a.AllGather = (decltype(a.AllGather))sym("ncclAllGather");
  if (!ok) {
    dlclose(lib);
    return nullptr;
  }
  a.lib = lib;
  g_nccl = a;
  return &g_nccl;
}

}  // namespace

struct KreaDist {
  const NcclApi* api = nullptr;
  ncclComm_t comm = nullptr;
  int rank = -1, nranks = 0;
  void* ws = nullptr;            // workspace of the reshard / sequence-parallel calls
  size_t ws_bytes = 0;
  cudaStream_t side = nullptr;   // second stream: exchanges that overlap the K normalisation pass
  cudaEvent_t ev[4] = {};        // 0 start, 1 K landed, 2 Q and V landed, 3 spare
  // Peer-store mode: every rank's workspace is mapped into every other rank's process (CUDA IPC), the pack
  // kernels and the attention epilogue store straight into the destination rank's memory over NVLink, and
  // NCCL only provides the barriers in between.
  bool p2p = false;              // agreed by all ranks at init
  void* sym = nullptr;           // this rank's symmetric workspace
  size_t sym_bytes = 0;
  void* peer[8] = {};            // peer[r]: rank r's symmetric workspace as seen from this process (peer[rank] == sym)
  unsigned char* xchg = nullptr; // device scratch: 8 IPC handles + the barrier word
};

#define NCCL_TRY(h, d, expr)                                                                               \
  do {                                                                                                     \
    ncclResult_t r_ = (expr);                                                                              \
    if (r_ != ncclSuccess) return fail(h, KREA_CUDA_E_COMM, "%s: %s", #expr, (d)->api->GetErrorString(r_)); \
  } while (0)

static int need_dist(krea_cuda* h, const char* who) {
  if (!h) return KREA_CUDA_E_ARG;
  if (!h->dist || !h->dist->comm) return fail(h, KREA_CUDA_E_COMM, "%s: krea_cuda_dist_init has not been called (or the communicator was aborted)", who);
  return KREA_CUDA_OK;
}

// Grows the workspace; the old block is released only after the stream that may still use it is idle.
static int dist_ws(krea_cuda* h, size_t bytes, void** out) {
  KreaDist* d = h->dist;
  if (d->ws_bytes < bytes) {
    CUDA_TRY(h, cudaStreamSynchronize(h->stream));
    CUDA_TRY(h, cudaStreamSynchronize(d->side));
    if (d->ws) cudaFree(d->ws);
    d->ws = nullptr;
    d->ws_bytes = 0;
    if (cudaMalloc(&d->ws, bytes) != cudaSuccess) {
      cudaGetLastError();
      return fail(h, KREA_CUDA_E_NOMEM, "sequence-parallel workspace: cannot allocate %zu bytes", bytes);
    }
    d->ws_bytes = bytes;
  }
  *out = d->ws;
  return KREA_CUDA_OK;
}

// Equal-block all-to-all: block p of `send` goes to rank p, block p of `recv` comes from rank p.
static int all_to_all(krea_cuda* h, const void* send, void* recv, size_t block_bytes, cudaStream_t stream) {
  KreaDist* d = h->dist;
  NCCL_TRY(h, d, d->api->GroupStart());
  for (int p = 0; p < d->nranks; p++) {
    NCCL_TRY(h, d, d->api->Send((const char*)send + (size_t)p * block_bytes, block_bytes, ncclInt8, p, d->comm, stream));
    NCCL_TRY(h, d, d->api->Recv((char*)recv + (size_t)p * block_bytes, block_bytes, ncclInt8, p, d->comm, stream));
  }
  NCCL_TRY(h, d, d->api->GroupEnd());
  return KREA_CUDA_OK;
}

static size_t round256(size_t b) { return (b + 255) & ~(size_t)255; }

// pack the local rows by destination head block into `stage`, then exchange into dst
static int seq_to_heads_on(krea_cuda* h, const void* src, void* dst, void* stage, int rows_local, int cols_per_rank, int src_ld,
                           int src_col0, cudaStream_t stream) {
  KreaDist* d = h->dist;
  ReshardParams p{};
  p.src = (const __nv_bfloat16*)src;
  p.dst = (__nv_bfloat16*)stage;
  p.nranks = d->nranks;
  p.rows = rows_local;
  p.cols_per_rank = cols_per_rank;
  p.src_ld = src_ld;
  p.src_col0 = src_col0;
  CUDA_TRY(h, launch_reshard_pack(p, stream));
  h->launches++;
  return all_to_all(h, stage, dst, (size_t)rows_local * cols_per_rank * 2, stream);
}

// exchange the row blocks of src as they are into `stage`, then merge the per-rank head blocks into dst
static int heads_to_seq_on(krea_cuda* h, const void* src, void* dst, void* stage, int rows_local, int cols_per_rank, int dst_ld,
                           int dst_col0, cudaStream_t stream) {
  KreaDist* d = h->dist;
  int rc = all_to_all(h, src, stage, (size_t)rows_local * cols_per_rank * 2, stream);
  if (rc) return rc;
  ReshardParams p{};
  p.src = (const __nv_bfloat16*)stage;
  p.dst = (__nv_bfloat16*)dst;
  p.nranks = d->nranks;
  p.rows = rows_local;
  p.cols_per_rank = cols_per_rank;
  p.dst_ld = dst_ld;
  p.dst_col0 = dst_col0;
  CUDA_TRY(h, launch_reshard_unpack(p, stream));
  h->launches++;
  return KREA_CUDA_OK;
}

// ---- peer-store mode ---------------------------------------------------------------------------------
constexpr size_t XCHG_BYTES = 8 * sizeof(cudaIpcMemHandle_t) + 256;

// All ranks reach this point of their streams: a one-float all-reduce (max, so the word stays bounded however
// many barriers pass).  Stream-ordered; kernels enqueued after it on any rank start only after every rank's
// earlier kernels (and their peer stores) have completed.
static int rank_barrier(krea_cuda* h, cudaStream_t stream, ncclRedOp_t op = ncclMax) {
  KreaDist* d = h->dist;
  float* w = (float*)(d->xchg + 8 * sizeof(cudaIpcMemHandle_t));
  NCCL_TRY(h, d, d->api->AllReduce(w, w, 1, ncclFloat, op, d->comm, stream));
  return KREA_CUDA_OK;
}

static void close_peers(KreaDist* d) {
  for (int r = 0; r < 8; r++) {
    if (d->peer[r] && r != d->rank) cudaIpcCloseMemHandle(d->peer[r]);
    d->peer[r] = nullptr;
  }
}

// (Re)allocates the symmetric workspace and maps every rank's copy.  Collective: every rank calls it with
// the same size at the same point of its call sequence.  Returns KREA_CUDA_OK with d->p2p possibly cleared
// (all ranks agree) when a mapping could not be made.
static int sym_alloc(krea_cuda* h, size_t bytes) {
  KreaDist* d = h->dist;
  // nobody may still be storing into the old block, and nobody may keep a mapping of it
  CUDA_TRY(h, cudaStreamSynchronize(h->stream));
  CUDA_TRY(h, cudaStreamSynchronize(d->side));
  int rc = rank_barrier(h, h->stream);
  if (rc) return rc;
  CUDA_TRY(h, cudaStreamSynchronize(h->stream));
  close_peers(d);
  if ((rc = rank_barrier(h, h->stream))) return rc;
  CUDA_TRY(h, cudaStreamSynchronize(h->stream));
  if (d->sym) cudaFree(d->sym);
  d->sym = nullptr;
  d->sym_bytes = 0;
  float* w = (float*)(d->xchg + 8 * sizeof(cudaIpcMemHandle_t));
  // the ranks agree on the outcome of a step (minimum of their flags) before any of them moves on: a rank
  // that failed alone would otherwise leave the others waiting in the next collective
  auto agree = [&](float mine_ok, float* all_ok) -> int {
    CUDA_TRY(h, cudaMemcpyAsync(w, &mine_ok, sizeof(float), cudaMemcpyHostToDevice, h->stream));
    const int r = rank_barrier(h, h->stream, ncclMin);
    if (r) return r;
    CUDA_TRY(h, cudaMemcpyAsync(all_ok, w, sizeof(float), cudaMemcpyDeviceToHost, h->stream));
    CUDA_TRY(h, cudaStreamSynchronize(h->stream));
    return KREA_CUDA_OK;
  };
  float ok = 1.f;
  if (cudaMalloc(&d->sym, bytes) != cudaSuccess) {
    cudaGetLastError();
    d->sym = nullptr;
    ok = 0.f;
  }
  float all_ok = 0.f;
  if ((rc = agree(ok, &all_ok))) return rc;
  if (all_ok < 0.5f) {
    if (d->sym) cudaFree(d->sym);
    d->sym = nullptr;
    return fail(h, KREA_CUDA_E_NOMEM, "sequence-parallel workspace: a rank could not allocate %zu bytes", bytes);
  }
  d->sym_bytes = bytes;
  // Every step below that can fail on one rank alone only lowers that rank's flag; the ranks compare flags
  // before the next collective, so they either all go on or all fall back to NCCL transfers together.
  cudaIpcMemHandle_t mine, all[8];
  ok = 1.f;
  if (cudaIpcGetMemHandle(&mine, d->sym) != cudaSuccess ||
      cudaMemcpyAsync(d->xchg + d->rank * sizeof(mine), &mine, sizeof(mine), cudaMemcpyHostToDevice, h->stream) != cudaSuccess) {
    cudaGetLastError();
    ok = 0.f;
  }
  if ((rc = agree(ok, &all_ok))) return rc;
  if (all_ok < 0.5f) {
    d->p2p = false;
    return KREA_CUDA_OK;
  }
  NCCL_TRY(h, d, d->api->AllGather(d->xchg + d->rank * sizeof(mine), d->xchg, sizeof(mine), ncclInt8, d->comm, h->stream));
  ok = 1.f;
  if (cudaMemcpyAsync(all, d->xchg, sizeof(mine) * d->nranks, cudaMemcpyDeviceToHost, h->stream) != cudaSuccess ||
      cudaStreamSynchronize(h->stream) != cudaSuccess) {
    cudaGetLastError();
    ok = 0.f;
  }
  for (int r = 0; r < d->nranks && ok > 0.5f; r++) {
    if (r == d->rank) {
      d->peer[r] = d->sym;
    } else if (cudaIpcOpenMemHandle(&d->peer[r], all[r], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
      cudaGetLastError();
      d->peer[r] = nullptr;
      ok = 0.f;
    }
  }
  // every rank must take the same path afterwards
  if ((rc = agree(ok, &all_ok))) return rc;
  if (all_ok < 0.5f) {
    close_peers(d);
    d->p2p = false;
  }
  return KREA_CUDA_OK;
}

static int validate_a2a(krea_cuda* h, const krea_cuda_a2a_args* a, bool to_heads) {
  if (!a) return fail(h, KREA_CUDA_E_ARG, "reshard: null arguments");
  if (a->rows_local < 0 || a->cols_per_rank < 0) return fail(h, KREA_CUDA_E_ARG, "reshard: negative size");
  if (a->rows_local == 0 || a->cols_per_rank == 0) return KREA_CUDA_OK;
  if (!a->src || !a->dst || !aligned16(a->src) || !aligned16(a->dst)) return fail(h, KREA_CUDA_E_ARG, "reshard: null or misaligned pointer");
  const int ld = to_heads ? a->src_ld : a->dst_ld, col0 = to_heads ? a->src_col0 : a->dst_col0;
  if (a->cols_per_rank % 8 || ld % 8 || col0 % 8 || col0 < 0) return fail(h, KREA_CUDA_E_ARG, "reshard: columns and leading dimension must be multiples of 8");
  if ((int64_t)col0 + (int64_t)h->dist->nranks * a->cols_per_rank > ld) return fail(h, KREA_CUDA_E_ARG, "reshard: column blocks exceed the leading dimension");
  return KREA_CUDA_OK;
}

void krea_dist_release(krea_cuda* h) {
  KreaDist* d = h ? h->dist : nullptr;
  if (!d) return;
  if (d->side) cudaStreamSynchronize(d->side);
  close_peers(d);
  if (d->comm) d->api->CommDestroy(d->comm);
  if (d->ws) cudaFree(d->ws);
  if (d->sym) cudaFree(d->sym);
  if (d->xchg) cudaFree(d->xchg);
  for (cudaEvent_t e : d->ev)
    if (e) cudaEventDestroy(e);
  if (d->side) cudaStreamDestroy(d->side);
  delete d;
  h->dist = nullptr;
}

extern "C" {

int krea_cuda_dist_unique_id(void* id_out, char* err, int errlen) {
  auto say = [&](const char* m) {
    if (err && errlen > 0) snprintf(err, (size_t)errlen, "%s", m);
  };
  if (!id_out) {
    say("krea_cuda_dist_unique_id: null output");
    return KREA_CUDA_E_ARG;
  }
  const NcclApi* api = nccl_api();
  if (!api) {
    say(g_nccl.why.c_str());
    return KREA_CUDA_E_COMM;
  }
  static_assert(sizeof(ncclUniqueId) == KREA_CUDA_DIST_ID_BYTES, "id size is part of the ABI");
  ncclUniqueId id;
  const ncclResult_t r = api->GetUniqueId(&id);
  if (r != ncclSuccess) {
    say(api->GetErrorString(r));
    return KREA_CUDA_E_COMM;
  }
  memcpy(id_out, &id, sizeof(id));
  return KREA_CUDA_OK;
}

int krea_cuda_dist_init(krea_cuda* h, int rank, int nranks, const void* id) {
  if (!h) return KREA_CUDA_E_ARG;
  if (!id || nranks < 1 || rank < 0 || rank >= nranks) return fail(h, KREA_CUDA_E_ARG, "dist_init: bad rank %d of %d or null id", rank, nranks);
  const NcclApi* api = nccl_api();
  if (!api) return fail(h, KREA_CUDA_E_COMM, "dist_init: %s", g_nccl.why.c_str());
  krea_dist_release(h);
  CUDA_TRY(h, cudaSetDevice(h->device));
  KreaDist* d = new KreaDist();
  d->api = api;
  h->dist = d;
  bool ok = cudaStreamCreateWithFlags(&d->side, cudaStreamNonBlocking) == cudaSuccess;
  for (int i = 0; i < 4 && ok; i++) ok = cudaEventCreateWithFlags(&d->ev[i], cudaEventDisableTiming) == cudaSuccess;
  if (!ok) {
    krea_dist_release(h);
    return fail(h, KREA_CUDA_E_CUDA, "dist_init: cannot create the side stream or its events");
  }
  ncclUniqueId uid;
  memcpy(&uid, id, sizeof(uid));
  const ncclResult_t r = api->CommInitRank(&d->comm, nranks, uid, rank);
  if (r != ncclSuccess) {
    d->comm = nullptr;
    krea_dist_release(h);
    return fail(h, KREA_CUDA_E_COMM, "ncclCommInitRank: %s", api->GetErrorString(r));
  }
  d->rank = rank;
  d->nranks = nranks;
  // exchange mode: peer stores unless the environment asks for NCCL transfers, the group is too large for
  // the kernels' tables, or a first small mapping round fails on any rank
  const char* mode = getenv("KREA_CUDA_SEQPAR_EXCHANGE");
  d->p2p = nranks >= 2 && nranks <= 8 && !(mode && strcmp(mode, "nccl") == 0);
  if (cudaMalloc((void**)&d->xchg, XCHG_BYTES) != cudaSuccess || cudaMemset(d->xchg, 0, XCHG_BYTES) != cudaSuccess) {
    cudaGetLastError();
    krea_dist_release(h);
    return fail(h, KREA_CUDA_E_NOMEM, "dist_init: cannot allocate the exchange scratch");
  }
  if (d->p2p) {
    const int rc = sym_alloc(h, 1 << 20);
    if (rc) {
      krea_dist_release(h);
      return rc;
    }
  }
  return KREA_CUDA_OK;
}

int krea_cuda_dist_exchange_mode(krea_cuda* h) { return (h && h->dist && h->dist->comm) ? (h->dist->p2p ? 1 : 0) : -1; }

int krea_cuda_dist_rank(krea_cuda* h) { return (h && h->dist && h->dist->comm) ? h->dist->rank : -1; }
int krea_cuda_dist_size(krea_cuda* h) { return (h && h->dist && h->dist->comm) ? h->dist->nranks : 0; }

int krea_cuda_dist_shutdown(krea_cuda* h) {
  if (!h) return KREA_CUDA_E_ARG;
  if (h->dist) {
    cudaSetDevice(h->device);
    cudaStreamSynchronize(h->stream);
  }
  krea_dist_release(h);
  return KREA_CUDA_OK;
}

int krea_cuda_dist_sync(krea_cuda* h, int timeout_ms) {
  int rc = need_dist(h, "dist_sync");
  if (rc) return rc;
  KreaDist* d = h->dist;
  CUDA_TRY(h, cudaSetDevice(h->device));
  struct timespec t0;
  clock_gettime(CLOCK_MONOTONIC, &t0);
  const char* what = nullptr;
  int code = KREA_CUDA_OK;
  for (;;) {
    const cudaError_t q = cudaStreamQuery(h->stream);
    if (q == cudaSuccess) break;
    if (q != cudaErrorNotReady) return fail(h, KREA_CUDA_E_CUDA, "dist_sync: %s", cudaGetErrorString(q));
    ncclResult_t async = ncclSuccess;
    const ncclResult_t r = d->api->CommGetAsyncError(d->comm, &async);
    if (r != ncclSuccess || (async != ncclSuccess && async != ncclInProgress)) {
      what = d->api->GetErrorString(r != ncclSuccess ? r : async);
      code = KREA_CUDA_E_COMM;
      break;
    }
    struct timespec t1;
    clock_gettime(CLOCK_MONOTONIC, &t1);
    const double ms = (t1.tv_sec - t0.tv_sec) * 1e3 + (t1.tv_nsec - t0.tv_nsec) * 1e-6;
    if (timeout_ms > 0 && ms > timeout_ms) {
      what = "timed out waiting for the stream";
      code = KREA_CUDA_E_TIMEOUT;
      break;
    }
    const struct timespec nap = {0, 200000};   // 0.2 ms
    nanosleep(&nap, nullptr);
  }
  if (code != KREA_CUDA_OK) {
    // Abort so that no collective of this rank keeps waiting for a peer; the handle falls back to
    // single-GPU service until dist_init is called again.
    d->api->CommAbort(d->comm);
    d->comm = nullptr;
    return fail(h, code, "dist_sync: %s; communicator aborted", what);
  }
  return krea_cuda_sync(h);
}

int krea_cuda_reshard_seq_to_heads(krea_cuda* h, const krea_cuda_a2a_args* a) {
  int rc = need_dist(h, "reshard_seq_to_heads");
  if (rc) return rc;
  if ((rc = validate_a2a(h, a, true))) return rc;
  if (a->rows_local == 0 || a->cols_per_rank == 0) return KREA_CUDA_OK;
  CUDA_TRY(h, cudaSetDevice(h->device));
  void* stage = nullptr;
  if ((rc = dist_ws(h, (size_t)h->dist->nranks * a->rows_local * a->cols_per_rank * 2, &stage))) return rc;
  return seq_to_heads_on(h, a->src, a->dst, stage, a->rows_local, a->cols_per_rank, a->src_ld, a->src_col0, h->stream);
}

int krea_cuda_reshard_heads_to_seq(krea_cuda* h, const krea_cuda_a2a_args* a) {
  int rc = need_dist(h, "reshard_heads_to_seq");
  if (rc) return rc;
  if ((rc = validate_a2a(h, a, false))) return rc;
  if (a->rows_local == 0 || a->cols_per_rank == 0) return KREA_CUDA_OK;
  CUDA_TRY(h, cudaSetDevice(h->device));
  void* stage = nullptr;
  if ((rc = dist_ws(h, (size_t)h->dist->nranks * a->rows_local * a->cols_per_rank * 2, &stage))) return rc;
  return heads_to_seq_on(h, a->src, a->dst, stage, a->rows_local, a->cols_per_rank, a->dst_ld, a->dst_col0, h->stream);
}

int krea_cuda_seqpar_joint_attention(krea_cuda* h, const krea_cuda_seqpar_args* a) {
  int rc = need_dist(h, "seqpar_joint_attention");
  if (rc) return rc;
  if (!a) return fail(h, KREA_CUDA_E_ARG, "seqpar_joint_attention: null arguments");
  KreaDist* d = h->dist;
  const int P = d->nranks;
  if (a->seq <= 0 || a->heads <= 0 || a->group < 1 || a->heads % a->group) return fail(h, KREA_CUDA_E_ARG, "seqpar_joint_attention: bad sizes");
  const int kvheads = a->heads / a->group;
  if (a->seq % P || a->heads % P || kvheads % P)
    return fail(h, KREA_CUDA_E_ARG, "seqpar_joint_attention: seq (%d), heads (%d) and kv heads (%d) must be multiples of the %d ranks", a->seq, a->heads, kvheads, P);
  const int rl = a->seq / P, hl = a->heads / P, kvl = kvheads / P;
  const int cl = hl * 128, kcl = kvl * 128;
  if (!a->Q || !a->K || !a->V || !a->O) return fail(h, KREA_CUDA_E_ARG, "seqpar_joint_attention: null tensor");
  if (!aligned16(a->Q) || !aligned16(a->K) || !aligned16(a->V) || !aligned16(a->O)) return fail(h, KREA_CUDA_E_ARG, "seqpar_joint_attention: pointers must be 16-byte aligned");
  if (a->ldq % 8 || a->ldk % 8 || a->ldv % 8 || a->ldo % 8 || a->ldq < a->heads * 128 || a->ldo < a->heads * 128 || a->ldk < kvheads * 128 || a->ldv < kvheads * 128)
    return fail(h, KREA_CUDA_E_ARG, "seqpar_joint_attention: leading dimensions must be multiples of 8 and cover all heads");

  // the local problem once the rows have been exchanged: every row of the sequence, this rank's heads
  krea_cuda_joint_args j{};
  j.batch = 1;
  j.Lq = j.Lk = a->seq;
  j.heads = hl;
  j.group = a->group;
  j.ldq = j.ldo = cl;
  j.ldk = j.ldv = kcl;
  j.wq = a->wq; j.wk = a->wk; j.cos = a->cos; j.sin = a->sin;
  j.eps = a->eps;
  j.rope_mode = a->rope_mode;

  CUDA_TRY(h, cudaSetDevice(h->device));
  const size_t q_bytes = round256((size_t)a->seq * cl * 2), kv_bytes = round256((size_t)a->seq * kcl * 2);
  if (d->p2p) {
    // ---- peer stores: no staging copies, no NCCL transfers ----
    // symmetric layout (same offsets on every rank): Q by heads | K | V | output by rows | normalised K (local use)
    const size_t o_bytes = round256((size_t)rl * a->heads * 128 * 2);
    const size_t need = q_bytes + 2 * kv_bytes + o_bytes + kv_bytes;
    if (d->sym_bytes < need && (rc = sym_alloc(h, need))) return rc;
  }
  if (d->p2p) {
    const size_t o_bytes = round256((size_t)rl * a->heads * 128 * 2);
    const size_t off_q = 0, off_k = q_bytes, off_v = q_bytes + kv_bytes, off_o = q_bytes + 2 * kv_bytes, off_kn = off_o + o_bytes;
    char* w = (char*)d->sym;
    j.Q = w + off_q; j.K = w + off_k; j.V = w + off_v;
    j.ldo = a->heads * 128;                  // the scattered output rows are full rows of all heads
    j.O = w + off_o;                          // (placeholder for validation; the kernel uses the block table)
    if ((rc = krea_validate_joint(h, &j))) return rc;
    // 1. every rank stores its rows of the head blocks straight into their owners' Q / K / V
    const void* srcs[3] = {a->K, a->V, a->Q};
    const int lds[3] = {a->ldk, a->ldv, a->ldq};
    const size_t offs[3] = {off_k, off_v, off_q};
    const int cols[3] = {kcl, kcl, cl};
    for (int t = 0; t < 3; t++) {
      ReshardParams p{};
      p.src = (const __nv_bfloat16*)srcs[t];
      p.dst = (__nv_bfloat16*)(w + offs[t]);
      for (int r = 0; r < 8; r++) p.dst_peer[r] = (__nv_bfloat16*)((char*)d->peer[r < P ? r : P - 1] + offs[t]);
      p.dst_row0 = d->rank * rl;
      p.nranks = P;
      p.rows = rl;
      p.cols_per_rank = cols[t];
      p.src_ld = lds[t];
      ProfileMark pm(h, 2);
      CUDA_TRY(h, launch_reshard_pack(p, h->stream));
      h->launches++;
    }
    // 2. all rows of my heads have landed once every rank has passed this point
    {
      ProfileMark pm(h, 3);
      if ((rc = rank_barrier(h, h->stream))) return rc;
    }
    if ((rc = krea_joint_prepass(h, &j, w + off_kn))) return rc;
    // 3. attention; the epilogue stores each query row into its home rank's output rows, at my heads' columns
    void* o_blk[8];
    for (int r = 0; r < P; r++) o_blk[r] = (char*)d->peer[r] + off_o + (size_t)d->rank * cl * 2;
    if ((rc = krea_joint_attend_scatter(h, &j, w + off_kn, o_blk, P, rl))) return rc;
    // 4. my output rows are complete once every rank's attention kernel has finished
    {
      ProfileMark pm(h, 3);
      if ((rc = rank_barrier(h, h->stream))) return rc;
    }
    ProfileMark pm(h, 2);
    CUDA_TRY(h, cudaMemcpy2DAsync(a->O, (size_t)a->ldo * 2, w + off_o, (size_t)a->heads * 128 * 2, (size_t)a->heads * 128 * 2, rl,
                                  cudaMemcpyDeviceToDevice, h->stream));
    return KREA_CUDA_OK;
  }
  void* base = nullptr;
  // send stage | Q (reused for the returning output blocks) | output by heads | K | V | normalised K
  if ((rc = dist_ws(h, 3 * q_bytes + 3 * kv_bytes, &base))) return rc;
  char* w = (char*)base;
  void* stage = w;
  void* qh = w + q_bytes;
  void* oh = w + 2 * q_bytes;
  void* kh = w + 3 * q_bytes;
  void* vh = w + 3 * q_bytes + kv_bytes;
  void* kn = w + 3 * q_bytes + 2 * kv_bytes;
  j.Q = qh; j.K = kh; j.V = vh; j.O = oh;
  if ((rc = krea_validate_joint(h, &j))) return rc;

  // The exchanges run on the side stream, K first; the main stream normalises K while V and Q travel.
  CUDA_TRY(h, cudaEventRecord(d->ev[0], h->stream));
  CUDA_TRY(h, cudaStreamWaitEvent(d->side, d->ev[0], 0));
  if ((rc = seq_to_heads_on(h, a->K, kh, stage, rl, kcl, a->ldk, 0, d->side))) return rc;
  CUDA_TRY(h, cudaEventRecord(d->ev[1], d->side));
  if ((rc = seq_to_heads_on(h, a->V, vh, stage, rl, kcl, a->ldv, 0, d->side))) return rc;
  if ((rc = seq_to_heads_on(h, a->Q, qh, stage, rl, cl, a->ldq, 0, d->side))) return rc;
  CUDA_TRY(h, cudaEventRecord(d->ev[2], d->side));
  CUDA_TRY(h, cudaStreamWaitEvent(h->stream, d->ev[1], 0));
  if ((rc = krea_joint_prepass(h, &j, kn))) return rc;
  CUDA_TRY(h, cudaStreamWaitEvent(h->stream, d->ev[2], 0));
  if ((rc = krea_joint_attend(h, &j, kn))) return rc;
  // the output goes home on the main stream; its blocks are received over the (now dead) Q rows
  ProfileMark pm(h, 2);
  return heads_to_seq_on(h, oh, a->O, qh, rl, cl, a->ldo, 0, h->stream);
}

}  // extern "C"
