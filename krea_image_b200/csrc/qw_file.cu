// Reader for the engine's `.qw` weight files (written by the reference's tools/convert.py:49-89, read by
// engine/src/weights.mm:16-81): the data format that supplies the QK-norm weights `L<l>.qn` / `L<l>.kn` of
// the attention path.  Layout: "QWTS", u32 version, u64 header length, a JSON header
//   {"tensors": {name: {"dtype", "shape", "offset", "nbytes"}}, "meta": {...}}
// and a data section starting at the next multiple of 16 KiB, tensor offsets relative to it and 16 KiB
// aligned.
//
// The reference wraps page ranges of the mapping in no-copy GPU buffers (unified memory).  A B200 has its
// own 180 GB: here the file is mapped read-only for the host-side queries, and byte ranges are uploaded
// to device memory through two pinned bounce buffers, so the copy engine always has a transfer in flight
// while the host fills the other buffer from the page cache.
#include <errno.h>
#include <fcntl.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <string>
#include <vector>

#include "handle.h"

namespace {

struct QwTensor {
  std::string name, dtype;
  std::vector<int64_t> shape;
  uint64_t offset = 0, nbytes = 0;
};

// Minimal JSON reader for the header: enough of the grammar for what the converter writes (objects,
// arrays, strings with escapes, numbers, true / false / null).
struct Json {
  const char* p;
  const char* end;
  std::string err;
  int depth = 0;            // nesting of the value being skipped: a header is a few levels deep, never hundreds

  void ws() {
    while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) p++;
  }
  bool lit(char c) {
    ws();
    if (p < end && *p == c) {
      p++;
      return true;
    }
    return false;
  }
  bool fail(const char* m) {
    if (err.empty()) err = m;
    return false;
  }
  bool string(std::string* out) {
    ws();
    if (p >= end || *p != '"') return fail("expected a string");
    p++;
    while (p < end && *p != '"') {
      if (*p == '\\') {
        if (++p >= end) return fail("unterminated escape");
        char c = *p;
        if (c == 'u') {   // \uXXXX: tensor names are ASCII; keep the low byte
          if (end - p < 5) return fail("short \\u escape");
          c = (char)strtol(std::string(p + 1, 4).c_str(), nullptr, 16);
          p += 4;
        } else if (c == 'n') c = '\n';
        else if (c == 't') c = '\t';
        else if (c == 'r') c = '\r';
        else if (c == 'b') c = '\b';
        else if (c == 'f') c = '\f';
        if (out) out->push_back(c);
        p++;
      } else {
        if (out) out->push_back(*p);
        p++;
      }
    }
    if (p >= end) return fail("unterminated string");
    p++;
    return true;
  }
  bool number(double* out) {
    ws();
    char* e = nullptr;
    const double v = strtod(p, &e);
    if (e == p || e > end) return fail("expected a number");
    p = e;
    if (out) *out = v;
    return true;
  }
  // a size, offset or dimension: a whole number that a double holds exactly (strtod also accepts "inf", "nan"
  // and values far beyond any file, and converting those to an integer is undefined)
  bool count(uint64_t* out) {
    double v = 0;
    if (!number(&v)) return false;
    if (!(v >= 0.0 && v <= 9007199254740992.0) || v != floor(v)) return fail("expected a non-negative whole number");
    *out = (uint64_t)v;
    return true;
  }
  // skips any value; used for members this reader does not interpret
  bool skip() {
    ws();
    if (p >= end) return fail("unexpected end of header");
    if (*p == '"') return string(nullptr);
    if (*p == '{' || *p == '[') {
      const char close = *p == '{' ? '}' : ']';
      const bool obj = *p == '{';
      p++;
      if (lit(close)) return true;
      if (++depth > 64) return fail("header nested too deeply");
      do {
        if (obj && (!string(nullptr) || !lit(':'))) return fail("bad object member");
        if (!skip()) return false;
      } while (lit(','));
      depth--;
      return lit(close) ? true : fail("unterminated container");
    }
    if (!strncmp(p, "true", 4)) { p += 4; return true; }
    if (!strncmp(p, "false", 5)) { p += 5; return true; }
    if (!strncmp(p, "null", 4)) { p += 4; return true; }
    return number(nullptr);
  }
};

bool parse_tensor(Json& j, QwTensor* t) {
  if (!j.lit('{')) return j.fail("tensor entry is not an object");
  if (j.lit('}')) return true;
  do {
    std::string key;
    if (!j.string(&key) || !j.lit(':')) return j.fail("bad tensor member");
    uint64_t v = 0;
    if (key == "dtype") {
      if (!j.string(&t->dtype)) return false;
    } else if (key == "shape") {
      if (!j.lit('[')) return j.fail("shape is not an array");
      if (!j.lit(']')) {
        do {
          if (!j.count(&v)) return false;
          t->shape.push_back((int64_t)v);
        } while (j.lit(','));
        if (!j.lit(']')) return j.fail("unterminated shape");
      }
    } else if (key == "offset") {
      if (!j.count(&v)) return false;
      t->offset = v;
    } else if (key == "nbytes") {
      if (!j.count(&v)) return false;
      t->nbytes = v;
    } else if (!j.skip()) {
      return false;
    }
  } while (j.lit(','));
  return j.lit('}') ? true : j.fail("unterminated tensor entry");
}

size_t dtype_size(const std::string& d) {
  if (d == "bf16" || d == "f16") return 2;
  if (d == "f32") return 4;
  if (d == "i8") return 1;
  return 0;
}

}  // namespace

struct krea_qw {
  std::string path, meta;
  void* base = MAP_FAILED;
  size_t size = 0, data_start = 0;
  std::vector<QwTensor> tensors;   // sorted by name
  const QwTensor* find(const char* name) const {
    auto it = std::lower_bound(tensors.begin(), tensors.end(), name, [](const QwTensor& t, const char* n) { return t.name < n; });
    return (it != tensors.end() && it->name == name) ? &*it : nullptr;
  }
};

static void fill_info(const QwTensor& t, krea_cuda_qw_info* out) {
  memset(out, 0, sizeof(*out));
  out->name = t.name.c_str();
  out->dtype = t.dtype.c_str();
  out->rank = (int)std::min<size_t>(t.shape.size(), 8);
  for (int i = 0; i < out->rank; i++) out->shape[i] = t.shape[i];
  out->offset = t.offset;
  out->nbytes = t.nbytes;
}

extern "C" {

krea_qw* krea_cuda_qw_open(const char* path, char* err, int errlen) {
  auto say = [&](const std::string& m) -> krea_qw* {
    if (err && errlen > 0) snprintf(err, (size_t)errlen, "%s", m.c_str());
    return nullptr;
  };
  if (!path) return say("qw_open: null path");
  const int fd = open(path, O_RDONLY);
  if (fd < 0) return say(std::string("cannot open weights: ") + path + ": " + strerror(errno));
  struct stat st;
  if (fstat(fd, &st) != 0 || st.st_size < 16) {
    close(fd);
    return say(std::string("weight file too short: ") + path);
  }
  krea_qw* q = new krea_qw();
  q->path = path;
  q->size = (size_t)st.st_size;
  q->base = mmap(nullptr, q->size, PROT_READ, MAP_PRIVATE, fd, 0);
  close(fd);
  auto bail = [&](const std::string& m) {
    krea_cuda_qw_close(q);
    return say(m);
  };
  if (q->base == MAP_FAILED) return bail(std::string("mmap failed: ") + path);
  const char* p = (const char*)q->base;
  if (memcmp(p, "QWTS", 4) != 0) return bail(std::string("bad weight file magic: ") + path);   // weights.mm:29
  uint64_t hlen = 0;
  memcpy(&hlen, p + 8, 8);
  if (hlen > q->size - 16) return bail(std::string("bad weight header length: ") + path);
  q->data_start = (size_t)((16 + hlen + 16383) / 16384 * 16384);                              // weights.mm:36
  const std::string header(p + 16, (size_t)hlen);   // NUL-terminated copy: the number parser may look one byte ahead
  Json j{header.data(), header.data() + header.size(), {}};
  bool ok = j.lit('{');
  if (ok && !j.lit('}')) {
    do {
      std::string key;
      if (!(ok = j.string(&key) && j.lit(':'))) break;
      if (key == "tensors") {
        if (!(ok = j.lit('{'))) break;
        if (!j.lit('}')) {
          do {
            QwTensor t;
            if (!(ok = j.string(&t.name) && j.lit(':') && parse_tensor(j, &t))) break;
            q->tensors.push_back(std::move(t));
          } while (j.lit(','));
          if (ok) ok = j.lit('}');
        }
      } else if (key == "meta") {
        j.ws();
        const char* m0 = j.p;
        if (!(ok = j.skip())) break;
        q->meta.assign(m0, j.p);
      } else {
        ok = j.skip();
      }
      if (!ok) break;
    } while (j.lit(','));
    if (ok) ok = j.lit('}');
  }
  if (!ok) return bail(std::string("bad weight header: ") + path + (j.err.empty() ? "" : " (" + j.err + ")"));
  std::sort(q->tensors.begin(), q->tensors.end(), [](const QwTensor& a, const QwTensor& b) { return a.name < b.name; });
  for (size_t i = 0; i < q->tensors.size(); i++) {
    const QwTensor& t = q->tensors[i];
    if (i > 0 && q->tensors[i - 1].name == t.name) return bail("duplicate tensor " + t.name + " in " + path);
    if (q->data_start > q->size || t.offset > q->size - q->data_start || t.nbytes > q->size - q->data_start - t.offset)
      return bail("tensor " + t.name + " lies outside " + path);
    uint64_t n = dtype_size(t.dtype);
    if (n == 0) return bail("tensor " + t.name + ": unknown dtype " + t.dtype);
    for (int64_t d : t.shape) {
      if (d != 0 && n > UINT64_MAX / (uint64_t)d) return bail("tensor " + t.name + ": shape overflows");
      n *= (uint64_t)d;
    }
    if (n != t.nbytes) return bail("tensor " + t.name + ": shape and nbytes disagree");
  }
  return q;
}

void krea_cuda_qw_close(krea_qw* q) {
  if (!q) return;
  if (q->base != MAP_FAILED) munmap(q->base, q->size);
  delete q;
}

int krea_cuda_qw_count(const krea_qw* q) { return q ? (int)q->tensors.size() : 0; }

int krea_cuda_qw_info_at(const krea_qw* q, int index, krea_cuda_qw_info* out) {
  if (!q || !out || index < 0 || index >= (int)q->tensors.size()) return KREA_CUDA_E_ARG;
  fill_info(q->tensors[index], out);
  return KREA_CUDA_OK;
}

int krea_cuda_qw_find(const krea_qw* q, const char* name, krea_cuda_qw_info* out) {
  if (!q || !name) return KREA_CUDA_E_ARG;
  const QwTensor* t = q->find(name);
  if (!t) return KREA_CUDA_E_ARG;
  if (out) fill_info(*t, out);
  return KREA_CUDA_OK;
}

const void* krea_cuda_qw_host_ptr(const krea_qw* q, uint64_t offset) {
  if (!q || q->data_start > q->size || offset > q->size - q->data_start) return nullptr;
  return (const char*)q->base + q->data_start + offset;
}

const char* krea_cuda_qw_meta(const krea_qw* q) { return q ? q->meta.c_str() : ""; }

uint64_t krea_cuda_qw_data_bytes(const krea_qw* q) { return (q && q->size >= q->data_start) ? q->size - q->data_start : 0; }

int krea_cuda_qw_span(const krea_qw* q, const char* prefix, uint64_t* off, uint64_t* len) {
  if (!q || !prefix || !off || !len) return KREA_CUDA_E_ARG;
  const size_t n = strlen(prefix);
  uint64_t lo = UINT64_MAX, hi = 0;
  for (const QwTensor& t : q->tensors)
    if (t.name.compare(0, n, prefix) == 0) {
      lo = std::min(lo, t.offset);
      hi = std::max(hi, t.offset + t.nbytes);
    }
  if (hi == 0 && lo == UINT64_MAX) return KREA_CUDA_E_ARG;   // weights.mm span(): no tensor has that prefix
  *off = lo;
  *len = hi - lo;
  return KREA_CUDA_OK;
}

int krea_cuda_qw_upload(krea_cuda* h, const krea_qw* q, uint64_t off, uint64_t len, void* dst_device) {
  if (!h || !q) return fail(h, KREA_CUDA_E_ARG, "qw_upload: null handle or file");
  const uint64_t data = krea_cuda_qw_data_bytes(q);
  if (off > data || len > data - off) return fail(h, KREA_CUDA_E_ARG, "qw_upload: byte range outside the data section of %s", q->path.c_str());
  if (len == 0) return KREA_CUDA_OK;
  if (!dst_device) return fail(h, KREA_CUDA_E_ARG, "qw_upload: null destination");
  CUDA_TRY(h, cudaSetDevice(h->device));
  // two pinned halves: while one travels, the host copies the next chunk out of the page cache
  const size_t chunk = 8u << 20;
  if (!h->qw_stage) {
    if (cudaMallocHost(&h->qw_stage, 2 * chunk) != cudaSuccess) {
      cudaGetLastError();
      h->qw_stage = nullptr;
      return fail(h, KREA_CUDA_E_NOMEM, "qw_upload: cannot allocate pinned staging memory");
    }
  }
  cudaEvent_t done[2] = {nullptr, nullptr};
  cudaError_t e = cudaSuccess;
  for (int i = 0; i < 2 && e == cudaSuccess; i++) e = cudaEventCreateWithFlags(&done[i], cudaEventDisableTiming);
  const char* src = (const char*)krea_cuda_qw_host_ptr(q, off);
  int rc = KREA_CUDA_OK;
  // (every upload ends with a stream synchronisation, so both halves are free here)
  if (e == cudaSuccess) e = cudaStreamSynchronize(h->stream);
  int k = 0;
  for (uint64_t o = 0; o < len && e == cudaSuccess; o += chunk, k ^= 1) {
    const size_t n = (size_t)std::min<uint64_t>(chunk, len - o);
    char* half = (char*)h->qw_stage + (size_t)k * chunk;
    if (o >= 2 * chunk) e = cudaEventSynchronize(done[k]);   // the copy that last used this half
    if (e != cudaSuccess) break;
    memcpy(half, src + o, n);
    e = cudaMemcpyAsync((char*)dst_device + o, half, n, cudaMemcpyHostToDevice, h->stream);
    if (e == cudaSuccess) e = cudaEventRecord(done[k], h->stream);
  }
  if (e == cudaSuccess) e = cudaStreamSynchronize(h->stream);   // the halves are free again on return
  if (e != cudaSuccess) rc = fail(h, KREA_CUDA_E_CUDA, "qw_upload: %s", cudaGetErrorString(e));
  for (int i = 0; i < 2; i++)
    if (done[i]) cudaEventDestroy(done[i]);
  return rc;
}

int krea_cuda_qw_big_dim(const float* qn, const float* kn, float gain_threshold) {
  // the head dimension whose |qn[d] * kn[d]| is largest among those above the threshold (model.mm:229-238)
  if (!qn || !kn) return -1;
  int best_d = -1;
  float best = 0.f;
  for (int d = 0; d < 128; d++) {
    const float g = fabsf(qn[d] * kn[d]);
    if (g > gain_threshold && g > best) {
      best = g;
      best_d = d;
    }
  }
  return best_d;
}

}  // extern "C"
