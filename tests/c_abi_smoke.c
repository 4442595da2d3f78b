/* Plain-C consumer of include/krea_cuda.h: the header must compile as C11 and the library must link and answer
 * from C, the way the reference's own C ABI (engine/src/krea.h) is consumed.  Needs no GPU: without one,
 * krea_cuda_create must fail with a message, and the host-side entry points must still work. */
#include <math.h>
#include <stdio.h>
#include <string.h>

#include "krea_cuda.h"

int main(int argc, char** argv) {
  char err[256] = "";
  krea_cuda* h = krea_cuda_create(0, err, (int)sizeof err);
  if (h == NULL) {
    if (err[0] == '\0') { printf("FAIL: no message from krea_cuda_create\n"); return 1; }
    printf("create: %s\n", err);
  }
  float c[6 * 64], s[6 * 64];
  if (krea_cuda_rope_tables_axial2d(c, s, 2, 2, 2, 10000.0) != KREA_CUDA_OK) { printf("FAIL: rope tables\n"); return 1; }
  /* text rows sit at position 0; image token 3 = (row 1, col 1): pair 0 turns by 1 rad, pair 32 too */
  if (c[0] != 1.0f || s[0] != 0.0f || fabsf(c[5 * 64] - cosf(1.0f)) > 1e-6f || fabsf(s[5 * 64 + 32] - sinf(1.0f)) > 1e-6f) { printf("FAIL: table values\n"); return 1; }
  krea_cuda_joint_args j;
  memset(&j, 0, sizeof j);
  j.Lk = 4608; j.heads = 24; j.group = 1; j.batch = 1;
  if (krea_cuda_joint_scratch_bytes(&j) != (size_t)4608 * 24 * 256) { printf("FAIL: scratch bytes\n"); return 1; }
  if (krea_cuda_attention(NULL, NULL) != KREA_CUDA_E_ARG || krea_cuda_gemm(NULL, NULL) != KREA_CUDA_E_ARG) { printf("FAIL: null handle\n"); return 1; }
  float qn[128], kn[128];
  for (int d = 0; d < 128; d++) { qn[d] = 1.0f; kn[d] = 1.0f; }
  qn[9] = 52.8f; kn[9] = 52.8f;
  if (krea_cuda_qw_big_dim(qn, kn, 256.0f) != 9) { printf("FAIL: big dim\n"); return 1; }
  if (argc > 1) {
    krea_qw* q = krea_cuda_qw_open(argv[1], err, (int)sizeof err);
    if (q == NULL) { printf("FAIL: qw_open: %s\n", err); return 1; }
    krea_cuda_qw_info info;
    if (krea_cuda_qw_find(q, "L0.qn", &info) != KREA_CUDA_OK || info.rank != 1 || info.shape[0] != 128 || strcmp(info.dtype, "f32") != 0) { printf("FAIL: qw_find\n"); return 1; }
    const float* p = (const float*)krea_cuda_qw_host_ptr(q, info.offset);
    printf("L0.qn[0] = %.6f, %d tensors\n", p[0], krea_cuda_qw_count(q));
    krea_cuda_qw_close(q);
  }
  if (h) krea_cuda_destroy(h);
  printf("OK\n");
  return 0;
}
