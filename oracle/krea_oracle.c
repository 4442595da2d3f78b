/*
 * CPU oracle for the Krea 2 Turbo DiT joint text+image attention path.
 *
 * THIS IS TEST INFRASTRUCTURE, NOT PRODUCT CODE.  Only the test-suite, the smoke check and the
 * CPU-baseline leg of the benchmark may load it; the CUDA library never calls into it.
 *
 * It restates, in plain C (fp32 arithmetic, OpenMP over independent rows), the math of the reference's
 * Metal kernels and their host glue:
 *   engine/kernels/norm.metal:81-134      qk_norm_rope  (per-head RMSNorm x f32 weight, RoPE, bf16 store)
 *   engine/kernels/attention.metal:131-333 attn_body    (scores, masks, softmax, bf16 P, PV, gate, store)
 *   engine/src/metal.mm:193-202           softmax scale 1/sqrt(128)
 *   engine/src/model.mm:290-315           DiT::set_grid (per-row cos/sin tables)
 *   engine/src/model.mm:17-24             bf16_round (round-to-nearest-even)
 *   engine/src/pipeline.mm:108-122        gaussian_noise (splitmix64 counter stream + Box-Muller)
 *
 * PARITY UNPINNED: the reference ships no test, golden vector or CPU implementation for this path
 * (its harness and fp32 PyTorch model live in a directory that is not part of the repository), and its
 * Metal sources cannot be compiled off macOS.  This file is therefore checked against (a) closed-form
 * cases, (b) an independent float64 numpy statement of the same formulas and (c) committed checksums of
 * its own outputs, not against outputs of the reference itself.
 *
 * Two rounding modes (argument `ref_rounding`):
 *   0  "fp32":  bf16 inputs are widened to fp32 and nothing is rounded afterwards (the contract the
 *               GPU result is held to: relative-L2 <= 5e-3 and max-abs <= 2e-2);
 *   1  "ref":   additionally applies the three roundings the reference kernels perform: normalised and
 *               rotated Q/K to bf16 (norm.metal:133), P to bf16 inside the PV product but not in the
 *               row sum (attention.metal:270-273), and the output to bf16 (attention.metal:330).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define KO_D 128

/* ---- bf16 helpers (model.mm:17-24: round to nearest even on the upper 16 bits) ---- */
static inline float bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
static inline uint16_t f32_to_bf16(float x) {
  uint32_t u;
  memcpy(&u, &x, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40); /* NaN stays NaN */
  u = u + 0x7FFFu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}
static inline float bf16_round(float x) { return bf16_to_f32(f32_to_bf16(x)); }

/* Launchers that start several ranks per node export OMP_NUM_THREADS=1; the benchmark's reference arm runs on one
 * rank and wants every host thread, so it can say so. */
void ko_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

int ko_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

void ko_f32_to_bf16(const float* in, uint16_t* out, int64_t n) {
  for (int64_t i = 0; i < n; i++) out[i] = f32_to_bf16(in[i]);
}
void ko_bf16_to_f32(const uint16_t* in, float* out, int64_t n) {
  for (int64_t i = 0; i < n; i++) out[i] = bf16_to_f32(in[i]);
}

/* ---- seeded generators (pipeline.mm:108-122), made counter-based so any slice can be produced ---- */
static inline uint64_t mix64(uint64_t z) {
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ULL;
  z = (z ^ (z >> 27)) * 0x94d049bb133111ebULL;
  return z ^ (z >> 31);
}
/* Element e of the stream `seed`: elements (2i, 2i+1) are the cos / sin branch of one Box-Muller pair
 * driven by counters 2i and 2i+1, exactly like the reference's loop. */
static inline float normal_at(uint64_t seed, uint64_t e) {
  const uint64_t i = e & ~1ULL;
  const uint64_t a = mix64(seed * 0x9E3779B97F4A7C15ULL + i), b = mix64(seed * 0x9E3779B97F4A7C15ULL + i + 1);
  const double u1 = ((double)(a >> 11) + 1.0) / 9007199254740993.0, u2 = (double)(b >> 11) / 9007199254740992.0;
  const double r = sqrt(-2.0 * log(u1));
  const double t = 2.0 * M_PI * u2;
  return (float)((e & 1) ? r * sin(t) : r * cos(t));
}
void ko_gen_normal_f32(uint64_t seed, uint64_t first, float* out, int64_t n) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; i++) out[i] = normal_at(seed, first + (uint64_t)i);
}
void ko_gen_normal_bf16(uint64_t seed, uint64_t first, uint16_t* out, int64_t n) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; i++) out[i] = f32_to_bf16(normal_at(seed, first + (uint64_t)i));
}
/* lo + (hi - lo) * U[0,1) from the same mixer. */
void ko_gen_uniform_f32(uint64_t seed, uint64_t first, float lo, float hi, float* out, int64_t n) {
  for (int64_t i = 0; i < n; i++) {
    const uint64_t a = mix64(seed * 0x9E3779B97F4A7C15ULL + first + (uint64_t)i);
    out[i] = (float)(lo + (double)(hi - lo) * ((double)(a >> 11) / 9007199254740992.0));
  }
}

/* ---- RoPE tables (model.mm:290-315): f32 cos/sin [T + gh*gw, 64]; text rows at position 0 ---- */
/* The reference's own 3-axis scheme: pairs 0-15 frame (always 0), 16-39 row, 40-63 column, theta 1000. */
void ko_rope_tables_ref3axis(float* c, float* s, int T, int gh, int gw) {
  double om[64];
  for (int p = 0; p < 64; p++) {
    const int ax = p < 16 ? 0 : p < 40 ? 1 : 2, k = p - (ax == 0 ? 0 : ax == 1 ? 16 : 40), d = ax == 0 ? 32 : 48;
    om[p] = 1.0 / pow(1000.0, (2.0 * k) / d);
  }
  const int R = T + gh * gw;
  for (int r = 0; r < R; r++) {
    const int k = r - T;
    const double pi = r < T ? 0 : k / gw, pj = r < T ? 0 : k % gw;
    for (int p = 0; p < 64; p++) {
      const double a = (p < 16 ? 0.0 : p < 40 ? pi : pj) * om[p];
      c[(size_t)r * 64 + p] = (float)cos(a);
      s[(size_t)r * 64 + p] = (float)sin(a);
    }
  }
}
/* The benchmark's 2-D axial scheme, same table mechanism: pairs 0-31 rotate by the grid row, 32-63 by
 * the grid column, frequency k of an axis = theta^(-2k/64). */
void ko_rope_tables_axial2d(float* c, float* s, int T, int gh, int gw, double theta) {
  double om[32];
  for (int k = 0; k < 32; k++) om[k] = 1.0 / pow(theta, (2.0 * k) / 64.0);
  const int R = T + gh * gw;
  for (int r = 0; r < R; r++) {
    const int k = r - T;
    const double pi = r < T ? 0 : k / gw, pj = r < T ? 0 : k % gw;
    for (int p = 0; p < 64; p++) {
      const double a = (p < 32 ? pi : pj) * om[p & 31];
      c[(size_t)r * 64 + p] = (float)cos(a);
      s[(size_t)r * 64 + p] = (float)sin(a);
    }
  }
}

/* ---- prologue on one head vector (norm.metal:98-126) ---- */
/* x[128] in place.  rope_mode 0: interleaved pairs; 1: rotate-half; 2: none.  cr/sr: this row's 64 entries. */
static void norm_rope_head(float* x, const float* w, const float* cr, const float* sr, float eps, int rope_mode) {
  float ss = 0.f;
  for (int d = 0; d < KO_D; d++) ss += x[d] * x[d];
  const float rrms = 1.0f / sqrtf(ss * (1.0f / KO_D) + eps);
  float y[KO_D];
  for (int d = 0; d < KO_D; d++) y[d] = x[d] * rrms * w[d];
  if (rope_mode == 0) {
    for (int i = 0; i < 64; i++) {
      x[2 * i] = y[2 * i] * cr[i] - y[2 * i + 1] * sr[i];
      x[2 * i + 1] = y[2 * i] * sr[i] + y[2 * i + 1] * cr[i];
    }
  } else if (rope_mode == 1) {
    for (int i = 0; i < 64; i++) {
      x[i] = y[i] * cr[i] - y[i + 64] * sr[i];
      x[i + 64] = y[i + 64] * cr[i] + y[i] * sr[i];
    }
  } else {
    for (int d = 0; d < KO_D; d++) x[d] = y[d];
  }
}

/* The operator Metal::qk_norm_rope (metal.h:80-82, metal.mm:182-191): in place on bf16 rows [rows, ld];
 * q heads at column q_off + h*128, k heads at k_off + h*128.  big_dim >= 0: that channel's value goes
 * to qbig [rows, n_q] / kbig [rows, n_k] in fp32 and is stored as zero (norm.metal:127-132). */
void ko_qk_norm_rope(uint16_t* qkv, const float* wq, const float* wk, const float* cosb, const float* sinb, int rows,
                     int ld, int q_off, int n_q, int k_off, int n_k, float eps, int rope_mode, int big_dim,
                     float* qbig, float* kbig) {
#pragma omp parallel for schedule(static)
  for (int row = 0; row < rows; row++) {
    for (int hh = 0; hh < n_q + n_k; hh++) {
      const int is_q = hh < n_q;
      const int col = is_q ? q_off + hh * KO_D : k_off + (hh - n_q) * KO_D;
      uint16_t* p = qkv + (size_t)row * ld + col;
      float x[KO_D];
      for (int d = 0; d < KO_D; d++) x[d] = bf16_to_f32(p[d]);
      norm_rope_head(x, is_q ? wq : wk, cosb ? cosb + (size_t)row * 64 : NULL, sinb ? sinb + (size_t)row * 64 : NULL,
                     eps, rope_mode);
      if (big_dim >= 0) {
        if (is_q) qbig[(size_t)row * n_q + hh] = x[big_dim];
        else kbig[(size_t)row * n_k + (hh - n_q)] = x[big_dim];
        x[big_dim] = 0.f;
      }
      for (int d = 0; d < KO_D; d++) p[d] = f32_to_bf16(x[d]);
    }
  }
}

/* ---- attention core on fp32 head-contiguous operands ---- */
/* q [Lq,128], kt [128,Lk] (transposed keys), v [Lk,128]; valid[k] != 0 marks usable keys (NULL = all);
 * causal: key k visible to row i iff k <= i + q_pos0 (attention.metal:237-249); qb/kb: optional fp32
 * rank-1 score term qb[i]*kb[k] (attention.metal:232-234).  out [Lq,128] fp32, row stride ldo. */
static void attend_head(const float* q, const float* kt, const float* v, const uint8_t* valid, int Lq, int Lk,
                        int causal, int q_pos0, const float* qb, const float* kb, int ref_rounding, float* out,
                        size_t ldo) {
  const float scale = (float)(1.0 / sqrt(128.0));
#pragma omp parallel
  {
    float* s = (float*)malloc(sizeof(float) * (size_t)Lk * 4);
#pragma omp for schedule(dynamic, 4)
    for (int i0 = 0; i0 < Lq; i0 += 4) {
      const int nr = Lq - i0 < 4 ? Lq - i0 : 4;
      for (int r = 0; r < nr; r++) memset(s + (size_t)r * Lk, 0, sizeof(float) * (size_t)Lk);
      for (int k0 = 0; k0 < Lk; k0 += 1024) { /* key chunks keep the working set in cache */
        const int kn = Lk - k0 < 1024 ? Lk - k0 : 1024;
        for (int d = 0; d < KO_D; d++) {
          const float* kr = kt + (size_t)d * Lk + k0;
          for (int r = 0; r < nr; r++) {
            const float qd = q[(size_t)(i0 + r) * KO_D + d];
            float* sr = s + (size_t)r * Lk + k0;
            for (int k = 0; k < kn; k++) sr[k] += qd * kr[k];
          }
        }
      }
      for (int r = 0; r < nr; r++) {
        const int i = i0 + r;
        float* sr = s + (size_t)r * Lk;
        float m = -INFINITY;
        for (int k = 0; k < Lk; k++) {
          float x = sr[k];
          if (qb) x += qb[i] * kb[k];
          x *= scale;
          const int ok = (!valid || valid[k]) && (!causal || k <= i + q_pos0);
          x = ok ? x : -INFINITY;
          sr[k] = x;
          m = x > m ? x : m;
        }
        float acc[KO_D];
        for (int d = 0; d < KO_D; d++) acc[d] = 0.f;
        float l = 0.f;
        if (m > -INFINITY) {
          for (int k = 0; k < Lk; k++) {
            if (sr[k] == -INFINITY) continue;
            const float p = expf(sr[k] - m);
            l += p;
            const float pv = ref_rounding ? bf16_round(p) : p;
            const float* vr = v + (size_t)k * KO_D;
            for (int d = 0; d < KO_D; d++) acc[d] += pv * vr[d];
          }
        }
        const float inv = l > 0.f ? 1.f / l : 0.f; /* a row with no visible key gives zeros (attention.metal:316) */
        for (int d = 0; d < KO_D; d++) out[(size_t)i * ldo + d] = acc[d] * inv;
      }
    }
    free(s);
  }
}

/* The operator Metal::attention (metal.h:83-88, metal.mm:193-202) on already-normalised bf16 operands.
 * Q [Lq, ldq] head h at column h*128; K/V [Lk, ldk/ldv] head h/group; G optional gate (bf16, stride ldg),
 * QB [Lq, heads] / KB [Lk, heads/group] optional fp32 rank-1 term.  Output: fp32 [Lq, heads*128]
 * (values are bf16-representable when ref_rounding). */
void ko_attention(const uint16_t* Q, const uint16_t* K, const uint16_t* V, float* O, int Lq, int Lk, int heads,
                  int ldq, int ldk, int ldv, int group, int causal, int q_pos0, const uint16_t* G, int ldg,
                  const float* QB, const float* KB, int ref_rounding) {
  const int kvheads = heads / group;
  float* q = (float*)malloc(sizeof(float) * (size_t)Lq * KO_D);
  float* kt = (float*)malloc(sizeof(float) * (size_t)Lk * KO_D);
  float* v = (float*)malloc(sizeof(float) * (size_t)Lk * KO_D);
  float* qb = QB ? (float*)malloc(sizeof(float) * (size_t)Lq) : NULL;
  float* kb = KB ? (float*)malloc(sizeof(float) * (size_t)Lk) : NULL;
  for (int h = 0; h < heads; h++) {
    const int kvh = h / group;
    for (int i = 0; i < Lq; i++)
      for (int d = 0; d < KO_D; d++) q[(size_t)i * KO_D + d] = bf16_to_f32(Q[(size_t)i * ldq + h * KO_D + d]);
    for (int k = 0; k < Lk; k++)
      for (int d = 0; d < KO_D; d++) {
        kt[(size_t)d * Lk + k] = bf16_to_f32(K[(size_t)k * ldk + kvh * KO_D + d]);
        v[(size_t)k * KO_D + d] = bf16_to_f32(V[(size_t)k * ldv + kvh * KO_D + d]);
      }
    if (QB) {
      for (int i = 0; i < Lq; i++) qb[i] = QB[(size_t)i * heads + h];
      for (int k = 0; k < Lk; k++) kb[k] = KB[(size_t)k * kvheads + kvh];
    }
    attend_head(q, kt, v, NULL, Lq, Lk, causal, q_pos0, qb, kb, ref_rounding, O + (size_t)h * KO_D,
                (size_t)heads * KO_D);
  }
  const size_t ldo = (size_t)heads * KO_D;
  if (G && ldg > 0) {
    for (int i = 0; i < Lq; i++)
      for (int c = 0; c < heads * KO_D; c++) {
        const float g = bf16_to_f32(G[(size_t)i * ldg + c]);
        O[i * ldo + c] *= 1.0f / (1.0f + expf(-g)); /* common.h:24 sigmoid, attention.metal:321-329 */
      }
  }
  if (ref_rounding)
    for (size_t i = 0; i < (size_t)Lq * ldo; i++) O[i] = bf16_round(O[i]);
  free(q); free(kt); free(v); free(qb); free(kb);
}

/* The whole path on raw projections: prologue + attention, with the batch and text key-padding
 * extensions the benchmark configs use.
 *   Q, K, V   bf16, sample b row s head h at  X + b*bs + s*ld + h*128   (bs, ld in elements)
 *   wq, wk    f32 [128], shared by all heads (tools/convert.py:212-213)
 *   cosb,sinb f32 [S, 64]
 *   text_len  NULL, or per-sample count of valid text rows out of `text_slots`: rows/keys in
 *             [text_len[b], text_slots) are padding.  Padded keys contribute nothing, padded query rows
 *             give zeros - identical to running the reference on the rows it would have kept, because
 *             the reference drops padding before the engine (ui/krea.py:3-6) and text sits at RoPE
 *             position 0.
 *   heads_sel NULL = all heads, else a list of n_sel head indices to evaluate (others left untouched)
 *   O         fp32 [B, S, heads*128]
 */
void ko_joint_attention(const uint16_t* Q, const uint16_t* K, const uint16_t* V, float* O, int B, int S, int heads,
                        int group, int64_t ld_q, int64_t ld_k, int64_t ld_v, int64_t bs_q, int64_t bs_k, int64_t bs_v,
                        const float* wq, const float* wk, const float* cosb, const float* sinb, float eps,
                        int rope_mode, const int32_t* text_len, int text_slots, const int32_t* heads_sel, int n_sel,
                        int ref_rounding) {
  float* q = (float*)malloc(sizeof(float) * (size_t)S * KO_D);
  float* kt = (float*)malloc(sizeof(float) * (size_t)S * KO_D);
  float* v = (float*)malloc(sizeof(float) * (size_t)S * KO_D);
  uint8_t* valid = (uint8_t*)malloc((size_t)S);
  const size_t ldo = (size_t)heads * KO_D;
  const int nh = heads_sel ? n_sel : heads;
  for (int b = 0; b < B; b++) {
    const int tl = text_len ? text_len[b] : text_slots;
    for (int s = 0; s < S; s++) valid[s] = !(text_len && s >= tl && s < text_slots);
    for (int hi = 0; hi < nh; hi++) {
      const int h = heads_sel ? heads_sel[hi] : hi;
      const int kvh = h / group;
#pragma omp parallel for schedule(static)
      for (int s = 0; s < S; s++) {
        float x[KO_D], y[KO_D];
        for (int d = 0; d < KO_D; d++) {
          x[d] = bf16_to_f32(Q[(size_t)b * bs_q + (size_t)s * ld_q + h * KO_D + d]);
          y[d] = bf16_to_f32(K[(size_t)b * bs_k + (size_t)s * ld_k + kvh * KO_D + d]);
          v[(size_t)s * KO_D + d] = bf16_to_f32(V[(size_t)b * bs_v + (size_t)s * ld_v + kvh * KO_D + d]);
        }
        norm_rope_head(x, wq, cosb + (size_t)s * 64, sinb + (size_t)s * 64, eps, rope_mode);
        norm_rope_head(y, wk, cosb + (size_t)s * 64, sinb + (size_t)s * 64, eps, rope_mode);
        for (int d = 0; d < KO_D; d++) {
          q[(size_t)s * KO_D + d] = ref_rounding ? bf16_round(x[d]) : x[d];
          kt[(size_t)d * S + s] = ref_rounding ? bf16_round(y[d]) : y[d];
        }
      }
      float* out = O + (size_t)b * S * ldo + (size_t)h * KO_D;
      attend_head(q, kt, v, text_len ? valid : NULL, S, S, 0, 0, NULL, NULL, ref_rounding, out, ldo);
      for (int s = 0; s < S; s++) {
        float* o = out + (size_t)s * ldo;
        if (!valid[s]) for (int d = 0; d < KO_D; d++) o[d] = 0.f;
        else if (ref_rounding) for (int d = 0; d < KO_D; d++) o[d] = bf16_round(o[d]);
      }
    }
  }
  free(q); free(kt); free(v); free(valid);
}

/* Selected query rows of one (sample, head) against the full key range: the sampled check used for the
 * long-sequence configs.  rows_sel: n_rows query indices; out fp32 [n_rows, 128]. */
void ko_joint_attention_rows(const uint16_t* Q, const uint16_t* K, const uint16_t* V, float* out, int S, int h,
                             int kvh, int64_t ld_q, int64_t ld_k, int64_t ld_v, const float* wq, const float* wk,
                             const float* cosb, const float* sinb, float eps, int rope_mode, int text_len,
                             int text_slots, const int32_t* rows_sel, int n_rows, int ref_rounding) {
  float* q = (float*)malloc(sizeof(float) * (size_t)n_rows * KO_D);
  float* kt = (float*)malloc(sizeof(float) * (size_t)S * KO_D);
  float* v = (float*)malloc(sizeof(float) * (size_t)S * KO_D);
  uint8_t* valid = (uint8_t*)malloc((size_t)S);
  for (int s = 0; s < S; s++) valid[s] = !(text_len >= 0 && s >= text_len && s < text_slots);
#pragma omp parallel for schedule(static)
  for (int s = 0; s < S; s++) {
    float y[KO_D];
    for (int d = 0; d < KO_D; d++) {
      y[d] = bf16_to_f32(K[(size_t)s * ld_k + kvh * KO_D + d]);
      v[(size_t)s * KO_D + d] = bf16_to_f32(V[(size_t)s * ld_v + kvh * KO_D + d]);
    }
    norm_rope_head(y, wk, cosb + (size_t)s * 64, sinb + (size_t)s * 64, eps, rope_mode);
    for (int d = 0; d < KO_D; d++) kt[(size_t)d * S + s] = ref_rounding ? bf16_round(y[d]) : y[d];
  }
  for (int r = 0; r < n_rows; r++) {
    const int s = rows_sel[r];
    float x[KO_D];
    for (int d = 0; d < KO_D; d++) x[d] = bf16_to_f32(Q[(size_t)s * ld_q + h * KO_D + d]);
    norm_rope_head(x, wq, cosb + (size_t)s * 64, sinb + (size_t)s * 64, eps, rope_mode);
    for (int d = 0; d < KO_D; d++) q[(size_t)r * KO_D + d] = ref_rounding ? bf16_round(x[d]) : x[d];
  }
  attend_head(q, kt, v, text_len >= 0 ? valid : NULL, n_rows, S, 0, 0, NULL, NULL, ref_rounding, out, KO_D);
  for (int r = 0; r < n_rows; r++) {
    float* o = out + (size_t)r * KO_D;
    if (!valid[rows_sel[r]]) for (int d = 0; d < KO_D; d++) o[d] = 0.f;
    else if (ref_rounding) for (int d = 0; d < KO_D; d++) o[d] = bf16_round(o[d]);
  }
  free(q); free(kt); free(v); free(valid);
}

/* ---- text-fusion layerwise attention (norm.metal:136-178, dispatch metal.mm:204-209) ----
 * Rows are token-major, row = t*12 + j; every row attends over the 12 rows of its own token:
 *   out[row, h*128 + d] = softmax_j(q[row] . k[base+j] / sqrt(128)) v[base+j] * sigmoid(gate[row])
 * with scores, softmax and the weighted sum in fp32 (P is NOT rounded here, unlike attn_body) and one
 * bf16 rounding at the store.  qkvg: fused bf16 rows [rows, ld], heads of 128 channels at q_off, k_off,
 * v_off, g_off.  Output fp32 [rows, heads*128]; ref_rounding rounds it to bf16. */
void ko_layerwise_attn(const uint16_t* qkvg, float* out, int rows, int ld, int heads, int q_off, int k_off, int v_off,
                       int g_off, int ref_rounding) {
  const int taps = 12;
  const float scale = (float)(1.0 / sqrt(128.0));
#pragma omp parallel for schedule(static)
  for (int row = 0; row < rows; row++) {
    const int base = row - row % taps;
    for (int h = 0; h < heads; h++) {
      const uint16_t* q = qkvg + (size_t)row * ld + q_off + h * KO_D;
      float s[12], mx = -INFINITY;
      for (int j = 0; j < taps; j++) {
        const uint16_t* k = qkvg + (size_t)(base + j) * ld + k_off + h * KO_D;
        double acc = 0.0;
        for (int d = 0; d < KO_D; d++) acc += (double)bf16_to_f32(q[d]) * (double)bf16_to_f32(k[d]);
        s[j] = (float)acc * scale;
        if (s[j] > mx) mx = s[j];
      }
      float l = 0.f, o[KO_D];
      for (int d = 0; d < KO_D; d++) o[d] = 0.f;
      for (int j = 0; j < taps; j++) {
        const float e = expf(s[j] - mx);
        l += e;
        const uint16_t* v = qkvg + (size_t)(base + j) * ld + v_off + h * KO_D;
        for (int d = 0; d < KO_D; d++) o[d] += e * bf16_to_f32(v[d]);
      }
      const uint16_t* g = qkvg + (size_t)row * ld + g_off + h * KO_D;
      float* dst = out + (size_t)row * heads * KO_D + (size_t)h * KO_D;
      for (int d = 0; d < KO_D; d++) {
        const float r = o[d] / l * (1.0f / (1.0f + expf(-bf16_to_f32(g[d]))));
        dst[d] = ref_rounding ? bf16_round(r) : r;
      }
    }
  }
}
