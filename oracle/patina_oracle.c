/*
 * patina_oracle.c -- CPU oracle for the Patina GEMM path (see patina_oracle.h).
 *
 * TEST INFRASTRUCTURE ONLY: never linked into, loaded by or called from the
 * shipped GEMM library.
 *
 * Numerical note used throughout: the product of two values that are exactly
 * representable with <= 24 significant bits is exact in double, so
 * "acc += (double)a * (double)b" rounds once per step (in the add) whether or
 * not the compiler fuses it. Any evaluation that keeps one accumulator per
 * output and adds k in ascending order is therefore bit-identical to the
 * reference loop (harness/gemm_check.cpp:165-178).
 */
#define _GNU_SOURCE
#include "patina_oracle.h"

#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

static inline uint32_t f32_bits(float x) {
  uint32_t u;
  memcpy(&u, &x, 4);
  return u;
}
static inline float bits_f32(uint32_t u) {
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* Shift `v` right by `s` (1 <= s <= 31) rounding to nearest, ties to even. */
static inline uint32_t shr_rne(uint32_t v, int s) {
  uint32_t q = v >> s;
  uint32_t rem = v & ((1u << s) - 1u);
  uint32_t half = 1u << (s - 1);
  if (rem > half || (rem == half && (q & 1u))) ++q;
  return q;
}

/* ---- f16 (harness/gemm_check.cpp:66-122 semantics) ---------------------- */
float po_f16_to_f32(uint16_t h) {
  uint32_t s = ((uint32_t)h & 0x8000u) << 16;
  uint32_t e = ((uint32_t)h >> 10) & 31u;
  uint32_t m = (uint32_t)h & 1023u;
  if (e == 31u) return bits_f32(s | 0x7f800000u | (m << 13)); /* inf, nan */
  if (e == 0u) {
    if (m == 0u) return bits_f32(s); /* signed zero */
    /* subnormal: value = m * 2^-24; normalise the 10-bit field */
    int lead = 31 - __builtin_clz(m); /* position of the top set bit, 0..9 */
    uint32_t frac = (m << (10 - lead)) & 1023u;
    uint32_t fe = (uint32_t)(lead - 24 + 127);
    return bits_f32(s | (fe << 23) | (frac << 13));
  }
  return bits_f32(s | ((e + 112u) << 23) | (m << 13));
}

uint16_t po_f32_to_f16(float x) {
  uint32_t u = f32_bits(x);
  uint16_t s = (uint16_t)((u >> 16) & 0x8000u);
  uint32_t e = (u >> 23) & 255u;
  uint32_t m = u & 0x7fffffu;
  if (e == 255u) /* inf keeps a zero payload; any nan becomes a quiet nan */
    return (uint16_t)(s | 0x7c00u | (m ? 0x200u : 0u));
  int he = (int)e - 112; /* re-biased exponent */
  if (he >= 31) return (uint16_t)(s | 0x7c00u); /* too large: inf */
  if (he <= 0) {
    if (he < -10) return s; /* below half the smallest subnormal: zero */
    /* subnormal result: 24-bit significand shifted into a 10-bit field */
    return (uint16_t)(s | shr_rne(m | 0x800000u, 14 - he));
  }
  /* normal: a carry out of the mantissa bumps the exponent (and reaches inf) */
  uint32_t packed = ((uint32_t)he << 23) | m;
  return (uint16_t)(s | shr_rne(packed, 13));
}

/* ---- bf16 ---------------------------------------------------------------- */
float po_bf16_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }

uint16_t po_f32_to_bf16(float x) {
  uint32_t u = f32_bits(x);
  if ((u & 0x7fffffffu) > 0x7f800000u) /* nan: keep sign, force quiet */
    return (uint16_t)((u >> 16) | 0x0040u);
  uint32_t bias = 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)((u + bias) >> 16);
}

/* ---- fp8 e4m3 (OCP "fn": no inf, 0x7f/0xff nan, max finite 448) ---------- */
float po_e4m3_to_f32(uint8_t v) {
  uint32_t s = ((uint32_t)v & 0x80u) << 24;
  uint32_t e = ((uint32_t)v >> 3) & 15u;
  uint32_t m = (uint32_t)v & 7u;
  if (e == 15u && m == 7u) return bits_f32(s | 0x7fc00000u);
  if (e == 0u) {
    float mag = (float)m * 0.001953125f; /* m * 2^-9 */
    return bits_f32(s | f32_bits(mag));
  }
  return bits_f32(s | ((e + 120u) << 23) | (m << 20));
}

uint8_t po_f32_to_e4m3_satfinite(float x) {
  uint32_t u = f32_bits(x);
  uint8_t s = (uint8_t)((u >> 24) & 0x80u);
  uint32_t a = u & 0x7fffffffu;
  if (a > 0x7f800000u) return (uint8_t)(s | 0x7fu); /* nan */
  if (a >= 0x43e80000u) return (uint8_t)(s | 0x7eu); /* >= 464 rounds past 448: clamp */
  uint32_t e = a >> 23;
  uint32_t m = a & 0x7fffffu;
  int ee = (int)e - 120; /* e4m3 biased exponent */
  uint32_t q;
  if (ee <= 0) {
    if (ee < -4) return s; /* < 2^-11: rounds to zero (ties included) */
    q = shr_rne(m | 0x800000u, 21 - ee); /* subnormal, units of 2^-9 */
  } else {
    q = shr_rne(((uint32_t)ee << 23) | m, 20);
  }
  if (q > 0x7eu) q = 0x7eu; /* 448 is the largest finite value */
  return (uint8_t)(s | q);
}

void po_f16_to_f32_n(const uint16_t* src, float* dst, size_t n) {
  for (size_t i = 0; i < n; ++i) dst[i] = po_f16_to_f32(src[i]);
}
void po_f32_to_f16_n(const float* src, uint16_t* dst, size_t n) {
  for (size_t i = 0; i < n; ++i) dst[i] = po_f32_to_f16(src[i]);
}
void po_bf16_to_f32_n(const uint16_t* src, float* dst, size_t n) {
  for (size_t i = 0; i < n; ++i) dst[i] = po_bf16_to_f32(src[i]);
}
void po_f32_to_bf16_n(const float* src, uint16_t* dst, size_t n) {
  for (size_t i = 0; i < n; ++i) dst[i] = po_f32_to_bf16(src[i]);
}
void po_e4m3_to_f32_n(const uint8_t* src, float* dst, size_t n) {
  for (size_t i = 0; i < n; ++i) dst[i] = po_e4m3_to_f32(src[i]);
}
void po_f32_to_e4m3_n(const float* src, uint8_t* dst, size_t n) {
  for (size_t i = 0; i < n; ++i) dst[i] = po_f32_to_e4m3_satfinite(src[i]);
}

/* ---- closed-form inputs (harness/gemm_check.cpp:152-163) ----------------- */
/* Single-precision sinf/cosf on single-precision arguments, as there; the
 * expression trees are kept in the same association order so the float
 * roundings coincide. */
void po_fill_legacy_f16(uint16_t* A, uint16_t* B, uint32_t rows, uint64_t K) {
  for (uint32_t r = 0; r < rows; ++r) {
    const float rp1 = (float)(r + 1u);
    for (uint64_t k = 0; k < K; ++k) {
      const float kf = (float)k;
      const float a_arg0 = 0.1f * rp1 + 0.7f * kf;
      const float a_arg1 = 0.05f * (kf + 1.0f);
      const float b_arg0 = 0.13f * rp1 + 0.11f * kf;
      const float b_arg1 = 0.03f * ((float)((uint64_t)r + k) + 1.0f);
      const float a = 0.9f * sinf(a_arg0) * cosf(a_arg1);
      const float b = 0.8f * cosf(b_arg0) * sinf(b_arg1);
      A[(uint64_t)r * K + k] = po_f32_to_f16(a);
      B[(uint64_t)r * K + k] = po_f32_to_f16(b);
    }
  }
}

/* ---- reference GEMM ------------------------------------------------------ */
int po_host_threads(void) {
  cpu_set_t set;
  if (sched_getaffinity(0, sizeof(set), &set) == 0) {
    int n = CPU_COUNT(&set);
    if (n > 0) return n;
  }
  long n = sysconf(_SC_NPROCESSORS_ONLN);
  return n > 0 ? (int)n : 1;
}

typedef struct {
  const float* A;
  int64_t lda;
  const float* B;
  int64_t ldb;
  double* C;
  int64_t ldc;
  const int64_t* rows; /* NULL: identity */
  int64_t row_begin, row_end;
  int64_t N, K;
} gemm_job;

#define PO_NB 8 /* outputs computed side by side; each keeps its own chain */

static void* gemm_worker(void* arg) {
  const gemm_job* j = (const gemm_job*)arg;
  for (int64_t i = j->row_begin; i < j->row_end; ++i) {
    const int64_t m = j->rows ? j->rows[i] : i;
    const float* a = j->A + m * j->lda;
    double* c = j->C + i * j->ldc;
    int64_t n = 0;
    for (; n + PO_NB <= j->N; n += PO_NB) {
      const float* b = j->B + n * j->ldb;
      double acc[PO_NB];
      for (int t = 0; t < PO_NB; ++t) acc[t] = 0.0;
      for (int64_t k = 0; k < j->K; ++k) {
        const double av = (double)a[k];
        for (int t = 0; t < PO_NB; ++t)
          acc[t] += av * (double)b[(int64_t)t * j->ldb + k];
      }
      for (int t = 0; t < PO_NB; ++t) c[n + t] = acc[t];
    }
    for (; n < j->N; ++n) {
      const float* b = j->B + n * j->ldb;
      double acc = 0.0;
      for (int64_t k = 0; k < j->K; ++k) acc += (double)a[k] * (double)b[k];
      c[n] = acc;
    }
  }
  return NULL;
}

static int run_gemm_jobs(gemm_job proto, int64_t n_rows, int threads) {
  if (threads <= 0) threads = po_host_threads();
  if ((int64_t)threads > n_rows) threads = (int)(n_rows > 0 ? n_rows : 1);
  if (threads > 256) threads = 256;
  pthread_t tid[256];
  gemm_job jobs[256];
  int64_t per = (n_rows + threads - 1) / threads;
  int started = 0;
  for (int t = 0; t < threads; ++t) {
    jobs[t] = proto;
    jobs[t].row_begin = (int64_t)t * per;
    jobs[t].row_end = jobs[t].row_begin + per;
    if (jobs[t].row_end > n_rows) jobs[t].row_end = n_rows;
    if (jobs[t].row_begin >= jobs[t].row_end) break;
    if (t == threads - 1 || pthread_create(&tid[t], NULL, gemm_worker, &jobs[t]) != 0) {
      /* last slab (or a failed spawn) runs on the calling thread, covering
       * everything that is left */
      jobs[t].row_end = n_rows;
      gemm_worker(&jobs[t]);
      break;
    }
    ++started;
  }
  for (int t = 0; t < started; ++t) pthread_join(tid[t], NULL);
  return started + 1;
}

int po_ref_gemm_tn(const float* A, int64_t lda, const float* B, int64_t ldb,
                   double* C, int64_t ldc, int64_t M, int64_t N, int64_t K,
                   int threads) {
  gemm_job p = {A, lda, B, ldb, C, ldc, NULL, 0, 0, N, K};
  return run_gemm_jobs(p, M, threads);
}

int po_ref_gemm_tn_rows(const float* A, int64_t lda, const float* B,
                        int64_t ldb, double* C, int64_t ldc,
                        const int64_t* rows, int64_t n_rows, int64_t N,
                        int64_t K, int threads) {
  gemm_job p = {A, lda, B, ldb, C, ldc, rows, 0, 0, N, K};
  return run_gemm_jobs(p, n_rows, threads);
}

void po_scale_round_bf16(const double* ref, double alpha, float* out, size_t n) {
  for (size_t i = 0; i < n; ++i)
    out[i] = po_bf16_to_f32(po_f32_to_bf16((float)(alpha * ref[i])));
}

/* ---- pass / fail rules ---------------------------------------------------- */
uint64_t po_compare_legacy(const float* got, const double* ref, size_t n,
                           double atol, double rtol, double* max_abs,
                           double* max_rel, double* sum_got) {
  double ma = 0.0, mr = 0.0, sum = 0.0;
  uint64_t bad = 0;
  for (size_t i = 0; i < n; ++i) {
    const double g = (double)got[i];
    const double abs_err = fabs(g - ref[i]);
    const double rel_err = abs_err / fmax(1.0, fabs(ref[i]));
    sum += g;
    if (abs_err > ma) ma = abs_err;
    if (rel_err > mr) mr = rel_err;
    if (abs_err > atol && rel_err > rtol) ++bad;
    if (g != g) ++bad; /* a NaN never satisfies the > tests: count it */
  }
  if (max_abs) *max_abs = ma;
  if (max_rel) *max_rel = mr;
  if (sum_got) *sum_got = sum;
  return bad;
}

int po_compare_norm(const float* got, const float* ref, size_t n,
                    double elem_tol, double fro_tol, double* max_abs_err,
                    double* max_abs_ref, double* fro_rel) {
  double me = 0.0, mx = 0.0, se = 0.0, sr = 0.0;
  int nan_seen = 0;
  for (size_t i = 0; i < n; ++i) {
    const double g = (double)got[i], r = (double)ref[i];
    const double d = fabs(g - r);
    if (g != g) nan_seen = 1;
    if (d > me) me = d;
    if (fabs(r) > mx) mx = fabs(r);
    se += d * d;
    sr += r * r;
  }
  const double fr = sr > 0.0 ? sqrt(se / sr) : (se > 0.0 ? INFINITY : 0.0);
  if (max_abs_err) *max_abs_err = me;
  if (max_abs_ref) *max_abs_ref = mx;
  if (fro_rel) *fro_rel = fr;
  return !nan_seen && me <= elem_tol * mx && fr <= fro_tol;
}
