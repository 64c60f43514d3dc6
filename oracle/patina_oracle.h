/*
 * patina_oracle.h -- CPU oracle for the Patina GEMM path.
 *
 * TEST INFRASTRUCTURE ONLY. This is a CPU restatement of the reference's own
 * numerical check (harness/gemm_check.cpp in neoming/Patina). The shipped
 * library never calls it; only the test-suite, the smoke check and the CPU
 * baseline leg of the benchmark do, and only as the checker / the baseline.
 *
 * Parity status: PINNED. The restatement is checked, bit for bit, against the
 * reference's own functions compiled from the reference sources
 * (oracle/_ref/libpatina_ref.so, built by oracle/Makefile) and against
 * fixtures generated from them (tests/golden/).
 */
#ifndef PATINA_ORACLE_H
#define PATINA_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- storage-type converters (software, round-to-nearest-even) --------- */
/* Follows harness/gemm_check.cpp:66-91 (f16 -> f32). */
float po_f16_to_f32(uint16_t h);
/* Follows harness/gemm_check.cpp:93-122 (f32 -> f16, RNE). */
uint16_t po_f32_to_f16(float x);
/* bf16 and e4m3 are not in the reference; same software-RNE style. */
float po_bf16_to_f32(uint16_t h);
uint16_t po_f32_to_bf16(float x);
float po_e4m3_to_f32(uint8_t v);
uint8_t po_f32_to_e4m3_satfinite(float x);

void po_f16_to_f32_n(const uint16_t* src, float* dst, size_t n);
void po_f32_to_f16_n(const float* src, uint16_t* dst, size_t n);
void po_bf16_to_f32_n(const uint16_t* src, float* dst, size_t n);
void po_f32_to_bf16_n(const float* src, uint16_t* dst, size_t n);
void po_e4m3_to_f32_n(const uint8_t* src, float* dst, size_t n);
void po_f32_to_e4m3_n(const float* src, uint8_t* dst, size_t n);

/* ---- the reference's closed-form inputs -------------------------------- */
/* Follows harness/gemm_check.cpp:152-163: A[rows,K], B[rows,K] as f16 bits.
 * The reference fixes rows = 128. */
void po_fill_legacy_f16(uint16_t* A, uint16_t* B, uint32_t rows, uint64_t K);

/* ---- the reference GEMM ------------------------------------------------- */
/* C[m,n] = sum_k (double)A[m,k] * (double)B[n,k], k ascending, one double
 * accumulator per output. Follows harness/gemm_check.cpp:165-178, with the
 * 128x128 extents and dense pitches generalised to M, N and lda/ldb/ldc
 * (element strides). A and B hold the storage values already widened to
 * float, which is exact for f16, bf16 and e4m3. `threads` <= 0 means all
 * host cores. Returns the number of threads used. */
int po_ref_gemm_tn(const float* A, int64_t lda, const float* B, int64_t ldb,
                   double* C, int64_t ldc, int64_t M, int64_t N, int64_t K,
                   int threads);

/* Same, but only for the listed rows of A (output row i = A row rows[i]). */
int po_ref_gemm_tn_rows(const float* A, int64_t lda, const float* B,
                        int64_t ldb, double* C, int64_t ldc,
                        const int64_t* rows, int64_t n_rows, int64_t N,
                        int64_t K, int threads);

/* out[i] = bf16_rne((float)(alpha * ref[i])) widened back to float. */
void po_scale_round_bf16(const double* ref, double alpha, float* out, size_t n);

/* ---- pass / fail rules --------------------------------------------------- */
/* The reference's rule (harness/gemm_check.cpp:303-321): an element is a
 * mismatch iff abs_err > atol AND abs_err / max(1, |ref|) > rtol. */
uint64_t po_compare_legacy(const float* got, const double* ref, size_t n,
                           double atol, double rtol, double* max_abs,
                           double* max_rel, double* sum_got);

/* The max-norm + Frobenius rule: returns 1 iff
 * max|got-ref| <= elem_tol * max|ref| and ||got-ref||_F <= fro_tol * ||ref||_F. */
int po_compare_norm(const float* got, const float* ref, size_t n,
                    double elem_tol, double fro_tol, double* max_abs_err,
                    double* max_abs_ref, double* fro_rel);

int po_host_threads(void);

#ifdef __cplusplus
}
#endif
#endif /* PATINA_ORACLE_H */
