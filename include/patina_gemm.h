/*
 * patina_gemm.h -- C ABI of the B200 (sm_100a) tcgen05 GEMM library.
 *
 * This is the boundary that replaces, for the GEMM hot path, what the reference
 * (neoming/Patina) exposes only as a generated PTX entry plus host runners:
 *   - the kernel ABI `tcgen05_gemm_v2(tma_a, tma_b, c, k_tiles)`
 *     (crates/patina/tests/golden/v2_gemm_pipelined.ptx:25-31),
 *   - the Rust runner `run_gemm(ptx, kernel, k, a, b)` (crates/patina/src/run.rs:462-529),
 *   - the C++ harness `gemm_check <ptx> <kernel> <K>` (harness/gemm_check.cpp:186-351).
 * Ownership and error conventions follow the reference's compiler C ABI
 * (mlir/include/patina-c/PatinaCAPI.h:3-39): opaque caller-owned contexts,
 * heap strings released by a *_string_free that accepts NULL, null arguments
 * produce a diagnostic and never a crash.
 *
 * All matrices are "TN": C[M,N] = alpha * A[M,K] * B[N,K]^T with A and B both
 * K-contiguous (row-major A, K-major B) and C row-major. Leading dimensions
 * are in ELEMENTS. Unless a function says otherwise, pointers are DEVICE
 * pointers owned by the caller, the call only enqueues work on `stream`
 * (a cudaStream_t passed as void*; NULL = the default stream) and does not
 * synchronise. There is no CPU fallback: without an sm_100 device every
 * compute entry point returns PATINA_GEMM_ERR_UNSUPPORTED_ARCH.
 *
 * Alignment rules (TMA): A, B, C base addresses 16-byte aligned;
 * lda, ldb, ldc times the element size a multiple of 16 bytes; lda,ldb >= K,
 * ldc >= N. M, N, K are otherwise free (ragged edges are zero-filled on load
 * and clipped on store: no element of C outside [M, N] is written, whatever
 * N's remainder). M == 0 or N == 0 is a no-op; K == 0 stores zeros.
 */
#ifndef PATINA_GEMM_H
#define PATINA_GEMM_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct PatinaGemmContext PatinaGemmContext;

enum {
  PATINA_GEMM_OK = 0,
  PATINA_GEMM_ERR_INVALID_ARG = 1,
  PATINA_GEMM_ERR_UNSUPPORTED_ARCH = 2, /* harness exit code 3 (gemm_check.cpp:233-238) */
  PATINA_GEMM_ERR_CUDA = 3,             /* harness exit code 2 (gemm_check.cpp:43-56) */
  PATINA_GEMM_ERR_TIMEOUT = 4           /* a bounded device-side wait expired */
};

enum { PATINA_IN_F16 = 0, PATINA_IN_BF16 = 1, PATINA_IN_E4M3 = 2,
       PATINA_IN_MXE4M3 = 3 /* block-scaled: patina_gemm_mxfp8_tn only */ };
enum { PATINA_OUT_BF16 = 0, PATINA_OUT_F32 = 1, PATINA_OUT_E4M3 = 2 /* fused epilogue only */ };

/* Tile configuration. Zero in any field means "choose for me". */
typedef struct PatinaGemmConfig {
  int32_t cta_group; /* 1 = one CTA per tile; 2 = CTA pair (tcgen05 cta_group::2) */
  int32_t block_n;   /* tile width: 128 ... 256 in steps of 16 for pair tiles with m_sub = 2,
                        128 or 256 otherwise */
  int32_t stages;    /* shared-memory ring depth */
  int32_t group_m;   /* scheduler band height in tiles */
  int32_t max_ctas;  /* cap on persistent CTAs (0 = number of SMs) */
  int32_t m_sub;     /* 128-row accumulator sub-tiles per CTA: 1 or 2;
                        tile height = 128 * cta_group * m_sub */
  int32_t stream_k;  /* skinny path (M <= 128; bf16 out, or f16 in / f32 out): 0 = library decides, 1 = force,
                        -1 = never; 2 = force, and sum shared tiles in the follow-up kernel;
                        3 = force, and let the last CTA to reach a tile sum it */
  int32_t cluster_k; /* few tiles, deep K, M > 128 (bf16): K cut across a thread-block cluster of
                        this many CTAs (2 or 4) per 128 x 256 tile, partial tiles summed through
                        distributed shared memory; 0 = library decides, -1 = never */
  int32_t k_order;   /* 0 = library decides: problems of at most one wave of 128 x 128 tiles take
                        kernels with two accumulators (C = sum over even k-blocks + sum over odd
                        k-blocks), a few take cluster_k; 1 = every output is summed over k in
                        ascending order in one accumulator, so the result does not depend on how
                        a problem is cut into column shards or row blocks (the sharded and
                        host-buffer entry points ask for this themselves) */
} PatinaGemmConfig;

/* What a call would launch; computed on the host without touching a device. */
typedef struct PatinaGemmPlan {
  int32_t cta_group, block_n, stages, group_m, m_sub;
  uint32_t tile_m;
  uint32_t tiles_m, tiles_n, num_tiles, k_blocks;
  uint32_t grid, block, cluster, smem_bytes, tmem_cols;
  uint32_t stage_bytes, expect_tx_bytes;
  uint32_t idesc;
  uint32_t half_tiles; /* tiles of the last wave run as two half tiles each (m_sub = 2 kernels, when
                          that wave fills at most half of the clusters): the persistent CTAs walk
                          num_tiles + half_tiles scheduler indices */
} PatinaGemmPlan;

/* ---- context (replaces run.rs `Cuda::init` / `Drop`, run.rs:256-394) ----- */
/* One context per device. Calls on one context are not thread-safe; different
 * contexts are independent. Returns PATINA_GEMM_ERR_UNSUPPORTED_ARCH when the
 * device is not compute capability 10.x (run.rs:476-481, gemm_check.cpp:233). */
int patina_gemm_context_create(int device, PatinaGemmContext** out);
void patina_gemm_context_destroy(PatinaGemmContext* ctx);

/* Last diagnostic of this context as a heap string (NULL if none). Mirrors
 * patina_verify's "NULL means success" (PatinaCAPI.h:25-28). */
char* patina_gemm_last_error(PatinaGemmContext* ctx);
/* Mirrors patina_string_free (PatinaCAPI.h:38-39). NULL-safe. */
void patina_gemm_string_free(char* s);

/* Bound, in nanoseconds, on every barrier wait inside the kernels
 * (the reference's waits are unbounded spins, v2_gemm_pipelined.ptx:111-113). */
int patina_gemm_set_wait_limit_ns(PatinaGemmContext* ctx, uint64_t ns);

/* Synchronise `stream` and report whether any kernel enqueued through this
 * context since the last call gave up on a wait (PATINA_GEMM_ERR_TIMEOUT).
 * Replaces the cuStreamSynchronize in gemm_check.cpp:297 / run.rs:375.
 * The context keeps ONE status record: with several streams on one context the report does not
 * say which stream's kernel gave up. After a suspected expiry call this before the context is
 * used again: it also clears the skinny path's arrival counters, which an abandoned launch can
 * leave half-way (later skinny launches would otherwise finish tiles early or not at all). */
int patina_gemm_status(PatinaGemmContext* ctx, void* stream);

/* Kernels this context has launched so far. */
uint64_t patina_gemm_launch_count(PatinaGemmContext* ctx);

/* ---- the GEMM entry points ------------------------------------------------ */
/* bf16 in, fp32 accumulate (TMEM), bf16 out. Replaces the cuLaunchKernel of the
 * generated kernel (gemm_check.cpp:286-296, run.rs:502-524) for bf16 problems. */
int patina_gemm_bf16_tn(PatinaGemmContext* ctx, const void* A, int64_t lda, const void* B,
                        int64_t ldb, void* C, int64_t ldc, int64_t M, int64_t N, int64_t K,
                        float alpha, void* stream);

/* fp8 e4m3 in, fp32 accumulate, bf16 out scaled by scale_a * scale_b. */
int patina_gemm_fp8e4m3_tn(PatinaGemmContext* ctx, const void* A, int64_t lda, const void* B,
                           int64_t ldb, void* C, int64_t ldc, int64_t M, int64_t N, int64_t K,
                           float scale_a, float scale_b, void* stream);

/* f16 in, fp32 out: the reference kernel's own types (gemm_check.cpp:9-10);
 * with M = N = 128 and K % 32 == 0 it computes exactly what tcgen05_gemm_v2 does. */
int patina_gemm_f16_tn_f32out(PatinaGemmContext* ctx, const void* A, int64_t lda, const void* B,
                              int64_t ldb, void* C, int64_t ldc, int64_t M, int64_t N, int64_t K,
                              float alpha, void* stream);

/* Any supported (in_type, out_type) pair with an explicit tile configuration
 * (cfg may be NULL). */
int patina_gemm_ex(PatinaGemmContext* ctx, int in_type, int out_type, const void* A, int64_t lda,
                   const void* B, int64_t ldb, void* C, int64_t ldc, int64_t M, int64_t N,
                   int64_t K, float alpha, const PatinaGemmConfig* cfg, void* stream);

/* Fused epilogue (no counterpart in the reference, whose kernel stores the raw accumulator,
 * v2_gemm_pipelined.ptx:252-330): C = act(alpha * A*B^T + bias[n] + beta * R[m,n]), evaluated in
 * fp32 on the accumulator before the single rounding to bf16. bias: N floats or NULL; residual:
 * [M, ldr] bf16 or NULL (may alias C only if ldr == ldc and it is the same buffer);
 * activation: 0 none, 1 relu, 2 gelu (erf form), 3 silu. */
typedef struct PatinaGemmEpilogue {
  const void* bias;
  const void* residual;
  int64_t ldr;
  float beta;
  int32_t activation;
} PatinaGemmEpilogue;
int patina_gemm_bf16_tn_fused(PatinaGemmContext* ctx, const void* A, int64_t lda, const void* B,
                              int64_t ldb, void* C, int64_t ldc, int64_t M, int64_t N, int64_t K,
                              float alpha, const PatinaGemmEpilogue* epi, void* stream);

/* The fused epilogue with an fp8 result (no counterpart in the reference): what a quantised
 * layer stack needs from the GEMM that feeds its next fp8 GEMM.
 *     y = act(alpha * A * B^T + bias + beta * R)          (fp32, as above)
 *     C[M, ldc] (e4m3, one byte per element) = saturate_e4m3(round_to_nearest_even(out_scale * y))
 *     *amax = max(*amax, max |y|)  over the M x N outputs (device float, atomic; may be NULL;
 *             the caller zeroes it when a new scale window starts)
 * ldc must be a multiple of 16 (bytes = elements); epi may be NULL (plain GEMM, quantised). */
int patina_gemm_bf16_tn_fused_fp8out(PatinaGemmContext* ctx, const void* A, int64_t lda, const void* B,
                                     int64_t ldb, void* C, int64_t ldc, int64_t M, int64_t N, int64_t K,
                                     float alpha, const PatinaGemmEpilogue* epi, float out_scale,
                                     float* amax, void* stream);

/* Column-shard scatter (no counterpart in the reference, which is single-GPU): the same bf16
 * GEMM, but every finished tile of C is stored to n_dests (1..8) destinations that share M, N
 * and ldc. On a multi-GPU node each GPU passes, for every GPU g, the address of ITS column block
 * inside g's full-width C (its own buffer plus peer buffers mapped into this process, e.g. with
 * CUDA IPC), so that when all GPUs are done each holds the whole C: the optional all-gather is
 * fused into the epilogue as peer writes over NVLink (TMA stores; nothing is loaded from a
 * peer, nothing is multicast, no GPU waits for another inside the kernel). The caller
 * synchronises the GPUs around the call (nobody may still read a C that is being written). */
int patina_gemm_bf16_tn_scatter(PatinaGemmContext* ctx, const void* A, int64_t lda, const void* B,
                                int64_t ldb, void* const* C_dests, int n_dests, int64_t ldc,
                                int64_t M, int64_t N, int64_t K, float alpha, void* stream);

/* Grouped GEMM (no counterpart in the reference, whose kernel runs one 128 x 128 problem; this
 * is its runtime `k_tiles` parameter, crates/patina/tests/golden/v2_gemm_pipelined.ptx:29, taken
 * one step further: the tile list itself is a runtime value). One launch computes
 *     C_g[M_g, N] = alpha * A_g[M_g, K] * B_g[N, K]^T     for g = 0 .. n_groups-1
 * for groups that share N and K, e.g. the experts of a mixture-of-experts layer:
 *   A  [total_rows, lda]   the groups' rows one after another (bf16, K-contiguous)
 *   B  [n_groups * N, ldb] group g's weights are rows g*N .. (g+1)*N-1
 *   C  [total_rows, ldc]   rows in the same order as A
 *   group_rows             DEVICE array of n_groups int32: M_g (negative counts as 0); the call
 *                          never reads it on the host, so it may be the output of a routing
 *                          kernel that is still running on `stream`
 * Rows of C from sum(M_g) up to total_rows are left untouched; if the sum exceeds total_rows the
 * excess is dropped. n_groups <= 128 per call. `config` may be NULL; only cta_group, m_sub,
 * group_m and max_ctas are looked at (tile height 128 * cta_group * m_sub, width 256). */
int patina_gemm_bf16_tn_grouped(PatinaGemmContext* ctx, const void* A, int64_t lda, const void* B,
                                int64_t ldb, void* C, int64_t ldc, const int32_t* group_rows,
                                int n_groups, int64_t total_rows, int64_t N, int64_t K, float alpha,
                                const PatinaGemmConfig* config, void* stream);

/* The same for e4m3 inputs with bf16 output: C_g = scale_a * group_scale_b[g] * (A_g * B_g^T).
 * group_scale_b is a DEVICE array of n_groups floats (each group's weight scale), or NULL for
 * a common factor of 1. */
int patina_gemm_fp8e4m3_tn_grouped(PatinaGemmContext* ctx, const void* A, int64_t lda, const void* B,
                                   int64_t ldb, void* C, int64_t ldc, const int32_t* group_rows,
                                   int n_groups, int64_t total_rows, int64_t N, int64_t K, float scale_a,
                                   const float* group_scale_b, const PatinaGemmConfig* config,
                                   void* stream);

/* Block-scaled fp8 ("MXFP8"; no counterpart in the reference, whose kernel is f16 only,
 * crates/patina/tests/golden/v2_gemm_pipelined.ptx:203,212): A and B hold e4m3 elements, and every
 * 32 consecutive K elements of a row share one E8M0 scale (a byte e: the factor 2^(e - 127); 0xFF is
 * NaN). The tensor core applies the scales (tcgen05.mma kind::mxf8f6f4.block_scale, scales in TMEM):
 *     C[M,N] (bf16) = alpha * sum_k (A[m,k] * sa[m, k/32]) * (B[n,k] * sb[n, k/32])
 * K must be a multiple of 32. The scales of a [rows, K] operand live in a buffer of
 * patina_gemm_mx_scale_bytes(rows, K) bytes, in atoms of 512 bytes that cover 128 rows x 128 elements
 * of K: atom index (row / 128) * ceil(K / 128) + k / 128, and inside the atom the scale of row r,
 * 32-element block j is byte (r % 32) * 16 + ((r % 128) / 32) * 4 + (j % 4), the layout the tensor
 * core's scale loads take (the "128x4 swizzled" layout other libraries use for MX scales).
 * patina_gemm_mx_scale_offset gives the byte offset of one scale. The buffer is padded to whole
 * atoms; padding bytes must be valid scales (anything but 0xFF), e.g. 127 (= 1.0). Scale buffers
 * are device pointers, 16-byte aligned. `config` may be NULL; block_n is 256, 192 or 128. */
int patina_gemm_mxfp8_tn(PatinaGemmContext* ctx, const void* A, int64_t lda, const void* scales_a,
                         const void* B, int64_t ldb, const void* scales_b, void* C, int64_t ldc, int64_t M,
                         int64_t N, int64_t K, float alpha, const PatinaGemmConfig* config, void* stream);
uint64_t patina_gemm_mx_scale_bytes(int64_t rows, int64_t K);
uint64_t patina_gemm_mx_scale_offset(int64_t row, int64_t k_block32, int64_t K);

/* N-column sharding over several GPUs (no counterpart in the reference, which uses device 0 only,
 * harness/gemm_check.cpp:222). patina_gemm_column_shard gives shard `rank` of `world` its columns
 * [*n0, *n1) of an N-wide problem: contiguous, in whole 256-column tiles while columns last
 * (trailing shards may be narrower or empty). patina_gemm_sharded_bf16_tn enqueues the whole
 * sharded bf16 GEMM from one host thread: for every shard g one launch on ctxs[g]'s device and
 * streams[g] (NULL array or entry: that device's default stream) computing
 *     C_shards[g][M, n1-n0] = alpha * A[g][M, K] * B_shards[g][n1-n0, K]^T
 * where A[g] is shard g's copy of the replicated A, B_shards[g] the rows [n0, n1) of B and
 * C_shards[g] the address of shard g's first column (its own buffer, or column n0 of a full-width
 * C with ldc = N). No GPU waits for another; call patina_gemm_status per context afterwards.
 * Two shards may share a device (two contexts, two streams). n_shards is 1..8. */
void patina_gemm_column_shard(int64_t n, int world, int rank, int64_t* n0, int64_t* n1);
int patina_gemm_sharded_bf16_tn(PatinaGemmContext* const* ctxs, int n_shards, const void* const* A, int64_t lda,
                                const void* const* B_shards, int64_t ldb, void* const* C_shards, int64_t ldc,
                                int64_t M, int64_t N, int64_t K, float alpha, void* const* streams);

/* Buffers for the scatter above (no counterpart in the reference). peer_alloc gives device
 * memory of this context's GPU plus a 64-byte handle that another PROCESS on the node passes
 * to peer_open (with its own context) to get a pointer its GPU can write through NVLink.
 * Close every opened pointer before the owner frees the buffer. */
int patina_gemm_peer_alloc(PatinaGemmContext* ctx, size_t bytes, void** ptr, unsigned char handle_out[64]);
int patina_gemm_peer_open(PatinaGemmContext* ctx, const unsigned char handle[64], void** ptr);
int patina_gemm_peer_close(PatinaGemmContext* ctx, void* ptr);
int patina_gemm_peer_free(PatinaGemmContext* ctx, void* ptr);

/* End-to-end form with HOST buffers, the shape of run.rs `run_gemm`
 * (alloc + memcpy_htod + launch + memcpy_dtoh, run.rs:484-528): copies A and B
 * to context-owned device buffers, runs the GEMM, copies C back, all on
 * `stream`, and returns without synchronising. Host buffers should be pinned. */
int patina_gemm_host(PatinaGemmContext* ctx, int in_type, int out_type, const void* hostA,
                     int64_t lda, const void* hostB, int64_t ldb, void* hostC, int64_t ldc,
                     int64_t M, int64_t N, int64_t K, float alpha, const PatinaGemmConfig* cfg,
                     void* stream);

/* ---- allocation-free entry point ---------------------------------------------- */
/* No counterpart in the reference (which allocates per run, gemm_check.cpp:266-272).
 *
 * For callers that must not allocate device memory: code running inside an allocator's own
 * callback, a process whose device memory is fully carved up and audited at start-up, a loop
 * that cannot afford cudaMalloc's implicit device-wide synchronisation. The context API
 * allocates (status word, scratch that grows on demand); this call allocates nothing after
 * its first call on a device (see below): no cudaMalloc, no cudaFree, no allocating library
 * routine, no host heap.
 *
 * It runs the skinny stream-K GEMM, bf16 in / bf16 out, C = alpha * A[M,K] * B[N,K]^T with
 * 1 <= M <= 128, on the CURRENT device, enqueued on `stream`, without synchronising. A, B, C
 * are device pointers under the usual alignment rules. Its scratch (partial tiles, arrival
 * counters, a wait-expiry record) is a fixed array inside the loaded module:
 * PATINA_GEMM_NOALLOC_PARTIAL_BYTES of partial-tile space plus 64 KiB of counters. Every GPU
 * that loads the library holds that array until the process exits. A problem whose partial
 * tiles do not fit is refused with PATINA_GEMM_ERR_INVALID_ARG and a message saying how many
 * bytes it would need (roughly: ceil(N/128) * 2 * round16(M) * 512 bytes).
 *
 * All calls on one GPU share the array and it keeps the last call's contents; the call clears
 * what must start at zero, on `stream`, before launching. Two calls that overlap on the same
 * GPU therefore race: issue them on one stream, or otherwise order them.
 *
 * The first call on each device does a one-time set-up (device queries, a driver entry-point
 * lookup, the address of the scratch array). With lazy module loading that first call is also
 * when the driver loads the module and reserves the array on that GPU, so treat it as part of
 * start-up: make one warm-up call per device before entering any region where allocation is
 * forbidden, and outside any stream capture. From the second call on, nothing is allocated
 * on the device or on the host heap, on success or on failure (diagnostics are formatted into
 * err_buf). The set-up is published with release/acquire ordering, so concurrent first calls
 * from several host threads are safe (they repeat the same work).
 *
 * Shared tiles are always summed by the last CTA to reach them (the follow-up reduce kernel of
 * the context API is not used here), which is the slower choice for M > 16 on narrow problems
 * (measured: about 15 us instead of 2 us for the sum at M = 128, N = 3584).
 * A device-side wait that runs out still ends the kernel after its bound, but this entry
 * point has no way to report it; use the context API when that report is needed.
 * err_buf (optional) receives a NUL-terminated diagnostic on failure. */
#define PATINA_GEMM_NOALLOC_PARTIAL_BYTES (16u * 1024u * 1024u)
int patina_gemm_bf16_tn_skinny_noalloc(const void* A, int64_t lda, const void* B, int64_t ldb,
                                       void* C, int64_t ldc, int64_t M, int64_t N, int64_t K,
                                       float alpha, void* stream, char* err_buf,
                                       size_t err_buf_len);

/* ---- host-only helpers (no device needed) ---------------------------------- */
/* Argument check used by every entry point; on failure returns
 * PATINA_GEMM_ERR_INVALID_ARG and, if err_out != NULL, a heap diagnostic. */
int patina_gemm_validate(int in_type, int out_type, const void* A, int64_t lda, const void* B,
                         int64_t ldb, const void* C, int64_t ldc, int64_t M, int64_t N, int64_t K,
                         char** err_out);

/* Launch plan for a problem on a device with `num_sms` SMs. */
int patina_gemm_plan(int in_type, int out_type, int64_t M, int64_t N, int64_t K,
                     const PatinaGemmConfig* cfg, int num_sms, PatinaGemmPlan* out);

/* The skinny (stream-K) path: the flat list of (128-row tile of B, k-block) units is cut
 * into one contiguous range per CTA; tiles shared by several CTAs are reduced through
 * context-owned scratch memory. These helpers expose the partition for host tests. */
typedef struct PatinaStreamKPlan {
  uint32_t grid, tiles, k_blocks, m_pad, max_contrib, stages, smem_bytes;
  uint64_t units, partial_bytes, counter_bytes;
} PatinaStreamKPlan;
int patina_gemm_streamk_plan(int in_type, int64_t M, int64_t N, int64_t K, int num_sms,
                             PatinaStreamKPlan* out);
void patina_gemm_streamk_range(uint64_t cta, uint64_t units, uint64_t parts, uint64_t* begin,
                               uint64_t* end);
/* 1 if a call without an explicit configuration would take the stream-K kernel for this
 * problem on a device with num_sms SMs, 0 if the large-tile kernel (host-only; for tests). */
int patina_gemm_streamk_chosen(int in_type, int out_type, int64_t M, int64_t N, int64_t K, int num_sms);
uint32_t patina_gemm_streamk_owner(uint64_t unit, uint64_t units, uint64_t parts);
/* The cluster size (2 or 4) a call without an explicit configuration would cut K across for this
 * problem on a device with num_sms SMs, or 0 (host-only; for tests). */
int patina_gemm_cluster_k_chosen(int in_type, int out_type, int64_t M, int64_t N, int64_t K, int num_sms);

/* Derived encodings, exported so tests can pin them against the reference's
 * constants (crates/patina/tests/layout.rs:33-68; v2_gemm_pipelined.ptx:192,197). */
uint64_t patina_gemm_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                               int swizzle_code);
uint32_t patina_gemm_idesc(int in_type, uint32_t umma_m, uint32_t umma_n);
/* instruction descriptor of the block-scaled form (E8M0 scales, e4m3 operands) */
uint32_t patina_gemm_idesc_mx(uint32_t umma_m, uint32_t umma_n, uint32_t a_sf_id, uint32_t b_sf_id);
uint32_t patina_gemm_k_advance_units(uint32_t k_elems, int in_type);
uint32_t patina_gemm_tmem_lane_offset(uint32_t warp_quarter);
void patina_gemm_tile_coord(uint32_t t, uint32_t tiles_m, uint32_t tiles_n, uint32_t group_m,
                            uint32_t* m_block, uint32_t* n_block);

const char* patina_gemm_version(void);

#ifdef __cplusplus
}
#endif
#endif /* PATINA_GEMM_H */
