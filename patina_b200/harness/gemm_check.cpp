// gemm_check -- numerical check and timing of the GEMM library from C++.
//
// Drop-in for the reference's harness CLI (harness/gemm_check.cpp:186-218 of
// neoming/Patina): the positional form
//
//     gemm_check <ptx_file> <kernel_name> <K>
//
// still runs C[128,128] f32 = A[128,K] f16 * B[128,K]^T with the same closed-form
// inputs, the same double-precision check, the same stdout lines and the same
// exit codes (0 PASS, 1 FAIL, 2 usage/CUDA error, 3 device is not sm_100). The
// <ptx_file> argument is accepted for compatibility and not read: the kernel is
// the library's own (patina_gemm_f16_tn_f32out), reached through the C ABI.
//
// The flag form covers the library's other entry points:
//
//     gemm_check --m M --n N --k K [--dtype bf16|fp8|f16] [--cta 1|2] [--block-n 128|256]
//                [--dist uniform|normal01|llm] [--seed S] [--alpha X] [--iters I]
//                [--check-rows R] [--splitk MODE] [--gpus G] [--allgather]
//
// and adds time_us / tflops / pct_peak lines. --splitk forces (1, 2, 3) or forbids (-1) the
// skinny stream-K path (PatinaGemmConfig::stream_k). --gpus G splits the N columns of a bf16
// problem over G GPUs of this node, one host thread and one library context per GPU, A
// replicated, no communication during the GEMM; with --allgather every GPU's epilogue stores
// its column block into every GPU's full-width C over NVLink (patina_gemm_bf16_tn_scatter:
// peer stores, nothing loaded from a peer, nothing multicast), and every GPU's copy of the
// whole C is verified. The reference harness is single-GPU (harness/gemm_check.cpp:222).
// Verification is this program's job, as in the reference: it carries its own CPU reference loop.
#include <cuda_runtime.h>

#include <algorithm>
#include <chrono>
#include <cmath>
#include <condition_variable>
#include <mutex>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "patina_gemm.h"

namespace {

constexpr int kExitPass = 0, kExitFail = 1, kExitError = 2, kExitNotSm100 = 3;

#define RT_CHECK(call)                                                                       \
  do {                                                                                       \
    cudaError_t e_ = (call);                                                                 \
    if (e_ != cudaSuccess) {                                                                 \
      std::fprintf(stderr, "CUDA error at %s:%d in %s: %s (%s)\n", __FILE__, __LINE__, #call, \
                   cudaGetErrorName(e_), cudaGetErrorString(e_));                            \
      std::exit(kExitError);                                                                 \
    }                                                                                        \
  } while (0)

// ---- storage types (software conversions, round to nearest even) -----------
uint32_t bits_of(float x) { uint32_t u; std::memcpy(&u, &x, 4); return u; }
float float_of(uint32_t u) { float f; std::memcpy(&f, &u, 4); return f; }

uint16_t to_bf16(float x) {
  uint32_t u = bits_of(x);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40u);
  return (uint16_t)((u + 0x7fffu + ((u >> 16) & 1u)) >> 16);
}
float from_bf16(uint16_t h) { return float_of((uint32_t)h << 16); }

uint32_t round_shift(uint32_t v, int s) {
  uint32_t q = v >> s, rem = v & ((1u << s) - 1u), half = 1u << (s - 1);
  return q + ((rem > half || (rem == half && (q & 1u))) ? 1u : 0u);
}
uint16_t to_f16(float x) {
  uint32_t u = bits_of(x), s = (u >> 16) & 0x8000u, e = (u >> 23) & 255u, m = u & 0x7fffffu;
  if (e == 255u) return (uint16_t)(s | 0x7c00u | (m ? 0x200u : 0u));
  int he = (int)e - 112;
  if (he >= 31) return (uint16_t)(s | 0x7c00u);
  if (he <= 0) return he < -10 ? (uint16_t)s : (uint16_t)(s | round_shift(m | 0x800000u, 14 - he));
  return (uint16_t)(s | round_shift(((uint32_t)he << 23) | m, 13));
}
float from_f16(uint16_t h) {
  uint32_t s = ((uint32_t)h & 0x8000u) << 16, e = (h >> 10) & 31u, m = h & 1023u;
  if (e == 31u) return float_of(s | 0x7f800000u | (m << 13));
  if (e == 0u) return float_of(s | bits_of((float)m * 5.9604644775390625e-8f));
  return float_of(s | ((e + 112u) << 23) | (m << 13));
}
uint8_t to_e4m3(float x) {
  uint32_t u = bits_of(x), a = u & 0x7fffffffu;
  uint8_t s = (uint8_t)((u >> 24) & 0x80u);
  if (a > 0x7f800000u) return (uint8_t)(s | 0x7fu);
  if (a >= 0x43e80000u) return (uint8_t)(s | 0x7eu);
  int ee = (int)(a >> 23) - 120;
  uint32_t m = a & 0x7fffffu, q;
  if (ee <= 0) q = ee < -4 ? 0u : round_shift(m | 0x800000u, 21 - ee);
  else q = round_shift(((uint32_t)ee << 23) | m, 20);
  return (uint8_t)(s | std::min(q, 0x7eu));
}
float from_e4m3(uint8_t v) {
  uint32_t s = ((uint32_t)v & 0x80u) << 24, e = (v >> 3) & 15u, m = v & 7u;
  if (e == 15u && m == 7u) return float_of(s | 0x7fc00000u);
  if (e == 0u) return float_of(s | bits_of((float)m * 0.001953125f));
  return float_of(s | ((e + 120u) << 23) | (m << 20));
}

// ---- inputs -------------------------------------------------------------------
// The reference's closed-form f16 inputs (harness/gemm_check.cpp:152-163).
void fill_closed_form(std::vector<uint16_t>& A, std::vector<uint16_t>& B, uint32_t rows, uint64_t K) {
  for (uint32_t r = 0; r < rows; ++r)
    for (uint64_t k = 0; k < K; ++k) {
      const float kf = (float)k, r1 = (float)(r + 1u);
      A[r * K + k] = to_f16(0.9f * std::sin(0.1f * r1 + 0.7f * kf) * std::cos(0.05f * (kf + 1.0f)));
      B[r * K + k] = to_f16(0.8f * std::cos(0.13f * r1 + 0.11f * kf) *
                            std::sin(0.03f * ((float)((uint64_t)r + k) + 1.0f)));
    }
}

// Counter-based generator: value i of tensor t under seed s depends only on (s, t, i).
uint64_t mix64(uint64_t z) {
  z += 0x9e3779b97f4a7c15ull;
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
  z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
  return z ^ (z >> 31);
}
double unit_uniform(uint64_t seed, uint64_t tensor, uint64_t i, uint64_t lane) {
  const uint64_t h = mix64(mix64(seed ^ (tensor << 56)) + 2 * i + lane);
  return ((double)(h >> 11) + 0.5) * (1.0 / 9007199254740992.0);  // (0, 1)
}
float draw(const std::string& dist, bool is_b, uint64_t seed, uint64_t i) {
  const uint64_t t = is_b ? 2 : 1;
  if (dist == "uniform") return (float)(2.0 * unit_uniform(seed, t, i, 0) - 1.0);
  const double u1 = unit_uniform(seed, t, i, 0), u2 = unit_uniform(seed, t, i, 1);
  const double n = std::sqrt(-2.0 * std::log(u1)) * std::cos(6.283185307179586 * u2);
  double sd = 1.0;
  if (dist == "normal01") sd = 0.1;
  if (dist == "llm" && is_b) sd = 0.02;
  return (float)(n * sd);
}

// ---- CPU reference (double accumulate, k ascending; gemm_check.cpp:165-178 generalised)
void reference_rows(const std::vector<float>& A, const std::vector<float>& B, int64_t N, int64_t K,
                    const std::vector<int64_t>& rows, std::vector<double>& C) {
  const unsigned nt = std::max(1u, std::thread::hardware_concurrency());
  std::vector<std::thread> pool;
  for (unsigned t = 0; t < nt; ++t)
    pool.emplace_back([&, t] {
      for (size_t i = t; i < rows.size(); i += nt) {
        const float* a = &A[(size_t)rows[i] * K];
        for (int64_t n = 0; n < N; ++n) {
          const float* b = &B[(size_t)n * K];
          double acc = 0.0;
          for (int64_t k = 0; k < K; ++k) acc += (double)a[k] * (double)b[k];
          C[i * (size_t)N + n] = acc;
        }
      }
    });
  for (auto& th : pool) th.join();
}

struct Options {
  int64_t m = 128, n = 128, k = 128;
  std::string dtype = "f16", dist = "closed_form";
  int cta = 0, block_n = 0, iters = 0, splitk = 0, gpus = 1;
  bool allgather = false;
  int64_t check_rows = 0;
  uint64_t seed = 0x5EED;
  float alpha = 1.0f;
  bool legacy = false;
  std::string kernel_name = "patina_gemm";
};

// ---- several GPUs: N-column shards, one host thread per GPU ---------------------------------
// Shards are contiguous, in whole 256-column tiles while columns last (the same split the
// Python side uses), so every listed projection width divides evenly over 2, 4 and 8 GPUs.
void column_shard(int64_t n, int world, int rank, int64_t* n0, int64_t* n1) {
  const int64_t blocks = (n + 255) / 256, per = (blocks + world - 1) / world;
  *n0 = std::min<int64_t>(n, (int64_t)rank * per * 256);
  *n1 = std::min<int64_t>(n, (int64_t)(rank + 1) * per * 256);
}

// A reusable barrier for the per-GPU host threads.
struct HostBarrier {
  std::mutex mu;
  std::condition_variable cv;
  int count, waiting = 0;
  uint64_t generation = 0;
  explicit HostBarrier(int n) : count(n) {}
  void wait() {
    std::unique_lock<std::mutex> lk(mu);
    const uint64_t gen = generation;
    if (++waiting == count) {
      waiting = 0;
      ++generation;
      cv.notify_all();
    } else {
      cv.wait(lk, [&] { return generation != gen; });
    }
  }
};

int run_sharded(const Options& o) {
  const int G = o.gpus;
  const int64_t M = o.m, N = o.n, K = o.k;
  const int64_t ldk = (K + 7) / 8 * 8, ldn = (N + 7) / 8 * 8;
  std::vector<float> Af((size_t)M * K), Bf((size_t)N * K);
  std::vector<uint16_t> Ab((size_t)M * ldk, 0), Bb((size_t)N * ldk, 0);
  for (size_t i = 0; i < Af.size(); ++i) Af[i] = draw(o.dist, false, o.seed, i);
  for (size_t i = 0; i < Bf.size(); ++i) Bf[i] = draw(o.dist, true, o.seed, i);
  for (int64_t r = 0; r < M; ++r)
    for (int64_t k = 0; k < K; ++k) {
      const uint16_t q = to_bf16(Af[(size_t)r * K + k]);
      Ab[(size_t)r * ldk + k] = q;
      Af[(size_t)r * K + k] = from_bf16(q);
    }
  for (int64_t r = 0; r < N; ++r)
    for (int64_t k = 0; k < K; ++k) {
      const uint16_t q = to_bf16(Bf[(size_t)r * K + k]);
      Bb[(size_t)r * ldk + k] = q;
      Bf[(size_t)r * K + k] = from_bf16(q);
    }
  std::vector<int64_t> rows;
  int64_t want_rows = o.check_rows > 0 ? o.check_rows : ((double)M * N * K <= 9e9 ? M : 64);
  want_rows = std::min(want_rows, M);
  for (int64_t i = 0; i < want_rows; ++i)
    rows.push_back(want_rows == M ? i : (i * (M - 1)) / std::max<int64_t>(1, want_rows - 1));
  std::vector<double> Cref(rows.size() * (size_t)N);
  reference_rows(Af, Bf, N, K, rows, Cref);

  struct Dev {
    PatinaGemmContext* ctx = nullptr;
    void *dA = nullptr, *dB = nullptr, *dC = nullptr;   // dC: the shard [M, ldn_shard], or with
    int64_t n0 = 0, n1 = 0, ldc = 0;                    // --allgather the whole C [M, ldn]
    std::vector<uint16_t> C;
    double device_us = 0, wall_us = 0;
    std::string error;
  };
  std::vector<Dev> dev(G);
  HostBarrier bar(G);
  std::chrono::steady_clock::time_point t_start;
  std::mutex start_mu;
  auto worker = [&](int g) {
    Dev& d = dev[g];
    auto fail = [&](const std::string& what) { if (d.error.empty()) d.error = what; };
    auto rt = [&](cudaError_t e, const char* what) {
      if (e != cudaSuccess) fail(std::string(what) + ": " + cudaGetErrorString(e));
      return e == cudaSuccess;
    };
    column_shard(N, G, g, &d.n0, &d.n1);
    const int64_t nw = d.n1 - d.n0;
    d.ldc = o.allgather ? ldn : (nw + 7) / 8 * 8;
    bool ok = rt(cudaSetDevice(g), "cudaSetDevice");
    if (ok && patina_gemm_context_create(g, &d.ctx) != PATINA_GEMM_OK) { fail("patina_gemm_context_create"); ok = false; }
    if (ok && o.allgather)
      for (int p = 0; p < G; ++p)
        if (p != g) {
          const cudaError_t e = cudaDeviceEnablePeerAccess(p, 0);
          if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) fail("cudaDeviceEnablePeerAccess");
          cudaGetLastError();
        }
    const size_t c_bytes = (size_t)M * std::max<int64_t>(d.ldc, 8) * 2;
    ok = ok && rt(cudaMalloc(&d.dA, Ab.size() * 2), "cudaMalloc(A)") &&
         rt(cudaMalloc(&d.dB, std::max<size_t>((size_t)nw * ldk * 2, 16)), "cudaMalloc(B)") &&
         rt(cudaMalloc(&d.dC, c_bytes), "cudaMalloc(C)") && rt(cudaMemset(d.dC, 0, c_bytes), "cudaMemset(C)") &&
         rt(cudaMemcpy(d.dA, Ab.data(), Ab.size() * 2, cudaMemcpyHostToDevice), "cudaMemcpy(A)");
    if (ok && nw > 0)
      ok = rt(cudaMemcpy(d.dB, &Bb[(size_t)d.n0 * ldk], (size_t)nw * ldk * 2, cudaMemcpyHostToDevice), "cudaMemcpy(B)");
    if (!ok) fail("set-up");
    bar.wait();                                   // every GPU's buffers exist from here on
    // destinations of this GPU's column block: its own C first, then (--allgather) every peer's
    std::vector<void*> dests;
    if (o.allgather) {
      dests.push_back(static_cast<char*>(d.dC) + 2 * d.n0);
      for (int p = 0; p < G; ++p)
        if (p != g) dests.push_back(static_cast<char*>(dev[p].dC) + 2 * d.n0);
    }
    auto launch = [&]() -> int {
      if (nw == 0 || !d.error.empty()) return PATINA_GEMM_OK;
      if (o.allgather)
        return patina_gemm_bf16_tn_scatter(d.ctx, d.dA, ldk, d.dB, ldk, dests.data(), (int)dests.size(), d.ldc, M, nw,
                                           K, o.alpha, nullptr);
      return patina_gemm_bf16_tn(d.ctx, d.dA, ldk, d.dB, ldk, d.dC, d.ldc, M, nw, K, o.alpha, nullptr);
    };
    auto run_checked = [&](const char* what) {
      int rc = launch();
      if (rc == PATINA_GEMM_OK && d.ctx) rc = patina_gemm_status(d.ctx, nullptr);
      if (rc != PATINA_GEMM_OK) {
        char* msg = d.ctx ? patina_gemm_last_error(d.ctx) : nullptr;
        fail(std::string(what) + ": " + (msg ? msg : "?"));
        patina_gemm_string_free(msg);
      }
    };
    run_checked("first launch");
    bar.wait();                                   // every block of every C has been written
    if (d.error.empty()) {
      d.C.resize((size_t)M * d.ldc);
      rt(cudaMemcpy(d.C.data(), d.dC, d.C.size() * 2, cudaMemcpyDeviceToHost), "cudaMemcpy(C)");
    }
    if (o.iters > 0) {
      cudaEvent_t e0 = nullptr, e1 = nullptr;
      cudaEventCreate(&e0);
      cudaEventCreate(&e1);
      for (int i = 0; i < 3; ++i) run_checked("warm-up");
      double best_dev = 1e30, best_wall = 1e30;
      for (int i = 0; i < o.iters; ++i) {
        bar.wait();
        if (g == 0) { std::lock_guard<std::mutex> lk(start_mu); t_start = std::chrono::steady_clock::now(); }
        bar.wait();                               // common host time stamp taken
        cudaEventRecord(e0, nullptr);
        launch();
        cudaEventRecord(e1, nullptr);
        cudaEventSynchronize(e1);
        const auto t1 = std::chrono::steady_clock::now();
        float ms = 0;
        cudaEventElapsedTime(&ms, e0, e1);
        best_dev = std::min(best_dev, (double)ms * 1e3);
        best_wall = std::min(best_wall, std::chrono::duration<double, std::micro>(t1 - t_start).count());
      }
      run_checked("timed launches");
      d.device_us = best_dev;
      d.wall_us = best_wall;
      cudaEventDestroy(e0);
      cudaEventDestroy(e1);
    }
    bar.wait();                                   // nobody still writes into anybody's C
    cudaFree(d.dA);
    cudaFree(d.dB);
    cudaFree(d.dC);
    if (d.ctx) patina_gemm_context_destroy(d.ctx);
  };
  std::vector<std::thread> pool;
  for (int g = 0; g < G; ++g) pool.emplace_back(worker, g);
  for (auto& t : pool) t.join();
  for (int g = 0; g < G; ++g)
    if (!dev[g].error.empty()) {
      std::fprintf(stderr, "GPU %d: %s\n", g, dev[g].error.c_str());
      return kExitError;
    }

  // every GPU's result against the CPU reference: its shard, or with --allgather the whole C
  double max_abs = 0, max_ref = 0, se = 0, sr = 0, sum = 0;
  uint64_t checked = 0;
  for (int g = 0; g < G; ++g) {
    const Dev& d = dev[g];
    const int64_t c0 = o.allgather ? 0 : d.n0, c1 = o.allgather ? N : d.n1;
    for (size_t i = 0; i < rows.size(); ++i)
      for (int64_t n = c0; n < c1; ++n) {
        const double ref = from_bf16(to_bf16((float)((double)o.alpha * Cref[i * (size_t)N + n])));
        const double got = from_bf16(d.C[(size_t)rows[i] * d.ldc + (o.allgather ? n : n - d.n0)]);
        const double abs_err = std::fabs(got - ref);
        if (g == 0 || !o.allgather) sum += got;
        max_abs = std::max(max_abs, abs_err);
        max_ref = std::max(max_ref, std::fabs(ref));
        se += abs_err * abs_err;
        sr += ref * ref;
        ++checked;
      }
  }
  const double fro = sr > 0 ? std::sqrt(se / sr) : 0.0;
  const bool pass = max_abs <= 1e-2 * max_ref && fro <= 1e-3 && checked > 0;
  std::printf("kernel: patina_gemm bf16  M=%lld N=%lld K=%lld  gpus=%d  shard_columns=%lld%s\n", (long long)M,
              (long long)N, (long long)K, G, (long long)(dev[0].n1 - dev[0].n0),
              o.allgather ? "  allgather=fused (peer stores)" : "");
  std::printf("max abs err: %.6e   fro rel err: %.6e   max|ref|: %.6e\n", max_abs, fro, max_ref);
  std::printf("elements checked: %llu (%zu rows on every GPU)\n", (unsigned long long)checked, rows.size());
  std::printf("sum(C):      %.9e\n", sum);
  if (o.iters > 0) {
    double dev_us = 0, wall_us = 0;
    for (const Dev& d : dev) { dev_us = std::max(dev_us, d.device_us); wall_us = std::max(wall_us, d.wall_us); }
    const double tflops = 2.0 * M * N * K / (dev_us * 1e-6) / 1e12;
    std::printf("time_us:     %.2f on the slowest GPU (CUDA events, best of %d); %.2f from a common host time stamp "
                "to the last GPU's completion\n", dev_us, o.iters, wall_us);
    std::printf("tflops:      %.1f aggregate   per_gpu: %.1f   pct_peak: %.1f (of 2250 nominal dense per GPU)\n", tflops,
                tflops / G, 100.0 * tflops / G / 2250.0);
  }
  std::printf("%s\n", pass ? "PASS" : "FAIL");
  return pass ? kExitPass : kExitFail;
}

int usage(const char* argv0) {
  std::fprintf(stderr,
               "usage: %s <ptx_file> <kernel_name> <K>\n"
               "  kernel_name: tcgen05_gemm_v1 (K=32) | tcgen05_gemm_v2 (K multiple of 32)\n"
               "   or: %s --m M --n N --k K [--dtype bf16|fp8|f16] [--cta 1|2] [--block-n 128|256]\n"
               "          [--dist uniform|normal01|llm] [--seed S] [--alpha X] [--iters I] [--check-rows R]\n"
               "          [--splitk -1|1|2|3] [--gpus G] [--allgather]\n",
               argv0, argv0);
  return kExitError;
}

}  // namespace

int main(int argc, char** argv) {
  Options o;
  if (argc == 4 && argv[1][0] != '-') {
    o.legacy = true;
    o.kernel_name = argv[2];
    o.k = (int64_t)std::strtoull(argv[3], nullptr, 10);
    if (o.kernel_name == "tcgen05_gemm_v1") {
      if (o.k != 32) {
        std::fprintf(stderr, "tcgen05_gemm_v1 requires K=32 (got %lld)\n", (long long)o.k);
        return kExitError;
      }
    } else if (o.kernel_name == "tcgen05_gemm_v2") {
      if (o.k % 32 != 0 || o.k == 0) {
        std::fprintf(stderr, "tcgen05_gemm_v2 requires K a multiple of 32 (got %lld)\n", (long long)o.k);
        return kExitError;
      }
    } else {
      std::fprintf(stderr, "unknown kernel '%s'\n", argv[2]);
      return kExitError;
    }
  } else {
    if (argc < 2) return usage(argv[0]);
    o.dtype = "bf16";
    o.dist = "uniform";
    for (int i = 1; i < argc; ++i) {
      std::string a = argv[i];
      auto val = [&]() -> const char* { return (i + 1 < argc) ? argv[++i] : ""; };
      if (a == "--m") o.m = std::atoll(val());
      else if (a == "--n") o.n = std::atoll(val());
      else if (a == "--k") o.k = std::atoll(val());
      else if (a == "--dtype") o.dtype = val();
      else if (a == "--dist") o.dist = val();
      else if (a == "--cta") o.cta = std::atoi(val());
      else if (a == "--block-n") o.block_n = std::atoi(val());
      else if (a == "--iters") o.iters = std::atoi(val());
      else if (a == "--check-rows") o.check_rows = std::atoll(val());
      else if (a == "--seed") o.seed = std::strtoull(val(), nullptr, 0);
      else if (a == "--alpha") o.alpha = (float)std::atof(val());
      else if (a == "--splitk") o.splitk = std::atoi(val());
      else if (a == "--gpus") o.gpus = std::atoi(val());
      else if (a == "--allgather") o.allgather = true;
      else return usage(argv[0]);
    }
    if (o.m <= 0 || o.n <= 0 || o.k <= 0) return usage(argv[0]);
    if (o.dtype != "bf16" && o.dtype != "fp8" && o.dtype != "f16") return usage(argv[0]);
    if (o.dist != "uniform" && o.dist != "normal01" && o.dist != "llm") return usage(argv[0]);
    if (o.gpus < 1 || o.gpus > 8 || o.splitk < -1 || o.splitk > 3) return usage(argv[0]);
    if ((o.gpus > 1 || o.allgather) && o.dtype != "bf16") {
      std::fprintf(stderr, "--gpus / --allgather take bf16 problems\n");
      return kExitError;
    }
  }

  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) {
    std::fprintf(stderr, "no CUDA device: tcgen05 needs sm_100a (Blackwell); there is no CPU path\n");
    return kExitNotSm100;
  }
  cudaDeviceProp prop;
  RT_CHECK(cudaGetDeviceProperties(&prop, 0));
  std::printf("device: %s (sm_%d%d)\n", prop.name, prop.major, prop.minor);
  if (o.gpus > 1 || o.allgather) {
    if (prop.major != 10) {
      std::fprintf(stderr, "device is sm_%d%d, but tcgen05 needs sm_100a (Blackwell). This GPU cannot run it.\n",
                   prop.major, prop.minor);
      return kExitNotSm100;
    }
    if (o.gpus > ndev) {
      std::fprintf(stderr, "--gpus %d, but only %d device(s) are visible\n", o.gpus, ndev);
      return kExitError;
    }
    return run_sharded(o);
  }
  PatinaGemmContext* ctx = nullptr;
  int rc = patina_gemm_context_create(0, &ctx);
  if (rc == PATINA_GEMM_ERR_UNSUPPORTED_ARCH) {
    std::fprintf(stderr, "device is sm_%d%d, but tcgen05 needs sm_100a (Blackwell). This GPU cannot run it.\n",
                 prop.major, prop.minor);
    return kExitNotSm100;
  }
  if (rc != PATINA_GEMM_OK) {
    std::fprintf(stderr, "patina_gemm_context_create failed (%d)\n", rc);
    return kExitError;
  }

  const int64_t M = o.m, N = o.n, K = o.k;
  const bool fp8 = o.dtype == "fp8", f16 = o.dtype == "f16";
  const int in_type = fp8 ? PATINA_IN_E4M3 : (f16 ? PATINA_IN_F16 : PATINA_IN_BF16);
  const int out_type = f16 ? PATINA_OUT_F32 : PATINA_OUT_BF16;
  const size_t ib = fp8 ? 1 : 2, ob = f16 ? 4 : 2;
  // pitches rounded up to 16 bytes
  const int64_t ldk = (int64_t)(((size_t)K * ib + 15) / 16 * 16 / ib);
  const int64_t ldc = (int64_t)(((size_t)N * ob + 15) / 16 * 16 / ob);

  // host operands: exact float images (for the check) and storage bytes (for the device)
  std::vector<float> Af((size_t)M * K), Bf((size_t)N * K);
  std::vector<uint8_t> Ab((size_t)M * ldk * ib, 0), Bb((size_t)N * ldk * ib, 0);
  float scale_a = 1.0f, scale_b = 1.0f;
  if (o.legacy) {
    std::vector<uint16_t> A16((size_t)M * K), B16((size_t)N * K);
    fill_closed_form(A16, B16, 128, (uint64_t)K);
    for (size_t i = 0; i < A16.size(); ++i) { Af[i] = from_f16(A16[i]); Bf[i] = from_f16(B16[i]); }
  } else {
    for (size_t i = 0; i < Af.size(); ++i) Af[i] = draw(o.dist, false, o.seed, i);
    for (size_t i = 0; i < Bf.size(); ++i) Bf[i] = draw(o.dist, true, o.seed, i);
    if (fp8) {  // per-tensor scale = amax / 448
      float amax = 0, bmax = 0;
      for (float v : Af) amax = std::max(amax, std::fabs(v));
      for (float v : Bf) bmax = std::max(bmax, std::fabs(v));
      scale_a = amax > 0 ? amax / 448.0f : 1.0f;
      scale_b = bmax > 0 ? bmax / 448.0f : 1.0f;
    }
  }
  auto store = [&](std::vector<float>& F, std::vector<uint8_t>& S, int64_t rows, float scale) {
    for (int64_t r = 0; r < rows; ++r)
      for (int64_t k = 0; k < K; ++k) {
        float& v = F[(size_t)r * K + k];
        uint8_t* dst = &S[((size_t)r * ldk + k) * ib];
        if (fp8) { uint8_t q = to_e4m3(v / scale); *dst = q; v = from_e4m3(q); }
        else if (f16) { uint16_t q = to_f16(v); std::memcpy(dst, &q, 2); v = from_f16(q); }
        else { uint16_t q = to_bf16(v); std::memcpy(dst, &q, 2); v = from_bf16(q); }
      }
  };
  store(Af, Ab, M, scale_a);
  store(Bf, Bb, N, scale_b);
  const float alpha = fp8 ? scale_a * scale_b * o.alpha : o.alpha;

  void *dA = nullptr, *dB = nullptr, *dC = nullptr;
  RT_CHECK(cudaMalloc(&dA, Ab.size()));
  RT_CHECK(cudaMalloc(&dB, Bb.size()));
  RT_CHECK(cudaMalloc(&dC, (size_t)M * ldc * ob));
  RT_CHECK(cudaMemset(dC, 0, (size_t)M * ldc * ob));
  RT_CHECK(cudaMemcpy(dA, Ab.data(), Ab.size(), cudaMemcpyHostToDevice));
  RT_CHECK(cudaMemcpy(dB, Bb.data(), Bb.size(), cudaMemcpyHostToDevice));

  PatinaGemmConfig cfg{};
  cfg.cta_group = o.cta;
  cfg.block_n = o.block_n;
  cfg.stream_k = o.splitk;
  PatinaGemmPlan plan{};
  patina_gemm_plan(in_type, out_type, M, N, K, &cfg, prop.multiProcessorCount, &plan);
  auto launch = [&]() {
    return patina_gemm_ex(ctx, in_type, out_type, dA, ldk, dB, ldk, dC, ldc, M, N, K, alpha, &cfg, nullptr);
  };
  auto die_on = [&](int code, const char* what) {
    if (code == PATINA_GEMM_OK) return;
    char* msg = patina_gemm_last_error(ctx);
    std::fprintf(stderr, "%s failed (%d): %s\n", what, code, msg ? msg : "?");
    patina_gemm_string_free(msg);
    std::exit(kExitError);
  };
  die_on(launch(), "patina_gemm_ex");
  die_on(patina_gemm_status(ctx, nullptr), "patina_gemm_status");

  std::vector<uint8_t> Cb((size_t)M * ldc * ob);
  RT_CHECK(cudaMemcpy(Cb.data(), dC, Cb.size(), cudaMemcpyDeviceToHost));

  // rows to verify: all of them for small problems, a spread sample otherwise
  std::vector<int64_t> rows;
  int64_t want_rows = o.check_rows > 0 ? o.check_rows : ((double)M * N * K <= 9e9 ? M : 64);
  want_rows = std::min(want_rows, M);
  for (int64_t i = 0; i < want_rows; ++i) rows.push_back(want_rows == M ? i : (i * (M - 1)) / std::max<int64_t>(1, want_rows - 1));
  std::vector<double> Cref(rows.size() * (size_t)N);
  reference_rows(Af, Bf, N, K, rows, Cref);

  double max_abs = 0, max_rel = 0, sum = 0, max_ref = 0, se = 0, sr = 0;
  uint64_t mismatches = 0;
  for (size_t i = 0; i < rows.size(); ++i)
    for (int64_t n = 0; n < N; ++n) {
      double got, ref = (double)alpha * Cref[i * (size_t)N + n];
      const uint8_t* src = &Cb[((size_t)rows[i] * ldc + n) * ob];
      if (f16) { float v; std::memcpy(&v, src, 4); got = v; }
      else { uint16_t h; std::memcpy(&h, src, 2); got = from_bf16(h); ref = from_bf16(to_bf16((float)ref)); }
      sum += got;
      const double abs_err = std::fabs(got - ref), rel_err = abs_err / std::fmax(1.0, std::fabs(ref));
      max_abs = std::max(max_abs, abs_err);
      max_rel = std::max(max_rel, rel_err);
      max_ref = std::max(max_ref, std::fabs(ref));
      se += abs_err * abs_err;
      sr += ref * ref;
      if ((abs_err > 1e-3 && rel_err > 1e-3) || got != got) ++mismatches;
    }
  const double fro = sr > 0 ? std::sqrt(se / sr) : 0.0;
  bool pass;
  if (f16) pass = mismatches == 0;                              // the reference's rule
  else pass = max_abs <= 1e-2 * max_ref && fro <= 1e-3;         // max-norm + Frobenius rule

  if (o.legacy)
    std::printf("kernel: %s  K=%llu  k_tiles=%u  block=%u  dyn_smem=%zu\n", o.kernel_name.c_str(),
                (unsigned long long)K, (unsigned)(K / 32), plan.block, (size_t)plan.smem_bytes);
  else
    std::printf("kernel: %s %s  M=%lld N=%lld K=%lld  cta_group=%d block_n=%d stages=%d grid=%u block=%u dyn_smem=%u\n",
                o.kernel_name.c_str(), o.dtype.c_str(), (long long)M, (long long)N, (long long)K,
                plan.cta_group, plan.block_n, plan.stages, plan.grid, plan.block, plan.smem_bytes);
  std::printf("max abs err: %.6e   max rel err: %.6e\n", max_abs, max_rel);
  std::printf("mismatches:  %llu / %llu\n", (unsigned long long)mismatches,
              (unsigned long long)(rows.size() * (size_t)N));
  std::printf("sum(C):      %.9e\n", sum);
  if (!f16) std::printf("fro rel err: %.6e   max|ref|: %.6e   rows checked: %zu of %lld\n", fro, max_ref, rows.size(), (long long)M);

  if (o.iters > 0) {
    cudaEvent_t e0, e1;
    RT_CHECK(cudaEventCreate(&e0));
    RT_CHECK(cudaEventCreate(&e1));
    for (int i = 0; i < 3; ++i) die_on(launch(), "warm-up");
    float best = 1e30f;
    for (int i = 0; i < o.iters; ++i) {
      RT_CHECK(cudaEventRecord(e0, nullptr));
      die_on(launch(), "timed launch");
      RT_CHECK(cudaEventRecord(e1, nullptr));
      RT_CHECK(cudaEventSynchronize(e1));
      float ms = 0;
      RT_CHECK(cudaEventElapsedTime(&ms, e0, e1));
      best = std::min(best, ms);
    }
    die_on(patina_gemm_status(ctx, nullptr), "patina_gemm_status");
    const double tflops = 2.0 * M * N * K / (best * 1e-3) / 1e12;
    const double peak = fp8 ? 4500.0 : 2250.0;
    std::printf("time_us:     %.2f (best of %d)\n", best * 1e3, o.iters);
    std::printf("tflops:      %.1f   pct_peak: %.1f (of %.0f nominal dense)\n", tflops, 100.0 * tflops / peak, peak);
  }
  std::printf("%s\n", pass ? "PASS" : "FAIL");

  cudaFree(dA);
  cudaFree(dB);
  cudaFree(dC);
  patina_gemm_context_destroy(ctx);
  return pass ? kExitPass : kExitFail;
}
