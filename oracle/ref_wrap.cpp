// ref_wrap.cpp -- exports the reference's OWN CPU functions for the GEMM check.
//
// TEST INFRASTRUCTURE ONLY. This translation unit #includes the reference's
// harness source (harness/gemm_check.cpp of neoming/Patina) from where it lies
// (the path arrives as -DPATINA_REF_SRC=...; nothing of it is copied here) and
// re-exports its file-static helpers -- f16_to_f32, f32_to_f16, fill_inputs,
// reference_gemm -- behind a C ABI, so that the CPU restatement in
// patina_oracle.c can be pinned against the real thing and the benchmark can
// time the reference's CPU GEMM itself.
//
// The reference's main() is renamed and never called. Its CUDA driver calls
// are only reachable from that main(), so the handful of cu* symbols it names
// are satisfied by inert definitions below instead of libcuda; the resulting
// library loads on machines without a GPU driver.
#include <cuda.h>

#define main patina_reference_harness_main
#include PATINA_REF_SRC
#undef main

#define PATINA_INERT(name, ...) \
  extern "C" CUresult name(__VA_ARGS__) { return CUDA_ERROR_NOT_INITIALIZED; }

PATINA_INERT(cuInit, unsigned int)
PATINA_INERT(cuDeviceGet, CUdevice*, int)
PATINA_INERT(cuDeviceGetAttribute, int*, CUdevice_attribute, CUdevice)
PATINA_INERT(cuDeviceGetName, char*, int, CUdevice)
PATINA_INERT(cuCtxCreate, CUcontext*, unsigned int, CUdevice)
PATINA_INERT(cuCtxDestroy, CUcontext)
PATINA_INERT(cuModuleLoadDataEx, CUmodule*, const void*, unsigned int, CUjit_option*, void**)
PATINA_INERT(cuModuleGetFunction, CUfunction*, CUmodule, const char*)
PATINA_INERT(cuModuleUnload, CUmodule)
PATINA_INERT(cuMemAlloc, CUdeviceptr*, size_t)
PATINA_INERT(cuMemFree, CUdeviceptr)
PATINA_INERT(cuMemsetD8, CUdeviceptr, unsigned char, size_t)
PATINA_INERT(cuMemcpyHtoD, CUdeviceptr, const void*, size_t)
PATINA_INERT(cuMemcpyDtoH, void*, CUdeviceptr, size_t)
PATINA_INERT(cuStreamCreate, CUstream*, unsigned int)
PATINA_INERT(cuStreamSynchronize, CUstream)
PATINA_INERT(cuLaunchKernel, CUfunction, unsigned int, unsigned int, unsigned int, unsigned int,
             unsigned int, unsigned int, unsigned int, CUstream, void**, void**)
PATINA_INERT(cuGetErrorName, CUresult, const char**)
PATINA_INERT(cuGetErrorString, CUresult, const char**)
PATINA_INERT(cuTensorMapEncodeTiled, CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
             const cuuint64_t*, const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
             CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
             CUtensorMapFloatOOBfill)

extern "C" {
// The reference's tile extents (harness/gemm_check.cpp:58-59).
uint32_t patina_ref_rows(void) { return M; }
uint32_t patina_ref_cols(void) { return N; }
float patina_ref_f16_to_f32(uint16_t h) { return f16_to_f32(h); }
uint16_t patina_ref_f32_to_f16(float x) { return f32_to_f16(x); }
// A, B: [128, K] f16 bits (harness/gemm_check.cpp:152-163).
void patina_ref_fill_inputs(uint16_t* A, uint16_t* B, uint64_t K) { fill_inputs(A, B, K); }
// C_ref: [128, 128] double (harness/gemm_check.cpp:165-178).
void patina_ref_reference_gemm(const uint16_t* A, const uint16_t* B, uint64_t K, double* C_ref) {
  reference_gemm(A, B, K, C_ref);
}
}
