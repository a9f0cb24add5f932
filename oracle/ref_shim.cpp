// C-linkage shim over the reference's own CPU GEMM, compiled together with the reference source
// file core/src/cpu_kernels.cpp taken from the mounted reference tree (never copied into this
// repository).  Test / benchmark infrastructure only.
#include <zenith/kernels.hpp>

extern "C" void ref_matmul_f32_avx2(const float* A, const float* B, float* C, int M, int N, int K) {
  // core/src/cpu_kernels.cpp:129-165; called directly because the dispatcher in matmul_f32
  // mis-detects AVX2 (cpuid leaf 7 without sub-leaf 0, core/src/cpu_kernels.cpp:33-35).
  zenith::kernels::matmul_f32_avx2(A, B, C, M, N, K);
}
extern "C" void ref_matmul_f32_naive(const float* A, const float* B, float* C, int M, int N, int K) {
  zenith::kernels::matmul_f32_naive(A, B, C, M, N, K);
}
