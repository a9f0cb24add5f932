// Device status word: folds the per-translation-unit words together for the host.
#include "zen_common.cuh"

extern "C" {
int zen_tu_status_gemm(int* out, int clear);
int zen_tu_status_rowwise(int* out, int clear);
int zen_tu_status_flash_attn(int* out, int clear);
int zen_tu_status_gemm_ln(int* out, int clear);
int zen_tu_status_selftest(int* out, int clear);
}

typedef int (*TuStatusFn)(int*, int);
static const TuStatusFn kTuStatus[] = {zen_tu_status_gemm, zen_tu_status_rowwise, zen_tu_status_flash_attn,
                                        zen_tu_status_gemm_ln, zen_tu_status_selftest};

static int fold_status(int* out, int clear) {
  if (cudaDeviceSynchronize() != cudaSuccess) {
    cudaGetLastError();
    return ZEN_ERR_LAUNCH;
  }
  int first = 0;
  for (TuStatusFn fn : kTuStatus) {
    int v = 0;
    const int st = fn(&v, clear);
    if (st != ZEN_OK) return st;
    if (first == 0) first = v;
  }
  if (out) *out = first;
  return ZEN_OK;
}

extern "C" int zen_device_status_read(int* status_host) {
  if (!status_host) return ZEN_ERR_INVALID_ARG;
  return fold_status(status_host, 0);
}

extern "C" int zen_device_status_clear(void) { return fold_status(nullptr, 1); }

// Copy-engine copy between any two ranges the calling process can address: device memory of the current or of a
// peer GPU (a CUDA IPC mapping included) and pinned host memory.  Stream-ordered, no kernel is launched.
extern "C" int zen_memcpy_async(void* dst, const void* src, size_t bytes, void* stream) {
  if (bytes == 0) return ZEN_OK;
  if (!dst || !src) return ZEN_ERR_INVALID_ARG;
  if (cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, static_cast<cudaStream_t>(stream)) != cudaSuccess) {
    cudaGetLastError();
    return ZEN_ERR_LAUNCH;
  }
  return ZEN_OK;
}
