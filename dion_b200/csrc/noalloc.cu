// Allocation-free variant of the batched Cholesky-inverse (see noalloc.h for the contract).
#include "noalloc.h"

#include <stdio.h>

#include <mutex>
#include <string>

#include "kernels.h"

namespace {

// Scratch of the factorisation (one r x r working copy per matrix).  Part of the library
// image: every GPU that loads the library holds these 8 MiB until the process exits.
static __device__ __align__(256) float g_noalloc_scratch[kDionNoAllocScratchFloats];

constexpr int kMaxDevices = 64;
float* g_scratch_addr[kMaxDevices] = {nullptr};
std::mutex g_setup_mutex;
thread_local std::string g_error;

// In host code the array's name is only a stand-in; the kernel needs the device address,
// which differs per device and is looked up once per device with that device current.
cudaError_t scratch_for_current_device(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_addr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_scratch);
    if (e != cudaSuccess) return e;
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return cudaSuccess;
}

}  // namespace

extern "C" const char* dion_noalloc_last_error(void) { return g_error.c_str(); }

extern "C" int dion_chol_inverse_noalloc(const float* G, float* Z, int* info, int batch, int r, long long ldg,
                                         long long g_batch_stride, float pivot_floor, cudaStream_t stream) {
  g_error.clear();
  char buf[256];
  if (G == nullptr || Z == nullptr || batch < 0 || r < 0 || ldg < r) {
    g_error = "dion_chol_inverse_noalloc: null pointer or negative / inconsistent size";
    return 1;
  }
  if (batch == 0 || r == 0) return 0;
  const long long need = (long long)batch * r * r;
  if (need > (long long)kDionNoAllocScratchFloats) {
    snprintf(buf, sizeof(buf),
             "dion_chol_inverse_noalloc: batch * r * r = %lld floats exceeds the built-in scratch of %d floats "
             "(batch %d, r %d); use the allocating entry point or split the batch",
             need, (int)kDionNoAllocScratchFloats, batch, r);
    g_error = buf;
    return 1;
  }
  float* scratch = nullptr;
  cudaError_t e = scratch_for_current_device(&scratch);
  if (e != cudaSuccess) {
    snprintf(buf, sizeof(buf), "dion_chol_inverse_noalloc: scratch set-up failed: %s", cudaGetErrorString(e));
    g_error = buf;
    return 2;
  }
  // The kernel writes every element of the working copy it later reads, so stale contents
  // of the shared scratch do not matter.
  e = dion::chol_inverse_launch(G, Z, scratch, info, batch, r, ldg, g_batch_stride, pivot_floor, stream);
  if (e == cudaErrorNotSupported) {  // the launcher's own size check, nothing was launched
    snprintf(buf, sizeof(buf), "dion_chol_inverse_noalloc: rank %d is larger than the kernel supports", r);
    g_error = buf;
    return 1;
  }
  if (e != cudaSuccess) {
    snprintf(buf, sizeof(buf), "dion_chol_inverse_noalloc: launch failed: %s", cudaGetErrorString(e));
    g_error = buf;
    return 2;
  }
  return 0;
}
