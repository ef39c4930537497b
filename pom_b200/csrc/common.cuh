// Host-side helpers shared by the translation units of libpom_b200.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <atomic>
#include <mutex>
#include <stdint.h>
#include "../../include/pom_b200.h"

namespace pomh {

extern std::atomic<long long> g_launches;

inline void count_launch(int n = 1) { g_launches.fetch_add(n, std::memory_order_relaxed); }

inline int check_launch() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? POM_OK : POM_ERR_CUDA;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline int sm_count() {
  static int cached = 0;
  if (cached == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return 148;
    cached = n;
  }
  return cached;
}

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Runs `f` (returning POM_OK or an error) once per device of this process: attributes of a kernel function
// (the opt-in to more than 48 KB of dynamic shared memory) belong to the device that is current when they are set.
// `done` holds one bit per device ordinal; beyond 64 devices, or when the current device cannot be read, `f` runs
// on every call.
template <class F>
inline int once_per_device(std::atomic<uint64_t>& done, F&& f) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return f();
  const uint64_t bit = 1ull << dev;
  if (done.load(std::memory_order_acquire) & bit) return POM_OK;
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  if (done.load(std::memory_order_relaxed) & bit) return POM_OK;
  const int rc = f();
  if (rc == POM_OK) done.fetch_or(bit, std::memory_order_release);
  return rc;
}

// Launch with programmatic stream serialization: the kernel may become resident while its predecessor in the stream
// drains.  Only for kernels that execute griddepcontrol.wait (pomk::griddep_wait) before they touch memory the
// predecessor may have written.
template <class Kern, class... Args>
inline cudaError_t launch_pdl(Kern kern, dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, args...);
}

// Rotary forms of the fused tensor-core phases (pom_gemm_rope.cu), reached through pom_ctx_gemm,
// pom_gate_gemm and pom_gate_bwd_gemm when their `rope` member names a rotary kind.
int ctx_gemm_rope(const pom_ctx_args* a, int* status, cudaStream_t st);
int gate_gemm_rope(const pom_gate_args* a, int* status, cudaStream_t st);
int gate_bwd_gemm_rope(const pom_gate_bwd_args* a, int* status, cudaStream_t st);
// Token-causal forms (pom_gemm_causal.cu), reached when the `causal` member of the arguments is set.
int ctx_gemm_causal(const pom_ctx_args* a, int* status, cudaStream_t st);
int gate_gemm_causal(const pom_gate_args* a, int* status, cudaStream_t st);
int gate_bwd_gemm_causal(const pom_gate_bwd_args* a, int* status, cudaStream_t st);

}  // namespace pomh
