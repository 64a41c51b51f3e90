// Process-wide pieces every library built from this directory carries: the launch counter behind
// kllm_launch_count(), the version string and the error names of include/kllm_b200.h.
#include <cuda_runtime.h>

#include <atomic>
#include <cstdint>

#include "kllm_host.h"

namespace kllm {
std::atomic<uint64_t>& launch_counter() {
  static std::atomic<uint64_t> c{0};
  return c;
}
}  // namespace kllm

extern "C" {
const char* kllm_version(void) { return "kllm_b200 0.1 (sm_100a)"; }

const char* kllm_error_string(int code) {
  switch (code) {
    case KLLM_OK: return "ok";
    case KLLM_E_INVALID: return "invalid argument";
    case KLLM_E_UNSUPPORTED: return "unsupported shape";
    case KLLM_E_STATE: return "invalid decoder state";
    case KLLM_E_NODEVICE: return "no CUDA device";
    case KLLM_E_COMM: return "tensor-parallel transport unavailable or failed";
    default: return code > 0 ? cudaGetErrorString(static_cast<cudaError_t>(code)) : "unknown";
  }
}

uint64_t kllm_launch_count(void) { return kllm::launch_counter().load(); }
}
