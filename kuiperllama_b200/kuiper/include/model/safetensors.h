// Reader of a .safetensors file: 8 bytes little-endian header length, that many bytes of JSON (name -> dtype, shape,
// data_offsets), then the tensor bytes.  The file is mapped read-only; tensors are views into the mapping.
#ifndef KLLM_KUIPER_MODEL_SAFETENSORS_H_
#define KLLM_KUIPER_MODEL_SAFETENSORS_H_
#include <cstddef>
#include <cstdint>
#include <map>
#include <string>
#include <vector>

#include "base/base.h"

namespace model {
struct StTensor {
  enum class Dtype { kBF16, kF32, kF16, kI32, kOther };
  Dtype dtype = Dtype::kOther;
  std::vector<int64_t> shape;
  const uint8_t* data = nullptr;
  size_t bytes = 0;
  int64_t numel() const {
    int64_t n = 1;
    for (int64_t s : shape) n *= s;
    return n;
  }
};

class SafetensorsFile : public base::NoCopyable {
 public:
  SafetensorsFile() = default;
  ~SafetensorsFile();
  base::Status open(const std::string& path);
  const StTensor* find(const std::string& name) const;
  const std::map<std::string, StTensor>& tensors() const { return tensors_; }

 private:
  int fd_ = -1;
  void* map_ = nullptr;
  size_t size_ = 0;
  std::map<std::string, StTensor> tensors_;
};

// element conversions used while packing weights for upload
float bf16_to_float(uint16_t v);
uint16_t float_to_bf16(float v);  // round to nearest even
// the tensor as fp32 / as bf16 bit patterns (whatever it is stored as: BF16, F32 or F16)
base::Status tensor_to_f32(const StTensor& t, float* out);
base::Status tensor_to_bf16(const StTensor& t, uint16_t* out);
}  // namespace model
#endif  // KLLM_KUIPER_MODEL_SAFETENSORS_H_
