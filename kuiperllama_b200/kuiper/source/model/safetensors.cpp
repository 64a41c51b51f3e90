#include "model/safetensors.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstring>

#include "model/json.h"

namespace model {
SafetensorsFile::~SafetensorsFile() {
  if (map_ != nullptr && map_ != MAP_FAILED) munmap(map_, size_);
  if (fd_ >= 0) ::close(fd_);
}

base::Status SafetensorsFile::open(const std::string& path) {
  fd_ = ::open(path.c_str(), O_RDONLY);
  if (fd_ < 0) return base::error::PathNotValid("cannot open " + path);
  struct stat st {};
  if (fstat(fd_, &st) != 0 || st.st_size < 8) return base::error::ModelParseError(path + ": too short");
  size_ = static_cast<size_t>(st.st_size);
  map_ = mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd_, 0);
  if (map_ == MAP_FAILED) return base::error::ModelParseError("mmap failed for " + path);
  const uint8_t* p = static_cast<const uint8_t*>(map_);
  uint64_t n = 0;
  for (int i = 7; i >= 0; --i) n = (n << 8) | p[i];
  if (n > size_ - 8) return base::error::ModelParseError(path + ": header length exceeds the file");
  const std::string header(reinterpret_cast<const char*>(p + 8), static_cast<size_t>(n));
  const uint8_t* data = p + 8 + n;
  const size_t data_bytes = size_ - 8 - static_cast<size_t>(n);
  try {
    const json::Value root = json::parse(header);
    if (!root.is_object()) return base::error::ModelParseError(path + ": header is not an object");
    for (const auto& kv : root.object) {
      if (kv.first == "__metadata__") continue;
      StTensor t;
      const std::string& dt = kv.second.at("dtype").as_string();
      t.dtype = dt == "BF16" ? StTensor::Dtype::kBF16 : dt == "F32" ? StTensor::Dtype::kF32
              : dt == "F16" ? StTensor::Dtype::kF16 : dt == "I32" ? StTensor::Dtype::kI32 : StTensor::Dtype::kOther;
      for (const json::Value& s : kv.second.at("shape").array) t.shape.push_back(s.as_int());
      const auto& off = kv.second.at("data_offsets").array;
      if (off.size() != 2) return base::error::ModelParseError(path + ": bad data_offsets of " + kv.first);
      const long long a = off[0].as_int(), b = off[1].as_int();
      if (a < 0 || b < a || static_cast<size_t>(b) > data_bytes)
        return base::error::ModelParseError(path + ": tensor " + kv.first + " lies outside the file");
      t.data = data + a;
      t.bytes = static_cast<size_t>(b - a);
      const size_t es = t.dtype == StTensor::Dtype::kF32 || t.dtype == StTensor::Dtype::kI32 ? 4
                      : t.dtype == StTensor::Dtype::kOther ? 0 : 2;
      if (es != 0 && t.bytes != es * static_cast<size_t>(t.numel()))
        return base::error::ModelParseError(path + ": size of " + kv.first + " does not fit its shape");
      tensors_.emplace(kv.first, std::move(t));
    }
  } catch (const std::exception& e) {
    return base::error::ModelParseError(path + ": " + e.what());
  }
  return base::error::Success();
}

const StTensor* SafetensorsFile::find(const std::string& name) const {
  const auto it = tensors_.find(name);
  return it == tensors_.end() ? nullptr : &it->second;
}

float bf16_to_float(uint16_t v) {
  const uint32_t u = static_cast<uint32_t>(v) << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}

uint16_t float_to_bf16(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((u >> 16) | 0x40);  // NaN stays NaN
  u += 0x7fffu + ((u >> 16) & 1u);
  return static_cast<uint16_t>(u >> 16);
}

static float f16_to_float(uint16_t h) {
  const uint32_t sign = (h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1f, man = h & 0x3ffu, u;
  if (exp == 0) {
    if (man == 0) {
      u = sign;
    } else {
      int e = -1;
      do {
        man <<= 1;
        ++e;
      } while (!(man & 0x400u));
      u = sign | ((127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
    }
  } else if (exp == 31) {
    u = sign | 0x7f800000u | (man << 13);
  } else {
    u = sign | ((exp + 112) << 23) | (man << 13);
  }
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}

base::Status tensor_to_f32(const StTensor& t, float* out) {
  const int64_t n = t.numel();
  switch (t.dtype) {
    case StTensor::Dtype::kF32: std::memcpy(out, t.data, static_cast<size_t>(n) * 4); break;
    case StTensor::Dtype::kBF16: {
      const uint16_t* s = reinterpret_cast<const uint16_t*>(t.data);
      for (int64_t i = 0; i < n; ++i) out[i] = bf16_to_float(s[i]);
      break;
    }
    case StTensor::Dtype::kF16: {
      const uint16_t* s = reinterpret_cast<const uint16_t*>(t.data);
      for (int64_t i = 0; i < n; ++i) out[i] = f16_to_float(s[i]);
      break;
    }
    default: return base::error::ModelParseError("tensor is not a floating-point tensor");
  }
  return base::error::Success();
}

base::Status tensor_to_bf16(const StTensor& t, uint16_t* out) {
  const int64_t n = t.numel();
  switch (t.dtype) {
    case StTensor::Dtype::kBF16: std::memcpy(out, t.data, static_cast<size_t>(n) * 2); break;
    case StTensor::Dtype::kF32: {
      const float* s = reinterpret_cast<const float*>(t.data);
      for (int64_t i = 0; i < n; ++i) out[i] = float_to_bf16(s[i]);
      break;
    }
    case StTensor::Dtype::kF16: {
      const uint16_t* s = reinterpret_cast<const uint16_t*>(t.data);
      for (int64_t i = 0; i < n; ++i) out[i] = float_to_bf16(f16_to_float(s[i]));
      break;
    }
    default: return base::error::ModelParseError("tensor is not a floating-point tensor");
  }
  return base::error::Success();
}
}  // namespace model
