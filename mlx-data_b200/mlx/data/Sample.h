// A sample is a dictionary of named arrays (mlx/data/Sample.h:13); an empty
// dictionary means "no sample" (end of stream, or dropped by an op).
#pragma once

#include <string>
#include <unordered_map>
#include <vector>

#include "mlx/data/Array.h"

namespace mlx {
namespace data {

typedef std::unordered_map<std::string, std::shared_ptr<Array>> Sample;

namespace sample {

inline std::vector<std::string> keys(const Sample& dict) {
  std::vector<std::string> out;
  out.reserve(dict.size());
  for (auto& kv : dict) {
    out.push_back(kv.first);
  }
  return out;
}

// The array stored under `key`; throws when the key is missing or, unless
// type is Any, when the array has another type (mlx/data/Sample.cpp:18-29).
inline std::shared_ptr<Array> check_key(const Sample& input, const std::string& key, ArrayType type) {
  auto it = input.find(key);
  if (it == input.end()) {
    throw std::runtime_error("key <" + key + "> expected");
  }
  if (type != ArrayType::Any && it->second->type() != type) {
    throw std::runtime_error("invalid Array type");
  }
  return it->second;
}

} // namespace sample
} // namespace data
} // namespace mlx
