// Dense, typed, row-major host array: the value type of every Sample entry.
// Same public surface as mlx-data's Array (mlx/data/Array.h:20-112 and the
// array:: helpers at :152-179) so pipelines and bindings written against it
// keep working; storage is a shared_ptr<void> that may be plain heap memory,
// page-locked memory from the GPU library, or memory owned by someone else
// (a numpy array) with a custom deleter.
#pragma once

#include <cstdint>
#include <cstring>
#include <memory>
#include <stdexcept>
#include <string>
#include <string_view>
#include <type_traits>
#include <vector>

namespace mlx {
namespace data {

enum ArrayType { Any, UInt8, Int8, Int32, Int64, Float, Double };

int64_t array_type_size(ArrayType t);

class Array {
 public:
  Array() : Array(Any, std::vector<int64_t>{0}) {}
  // Shares storage with src (no copy), like the reference's copy-from-pointer.
  Array(const std::shared_ptr<const Array>& src);
  explicit Array(ArrayType type) : Array(type, std::vector<int64_t>{0}) {}
  Array(const std::string& str);
  Array(std::string_view str);
  Array(ArrayType type, const std::vector<int64_t>& shape);
  // Adopt external storage; `data` keeps it alive and releases it.  device >= 0
  // marks storage that lives in that GPU's memory (an addition: mlx-data's
  // arrays are host-only); host code must not dereference it.
  Array(ArrayType type, const std::vector<int64_t>& shape, std::shared_ptr<void> data, int device = -1);

  template <class... Dims, class = std::enable_if_t<(std::is_integral_v<Dims> && ...) && (sizeof...(Dims) > 0)>>
  Array(ArrayType type, Dims... dims) : Array(type, std::vector<int64_t>{static_cast<int64_t>(dims)...}) {}

  template <class T>
  Array(const std::vector<T>& vec) : Array(to_array_type<T>(), std::vector<int64_t>{static_cast<int64_t>(vec.size())}) {
    if (!vec.empty()) {
      std::memcpy(data_.get(), vec.data(), vec.size() * sizeof(T));
    }
  }

  template <class T, class = std::enable_if_t<std::is_arithmetic_v<T>>>
  Array(T scalar) : Array(to_array_type<T>(), std::vector<int64_t>{}) {
    *static_cast<T*>(data_.get()) = scalar;
  }

  template <class T>
  static constexpr ArrayType to_array_type() {
    if constexpr (std::is_same_v<T, char>) {
      return Int8;
    } else if constexpr (std::is_same_v<T, unsigned char>) {
      return UInt8;
    } else if constexpr (std::is_same_v<T, int32_t>) {
      return Int32;
    } else if constexpr (std::is_same_v<T, int64_t>) {
      return Int64;
    } else if constexpr (std::is_same_v<T, float>) {
      return Float;
    } else if constexpr (std::is_same_v<T, double>) {
      return Double;
    } else {
      static_assert(sizeof(T) == 0, "unsupported element type");
    }
  }

  const std::vector<int64_t>& shape() const { return shape_; }
  int64_t shape(int d) const { return shape_[checkdim(d)]; }
  int ndim() const { return static_cast<int>(shape_.size()); }
  int64_t itemsize() const { return itemsize_; }
  int64_t size() const;
  ArrayType type() const { return type_; }
  void* data() const { return data_.get(); }
  const std::shared_ptr<void>& storage() const { return data_; }
  // -1: host memory; otherwise the CUDA device holding the storage.
  int device() const { return device_; }
  // Throws when the storage is on a GPU; host-side array helpers call this.
  void require_host(const char* what) const;

  template <class T>
  T* data() const {
    if (type_ != to_array_type<T>()) {
      throw std::runtime_error("Array: incompatible array type");
    }
    return static_cast<T*>(data_.get());
  }

  template <class T>
  T scalar() const {
    if (size() != 1) {
      throw std::runtime_error("Array: expected a scalar array");
    }
    return *data<T>();
  }

  void fill(double value);
  void squeeze(const std::vector<int>& dims);
  void reshape(const std::vector<int64_t>& shape);
  // Normalise a possibly negative dimension index; throws when out of range.
  int checkdim(int dim) const;

 private:
  ArrayType type_ = Any;
  std::vector<int64_t> shape_;
  std::shared_ptr<void> data_;
  int64_t itemsize_ = 0;
  int device_ = -1;
};

namespace array {

std::shared_ptr<Array> clone(const std::shared_ptr<const Array>& arr);
std::shared_ptr<Array> reshape(const std::shared_ptr<const Array>& arr, const std::vector<int64_t>& shape);
std::shared_ptr<Array> squeeze(const std::shared_ptr<const Array>& arr, const std::vector<int>& dims);
std::shared_ptr<Array> pad(const std::shared_ptr<const Array>& arr, int dim, int64_t lpad, int64_t rpad, double value);
// View of arr[index0] sharing storage.
std::shared_ptr<Array> slice(const std::shared_ptr<const Array>& arr, int index0);
void copy(const std::shared_ptr<Array>& dst, const std::shared_ptr<const Array>& src);
// Stack along a new leading dimension, padding every other dimension to the
// largest extent with pad_value.
std::shared_ptr<Array> batch(const std::vector<std::shared_ptr<Array>>& arrs, double pad_value);
// Concatenate along `dim`, padding the other dimensions.
std::shared_ptr<Array> batch(const std::vector<std::shared_ptr<Array>>& arrs, int dim, double pad_value);
// Rectangular sub-array; -1 in shape means "to the end of that dimension".
std::shared_ptr<Array> sub(const std::shared_ptr<const Array>& arr, std::vector<int64_t> offset, std::vector<int64_t> shape);

} // namespace array
} // namespace data
} // namespace mlx
