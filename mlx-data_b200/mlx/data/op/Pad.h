// Explicit per-sample padding ops (mlx/data/op/Pad.cpp:9-81): host-side array
// ops like in mlx-data, on any array type; they end a run of fusable image ops.
#pragma once

#include <limits>
#include <stdexcept>
#include <vector>

#include "mlx/data/op/KeyTransform.h"

namespace mlx {
namespace data {
namespace op {

// lpad elements of `value` before and rpad after, along `dim`.
class Pad : public KeyTransformOp {
 public:
  Pad(const std::string& ikey, int dim, int64_t lpad, int64_t rpad, double value, const std::string& okey = "")
      : KeyTransformOp(ikey, okey), dim_(dim), lpad_(lpad), rpad_(rpad), value_(value) {
    if (lpad_ < 0 || rpad_ < 0) {
      throw std::runtime_error("Pad: pad value must be positive");
    }
  }
  std::shared_ptr<Array> apply_key(const std::shared_ptr<const Array>& src) const override {
    return array::pad(src, src->checkdim(dim_), lpad_, rpad_, value_);
  }

 private:
  int dim_;
  int64_t lpad_, rpad_;
  double value_;
};

// Pad at the end of `dim` up to the nearest listed size above the current one;
// an array already at or beyond every listed size is copied unchanged.
class PadToSize : public KeyTransformOp {
 public:
  PadToSize(const std::string& ikey, int dim, const std::vector<int64_t>& sizes, double value, const std::string& okey = "")
      : KeyTransformOp(ikey, okey), dim_(dim), sizes_(sizes), value_(value) {}
  std::shared_ptr<Array> apply_key(const std::shared_ptr<const Array>& src) const override {
    const int dim = src->checkdim(dim_);
    const int64_t have = src->shape(dim);
    int64_t best = std::numeric_limits<int64_t>::max();
    for (auto s : sizes_) {
      const int64_t missing = s - have;
      if (missing > 0 && missing < best) {
        best = missing;
      }
    }
    if (best == std::numeric_limits<int64_t>::max()) {
      return array::clone(src);
    }
    return array::pad(src, dim, 0, best, value_);
  }

 private:
  int dim_;
  std::vector<int64_t> sizes_;
  double value_;
};

// Pad at the end of `dim` up to the next multiple of `size`.
class PadToMultiple : public KeyTransformOp {
 public:
  PadToMultiple(const std::string& ikey, int dim, int64_t size, double value, const std::string& okey = "")
      : KeyTransformOp(ikey, okey), dim_(dim), size_(size), value_(value) {}
  std::shared_ptr<Array> apply_key(const std::shared_ptr<const Array>& src) const override {
    const int dim = src->checkdim(dim_);
    const int64_t rest = src->shape(dim) % size_;
    if (rest == 0) {
      return array::clone(src);
    }
    return array::pad(src, dim, 0, size_ - rest, value_);
  }

 private:
  int dim_;
  int64_t size_;
  double value_;
};

} // namespace op
} // namespace data
} // namespace mlx
