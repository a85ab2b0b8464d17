// Explicit per-sample padding ops (mlx/data/op/Pad.cpp:9-81).  On any array
// they are host-side array ops like in mlx-data.  Under a batch node, padding
// at the end of the rows or columns of a uint8 image joins the fused run: the
// image claims a larger rectangle of its batch slot and the batch kernel's pad
// fill supplies the values (when the op's value and the batch's pad value for
// the key agree; else the image is computed first, in a launch of its own).
#pragma once

#include <limits>
#include <stdexcept>
#include <vector>

#include "mlx/data/gpu/Runtime.h"
#include "mlx/data/op/KeyTransform.h"

namespace mlx {
namespace data {
namespace op {

// lpad elements of `value` before and rpad after, along `dim`.
class Pad : public FusableOp {
 public:
  Pad(const std::string& ikey, int dim, int64_t lpad, int64_t rpad, double value, const std::string& okey = "")
      : FusableOp(ikey, okey), dim_(dim), lpad_(lpad), rpad_(rpad), value_(value) {
    if (lpad_ < 0 || rpad_ < 0) {
      throw std::runtime_error("Pad: pad value must be positive");
    }
  }
  std::shared_ptr<Array> apply_key(const std::shared_ptr<const Array>& src) const override {
    return array::pad(src, src->checkdim(dim_), lpad_, rpad_, value_);
  }
  bool fold(gpu::LazyImage& image) const override {
    // padding in front would move the image inside its slot: host op
    return lpad_ == 0 && image.pad_end(dim_ < 0 ? dim_ + 3 : dim_, rpad_, value_);
  }
  bool extends_only() const override { return true; }

 private:
  int dim_;
  int64_t lpad_, rpad_;
  double value_;
};

// Pad at the end of `dim` up to the nearest listed size above the current one;
// an array already at or beyond every listed size is copied unchanged.
class PadToSize : public FusableOp {
 public:
  PadToSize(const std::string& ikey, int dim, const std::vector<int64_t>& sizes, double value, const std::string& okey = "")
      : FusableOp(ikey, okey), dim_(dim), sizes_(sizes), value_(value) {}
  std::shared_ptr<Array> apply_key(const std::shared_ptr<const Array>& src) const override {
    const int dim = src->checkdim(dim_);
    const int64_t best = missing(src->shape(dim));
    if (best == 0) {
      return array::clone(src);
    }
    return array::pad(src, dim, 0, best, value_);
  }
  bool fold(gpu::LazyImage& image) const override {
    const int dim = dim_ < 0 ? dim_ + 3 : dim_;
    if (dim != 0 && dim != 1) {
      return false;
    }
    return image.pad_end(dim, missing(dim == 0 ? image.height() : image.width()), value_);
  }
  bool extends_only() const override { return true; }

 private:
  // elements to add to reach the nearest listed size above `have`; 0 when there is none
  int64_t missing(int64_t have) const {
    int64_t best = std::numeric_limits<int64_t>::max();
    for (auto s : sizes_) {
      const int64_t m = s - have;
      if (m > 0 && m < best) {
        best = m;
      }
    }
    return best == std::numeric_limits<int64_t>::max() ? 0 : best;
  }
  int dim_;
  std::vector<int64_t> sizes_;
  double value_;
};

// Pad at the end of `dim` up to the next multiple of `size`.
class PadToMultiple : public FusableOp {
 public:
  PadToMultiple(const std::string& ikey, int dim, int64_t size, double value, const std::string& okey = "")
      : FusableOp(ikey, okey), dim_(dim), size_(size), value_(value) {}
  std::shared_ptr<Array> apply_key(const std::shared_ptr<const Array>& src) const override {
    const int dim = src->checkdim(dim_);
    const int64_t rest = src->shape(dim) % size_;
    if (rest == 0) {
      return array::clone(src);
    }
    return array::pad(src, dim, 0, size_ - rest, value_);
  }
  bool fold(gpu::LazyImage& image) const override {
    const int dim = dim_ < 0 ? dim_ + 3 : dim_;
    if ((dim != 0 && dim != 1) || size_ <= 0) {
      return false;
    }
    const int64_t rest = (dim == 0 ? image.height() : image.width()) % size_;
    return image.pad_end(dim, rest == 0 ? 0 : size_ - rest, value_);
  }
  bool extends_only() const override { return true; }

 private:
  int dim_;
  int64_t size_;
  double value_;
};

} // namespace op
} // namespace data
} // namespace mlx
