// slice / random_slice (mlx/data/op/Slice.cpp:12-86): host-side sub-array ops
// on any array type.  Under a batch node a slice of the rows and columns of a
// uint8 image is a crop and joins the fused run; a slice that touches the
// channel dimension is computed on the host.
#pragma once

#include <algorithm>
#include <random>
#include <stdexcept>
#include <vector>

#include "mlx/data/core/State.h"
#include "mlx/data/gpu/Runtime.h"
#include "mlx/data/op/KeyTransform.h"

namespace mlx {
namespace data {
namespace op {

// [starts[i], ends[i]) along dims[i], clipped to the array's extent.
class Slice : public FusableOp {
 public:
  Slice(const std::string& ikey, std::vector<int> dims, std::vector<int64_t> starts, std::vector<int64_t> ends,
        const std::string& okey = "")
      : FusableOp(ikey, okey), dims_(std::move(dims)), starts_(std::move(starts)), ends_(std::move(ends)) {
    if (dims_.size() != starts_.size() || dims_.size() != ends_.size()) {
      throw std::invalid_argument("Slice: number of dims much match provided starts and ends");
    }
  }
  std::shared_ptr<Array> apply_key(const std::shared_ptr<const Array>& src) const override {
    std::vector<int64_t> offsets(src->ndim(), 0);
    std::vector<int64_t> shape = src->shape();
    for (size_t i = 0; i < dims_.size(); i++) {
      const int d = src->checkdim(dims_[i]);
      offsets[d] = starts_[i];
      shape[d] = std::min(shape[d] - starts_[i], ends_[i] - starts_[i]);
    }
    return array::sub(src, std::move(offsets), std::move(shape));
  }
  bool fold(gpu::LazyImage& image) const override {
    if (image.extended()) {
      return false;
    }
    int64_t off[2] = {0, 0};
    int64_t len[2] = {image.height(), image.width()};
    for (size_t i = 0; i < dims_.size(); i++) {
      const int d = dims_[i] < 0 ? dims_[i] + 3 : dims_[i];
      if (d != 0 && d != 1) {
        return false;
      }
      off[d] = starts_[i];
      len[d] = std::min(len[d] - starts_[i], ends_[i] - starts_[i]);
    }
    // anything the sub-array code would refuse is left to it, with its messages
    if (off[0] < 0 || off[1] < 0 || len[0] <= 0 || len[1] <= 0 || off[0] + len[0] > image.height() ||
        off[1] + len[1] > image.width()) {
      return false;
    }
    return image.crop(off[1], off[0], len[1], len[0]);
  }

 private:
  std::vector<int> dims_;
  std::vector<int64_t> starts_, ends_;
};

// A window of sizes[i] along dims[i] at a uniformly random offset (one double
// draw per listed dimension that is longer than its window, in list order).
class RandomSlice : public FusableOp {
 public:
  RandomSlice(const std::string& ikey, std::vector<int> dims, std::vector<int64_t> sizes, const std::string& okey = "")
      : FusableOp(ikey, okey), dims_(std::move(dims)), sizes_(std::move(sizes)) {
    if (dims_.size() != sizes_.size()) {
      throw std::invalid_argument("RandomSlice: number of dims much match provided sizes");
    }
  }
  std::shared_ptr<Array> apply_key(const std::shared_ptr<const Array>& src) const override {
    std::uniform_real_distribution<> draw(0.0, 1.0);
    std::vector<int64_t> offsets(src->ndim(), 0);
    std::vector<int64_t> shape = src->shape();
    auto state = core::get_state();
    for (size_t i = 0; i < dims_.size(); i++) {
      const int d = src->checkdim(dims_[i]);
      const int64_t room = shape[d] - sizes_[i];
      if (room > 0) {
        shape[d] = sizes_[i];
        offsets[d] = static_cast<int64_t>((room + 1) * draw(state->randomGenerator));
      }
    }
    return array::sub(src, std::move(offsets), std::move(shape));
  }
  bool fold(gpu::LazyImage& image) const override {
    // decide before anything is drawn: a refusal must leave the generator alone
    if (image.extended()) {
      return false;
    }
    for (size_t i = 0; i < dims_.size(); i++) {
      const int d = dims_[i] < 0 ? dims_[i] + 3 : dims_[i];
      if ((d != 0 && d != 1) || sizes_[i] <= 0) {
        return false;
      }
    }
    std::uniform_real_distribution<> draw(0.0, 1.0);
    int64_t off[2] = {0, 0};
    int64_t len[2] = {image.height(), image.width()};
    auto state = core::get_state();
    for (size_t i = 0; i < dims_.size(); i++) {
      const int d = dims_[i] < 0 ? dims_[i] + 3 : dims_[i];
      const int64_t room = len[d] - sizes_[i];
      if (room > 0) {
        len[d] = sizes_[i];
        off[d] = static_cast<int64_t>((room + 1) * draw(state->randomGenerator));
      }
    }
    return image.crop(off[1], off[0], len[1], len[0]);
  }

  bool draws() const override { return true; }

 private:
  std::vector<int> dims_;
  std::vector<int64_t> sizes_;
};

} // namespace op
} // namespace data
} // namespace mlx
