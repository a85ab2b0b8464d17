// Ops that rewrite one key of a sample (mlx/data/op/KeyTransform.h:12-40):
// read the array at ikey, store the result at okey (ikey when okey is empty).
#pragma once

#include <functional>
#include <string>

#include "mlx/data/op/Op.h"

namespace mlx {
namespace data {
namespace gpu {
class LazyImage;
}
namespace op {

class KeyTransformOp : public Op {
 public:
  KeyTransformOp(const std::string& ikey, const std::string& okey = "") : ikey_(ikey), okey_(okey) {}
  virtual std::shared_ptr<Array> apply_key(const std::shared_ptr<const Array>& src) const = 0;
  Sample apply(const Sample& sample) const override;

  const std::string& input_key() const { return ikey_; }
  const std::string& output_key() const { return okey_.empty() ? ikey_ : okey_; }

 protected:
  std::string ikey_;
  std::string okey_;
};

// A key op that a batch node can absorb when the key holds a uint8 image: it
// records itself on a LazyImage (source array + program) instead of producing
// pixels, and the whole run of such ops, the batching and the cast execute as
// one GPU launch.  On any other kind of array the op's apply_key() runs as usual.
class FusableOp : public KeyTransformOp {
 public:
  FusableOp(const std::string& ikey, const std::string& okey = "") : KeyTransformOp(ikey, okey) {}
  // Record this op on `image`.  Returns false when it cannot join the program
  // already recorded; the caller then materialises the image and folds again,
  // and if the op cannot join an empty program either, runs apply_key() on
  // the pixels.
  virtual bool fold(gpu::LazyImage& image) const = 0;
  // fold() for ops whose parameters may come from other entries of the sample
  // (`sample` holds the entries that are concrete arrays).
  virtual bool fold_in(gpu::LazyImage& image, const Sample& sample) const {
    (void)sample;
    return fold(image);
  }
  virtual bool reads_sample() const { return false; }
  // True for ops that only enlarge the image's claim on its batch slot (end
  // padding): they may follow one another; any other op after them needs the
  // pixels first.  The batch node checks this before it lets an op draw random
  // parameters, so nothing is drawn twice.
  virtual bool extends_only() const { return false; }
  // True for ops that draw random parameters: running them twice on a sample
  // gives two different results.
  virtual bool draws() const { return false; }
};

// Arbitrary host callback on one key (this is how Python lambdas enter a pipeline).
class KeyTransform : public KeyTransformOp {
 public:
  using Fn = std::function<std::shared_ptr<Array>(const std::shared_ptr<const Array>&)>;
  KeyTransform(const std::string& ikey, Fn op, const std::string& okey = "")
      : KeyTransformOp(ikey, okey), op_(std::move(op)) {}
  std::shared_ptr<Array> apply_key(const std::shared_ptr<const Array>& src) const override { return op_(src); }

 private:
  Fn op_;
};

// Arbitrary host callback on the whole sample.
class SampleTransform : public Op {
 public:
  using Fn = std::function<Sample(const Sample&)>;
  explicit SampleTransform(Fn op) : op_(std::move(op)) {}
  Sample apply(const Sample& sample) const override { return op_(sample); }

 private:
  Fn op_;
};

} // namespace op
} // namespace data
} // namespace mlx
