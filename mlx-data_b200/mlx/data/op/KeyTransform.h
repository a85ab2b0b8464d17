// Ops that rewrite one key of a sample (mlx/data/op/KeyTransform.h:12-40):
// read the array at ikey, store the result at okey (ikey when okey is empty).
#pragma once

#include <functional>
#include <string>

#include "mlx/data/op/Op.h"

namespace mlx {
namespace data {
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
