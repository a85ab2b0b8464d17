// A sample-to-sample transformation (mlx/data/op/Op.h:16-24).  An op returning
// an empty sample drops it from a stream.
#pragma once

#include <memory>

#include "mlx/data/Sample.h"

namespace mlx {
namespace data {
namespace op {

class Op {
 public:
  virtual Sample apply(const Sample& sample) const = 0;
  virtual ~Op() {}
};

} // namespace op
} // namespace data
} // namespace mlx
