// Random-access pipeline node (mlx/data/buffer/Buffer.h:11-20).
#pragma once

#include "mlx/data/Sample.h"

namespace mlx {
namespace data {
namespace buffer {

class Buffer {
 public:
  virtual Sample get(int64_t idx) const = 0;
  virtual int64_t size() const = 0;
  virtual ~Buffer() {}
};

} // namespace buffer
} // namespace data
} // namespace mlx
