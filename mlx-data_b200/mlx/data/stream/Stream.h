// Pull-based pipeline node (mlx/data/stream/Stream.h:15-26): next() yields
// samples until it returns an empty one; reset() rewinds.
#pragma once

#include "mlx/data/Sample.h"

namespace mlx {
namespace data {
namespace stream {

class Stream {
 public:
  virtual Sample next() const = 0;
  virtual void reset() = 0;
  virtual ~Stream() {}
};

} // namespace stream
} // namespace data
} // namespace mlx
