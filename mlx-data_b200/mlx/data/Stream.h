// Public stream pipeline (mlx/data/Stream.h:18-79, the hot-path subset).
#pragma once

#include <unordered_map>

#include "mlx/data/Dataset.h"
#include "mlx/data/stream/Stream.h"

namespace mlx {
namespace data {

class Buffer;

class Stream : public Dataset<Stream, stream::Stream> {
 public:
  Stream(const std::shared_ptr<stream::Stream>& self) : Dataset<Stream, stream::Stream>(self) {}

  Sample next() const { return self_->next(); }
  void reset() { self_->reset(); }

  Stream batch(
      int64_t batch_size, const std::unordered_map<std::string, double>& pad_values = {},
      const std::unordered_map<std::string, int>& batch_dims = {}) const;
  Stream partition(int64_t num_partitions, int64_t partition) const;
  Stream partition_if(bool cond, int64_t num_partitions, int64_t partition) const;
  Stream prefetch(int prefetch_size, int num_thread) const;
  Stream prefetch_if(bool cond, int prefetch_size, int num_thread) const;
  Buffer to_buffer();

  // used by Dataset
  Stream transform_(const std::shared_ptr<op::Op>& op) const;
  Stream cast_(const std::string& ikey, const gpu::CastSpec& spec, const std::string& okey) const;
};

} // namespace data
} // namespace mlx
