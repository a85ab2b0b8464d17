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
  Stream dynamic_batch(
      int64_t buffer_size, const std::string& key, int64_t min_data_size = -1, int64_t max_data_size = -1,
      const std::unordered_map<std::string, double>& pad_values = {},
      const std::unordered_map<std::string, int>& batch_dims = {}, bool shuffle = false, bool drop_outliers = false,
      int64_t max_skipped_samples = 1000, int num_thread = 1) const;
  Stream partition(int64_t num_partitions, int64_t partition) const;
  Stream partition_if(bool cond, int64_t num_partitions, int64_t partition) const;
  Stream prefetch(int prefetch_size, int num_thread) const;
  Stream prefetch_if(bool cond, int prefetch_size, int num_thread) const;
  Stream repeat(int64_t num_time) const;
  Buffer to_buffer();

  // used by Dataset
  Stream transform_(const std::shared_ptr<op::Op>& op) const;
  Stream cast_(const std::string& ikey, const gpu::CastSpec& spec, const std::string& okey) const;
};

} // namespace data
} // namespace mlx
