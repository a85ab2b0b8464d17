// Public random-access pipeline (mlx/data/Buffer.h:18-68, the hot-path subset).
#pragma once

#include <unordered_map>
#include <vector>

#include "mlx/data/Dataset.h"
#include "mlx/data/buffer/Buffer.h"

namespace mlx {
namespace data {

class Stream;

class Buffer : public Dataset<Buffer, buffer::Buffer> {
 public:
  Buffer(const std::shared_ptr<buffer::Buffer>& self) : Dataset<Buffer, buffer::Buffer>(self) {}

  Sample get(int64_t idx) const { return self_->get(idx); }
  int64_t size() const { return self_->size(); }

  Buffer batch(
      int64_t batch_size, const std::unordered_map<std::string, double>& pad_values = {},
      const std::unordered_map<std::string, int>& batch_dims = {}) const;
  Buffer batch(
      const std::vector<int64_t>& batch_sizes, const std::unordered_map<std::string, double>& pad_values = {},
      const std::unordered_map<std::string, int>& batch_dims = {}) const;
  // Batches of about the same padded element count (mlx/data/Buffer.h dynamic_batch).
  Buffer dynamic_batch(
      const std::string& key, int64_t min_data_size = -1, int64_t max_data_size = -1,
      const std::unordered_map<std::string, double>& pad_values = {},
      const std::unordered_map<std::string, int>& batch_dims = {}, bool drop_outliers = false) const;
  Buffer dynamic_batch(
      const Buffer& size_buffer, const std::string& key, int64_t min_data_size = -1, int64_t max_data_size = -1,
      const std::unordered_map<std::string, double>& pad_values = {},
      const std::unordered_map<std::string, int>& batch_dims = {}, bool drop_outliers = false) const;
  Stream ordered_prefetch(int prefetch_size, int num_thread) const;
  Buffer partition(int64_t num_partitions, int64_t partition) const;
  Buffer partition_if(bool cond, int64_t num_partitions, int64_t partition) const;
  Buffer perm(const std::vector<int64_t>& order) const;
  Buffer shuffle() const;
  Buffer shuffle_if(bool cond) const;
  Stream to_stream();

  // used by Dataset
  Buffer transform_(const std::shared_ptr<op::Op>& op) const;
  Buffer cast_(const std::string& ikey, const gpu::CastSpec& spec, const std::string& okey) const;
};

Buffer buffer_from_vector(const std::vector<Sample>& data);
Buffer buffer_from_vector(std::vector<Sample>&& data);

} // namespace data
} // namespace mlx
