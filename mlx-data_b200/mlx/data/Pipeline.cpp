// Bodies of the Stream and Buffer façades: each call wraps the current top
// node in one more node.
#include "mlx/data/Buffer.h"
#include "mlx/data/Stream.h"
#include "mlx/data/buffer/Nodes.h"
#include "mlx/data/stream/Nodes.h"

namespace mlx {
namespace data {

// ------------------------------------------------------------ Stream
Stream Stream::transform_(const std::shared_ptr<op::Op>& op) const {
  return Stream(std::make_shared<stream::Transform>(self_, op));
}

Stream Stream::cast_(const std::string& ikey, const gpu::CastSpec& spec, const std::string& okey) const {
  if (auto b = std::dynamic_pointer_cast<stream::Batch>(self_)) {
    return Stream(b->with_cast(core::CastRequest{ikey, okey, spec}));
  }
  return transform_(std::make_shared<op::Cast>(ikey, spec, okey));
}

Stream Stream::batch(
    int64_t batch_size, const std::unordered_map<std::string, double>& pad_values,
    const std::unordered_map<std::string, int>& batch_dims) const {
  return Stream(std::make_shared<stream::Batch>(self_, batch_size, pad_values, batch_dims));
}

Stream Stream::dynamic_batch(
    int64_t buffer_size, const std::string& key, int64_t min_data_size, int64_t max_data_size,
    const std::unordered_map<std::string, double>& pad_values, const std::unordered_map<std::string, int>& batch_dims,
    bool shuffle, bool drop_outliers, int64_t max_skipped_samples, int num_thread) const {
  return Stream(std::make_shared<stream::DynamicBatch>(
      self_, buffer_size, key, min_data_size, max_data_size, pad_values, batch_dims, shuffle, drop_outliers,
      max_skipped_samples, num_thread));
}

Stream Stream::repeat(int64_t num_time) const {
  return Stream(std::make_shared<stream::Repeat>(self_, num_time));
}

Stream Stream::partition(int64_t num_partitions, int64_t partition) const {
  return Stream(std::make_shared<stream::Partition>(self_, num_partitions, partition));
}

Stream Stream::partition_if(bool cond, int64_t num_partitions, int64_t partition) const {
  return cond ? this->partition(num_partitions, partition) : Stream(self_);
}

Stream Stream::prefetch(int prefetch_size, int num_thread) const {
  return Stream(std::make_shared<stream::Prefetch>(self_, prefetch_size, num_thread));
}

Stream Stream::prefetch_if(bool cond, int prefetch_size, int num_thread) const {
  return cond ? this->prefetch(prefetch_size, num_thread) : Stream(self_);
}

Buffer Stream::to_buffer() {
  std::vector<Sample> all;
  for (;;) {
    Sample s = self_->next();
    if (s.empty()) {
      break;
    }
    all.push_back(std::move(s));
  }
  return buffer_from_vector(std::move(all));
}

// ------------------------------------------------------------ Buffer
Buffer Buffer::transform_(const std::shared_ptr<op::Op>& op) const {
  return Buffer(std::make_shared<buffer::Transform>(self_, op));
}

Buffer Buffer::cast_(const std::string& ikey, const gpu::CastSpec& spec, const std::string& okey) const {
  if (auto b = std::dynamic_pointer_cast<buffer::Batch>(self_)) {
    return Buffer(b->with_cast(core::CastRequest{ikey, okey, spec}));
  }
  return transform_(std::make_shared<op::Cast>(ikey, spec, okey));
}

Buffer Buffer::batch(
    int64_t batch_size, const std::unordered_map<std::string, double>& pad_values,
    const std::unordered_map<std::string, int>& batch_dims) const {
  return Buffer(std::make_shared<buffer::Batch>(self_, batch_size, pad_values, batch_dims));
}

Buffer Buffer::batch(
    const std::vector<int64_t>& batch_sizes, const std::unordered_map<std::string, double>& pad_values,
    const std::unordered_map<std::string, int>& batch_dims) const {
  return Buffer(std::make_shared<buffer::Batch>(self_, batch_sizes, pad_values, batch_dims));
}

Buffer Buffer::dynamic_batch(
    const std::string& key, int64_t min_data_size, int64_t max_data_size,
    const std::unordered_map<std::string, double>& pad_values, const std::unordered_map<std::string, int>& batch_dims,
    bool drop_outliers) const {
  return Buffer(buffer::dynamic_batch(
      self_, nullptr, key, min_data_size, max_data_size, pad_values, batch_dims, drop_outliers));
}

Buffer Buffer::dynamic_batch(
    const Buffer& size_buffer, const std::string& key, int64_t min_data_size, int64_t max_data_size,
    const std::unordered_map<std::string, double>& pad_values, const std::unordered_map<std::string, int>& batch_dims,
    bool drop_outliers) const {
  return Buffer(buffer::dynamic_batch(
      self_, size_buffer.self_, key, min_data_size, max_data_size, pad_values, batch_dims, drop_outliers));
}

Stream Buffer::ordered_prefetch(int prefetch_size, int num_thread) const {
  return Stream(std::make_shared<stream::OrderedPrefetch>(self_, prefetch_size, num_thread));
}

Buffer Buffer::partition(int64_t num_partitions, int64_t partition) const {
  return Buffer(std::make_shared<buffer::Partition>(self_, num_partitions, partition));
}

Buffer Buffer::partition_if(bool cond, int64_t num_partitions, int64_t partition) const {
  return cond ? this->partition(num_partitions, partition) : Buffer(self_);
}

Buffer Buffer::perm(const std::vector<int64_t>& order) const {
  return Buffer(std::make_shared<buffer::Perm>(self_, order));
}

Buffer Buffer::shuffle() const {
  return Buffer(buffer::shuffled(self_));
}

Buffer Buffer::shuffle_if(bool cond) const {
  return cond ? this->shuffle() : Buffer(self_);
}

Stream Buffer::to_stream() {
  return Stream(std::make_shared<stream::FromBuffer>(self_));
}

Buffer buffer_from_vector(const std::vector<Sample>& data) {
  return Buffer(std::make_shared<buffer::FromVector>(data));
}

Buffer buffer_from_vector(std::vector<Sample>&& data) {
  return Buffer(std::make_shared<buffer::FromVector>(std::move(data)));
}

} // namespace data
} // namespace mlx
