#include "mlx/data/buffer/Nodes.h"

#include <algorithm>
#include <stdexcept>

namespace mlx {
namespace data {
namespace buffer {

// ------------------------------------------------------------ FromVector
FromVector::FromVector(const std::vector<Sample>& data) : data_(data) {
  check();
}

FromVector::FromVector(std::vector<Sample>&& data) : data_(std::move(data)) {
  check();
}

void FromVector::check() const {
  for (auto& s : data_) {
    if (s.empty()) {
      throw std::runtime_error("FromVector: unexpected empty sample");
    }
  }
}

Sample FromVector::get(int64_t idx) const {
  if (idx < 0 || idx >= static_cast<int64_t>(data_.size())) {
    throw std::out_of_range("FromVector: index out of range");
  }
  return data_[idx];
}

int64_t FromVector::size() const {
  return static_cast<int64_t>(data_.size());
}

// ------------------------------------------------------------ Transform
Transform::Transform(const std::shared_ptr<Buffer>& source, const std::shared_ptr<op::Op>& op)
    : source_(source), ops_({op}) {}

Transform::Transform(const std::shared_ptr<Buffer>& source, const std::vector<std::shared_ptr<op::Op>>& ops)
    : source_(source), ops_(ops) {}

Sample Transform::get(int64_t idx) const {
  Sample s = source_->get(idx);
  for (auto& op : ops_) {
    s = op->apply(s);
    if (s.empty()) {
      throw std::runtime_error("Transform: a buffer transform cannot drop samples (empty sample returned)");
    }
  }
  return s;
}

int64_t Transform::size() const {
  return source_->size();
}

std::shared_ptr<Buffer> peel_image_ops(
    const std::shared_ptr<Buffer>& top, std::vector<std::shared_ptr<op::ImageTransformOp>>& ops) {
  std::shared_ptr<Buffer> cur = top;
  std::vector<std::shared_ptr<op::ImageTransformOp>> rev;
  for (;;) {
    auto t = std::dynamic_pointer_cast<Transform>(cur);
    if (!t) {
      break;
    }
    std::vector<std::shared_ptr<op::ImageTransformOp>> mine;
    for (auto& o : t->ops()) {
      auto io = std::dynamic_pointer_cast<op::ImageTransformOp>(o);
      if (!io) {
        mine.clear();
        break;
      }
      mine.push_back(io);
    }
    if (mine.size() != t->ops().size() || mine.empty()) {
      break;
    }
    rev.insert(rev.end(), mine.rbegin(), mine.rend());
    cur = t->source();
  }
  ops.assign(rev.rbegin(), rev.rend());
  return cur;
}

// ------------------------------------------------------------ Batch
void Batch::absorb(
    const std::shared_ptr<Buffer>& source,
    const std::unordered_map<std::string, double>& pad_values,
    const std::unordered_map<std::string, int>& batch_dims) {
  std::vector<std::shared_ptr<op::ImageTransformOp>> ops;
  base_ = peel_image_ops(source, ops);
  batcher_ = std::make_shared<core::Batcher>(ops, pad_values, batch_dims);
}

Batch::Batch(
    const std::shared_ptr<Buffer>& source, int64_t batch_size,
    const std::unordered_map<std::string, double>& pad_values,
    const std::unordered_map<std::string, int>& batch_dims)
    : batch_size_(batch_size) {
  if (batch_size <= 0) {
    throw std::runtime_error("Batch: batch size must be positive");
  }
  absorb(source, pad_values, batch_dims);
  const int64_t n = base_->size();
  count_ = (n + batch_size - 1) / batch_size;
}

Batch::Batch(
    const std::shared_ptr<Buffer>& source, const std::vector<int64_t>& batch_sizes,
    const std::unordered_map<std::string, double>& pad_values,
    const std::unordered_map<std::string, int>& batch_dims) {
  absorb(source, pad_values, batch_dims);
  int64_t at = 0;
  starts_.push_back(0);
  for (auto b : batch_sizes) {
    if (b <= 0) {
      throw std::runtime_error("Batch: batch size must be positive");
    }
    at += b;
    starts_.push_back(at);
  }
  if (at > base_->size()) {
    throw std::runtime_error("Batch: sum of batch sizes exceeds buffer size");
  }
  count_ = static_cast<int64_t>(batch_sizes.size());
}

std::shared_ptr<Batch> Batch::with_cast(const core::CastRequest& cast) const {
  std::shared_ptr<Batch> b(new Batch());
  b->base_ = base_;
  b->batch_size_ = batch_size_;
  b->starts_ = starts_;
  b->count_ = count_;
  auto casts = batcher_->casts();
  casts.push_back(cast);
  b->batcher_ = std::make_shared<core::Batcher>(
      batcher_->ops(), batcher_->pad_values(), batcher_->batch_dims(), casts);
  return b;
}

Sample Batch::get(int64_t idx) const {
  if (idx < 0 || idx >= count_) {
    throw std::out_of_range("Batch: index out of range");
  }
  int64_t lo, hi;
  if (starts_.empty()) {
    lo = idx * batch_size_;
    hi = std::min(lo + batch_size_, base_->size());
  } else {
    lo = starts_[idx];
    hi = starts_[idx + 1];
  }
  std::vector<Sample> raw;
  raw.reserve(hi - lo);
  for (int64_t i = lo; i < hi; i++) {
    raw.push_back(base_->get(i));
  }
  return batcher_->run(raw);
}

int64_t Batch::size() const {
  return count_;
}

// ------------------------------------------------------------ Partition
Partition::Partition(const std::shared_ptr<Buffer>& source, int64_t num_partitions, int64_t partition)
    : source_(source), num_partitions_(num_partitions), partition_(partition) {
  if (num_partitions <= 0) {
    throw std::runtime_error("Partition: number of partitions must be positive");
  }
  if (partition < 0 || partition >= num_partitions) {
    throw std::runtime_error("Partition: selected partition is out of range");
  }
  const int64_t n = source->size();
  size_ = n / num_partitions + (partition < n % num_partitions ? 1 : 0);
}

Sample Partition::get(int64_t idx) const {
  if (idx < 0 || idx >= size_) {
    throw std::runtime_error("Partition: index out of range");
  }
  return source_->get(idx * num_partitions_ + partition_);
}

int64_t Partition::size() const {
  return size_;
}

} // namespace buffer
} // namespace data
} // namespace mlx
