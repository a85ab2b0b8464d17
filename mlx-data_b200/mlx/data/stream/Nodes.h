// Stream nodes of the transform-and-batch path: FromBuffer, Transform, Batch,
// Prefetch, OrderedPrefetch, Partition (roles of the same-named files under
// mlx/data/stream/).
#pragma once

#include <deque>
#include <future>
#include <memory>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "mlx/data/buffer/Buffer.h"
#include "mlx/data/core/Batcher.h"
#include "mlx/data/core/ThreadPool.h"
#include "mlx/data/op/Op.h"
#include "mlx/data/stream/Stream.h"

namespace mlx {
namespace data {
namespace stream {

// Walk a buffer front to back.
class FromBuffer : public Stream {
 public:
  explicit FromBuffer(const std::shared_ptr<buffer::Buffer>& buffer) : buffer_(buffer) {}
  Sample next() const override;
  void reset() override;

 private:
  std::shared_ptr<buffer::Buffer> buffer_;
  mutable int64_t cursor_ = 0;
  mutable std::mutex mu_;
};

// Apply ops to every sample; samples an op turns empty are skipped.
class Transform : public Stream {
 public:
  Transform(const std::shared_ptr<Stream>& source, const std::shared_ptr<op::Op>& op) : source_(source), ops_({op}) {}
  Transform(const std::shared_ptr<Stream>& source, const std::vector<std::shared_ptr<op::Op>>& ops)
      : source_(source), ops_(ops) {}
  Sample next() const override;
  void reset() override { source_->reset(); }
  const std::shared_ptr<Stream>& source() const { return source_; }
  const std::vector<std::shared_ptr<op::Op>>& ops() const { return ops_; }

 private:
  std::shared_ptr<Stream> source_;
  std::vector<std::shared_ptr<op::Op>> ops_;
};

// Group consecutive samples; the last batch may be short.  Image ops sitting
// directly under the batch node are absorbed and run fused with it on the GPU.
class Batch : public Stream {
 public:
  Batch(
      const std::shared_ptr<Stream>& source, int64_t batch_size,
      const std::unordered_map<std::string, double>& pad_values = {},
      const std::unordered_map<std::string, int>& batch_dims = {});
  Sample next() const override;
  void reset() override;
  std::shared_ptr<Batch> with_cast(const core::CastRequest& cast) const;

 private:
  Batch() = default;
  std::shared_ptr<Stream> base_;
  std::shared_ptr<core::Batcher> batcher_;
  int64_t batch_size_ = 0;
  mutable std::mutex pull_mu_;  // a batch takes consecutive samples even with several consumers
};

// Keep prefetch_size next() calls of the source in flight on num_thread
// workers; order of results follows completion of the queue head only, so with
// several workers the sample order may differ from the source order.
class Prefetch : public Stream {
 public:
  Prefetch(const std::shared_ptr<Stream>& source, int prefetch_size, int num_thread);
  ~Prefetch();
  Sample next() const override;
  void reset() override;

 private:
  void drain() const;
  std::shared_ptr<Stream> source_;
  std::shared_ptr<core::ThreadPool> pool_;
  int prefetch_size_;
  mutable std::deque<std::future<Sample>> inflight_;
  mutable std::mutex mu_;
};

// Prefetch over a buffer that preserves the buffer's order.
class OrderedPrefetch : public Stream {
 public:
  OrderedPrefetch(const std::shared_ptr<buffer::Buffer>& buffer, int prefetch_size, int num_thread);
  ~OrderedPrefetch();
  Sample next() const override;
  void reset() override;

 private:
  std::shared_ptr<buffer::Buffer> buffer_;
  std::shared_ptr<core::ThreadPool> pool_;
  int64_t prefetch_size_;
  mutable int64_t cursor_ = 0;
  mutable std::vector<std::future<Sample>> ring_;
  mutable std::mutex mu_;
};

// Of every num_partitions consecutive samples keep the one at `partition`.
class Partition : public Stream {
 public:
  Partition(const std::shared_ptr<Stream>& source, int64_t num_partitions, int64_t partition);
  Sample next() const override;
  void reset() override;

 private:
  std::shared_ptr<Stream> source_;
  int64_t num_partitions_, partition_;
  mutable std::mutex mu_;
};

} // namespace stream
} // namespace data
} // namespace mlx
