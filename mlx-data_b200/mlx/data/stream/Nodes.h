// Stream nodes of the transform-and-batch path: FromBuffer, Transform, Batch,
// DynamicBatch, Prefetch, OrderedPrefetch, Partition, Repeat (roles of the
// same-named files under mlx/data/stream/).
#pragma once

#include <deque>
#include <future>
#include <memory>
#include <mutex>
#include <shared_mutex>
#include <string>
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

// Start the source over when it runs dry: num_time more passes after the
// first, without end when num_time <= 0 (mlx/data/stream/Repeat.cpp:14-48).
class Repeat : public Stream {
 public:
  Repeat(const std::shared_ptr<Stream>& source, int64_t num_time) : source_(source), num_time_(num_time) {}
  Sample next() const override;
  void reset() override;

 private:
  std::shared_ptr<Stream> source_;
  int64_t num_time_;
  mutable int64_t restarts_ = 0;
  mutable std::shared_mutex mu_;  // shared: pulling; exclusive: restarting the source
};

// Size-aware batching over a stream (mlx/data/stream/DynamicBatch.cpp:35-70 on
// top of stream/Buffered.cpp:22-98): pull `buffer_size` samples, append the
// samples the previous round left out, group them with buffer::dynamic_batch,
// optionally shuffle the batches, hand them out one by one; then pull again.
// Samples a round leaves out (at most max_skipped_samples of them when that is
// positive) get another chance in the next round.  The stream ends with the
// first round that yields no batch.  The next round is prepared on a worker
// thread while the current one is handed out; its samples are pulled by
// num_thread workers.  A run of fusable ops directly under this node that draw
// nothing at random is absorbed: raw samples are pulled, sized symbolically and
// the ops run fused with each batch.  With an op that draws (random crop, flip,
// slice) samples are taken as the source delivers them - the ops have run by
// then, so the sizes that drive the grouping are the sizes that get batched -
// and padding and stacking of image keys still run as one launch per batch.
class DynamicBatch : public Stream {
 public:
  DynamicBatch(
      const std::shared_ptr<Stream>& source, int64_t buffer_size, const std::string& key, int64_t min_data_size,
      int64_t max_data_size, const std::unordered_map<std::string, double>& pad_values,
      const std::unordered_map<std::string, int>& batch_dims, bool shuffle, bool drop_outliers,
      int64_t max_skipped_samples, int num_thread);
  ~DynamicBatch();
  Sample next() const override;
  void reset() override;

 private:
  std::shared_ptr<buffer::Buffer> make_round() const;
  std::future<std::shared_ptr<buffer::Buffer>> start_round() const;

  std::shared_ptr<Stream> source_;                       // what samples are pulled from
  std::vector<std::shared_ptr<op::Op>> absorbed_;        // deterministic fusable ops re-applied above each round
  int64_t buffer_size_;
  std::string key_;
  int64_t min_data_size_, max_data_size_;
  std::unordered_map<std::string, double> pad_values_;
  std::unordered_map<std::string, int> batch_dims_;
  bool shuffle_, drop_outliers_;
  int64_t max_skipped_samples_;
  std::shared_ptr<core::ThreadPool> pullers_;               // num_thread workers calling the source
  std::shared_ptr<core::ThreadPool> planner_;               // one worker building the next round
  mutable std::vector<Sample> left_out_;                    // only touched by the planner thread's task
  mutable std::shared_ptr<buffer::Buffer> round_;
  mutable std::future<std::shared_ptr<buffer::Buffer>> next_round_;
  mutable int64_t cursor_ = 0;
  mutable std::mutex mu_;
};

} // namespace stream
} // namespace data
} // namespace mlx
