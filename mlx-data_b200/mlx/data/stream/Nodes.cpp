#include "mlx/data/stream/Nodes.h"

#include <algorithm>
#include <stdexcept>

#include "mlx/data/buffer/Nodes.h"

namespace mlx {
namespace data {
namespace stream {

// ------------------------------------------------------------ FromBuffer
Sample FromBuffer::next() const {
  int64_t idx;
  {
    std::lock_guard<std::mutex> g(mu_);
    if (cursor_ >= buffer_->size()) {
      return Sample();
    }
    idx = cursor_++;
  }
  return buffer_->get(idx);
}

void FromBuffer::reset() {
  std::lock_guard<std::mutex> g(mu_);
  cursor_ = 0;
}

// ------------------------------------------------------------ Transform
Sample Transform::next() const {
  for (;;) {
    Sample s = source_->next();
    if (s.empty()) {
      return s;  // source exhausted
    }
    for (auto& op : ops_) {
      s = op->apply(s);
      if (s.empty()) {
        break;  // dropped: pull the next one
      }
    }
    if (!s.empty()) {
      return s;
    }
  }
}

// ------------------------------------------------------------ Batch
namespace {
std::shared_ptr<Stream> peel_image_ops(
    const std::shared_ptr<Stream>& top, std::vector<std::shared_ptr<op::FusableOp>>& ops) {
  std::shared_ptr<Stream> cur = top;
  std::vector<std::vector<std::shared_ptr<op::FusableOp>>> layers;
  for (;;) {
    auto t = std::dynamic_pointer_cast<Transform>(cur);
    if (!t || t->ops().empty()) {
      break;
    }
    std::vector<std::shared_ptr<op::FusableOp>> mine;
    for (auto& o : t->ops()) {
      if (auto io = std::dynamic_pointer_cast<op::FusableOp>(o)) {
        mine.push_back(io);
      }
    }
    if (mine.size() != t->ops().size()) {
      break;  // some other kind of op: the fusable run ends here
    }
    layers.push_back(mine);
    cur = t->source();
  }
  ops.clear();
  for (auto it = layers.rbegin(); it != layers.rend(); ++it) {
    ops.insert(ops.end(), it->begin(), it->end());
  }
  return cur;
}
} // namespace

Batch::Batch(
    const std::shared_ptr<Stream>& source, int64_t batch_size,
    const std::unordered_map<std::string, double>& pad_values,
    const std::unordered_map<std::string, int>& batch_dims)
    : batch_size_(batch_size) {
  if (batch_size <= 0) {
    throw std::runtime_error("Batch: batch size must be positive");
  }
  std::vector<std::shared_ptr<op::FusableOp>> ops;
  base_ = peel_image_ops(source, ops);
  batcher_ = std::make_shared<core::Batcher>(ops, pad_values, batch_dims);
}

std::shared_ptr<Batch> Batch::with_cast(const core::CastRequest& cast) const {
  std::shared_ptr<Batch> b(new Batch());
  b->base_ = base_;
  b->batch_size_ = batch_size_;
  auto casts = batcher_->casts();
  casts.push_back(cast);
  b->batcher_ = std::make_shared<core::Batcher>(
      batcher_->ops(), batcher_->pad_values(), batcher_->batch_dims(), casts);
  return b;
}

Sample Batch::next() const {
  std::vector<Sample> raw;
  raw.reserve(batch_size_);
  {
    std::lock_guard<std::mutex> g(pull_mu_);
    for (int64_t i = 0; i < batch_size_; i++) {
      Sample s = base_->next();
      if (s.empty()) {
        break;
      }
      raw.push_back(std::move(s));
    }
  }
  return batcher_->run(raw);
}

void Batch::reset() {
  std::lock_guard<std::mutex> g(pull_mu_);
  base_->reset();
}

// ------------------------------------------------------------ Prefetch
Prefetch::Prefetch(const std::shared_ptr<Stream>& source, int prefetch_size, int num_thread)
    : source_(source), pool_(std::make_shared<core::ThreadPool>(num_thread)), prefetch_size_(prefetch_size) {
  if (prefetch_size < 0) {
    throw std::runtime_error("Prefetch: prefetch size must be positive");
  }
}

void Prefetch::drain() const {
  while (!inflight_.empty()) {
    try {
      inflight_.front().get();
    } catch (...) {
      // a failed look-ahead is dropped with the rest
    }
    inflight_.pop_front();
  }
}

Prefetch::~Prefetch() {
  std::lock_guard<std::mutex> g(mu_);
  drain();
}

Sample Prefetch::next() const {
  std::lock_guard<std::mutex> g(mu_);
  auto more = [this] { inflight_.push_back(pool_->enqueue([s = source_] { return s->next(); })); };
  while (static_cast<int>(inflight_.size()) < prefetch_size_) {
    more();
  }
  // An empty result may only mean that one worker hit the end early: look at
  // up to prefetch_size results before declaring the stream exhausted.
  Sample res;
  for (int i = 0; i < prefetch_size_; i++) {
    std::future<Sample> head = std::move(inflight_.front());
    inflight_.pop_front();
    more();
    res = head.get();
    if (!res.empty()) {
      break;
    }
  }
  return res;
}

void Prefetch::reset() {
  std::lock_guard<std::mutex> g(mu_);
  drain();
  source_->reset();
}

// ------------------------------------------------------------ OrderedPrefetch
OrderedPrefetch::OrderedPrefetch(const std::shared_ptr<buffer::Buffer>& buffer, int prefetch_size, int num_thread)
    : buffer_(buffer), pool_(std::make_shared<core::ThreadPool>(num_thread)), prefetch_size_(prefetch_size) {
  if (prefetch_size <= 0) {
    throw std::runtime_error("Prefetch: prefetch size must be strictly positive");
  }
}

OrderedPrefetch::~OrderedPrefetch() {
  std::lock_guard<std::mutex> g(mu_);
  for (auto& f : ring_) {
    if (f.valid()) {
      f.wait();
    }
  }
  ring_.clear();
}

Sample OrderedPrefetch::next() const {
  std::future<Sample> mine;
  {
    std::lock_guard<std::mutex> g(mu_);
    const int64_t n = buffer_->size();
    if (ring_.empty()) {
      // slot i % prefetch_size always holds the request for index i
      ring_.resize(prefetch_size_);
      for (int64_t i = cursor_; i < std::min(cursor_ + prefetch_size_, n); i++) {
        ring_[i % prefetch_size_] = pool_->enqueue([b = buffer_, i] { return b->get(i); });
      }
    }
    if (cursor_ >= n) {
      return Sample();
    }
    const int64_t idx = cursor_++;
    const int64_t slot = idx % prefetch_size_;
    mine = std::move(ring_[slot]);
    const int64_t ahead = idx + prefetch_size_;
    if (ahead < n) {
      ring_[slot] = pool_->enqueue([b = buffer_, ahead] { return b->get(ahead); });
    }
  }
  return mine.get();
}

void OrderedPrefetch::reset() {
  std::lock_guard<std::mutex> g(mu_);
  for (auto& f : ring_) {
    if (f.valid()) {
      f.wait();
    }
  }
  ring_.clear();
  cursor_ = 0;
}

// ------------------------------------------------------------ Partition
Partition::Partition(const std::shared_ptr<Stream>& source, int64_t num_partitions, int64_t partition)
    : source_(source), num_partitions_(num_partitions), partition_(partition) {
  if (num_partitions <= 0) {
    throw std::runtime_error("Partition: number of partitions must be positive");
  }
  if (partition < 0 || partition >= num_partitions) {
    throw std::runtime_error("Partition: selected partition is out of range");
  }
}

Sample Partition::next() const {
  std::lock_guard<std::mutex> g(mu_);
  Sample keep;
  for (int64_t i = 0; i < num_partitions_; i++) {
    Sample s = source_->next();
    if (i == partition_) {
      keep = std::move(s);
    }
  }
  return keep;
}

void Partition::reset() {
  std::lock_guard<std::mutex> g(mu_);
  source_->reset();
}

// ------------------------------------------------------------ Repeat
Sample Repeat::next() const {
  {
    std::shared_lock<std::shared_mutex> pulling(mu_);
    Sample s = source_->next();
    if (!s.empty()) {
      return s;
    }
  }
  // The source looked dry.  Whoever gets the exclusive lock first restarts it;
  // the others find samples again when their turn comes.
  std::unique_lock<std::shared_mutex> restarting(mu_);
  Sample s = source_->next();
  if (!s.empty()) {
    return s;
  }
  if (num_time_ > 0 && restarts_ >= num_time_) {
    return s;  // all passes done
  }
  restarts_++;
  source_->reset();
  return source_->next();
}

void Repeat::reset() {
  std::unique_lock<std::shared_mutex> restarting(mu_);
  source_->reset();
  restarts_ = 0;
}

// ------------------------------------------------------------ DynamicBatch
DynamicBatch::DynamicBatch(
    const std::shared_ptr<Stream>& source, int64_t buffer_size, const std::string& key, int64_t min_data_size,
    int64_t max_data_size, const std::unordered_map<std::string, double>& pad_values,
    const std::unordered_map<std::string, int>& batch_dims, bool shuffle, bool drop_outliers,
    int64_t max_skipped_samples, int num_thread)
    : source_(source),
      buffer_size_(buffer_size),
      key_(key),
      min_data_size_(min_data_size),
      max_data_size_(max_data_size),
      pad_values_(pad_values),
      batch_dims_(batch_dims),
      shuffle_(shuffle),
      drop_outliers_(drop_outliers),
      max_skipped_samples_(max_skipped_samples),
      pullers_(std::make_shared<core::ThreadPool>(std::max(num_thread, 1))),
      planner_(std::make_shared<core::ThreadPool>(1)) {
  if (buffer_size <= 0) {
    throw std::runtime_error("DynamicBatch: buffer size must be positive");
  }
  std::vector<std::shared_ptr<op::FusableOp>> ops;
  auto below = peel_image_ops(source, ops);
  bool any_draws = false;
  for (auto& o : ops) {
    any_draws = any_draws || o->draws();
  }
  if (!ops.empty() && !any_draws) {
    source_ = below;
    absorbed_.assign(ops.begin(), ops.end());
  }
}

DynamicBatch::~DynamicBatch() {
  if (next_round_.valid()) {
    next_round_.wait();
  }
  planner_.reset();  // joins; its task is the only user of pullers_ and left_out_
  pullers_.reset();
}

std::shared_ptr<buffer::Buffer> DynamicBatch::make_round() const {
  std::vector<std::future<Sample>> pulls;
  pulls.reserve(buffer_size_);
  for (int64_t i = 0; i < buffer_size_; i++) {
    pulls.push_back(pullers_->enqueue([s = source_] { return s->next(); }));
  }
  std::vector<Sample> samples;
  samples.reserve(buffer_size_ + left_out_.size());
  std::exception_ptr failed;
  for (auto& f : pulls) {
    try {
      Sample s = f.get();
      if (!s.empty()) {
        samples.push_back(std::move(s));
      }
    } catch (...) {
      failed = failed ? failed : std::current_exception();  // still collect the rest: they hold the source
    }
  }
  if (failed) {
    std::rethrow_exception(failed);
  }
  // new samples first, then the ones carried over
  samples.insert(samples.end(), left_out_.begin(), left_out_.end());
  left_out_.clear();

  std::shared_ptr<buffer::Buffer> pulled = std::make_shared<buffer::FromVector>(samples);
  if (!absorbed_.empty()) {
    pulled = std::make_shared<buffer::Transform>(pulled, absorbed_);
  }
  std::vector<int64_t> skipped;
  std::shared_ptr<buffer::Buffer> batches = buffer::dynamic_batch(
      pulled, nullptr, key_, min_data_size_, max_data_size_, pad_values_, batch_dims_, drop_outliers_, &skipped);
  if (max_skipped_samples_ > 0 && static_cast<int64_t>(skipped.size()) > max_skipped_samples_) {
    skipped.resize(max_skipped_samples_);
  }
  for (auto idx : skipped) {
    left_out_.push_back(samples[idx]);
  }
  return shuffle_ ? buffer::shuffled(batches) : batches;
}

std::future<std::shared_ptr<buffer::Buffer>> DynamicBatch::start_round() const {
  return planner_->enqueue([this] { return make_round(); });
}

Sample DynamicBatch::next() const {
  std::lock_guard<std::mutex> g(mu_);
  if (!round_) {
    round_ = start_round().get();
    next_round_ = start_round();
  } else if (round_->size() > 0 && cursor_ >= round_->size()) {
    cursor_ = 0;
    round_ = next_round_.get();
    next_round_ = start_round();
  }
  if (round_->size() == 0) {
    return Sample();  // a round without a batch ends the stream (until reset)
  }
  return round_->get(cursor_++);
}

void DynamicBatch::reset() {
  std::lock_guard<std::mutex> g(mu_);
  if (next_round_.valid()) {
    try {
      next_round_.get();  // its samples are discarded with it
    } catch (...) {
    }
  }
  round_.reset();
  cursor_ = 0;
  source_->reset();
  // samples left out so far stay in line for the next round, as in the reference
}

} // namespace stream
} // namespace data
} // namespace mlx
