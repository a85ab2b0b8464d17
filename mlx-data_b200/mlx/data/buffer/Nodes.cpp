#include "mlx/data/buffer/Nodes.h"

#include <algorithm>
#include <stdexcept>

#include "mlx/data/core/State.h"

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
    const std::shared_ptr<Buffer>& top, std::vector<std::shared_ptr<op::FusableOp>>& ops) {
  std::shared_ptr<Buffer> cur = top;
  std::vector<std::shared_ptr<op::FusableOp>> rev;
  for (;;) {
    auto t = std::dynamic_pointer_cast<Transform>(cur);
    if (!t) {
      break;
    }
    std::vector<std::shared_ptr<op::FusableOp>> mine;
    for (auto& o : t->ops()) {
      auto io = std::dynamic_pointer_cast<op::FusableOp>(o);
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
  std::vector<std::shared_ptr<op::FusableOp>> ops;
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

// ------------------------------------------------------------ Perm
Perm::Perm(const std::shared_ptr<Buffer>& source, const std::vector<int64_t>& perm) : source_(source), perm_(perm) {
  const int64_t n = source->size();
  for (auto i : perm_) {
    if (i < 0 || i >= n) {
      throw std::runtime_error("Perm: index out of range");
    }
  }
}

Sample Perm::get(int64_t idx) const {
  if (idx < 0 || idx >= static_cast<int64_t>(perm_.size())) {
    throw std::out_of_range("Perm: index out of range");
  }
  return source_->get(perm_[idx]);
}

int64_t Perm::size() const {
  return static_cast<int64_t>(perm_.size());
}

// ------------------------------------------------------------ dynamic batching
namespace {

// Shape of the batch that a run of samples would make (the bookkeeping of
// mlx/data/core/BatchShape.cpp:26-66): a leading sample count over the largest
// extents, or - with a batch dimension - extents summed along it.
class RunShape {
 public:
  RunShape(bool has_dim, int dim) : has_dim_(has_dim), dim_(dim) {}

  void add(const std::vector<int64_t>& shape) {
    const int64_t nd = static_cast<int64_t>(shape.size());
    if (!has_dim_) {
      if (count_ == 0) {
        shape_.assign(nd + 1, 0);
        std::copy(shape.begin(), shape.end(), shape_.begin() + 1);
      } else {
        if (nd + 1 != static_cast<int64_t>(shape_.size())) {
          throw std::runtime_error("BatchShape: batched arrays expected to have consistent shapes");
        }
        for (int64_t d = 0; d < nd; d++) {
          shape_[d + 1] = std::max(shape_[d + 1], shape[d]);
        }
      }
      shape_[0] += 1;
    } else {
      const int64_t dim = dim_ < 0 ? nd + dim_ : dim_;
      if (dim >= nd) {
        throw std::runtime_error("BatchShape: dimension out of bound");
      }
      if (count_ == 0) {
        shape_ = shape;
      } else {
        if (nd != static_cast<int64_t>(shape_.size())) {
          throw std::runtime_error("BatchShape: batched arrays expected to have consistent shapes");
        }
        for (int64_t d = 0; d < nd; d++) {
          shape_[d] = d == dim ? shape_[d] + shape[d] : std::max(shape_[d], shape[d]);
        }
      }
    }
    count_++;
  }

  int64_t elements() const {
    int64_t n = 1;
    for (auto d : shape_) {
      n *= d;
    }
    return n;
  }

  int64_t count() const { return count_; }

  void clear() {
    shape_.clear();
    count_ = 0;
  }

 private:
  bool has_dim_;
  int dim_;
  std::vector<int64_t> shape_;
  int64_t count_ = 0;
};

} // namespace

// The grouping rule, stated over the (size-ordered) sequence of samples:
//
//   a run starts at the first sample not yet placed and grows one sample at a
//   time; after every sample the padded size of the run is looked at and the
//   run ends by one of four verdicts, else keeps growing.
//     Emit      - both limits are given and the size lies between them;
//                 also a lone sample over the upper limit when outliers are kept
//     Drop      - a lone sample over the upper limit when outliers are dropped
//     EmitShort - over the upper limit and no lower limit: the run without its
//                 last sample is a batch; the last sample starts the next run
//                 and is not looked at on its own there (so an oversized
//                 sample arriving this way leaves as a batch of one when the
//                 next sample comes, whatever drop_outliers says)
//     LeaveOut  - over the upper limit with a lower limit (the run was too
//                 small before this sample and is too large with it)
//   A run still growing when the samples end is emitted if it respects the
//   limits that are given and left out otherwise.
//
// This restates what mlx/data/buffer/DynamicBatch.cpp:101-204 computes (same
// batches, same skipped samples, in the same order); the statement above is
// the specification, the reference is where it was read from.
namespace {
enum class Verdict { Grow, Emit, Drop, EmitShort, LeaveOut };

struct Limits {
  int64_t lo, hi;  // <= 0: not given
  bool drop_outliers;

  bool above(int64_t size) const { return hi > 0 && size > hi; }
  bool respects(int64_t size) const { return (lo <= 0 || size >= lo) && !above(size); }

  Verdict after_adding(int64_t size, int64_t run_length, bool inherited_first) const {
    if (run_length == 1 && inherited_first) {
      return Verdict::Grow;
    }
    if (lo > 0 && hi > 0 && respects(size)) {
      return Verdict::Emit;
    }
    if (!above(size)) {
      return Verdict::Grow;
    }
    if (run_length == 1) {
      return drop_outliers ? Verdict::Drop : Verdict::Emit;
    }
    return lo > 0 ? Verdict::LeaveOut : Verdict::EmitShort;
  }
};
} // namespace

DynamicGroups dynamic_groups(
    const std::vector<std::vector<int64_t>>& shapes, int64_t min_data_size, int64_t max_data_size,
    bool has_batch_dim, int batch_dim, bool drop_outliers) {
  const int64_t n = static_cast<int64_t>(shapes.size());
  std::vector<int64_t> by_size(n);
  for (int64_t i = 0; i < n; i++) {
    by_size[i] = i;
  }
  if (max_data_size > 0) {
    // an array without dimensions counts as empty here
    std::vector<int64_t> volume(n, 0);
    for (int64_t i = 0; i < n; i++) {
      if (!shapes[i].empty()) {
        volume[i] = 1;
        for (auto d : shapes[i]) {
          volume[i] *= d;
        }
      }
    }
    std::stable_sort(by_size.begin(), by_size.end(), [&](int64_t a, int64_t b) { return volume[a] < volume[b]; });
  }

  const Limits limits{min_data_size, max_data_size, drop_outliers};
  DynamicGroups out;
  out.order.reserve(n);
  auto emit = [&](int64_t first, int64_t past) {
    out.batch_sizes.push_back(past - first);
    out.order.insert(out.order.end(), by_size.begin() + first, by_size.begin() + past);
  };
  auto leave_out = [&](int64_t first, int64_t past) {
    out.skipped.insert(out.skipped.end(), by_size.begin() + first, by_size.begin() + past);
  };

  int64_t first = 0;  // where the current run starts in by_size
  bool inherited_first = false;  // the run's first sample is the one an EmitShort pushed out
  while (first < n) {
    RunShape run(has_batch_dim, batch_dim);
    Verdict verdict = Verdict::Grow;
    int64_t past = first;  // one past the run's last sample
    while (past < n && verdict == Verdict::Grow) {
      run.add(shapes[by_size[past++]]);
      verdict = limits.after_adding(run.elements(), past - first, inherited_first);
    }
    inherited_first = verdict == Verdict::EmitShort;
    switch (verdict) {
      case Verdict::Grow:  // the samples ended first
        if (limits.respects(run.elements())) {
          emit(first, past);
        } else {
          leave_out(first, past);
        }
        break;
      case Verdict::Emit:
        emit(first, past);
        break;
      case Verdict::Drop:
        break;
      case Verdict::EmitShort:
        past -= 1;
        emit(first, past);
        break;
      case Verdict::LeaveOut:
        leave_out(first, past);
        break;
    }
    first = past;
  }
  return out;
}

std::shared_ptr<Buffer> dynamic_batch(
    const std::shared_ptr<Buffer>& source, const std::shared_ptr<Buffer>& size_source, const std::string& key,
    int64_t min_data_size, int64_t max_data_size, const std::unordered_map<std::string, double>& pad_values,
    const std::unordered_map<std::string, int>& batch_dims, bool drop_outliers, std::vector<int64_t>* skipped) {
  const int64_t n = source->size();
  if (size_source && size_source->size() != n) {
    throw std::runtime_error("DynamicBatch: buffer and reference size buffer do not match in size");
  }
  // the image ops on top of the source: sized symbolically here, fused into the batches below
  std::vector<std::shared_ptr<op::FusableOp>> ops;
  const std::shared_ptr<Buffer> base = peel_image_ops(source, ops);
  std::vector<std::vector<int64_t>> shapes(n);
  for (int64_t i = 0; i < n; i++) {
    if (size_source) {
      auto arr = sample::check_key(size_source->get(i), key, ArrayType::Int64);
      const int64_t* v = arr->data<int64_t>();
      shapes[i].assign(v, v + arr->size());
    } else if (!ops.empty()) {
      shapes[i] = core::folded_shape(ops, base->get(i), key);
    } else {
      shapes[i] = sample::check_key(source->get(i), key, ArrayType::Any)->shape();
    }
  }
  const auto dim = batch_dims.find(key);
  const DynamicGroups g = dynamic_groups(
      shapes, min_data_size, max_data_size, dim != batch_dims.end(), dim != batch_dims.end() ? dim->second : 0,
      drop_outliers);
  if (skipped) {
    *skipped = g.skipped;
  }
  // keep the image ops on top of the permutation, where Batch can fuse them
  std::shared_ptr<Buffer> top = std::make_shared<Perm>(base, g.order);
  if (!ops.empty()) {
    std::vector<std::shared_ptr<op::Op>> generic(ops.begin(), ops.end());
    top = std::make_shared<Transform>(top, generic);
  }
  return std::make_shared<Batch>(top, g.batch_sizes, pad_values, batch_dims);
}

std::shared_ptr<Buffer> shuffled(const std::shared_ptr<Buffer>& source) {
  std::vector<int64_t> order(source->size());
  for (size_t i = 0; i < order.size(); i++) {
    order[i] = static_cast<int64_t>(i);
  }
  std::shuffle(order.begin(), order.end(), core::get_state()->randomGenerator);
  return std::make_shared<Perm>(source, order);
}

} // namespace buffer
} // namespace data
} // namespace mlx
