// Buffer nodes of the transform-and-batch path: FromVector, Transform, Batch,
// Partition (roles of mlx/data/buffer/{FromVector,Transform,Batch,Partition}.h).
#pragma once

#include <memory>
#include <unordered_map>
#include <vector>

#include "mlx/data/buffer/Buffer.h"
#include "mlx/data/core/Batcher.h"
#include "mlx/data/op/Op.h"

namespace mlx {
namespace data {
namespace buffer {

// Samples held in memory.  Empty samples are rejected at construction.
class FromVector : public Buffer {
 public:
  explicit FromVector(const std::vector<Sample>& data);
  explicit FromVector(std::vector<Sample>&& data);
  Sample get(int64_t idx) const override;  // throws std::out_of_range
  int64_t size() const override;

 private:
  void check() const;
  std::vector<Sample> data_;
};

class Transform : public Buffer {
 public:
  Transform(const std::shared_ptr<Buffer>& source, const std::shared_ptr<op::Op>& op);
  Transform(const std::shared_ptr<Buffer>& source, const std::vector<std::shared_ptr<op::Op>>& ops);
  Sample get(int64_t idx) const override;  // an op returning an empty sample is an error here
  int64_t size() const override;
  const std::shared_ptr<Buffer>& source() const { return source_; }
  const std::vector<std::shared_ptr<op::Op>>& ops() const { return ops_; }

 private:
  std::shared_ptr<Buffer> source_;
  std::vector<std::shared_ptr<op::Op>> ops_;
};

// Batches of fixed or listed sizes.  Image ops sitting directly under the
// batch node are absorbed and run fused with it on the GPU.
class Batch : public Buffer {
 public:
  Batch(
      const std::shared_ptr<Buffer>& source, int64_t batch_size,
      const std::unordered_map<std::string, double>& pad_values = {},
      const std::unordered_map<std::string, int>& batch_dims = {});
  Batch(
      const std::shared_ptr<Buffer>& source, const std::vector<int64_t>& batch_sizes,
      const std::unordered_map<std::string, double>& pad_values = {},
      const std::unordered_map<std::string, int>& batch_dims = {});
  Sample get(int64_t idx) const override;
  int64_t size() const override;
  // Same node with one more fused cast.
  std::shared_ptr<Batch> with_cast(const core::CastRequest& cast) const;

 private:
  Batch() = default;
  void absorb(const std::shared_ptr<Buffer>& source,
              const std::unordered_map<std::string, double>& pad_values,
              const std::unordered_map<std::string, int>& batch_dims);
  std::shared_ptr<Buffer> base_;
  std::shared_ptr<core::Batcher> batcher_;
  int64_t batch_size_ = 0;
  std::vector<int64_t> starts_;  // listed sizes: first sample of every batch, plus the end
  int64_t count_ = 0;
};

// Every num_partitions-th sample starting at `partition`.
class Partition : public Buffer {
 public:
  Partition(const std::shared_ptr<Buffer>& source, int64_t num_partitions, int64_t partition);
  Sample get(int64_t idx) const override;
  int64_t size() const override;

 private:
  std::shared_ptr<Buffer> source_;
  int64_t num_partitions_, partition_, size_;
};

// The samples of `source` listed in `perm`, in that order.
class Perm : public Buffer {
 public:
  Perm(const std::shared_ptr<Buffer>& source, const std::vector<int64_t>& perm);
  Sample get(int64_t idx) const override;
  int64_t size() const override;

 private:
  std::shared_ptr<Buffer> source_;
  std::vector<int64_t> perm_;
};

// Size-aware grouping of mlx/data/buffer/DynamicBatch.cpp:68-207: samples are
// ordered by the element count of `key` (stable; only when max_data_size > 0)
// and cut into runs whose padded batch - largest extent per dimension times
// the sample count, or the summed extent along batch_dims[key] - holds between
// min_data_size and max_data_size elements.  Returns the accepted samples in
// batch order, the size of every batch and the samples left out.
struct DynamicGroups {
  std::vector<int64_t> order;
  std::vector<int64_t> batch_sizes;
  std::vector<int64_t> skipped;
};
DynamicGroups dynamic_groups(
    const std::vector<std::vector<int64_t>>& shapes, int64_t min_data_size, int64_t max_data_size,
    bool has_batch_dim, int batch_dim, bool drop_outliers);

// source.dynamic_batch(...): the shapes come from `size_source` (int64 arrays
// under `key`) when given, else from the samples themselves.  `skipped`, when
// given, receives the indices of the samples that ended up in no batch.
std::shared_ptr<Buffer> dynamic_batch(
    const std::shared_ptr<Buffer>& source, const std::shared_ptr<Buffer>& size_source, const std::string& key,
    int64_t min_data_size, int64_t max_data_size, const std::unordered_map<std::string, double>& pad_values,
    const std::unordered_map<std::string, int>& batch_dims, bool drop_outliers,
    std::vector<int64_t>* skipped = nullptr);

// The buffer in a random order drawn from the calling thread's core::State
// (std::shuffle of the identity, as mlx/data/buffer/Shuffle.cpp:16-22 draws it).
std::shared_ptr<Buffer> shuffled(const std::shared_ptr<Buffer>& source);

// Split a chain "source -> Transform(image op) -> ... -> Transform(image op)"
// into its non-image base and the list of image ops above it.
std::shared_ptr<Buffer> peel_image_ops(
    const std::shared_ptr<Buffer>& top, std::vector<std::shared_ptr<op::FusableOp>>& ops);

} // namespace buffer
} // namespace data
} // namespace mlx
