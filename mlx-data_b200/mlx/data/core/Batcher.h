// Turns "a run of image ops, then batch, then cast" into one GPU launch per key.
//
// A batch node hands the batcher the raw samples it pulled and the image ops
// that sat between the source and the batch node.  The batcher executes those
// ops symbolically, sample by sample and op by op - the order in which the
// reference pipeline would run them, so random parameters are drawn from
// core::State in the same sequence - and then asks the GPU runtime for each
// key's batch tensor: resize/crop/flip/rotate/gray, pad-to-max-shape, stacking
// and the float32 cast in a single kernel.
#pragma once

#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "mlx/data/Sample.h"
#include "mlx/data/gpu/Runtime.h"
#include "mlx/data/op/ImageTransform.h"

namespace mlx {
namespace data {
namespace core {

struct CastRequest {
  std::string ikey;
  std::string okey;  // empty: replace ikey
  gpu::CastSpec spec;
};

class Batcher {
 public:
  Batcher(
      std::vector<std::shared_ptr<op::FusableOp>> ops,
      std::unordered_map<std::string, double> pad_values,
      std::unordered_map<std::string, int> batch_dims,
      std::vector<CastRequest> casts = {});

  // Empty input gives an empty sample (end of stream).
  Sample run(const std::vector<Sample>& raw) const;

  const std::vector<std::shared_ptr<op::FusableOp>>& ops() const { return ops_; }
  const std::unordered_map<std::string, double>& pad_values() const { return pad_values_; }
  const std::unordered_map<std::string, int>& batch_dims() const { return batch_dims_; }
  const std::vector<CastRequest>& casts() const { return casts_; }
  const gpu::Placement& placement() const { return placement_; }

 private:
  std::vector<std::shared_ptr<op::FusableOp>> ops_;
  std::unordered_map<std::string, double> pad_values_;
  std::unordered_map<std::string, int> batch_dims_;
  std::vector<CastRequest> casts_;
  gpu::Placement placement_;   // the process-wide defaults at the time the node was built
};

// Shape the array at `key` has after `ops` ran on `raw`, without computing
// pixels where the ops fold into an image program (random parameters are drawn
// from core::State exactly as when the ops run for real).  Size-aware batching
// sizes its samples with this instead of one GPU launch per sample.
std::vector<int64_t> folded_shape(
    const std::vector<std::shared_ptr<op::FusableOp>>& ops, const Sample& raw, const std::string& key);

} // namespace core
} // namespace data
} // namespace mlx
