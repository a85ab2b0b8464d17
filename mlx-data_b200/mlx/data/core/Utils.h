// Batch assembly (mlx/data/core/Utils.h:29-32).
#pragma once

#include <string>
#include <unordered_map>
#include <vector>

#include "mlx/data/Sample.h"

namespace mlx {
namespace data {
namespace core {

// One batch sample out of many: per key, array::batch with that key's pad
// value (default 0) or, when the key has a batch dimension, concatenation
// along it.  Keys come from the first sample; a later sample missing one of
// them is an error, extra keys are ignored.  uint8 images take the GPU path.
Sample merge_batch(
    const std::vector<Sample>& samples,
    const std::unordered_map<std::string, double>& pad_values = {},
    const std::unordered_map<std::string, int>& batch_dims = {});

} // namespace core
} // namespace data
} // namespace mlx
