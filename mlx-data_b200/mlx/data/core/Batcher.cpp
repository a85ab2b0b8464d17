#include "mlx/data/core/Batcher.h"

#include <map>
#include <stdexcept>

#include "mlx/data/core/Utils.h"

namespace mlx {
namespace data {
namespace core {

namespace {

// A sample whose image entries may still be programs rather than pixels.
struct Entry {
  std::shared_ptr<Array> array;            // set when concrete
  std::shared_ptr<gpu::LazyImage> lazy;    // set when pending
};
using LazySample = std::unordered_map<std::string, Entry>;

bool gpu_image(const std::shared_ptr<Array>& a) {
  return a && a->type() == UInt8 && a->ndim() == 3 && a->shape(2) >= 1 && a->shape(2) <= 4 && a->size() > 0;
}

std::shared_ptr<Array> lazy_pixels(const Entry& e) {
  if (e.array) {
    return e.array;
  }
  if (e.lazy->untouched()) {
    return std::make_shared<Array>(e.lazy->source());
  }
  return e.lazy->materialise();
}

void run_op(LazySample& s, const op::FusableOp& op) {
  auto it = s.find(op.input_key());
  if (it == s.end()) {
    throw std::runtime_error("key <" + op.input_key() + "> expected");
  }
  Entry in = it->second;
  Entry out;
  if (!in.lazy && !gpu_image(in.array)) {
    // videos, non-uint8 arrays, token arrays, malformed images: the op decides (and throws)
    out.array = op.apply_key(in.array);
  } else {
    auto lazy = in.lazy ? std::make_shared<gpu::LazyImage>(*in.lazy) : std::make_shared<gpu::LazyImage>(in.array);
    Sample concrete_entries;
    if (op.reads_sample()) {
      for (auto& kv : s) {
        if (kv.second.array) {
          concrete_entries[kv.first] = kv.second.array;
        }
      }
    }
    // An image that claims padding takes no further op except more padding:
    // compute it before the op gets to draw anything.
    bool joined = !(lazy->extended() && !op.extends_only()) && op.fold_in(*lazy, concrete_entries);
    if (!joined && !lazy->untouched()) {
      // the program is full: compute what we have, start a new one
      auto pixels = lazy_pixels(in);
      lazy = std::make_shared<gpu::LazyImage>(pixels);
      joined = op.fold_in(*lazy, concrete_entries);
    }
    if (joined) {
      out.lazy = lazy;
    } else {
      // not an op the kernels run (padding in front, a slice of the channels): the host op on the pixels
      out.array = op.apply_key(lazy_pixels(in));
    }
  }
  s[op.output_key()] = out;
}

} // namespace

Batcher::Batcher(
    std::vector<std::shared_ptr<op::FusableOp>> ops,
    std::unordered_map<std::string, double> pad_values,
    std::unordered_map<std::string, int> batch_dims,
    std::vector<CastRequest> casts)
    : ops_(std::move(ops)),
      pad_values_(std::move(pad_values)),
      batch_dims_(std::move(batch_dims)),
      casts_(std::move(casts)),
      placement_(gpu::Runtime::get().placement()) {}

Sample Batcher::run(const std::vector<Sample>& raw) const {
  if (raw.empty()) {
    return Sample();
  }
  // 1. symbolic execution, sample-major like a pull pipeline
  std::vector<LazySample> lazy(raw.size());
  for (size_t i = 0; i < raw.size(); i++) {
    for (auto& kv : raw[i]) {
      lazy[i][kv.first].array = kv.second;
    }
    for (auto& op : ops_) {
      run_op(lazy[i], *op);
    }
  }
  // 2. per key of the first sample: one batch tensor
  Sample out;
  for (auto& first_kv : lazy.front()) {
    const std::string& key = first_kv.first;
    std::vector<Entry> col;
    col.reserve(lazy.size());
    for (auto& s : lazy) {
      auto it = s.find(key);
      if (it == s.end()) {
        throw std::runtime_error("mergeBatch: inconsistent sample keys in batch (unknown key: <" + key + ">)");
      }
      col.push_back(it->second);
    }
    double pad = 0.0;
    if (auto p = pad_values_.find(key); p != pad_values_.end()) {
      pad = p->second;
    }
    const auto dim = batch_dims_.find(key);
    bool on_gpu = dim == batch_dims_.end();
    for (auto& e : col) {
      on_gpu = on_gpu && (e.lazy || gpu_image(e.array));
    }
    if (on_gpu) {
      std::vector<gpu::LazyImage> images;
      images.reserve(col.size());
      bool same = true;
      for (auto& e : col) {
        if (e.lazy && !e.lazy->extension_matches(pad)) {
          // explicit padding with another value than the batch's: that image is computed on its own first
          images.push_back(gpu::LazyImage(e.lazy->materialise()));
        } else {
          images.push_back(e.lazy ? *e.lazy : gpu::LazyImage(e.array));
        }
        same = same && images.back().source_channels() == images.front().source_channels() &&
            images.back().is_gray() == images.front().is_gray();
      }
      if (!same) {
        throw std::runtime_error("BatchShape: batched arrays expected to have consistent shapes");
      }
      bool replaced = false;
      for (auto& c : casts_) {
        if (c.ikey != key) {
          continue;
        }
        auto f32 = gpu::Runtime::get().batch(images, pad, &c.spec, placement_);
        if (c.okey.empty() || c.okey == key) {
          out[key] = f32;
          replaced = true;
        } else {
          out[c.okey] = f32;
        }
      }
      if (!replaced) {
        out[key] = gpu::Runtime::get().batch(images, pad, nullptr, placement_);
      }
      continue;
    }
    std::vector<std::shared_ptr<Array>> arrs;
    arrs.reserve(col.size());
    for (auto& e : col) {
      arrs.push_back(lazy_pixels(e));
    }
    std::shared_ptr<Array> merged =
        dim == batch_dims_.end() ? array::batch(arrs, pad) : array::batch(arrs, dim->second, pad);
    out[key] = merged;
    for (auto& c : casts_) {
      if (c.ikey == key) {
        out[c.okey.empty() ? key : c.okey] = gpu::Runtime::get().cast(merged, c.spec);
      }
    }
  }
  return out;
}

std::vector<int64_t> folded_shape(
    const std::vector<std::shared_ptr<op::FusableOp>>& ops, const Sample& raw, const std::string& key) {
  LazySample lazy;
  for (auto& kv : raw) {
    lazy[kv.first].array = kv.second;
  }
  for (auto& op : ops) {
    run_op(lazy, *op);
  }
  auto it = lazy.find(key);
  if (it == lazy.end()) {
    throw std::runtime_error("key <" + key + "> expected");
  }
  if (it->second.lazy) {
    const auto& im = *it->second.lazy;
    return {im.height(), im.width(), im.channels()};
  }
  return it->second.array->shape();
}

Sample merge_batch(
    const std::vector<Sample>& samples,
    const std::unordered_map<std::string, double>& pad_values,
    const std::unordered_map<std::string, int>& batch_dims) {
  return Batcher({}, pad_values, batch_dims).run(samples);
}

} // namespace core
} // namespace data
} // namespace mlx
