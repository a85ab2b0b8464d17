// The fluent op methods shared by Stream and Buffer
// (mlx/data/Dataset.h:22-494, the subset on the image-transform-and-batch
// path).  Every method returns a new pipeline whose top node applies one more
// op; `_if` twins apply it only when `cond` holds.
#pragma once

#include <functional>
#include <memory>
#include <string>
#include <utility>

#include "mlx/data/Array.h"
#include "mlx/data/Sample.h"
#include "mlx/data/op/ImageTransform.h"
#include "mlx/data/op/LoadImage.h"
#include "mlx/data/op/Pad.h"
#include "mlx/data/op/Slice.h"
#include "mlx/data/op/KeyTransform.h"
#include "mlx/data/op/Op.h"

namespace mlx {
namespace data {

// T: the public class (Stream or Buffer); B: its node base class.
// T must provide `T transform_(std::shared_ptr<op::Op>) const`.
template <class T, class B>
class Dataset {
 public:
  explicit Dataset(const std::shared_ptr<B>& self) : self_(self) {}
  const std::shared_ptr<B>& node() const { return self_; }

#define MLXD_IF_TWIN(name, ...)                        \
  if (!cond) {                                         \
    return T(self_);                                   \
  }                                                    \
  return name(__VA_ARGS__)

  T image_center_crop(const std::string& ikey, int64_t w, int64_t h, const std::string& okey = "") const {
    return add_(std::make_shared<op::ImageCenterCrop>(ikey, w, h, okey));
  }
  T image_center_crop_if(bool cond, const std::string& ikey, int64_t w, int64_t h, const std::string& okey = "") const {
    MLXD_IF_TWIN(image_center_crop, ikey, w, h, okey);
  }

  T image_channel_reduction(const std::string& ikey, std::string preset = "default", const std::string& okey = "") const {
    return add_(std::make_shared<op::ImageChannelReduction>(ikey, preset, okey));
  }
  T image_channel_reduction_if(bool cond, const std::string& ikey, std::string preset = "default", const std::string& okey = "") const {
    MLXD_IF_TWIN(image_channel_reduction, ikey, preset, okey);
  }

  T image_random_area_crop(
      const std::string& ikey, std::pair<float, float> area_range, std::pair<float, float> aspect_ratio_range,
      int num_trial = 10, const std::string& okey = "") const {
    return add_(std::make_shared<op::ImageRandomAreaCrop>(ikey, area_range, aspect_ratio_range, num_trial, okey));
  }
  T image_random_area_crop_if(
      bool cond, const std::string& ikey, std::pair<float, float> area_range,
      std::pair<float, float> aspect_ratio_range, int num_trial = 10, const std::string& okey = "") const {
    MLXD_IF_TWIN(image_random_area_crop, ikey, area_range, aspect_ratio_range, num_trial, okey);
  }

  T image_random_crop(const std::string& ikey, int64_t w, int64_t h, const std::string& okey = "") const {
    return add_(std::make_shared<op::ImageRandomCrop>(ikey, w, h, okey));
  }
  T image_random_crop_if(bool cond, const std::string& ikey, int64_t w, int64_t h, const std::string& okey = "") const {
    MLXD_IF_TWIN(image_random_crop, ikey, w, h, okey);
  }

  T image_random_h_flip(const std::string& ikey, float prob, const std::string& okey = "") const {
    return add_(std::make_shared<op::ImageRandomHFlip>(ikey, prob, okey));
  }
  T image_random_h_flip_if(bool cond, const std::string& ikey, float prob, const std::string& okey = "") const {
    MLXD_IF_TWIN(image_random_h_flip, ikey, prob, okey);
  }

  T image_resize(const std::string& ikey, int64_t w, int64_t h, const std::string& okey = "") const {
    return add_(std::make_shared<op::ImageResize>(ikey, w, h, okey));
  }
  T image_resize_if(bool cond, const std::string& ikey, int64_t w, int64_t h, const std::string& okey = "") const {
    MLXD_IF_TWIN(image_resize, ikey, w, h, okey);
  }

  T image_resize_smallest_side(const std::string& ikey, int64_t size, const std::string& okey = "") const {
    return add_(std::make_shared<op::ImageResizeSmallestSide>(ikey, size, okey));
  }
  T image_resize_smallest_side_if(bool cond, const std::string& ikey, int64_t size, const std::string& okey = "") const {
    MLXD_IF_TWIN(image_resize_smallest_side, ikey, size, okey);
  }

  T image_rotate(const std::string& ikey, double angle, bool crop = false, const std::string& okey = "",
                 const std::string& angle_key = "") const {
    return add_(std::make_shared<op::ImageRotate>(ikey, angle, crop, okey, angle_key));
  }
  T image_rotate_if(bool cond, const std::string& ikey, double angle, bool crop = false,
                    const std::string& okey = "", const std::string& angle_key = "") const {
    MLXD_IF_TWIN(image_rotate, ikey, angle, crop, okey, angle_key);
  }

  T pad(const std::string& ikey, int dim, int64_t lpad, int64_t rpad, double pad_value, const std::string& okey = "") const {
    return add_(std::make_shared<op::Pad>(ikey, dim, lpad, rpad, pad_value, okey));
  }
  T pad_if(bool cond, const std::string& ikey, int dim, int64_t lpad, int64_t rpad, double pad_value,
           const std::string& okey = "") const {
    MLXD_IF_TWIN(pad, ikey, dim, lpad, rpad, pad_value, okey);
  }

  T pad_to_multiple(const std::string& ikey, int dim, int64_t pad_multiple, double pad_value,
                    const std::string& okey = "") const {
    return add_(std::make_shared<op::PadToMultiple>(ikey, dim, pad_multiple, pad_value, okey));
  }
  T pad_to_multiple_if(bool cond, const std::string& ikey, int dim, int64_t pad_multiple, double pad_value,
                       const std::string& okey = "") const {
    MLXD_IF_TWIN(pad_to_multiple, ikey, dim, pad_multiple, pad_value, okey);
  }

  T pad_to_size(const std::string& ikey, int dim, const std::vector<int64_t>& sizes, double pad_value,
                const std::string& okey = "") const {
    return add_(std::make_shared<op::PadToSize>(ikey, dim, sizes, pad_value, okey));
  }
  T pad_to_size_if(bool cond, const std::string& ikey, int dim, const std::vector<int64_t>& sizes, double pad_value,
                   const std::string& okey = "") const {
    MLXD_IF_TWIN(pad_to_size, ikey, dim, sizes, pad_value, okey);
  }

  T slice(const std::string& ikey, std::vector<int> dims, std::vector<int64_t> starts, std::vector<int64_t> ends,
          const std::string& okey = "") const {
    return add_(std::make_shared<op::Slice>(ikey, std::move(dims), std::move(starts), std::move(ends), okey));
  }
  T slice_if(bool cond, const std::string& ikey, std::vector<int> dims, std::vector<int64_t> starts,
             std::vector<int64_t> ends, const std::string& okey = "") const {
    MLXD_IF_TWIN(slice, ikey, std::move(dims), std::move(starts), std::move(ends), okey);
  }

  T random_slice(const std::string& ikey, std::vector<int> dims, std::vector<int64_t> sizes,
                 const std::string& okey = "") const {
    return add_(std::make_shared<op::RandomSlice>(ikey, std::move(dims), std::move(sizes), okey));
  }
  T random_slice_if(bool cond, const std::string& ikey, std::vector<int> dims, std::vector<int64_t> sizes,
                    const std::string& okey = "") const {
    MLXD_IF_TWIN(random_slice, ikey, std::move(dims), std::move(sizes), okey);
  }

  T load_image(const std::string& ikey, const std::string& prefix = "", bool info = false,
               const std::string& format = "RGB", bool from_memory = false, const std::string& okey = "") const {
    return add_(std::make_shared<op::LoadImage>(ikey, prefix, info, format, from_memory, okey));
  }
  T load_image_if(bool cond, const std::string& ikey, const std::string& prefix = "", bool info = false,
                  const std::string& format = "RGB", bool from_memory = false, const std::string& okey = "") const {
    MLXD_IF_TWIN(load_image, ikey, prefix, info, format, from_memory, okey);
  }

  T key_transform(const std::string& ikey, op::KeyTransform::Fn fn, const std::string& okey = "") const {
    return add_(std::make_shared<op::KeyTransform>(ikey, std::move(fn), okey));
  }
  T key_transform_if(bool cond, const std::string& ikey, op::KeyTransform::Fn fn, const std::string& okey = "") const {
    MLXD_IF_TWIN(key_transform, ikey, std::move(fn), okey);
  }

  T sample_transform(op::SampleTransform::Fn fn) const {
    return add_(std::make_shared<op::SampleTransform>(std::move(fn)));
  }
  T sample_transform_if(bool cond, op::SampleTransform::Fn fn) const {
    MLXD_IF_TWIN(sample_transform, std::move(fn));
  }

  // Addition to the reference API: the uint8 -> float32 cast as a native op.
  // Directly after batch() it is fused into the batch kernel; anywhere else it
  // runs as its own GPU launch.
  T key_cast(const std::string& ikey, const gpu::CastSpec& spec, const std::string& okey = "") const {
    return static_cast<const T*>(this)->cast_(ikey, spec, okey);
  }
  T key_cast_if(bool cond, const std::string& ikey, const gpu::CastSpec& spec, const std::string& okey = "") const {
    MLXD_IF_TWIN(key_cast, ikey, spec, okey);
  }

#undef MLXD_IF_TWIN

 protected:
  T add_(const std::shared_ptr<op::Op>& op) const { return static_cast<const T*>(this)->transform_(op); }
  std::shared_ptr<B> self_;
};

} // namespace data
} // namespace mlx
