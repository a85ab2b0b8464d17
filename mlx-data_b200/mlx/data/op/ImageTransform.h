// The image ops of the transform-and-batch path, same names, constructor
// arguments and error behaviour as mlx/data/op/ImageTransform.h:12-167.
//
// Every op has two faces.  fold() records the op on a LazyImage - drawing any
// random parameter from core::State right there, in the reference's order -
// so that a batch node can run a whole chain for a whole batch as one kernel
// launch.  apply_image() is fold() followed by running the one-op program on
// the GPU immediately; it is what a pipeline without a batch node uses.
#pragma once

#include <string>
#include <utility>

#include "mlx/data/gpu/Runtime.h"
#include "mlx/data/op/KeyTransform.h"

namespace mlx {
namespace data {
namespace op {

class ImageTransformOp : public FusableOp {
 public:
  ImageTransformOp(const std::string& ikey, const std::string& okey = "") : FusableOp(ikey, okey) {}
  Sample apply(const Sample& sample) const override;
  std::shared_ptr<Array> apply_key(const std::shared_ptr<const Array>& src) const override;
  virtual std::shared_ptr<Array> apply_image(const std::shared_ptr<const Array>& image) const;
  virtual std::shared_ptr<Array> apply_video(const std::shared_ptr<const Array>& video) const;

 private:
  // A clip [F, H, W, C]: the op is recorded once, on the first frame - so random
  // parameters are drawn once per clip, as the per-op video variants of
  // mlx-data do (mlx/data/op/ImageTransform.cpp:33-70, 160-182, 293-357) - and
  // every frame runs that program in one launch.
  std::shared_ptr<Array> apply_clip(const std::shared_ptr<const Array>& video, const Sample* sample) const;
};

class ImageResizeSmallestSide : public ImageTransformOp {
 public:
  ImageResizeSmallestSide(const std::string& ikey, int64_t size, const std::string& okey = "")
      : ImageTransformOp(ikey, okey), size_(size) {}
  bool fold(gpu::LazyImage& image) const override;

 private:
  int64_t size_;
};

class ImageResize : public ImageTransformOp {
 public:
  ImageResize(const std::string& ikey, int64_t w, int64_t h, const std::string& okey = "")
      : ImageTransformOp(ikey, okey), w_(w), h_(h) {}
  bool fold(gpu::LazyImage& image) const override;

 private:
  int64_t w_, h_;
};

class ImageCenterCrop : public ImageTransformOp {
 public:
  ImageCenterCrop(const std::string& ikey, int64_t w, int64_t h, const std::string& okey = "")
      : ImageTransformOp(ikey, okey), w_(w), h_(h) {}
  bool fold(gpu::LazyImage& image) const override;

 private:
  int64_t w_, h_;
};

class ImageRandomCrop : public ImageTransformOp {
 public:
  ImageRandomCrop(const std::string& ikey, int64_t w, int64_t h, const std::string& okey = "")
      : ImageTransformOp(ikey, okey), w_(w), h_(h) {}
  bool fold(gpu::LazyImage& image) const override;
  bool draws() const override { return true; }

 private:
  int64_t w_, h_;
};

class ImageRandomAreaCrop : public ImageTransformOp {
 public:
  ImageRandomAreaCrop(
      const std::string& ikey, std::pair<float, float> area_range, std::pair<float, float> aspect_ratio_range,
      int num_trial = 10, const std::string& okey = "");
  bool fold(gpu::LazyImage& image) const override;
  bool draws() const override { return true; }

  struct Rect {
    int64_t tx, ty, tw, th;
  };
  // The rectangle for a w x h image; all zero means "keep the image".
  Rect draw(int64_t w, int64_t h) const;

 private:
  std::pair<float, float> area_;
  std::pair<float, float> ratio_;
  int num_trial_;
};

class ImageRandomHFlip : public ImageTransformOp {
 public:
  ImageRandomHFlip(const std::string& ikey, float prob, const std::string& okey = "")
      : ImageTransformOp(ikey, okey), prob_(prob) {}
  bool fold(gpu::LazyImage& image) const override;
  bool draws() const override { return true; }

 private:
  float prob_;
};

class ImageRotate : public ImageTransformOp {
 public:
  // angle_key (an addition to the reference op, which has one fixed angle per
  // op instance): when not empty, the angle in degrees is read per sample from
  // the float scalar stored under that key.
  ImageRotate(const std::string& ikey, double angle, bool crop = false, const std::string& okey = "",
              const std::string& angle_key = "")
      : ImageTransformOp(ikey, okey), angle_(angle), crop_(crop), angle_key_(angle_key) {}
  bool fold(gpu::LazyImage& image) const override;
  bool fold_in(gpu::LazyImage& image, const Sample& sample) const override;
  bool reads_sample() const override { return !angle_key_.empty(); }

 private:
  bool fold_angle(gpu::LazyImage& image, double angle) const;
  double angle_;
  bool crop_;
  std::string angle_key_;
};

class ImageChannelReduction : public ImageTransformOp {
 public:
  ImageChannelReduction(const std::string& ikey, std::string preset = "default", const std::string& okey = "");
  bool fold(gpu::LazyImage& image) const override;

 private:
  float bias_;
  float m_[3];
};

// uint8 -> float32 cast with scale and optional per-channel normalisation, the
// native form of the Python lambda reference pipelines pass to key_transform
// (README.md:55-57).  Not an image op of the reference: an addition.
class Cast : public KeyTransformOp {
 public:
  Cast(const std::string& ikey, const gpu::CastSpec& spec, const std::string& okey = "")
      : KeyTransformOp(ikey, okey), spec_(spec) {}
  std::shared_ptr<Array> apply_key(const std::shared_ptr<const Array>& src) const override;
  const gpu::CastSpec& spec() const { return spec_; }

 private:
  gpu::CastSpec spec_;
};

} // namespace op
} // namespace data
} // namespace mlx
