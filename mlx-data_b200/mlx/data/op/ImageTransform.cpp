#include "mlx/data/op/ImageTransform.h"

#include <algorithm>
#include <cmath>
#include <random>
#include <stdexcept>
#include <unordered_map>

#include "mlx/data/core/State.h"

namespace mlx {
namespace data {
namespace op {

Sample KeyTransformOp::apply(const Sample& sample) const {
  auto src = sample::check_key(sample, ikey_, ArrayType::Any);
  Sample res = sample;
  res[output_key()] = apply_key(src);
  return res;
}

// ------------------------------------------------------------ dispatch
Sample ImageTransformOp::apply(const Sample& sample) const {
  if (!reads_sample()) {
    return KeyTransformOp::apply(sample);
  }
  auto src = sample::check_key(sample, ikey_, ArrayType::Any);
  Sample res = sample;
  if (src->ndim() == 4) {
    res[output_key()] = apply_clip(src, &sample);
    return res;
  }
  gpu::LazyImage lazy(src);
  if (!fold_in(lazy, sample)) {
    throw std::runtime_error("ImageTransformOp: internal error: op does not fold into an empty program");
  }
  res[output_key()] = lazy.untouched() ? std::make_shared<Array>(src) : lazy.materialise();
  return res;
}

std::shared_ptr<Array> ImageTransformOp::apply_key(const std::shared_ptr<const Array>& src) const {
  if (src->ndim() == 4) {
    return apply_video(src);
  }
  return apply_image(src);
}

std::shared_ptr<Array> ImageTransformOp::apply_image(const std::shared_ptr<const Array>& image) const {
  gpu::LazyImage lazy(image);
  if (!fold(lazy)) {
    throw std::runtime_error("ImageTransformOp: internal error: op does not fold into an empty program");
  }
  if (lazy.untouched()) {
    // the op decided to leave the image alone: share its storage
    return std::make_shared<Array>(image);
  }
  return lazy.materialise();
}

std::shared_ptr<Array> ImageTransformOp::apply_video(const std::shared_ptr<const Array>& video) const {
  return apply_clip(video, nullptr);
}

std::shared_ptr<Array> ImageTransformOp::apply_clip(
    const std::shared_ptr<const Array>& video, const Sample* sample) const {
  // the checks of core::video::verify_video
  if (video->ndim() != 4) {
    throw std::runtime_error("verifyVideo: video must be 4 dimension Array (FHWC)");
  }
  const int64_t frames = video->shape(0);
  const int64_t h = video->shape(1);
  const int64_t w = video->shape(2);
  const int64_t c = video->shape(3);
  if (c == 0 || c > 4) {
    throw std::runtime_error("verifyVideo: channels must be 0 <= c <= 4");
  }
  if (video->type() != ArrayType::UInt8) {
    throw std::runtime_error("ImageTransformOp: clips must be uint8");
  }
  if (frames == 0) {
    throw std::runtime_error("ImageTransformOp: clip without frames");
  }
  const size_t frame_bytes = static_cast<size_t>(h) * w * c;
  auto frame = [&](int64_t f) {
    // a view of frame f that keeps the clip's storage alive
    std::shared_ptr<void> at(video->storage(), static_cast<uint8_t*>(video->data()) + f * frame_bytes);
    return std::make_shared<const Array>(ArrayType::UInt8, std::vector<int64_t>{h, w, c}, at, video->device());
  };
  gpu::LazyImage first(frame(0));
  const bool ok = sample ? fold_in(first, *sample) : fold(first);
  if (!ok) {
    throw std::runtime_error("ImageTransformOp: internal error: op does not fold into an empty program");
  }
  if (first.untouched()) {
    return std::make_shared<Array>(video);
  }
  std::vector<gpu::LazyImage> all;
  all.reserve(frames);
  all.push_back(first);
  for (int64_t f = 1; f < frames; f++) {
    all.push_back(first.with_source(frame(f)));
  }
  // every frame has the same result size: the "batch" is the clip, nothing is padded
  return gpu::Runtime::get().batch(all, 0.0, nullptr, gpu::Placement());
}

// ------------------------------------------------------------ resize
bool ImageResizeSmallestSide::fold(gpu::LazyImage& image) const {
  if (size_ <= 0) {
    throw std::runtime_error("ImageResizeSmallestSide: illegal target size: " + std::to_string(size_));
  }
  const int64_t w = image.width();
  const int64_t h = image.height();
  // scale from the shorter side, both targets rounded half away from zero
  const double scale = static_cast<double>(size_) / static_cast<double>(h > w ? w : h);
  const int64_t tw = std::lround(scale * w);
  const int64_t th = std::lround(scale * h);
  return image.resize(tw, th);
}

bool ImageResize::fold(gpu::LazyImage& image) const {
  return image.resize(w_, h_);
}

// ------------------------------------------------------------ crops
bool ImageCenterCrop::fold(gpu::LazyImage& image) const {
  const int64_t w = image.width();
  const int64_t h = image.height();
  if (h_ > h || w_ > w) {
    throw std::runtime_error("ImageCenterCrop: target image size larger than input image");
  }
  return image.crop((w - w_) / 2, (h - h_) / 2, w_, h_);
}

bool ImageRandomCrop::fold(gpu::LazyImage& image) const {
  const int64_t w = image.width();
  const int64_t h = image.height();
  if (h_ > h || w_ > w) {
    throw std::runtime_error("ImageRandomCrop: target image size larger than input image");
  }
  auto state = core::get_state();
  // x is drawn before y
  std::uniform_int_distribution<int64_t> draw_x{0, w - w_};
  std::uniform_int_distribution<int64_t> draw_y{0, h - h_};
  const int64_t x = draw_x(state->randomGenerator);
  const int64_t y = draw_y(state->randomGenerator);
  return image.crop(x, y, w_, h_);
}

ImageRandomAreaCrop::ImageRandomAreaCrop(
    const std::string& ikey, std::pair<float, float> area_range, std::pair<float, float> aspect_ratio_range,
    int num_trial, const std::string& okey)
    : ImageTransformOp(ikey, okey), area_(area_range), ratio_(aspect_ratio_range), num_trial_(num_trial) {
  if (area_.first > area_.second || area_.first <= 0 || area_.second > 1.0) {
    throw std::runtime_error("ImageRandomAreaCrop: invalid area range");
  }
  if (ratio_.first > ratio_.second || ratio_.first <= 0) {
    throw std::runtime_error("ImageRandomAreaCrop: invalid aspect ratio range");
  }
  if (area_.first * ratio_.first > 1 || area_.first > ratio_.second) {
    throw std::runtime_error(
        "ImageRandomAreaCrop: provided area range and aspect ratio range cannot be fullfilled");
  }
  if (num_trial_ <= 0) {
    throw std::runtime_error("ImageRandomAreaCrop: number of trial must be positive");
  }
}

// Sampler of mlx/data/op/ImageTransform.cpp:213-280.  All real arithmetic is
// float32 and integers enter it by conversion to float, exactly as there; a
// width is drawn per trial, a height only when its admissible range is not
// empty, and when every trial is rejected the last drawn sizes are used.
ImageRandomAreaCrop::Rect ImageRandomAreaCrop::draw(int64_t w, int64_t h) const {
  const Rect keep{0, 0, 0, 0};
  if (w == 0 || h == 0) {
    return keep;
  }
  const float fw = static_cast<float>(w);
  const float fh = static_cast<float>(h);
  const float aspect = fw / fh;
  const float a_lo = area_.first, a_hi = area_.second;
  const float r_lo = ratio_.first, r_hi = ratio_.second;

  const float w_lo_f = std::sqrt(a_lo * r_lo) * fw;
  const float w_hi_f = std::min(std::sqrt(a_hi * r_hi) * fw, fw);
  const int64_t w_lo = static_cast<int64_t>(std::ceil(w_lo_f));
  const int64_t w_hi = static_cast<int64_t>(std::floor(w_hi_f));
  if (w_lo > w_hi) {
    return keep;
  }
  auto state = core::get_state();
  std::uniform_int_distribution<int64_t> draw_w{w_lo, w_hi};
  int64_t tw = 0, th = 0;
  for (int trial = 0; trial < num_trial_; trial++) {
    tw = draw_w(state->randomGenerator);
    const float ftw = static_cast<float>(tw);
    const float h_from_ratio_hi = 1.0f / (aspect * r_hi) * ftw;
    const float h_from_area_lo = a_lo * fw * fh / ftw;
    const float h_from_ratio_lo = 1.0f / (aspect * r_lo) * ftw;
    const float h_from_area_hi = a_hi * fw * fh / ftw;
    const int64_t h_lo = static_cast<int64_t>(std::ceil(std::max(h_from_ratio_hi, h_from_area_lo)));
    const int64_t h_hi =
        static_cast<int64_t>(std::floor(std::min(std::min(h_from_ratio_lo, h_from_area_hi), fh)));
    if (h_lo > h_hi) {
      continue;  // th keeps its previous value
    }
    std::uniform_int_distribution<int64_t> draw_h{h_lo, h_hi};
    th = draw_h(state->randomGenerator);
    const float got_aspect = static_cast<float>(tw) / static_cast<float>(th);
    const float got_area = static_cast<float>(tw * th);
    const float area_floor = a_lo * static_cast<float>(w) * static_cast<float>(h);
    const float area_ceil = a_hi * static_cast<float>(w) * static_cast<float>(h);
    const bool area_ok = !(area_floor > got_area) && !(area_ceil < got_area);
    const bool aspect_ok = !(r_lo * aspect > got_aspect) && !(r_hi * aspect < got_aspect);
    const bool fits = tw > 0 && tw <= w && th > 0 && th <= h;
    if (area_ok && aspect_ok && fits) {
      break;
    }
  }
  if (tw == 0 || th == 0) {
    return keep;
  }
  std::uniform_int_distribution<int64_t> draw_x{0, w - tw};
  std::uniform_int_distribution<int64_t> draw_y{0, h - th};
  Rect r;
  r.tw = tw;
  r.th = th;
  r.tx = draw_x(state->randomGenerator);
  r.ty = draw_y(state->randomGenerator);
  return r;
}

bool ImageRandomAreaCrop::fold(gpu::LazyImage& image) const {
  const Rect r = draw(image.width(), image.height());
  if (r.tw == 0 || r.th == 0) {
    return true;  // image unchanged
  }
  return image.crop(r.tx, r.ty, r.tw, r.th);
}

// ------------------------------------------------------------ flip
bool ImageRandomHFlip::fold(gpu::LazyImage& image) const {
  auto state = core::get_state();
  std::uniform_real_distribution<float> unit{0, 1.0};
  if (unit(state->randomGenerator) <= prob_) {
    return image.hflip();
  }
  return true;
}

// ------------------------------------------------------------ rotate
bool ImageRotate::fold(gpu::LazyImage& image) const {
  if (!angle_key_.empty()) {
    throw std::runtime_error("ImageRotate: the angle comes from key <" + angle_key_ + ">, a sample is needed");
  }
  return fold_angle(image, angle_);
}

bool ImageRotate::fold_in(gpu::LazyImage& image, const Sample& sample) const {
  if (angle_key_.empty()) {
    return fold_angle(image, angle_);
  }
  auto a = sample::check_key(sample, angle_key_, ArrayType::Any);
  double angle;
  if (a->type() == Double) {
    angle = a->scalar<double>();
  } else if (a->type() == Float) {
    angle = a->scalar<float>();
  } else if (a->type() == Int64) {
    angle = static_cast<double>(a->scalar<int64_t>());
  } else {
    throw std::runtime_error("ImageRotate: the angle at key <" + angle_key_ + "> must be a float scalar");
  }
  return fold_angle(image, angle);
}

bool ImageRotate::fold_angle(gpu::LazyImage& image, double angle_) const {
  // pi, the angle in radians, cos and sin are float32; the matrix is
  // {c, s, 0, -s, c, 0} (mlx/data/core/image/ImageTransform.cpp:113-121).
  const float pi = static_cast<float>(std::atan(1.0) * 4);
  const float radians = static_cast<float>(angle_ * pi / 180.);
  const float c = std::cos(radians);
  const float s = std::sin(radians);
  const float mx[6] = {c, s, 0, -s, c, 0};
  const int64_t w = image.width();
  const int64_t h = image.height();
  int64_t tw = w, th = h;
  if (!crop_) {
    // Output size when not cropping (:80-86): integer sizes times float32
    // magnitudes, summed in float32, truncated.  The second line pairs h with
    // mx[3] and w with mx[4], so both sizes come out equal.
    tw = static_cast<int64_t>(w * std::fabs(mx[0]) + h * std::fabs(mx[1]));
    th = static_cast<int64_t>(h * std::fabs(mx[3]) + w * std::fabs(mx[4]));
  }
  return image.affine(mx, tw, th);
}

// ------------------------------------------------------------ gray
namespace {
struct Mix {
  float bias;
  float m[3];
};
const std::unordered_map<std::string, Mix>& presets() {
  // Full-range luma mixes (mlx/data/op/ImageTransform.cpp:384-404).
  static const std::unordered_map<std::string, Mix> p = {
      {"default", {0, {0.299, 0.587, 0.114}}},
      {"rec601", {0, {0.299, 0.587, 0.114}}},
      {"rec709", {0, {0.2126, 0.7152, 0.0722}}},
      {"rec2020", {0, {0.2627, 0.678, 0.0593}}},
      {"green", {0, {0, 1, 0}}},
  };
  return p;
}
} // namespace

ImageChannelReduction::ImageChannelReduction(const std::string& ikey, std::string preset, const std::string& okey)
    : ImageTransformOp(ikey, okey) {
  auto it = presets().find(preset);
  if (it == presets().end()) {
    throw std::runtime_error("ImageChannelReduction: unable to find preset " + preset);
  }
  bias_ = it->second.bias;
  for (int i = 0; i < 3; i++) {
    m_[i] = it->second.m[i];
  }
}

bool ImageChannelReduction::fold(gpu::LazyImage& image) const {
  return image.channel_reduction(bias_, m_);
}

// ------------------------------------------------------------ cast
std::shared_ptr<Array> Cast::apply_key(const std::shared_ptr<const Array>& src) const {
  return gpu::Runtime::get().cast(src, spec_);
}

} // namespace op
} // namespace data
} // namespace mlx
