#include "mlx/data/core/image/Image.h"

#include <cmath>

#include "mlx/data/gpu/Runtime.h"

namespace mlx {
namespace data {
namespace core {
namespace image {

void verify_image(const std::shared_ptr<const Array>& image) {
  gpu::LazyImage probe(image);  // throws the verifyImage errors
  (void)probe;
}

std::shared_ptr<Array> scale(const std::shared_ptr<const Array>& image, double scale) {
  const int64_t tw = std::lround(scale * width(image));
  const int64_t th = std::lround(scale * height(image));
  return resize(image, tw, th);
}

std::shared_ptr<Array> resize(const std::shared_ptr<const Array>& image, int64_t dw, int64_t dh) {
  gpu::LazyImage lazy(image);
  lazy.resize(dw, dh);
  return lazy.materialise();
}

std::shared_ptr<Array> crop(const std::shared_ptr<const Array>& image, int64_t x, int64_t y, int64_t w, int64_t h) {
  gpu::LazyImage lazy(image);
  lazy.crop(x, y, w, h);
  return lazy.materialise();
}

std::shared_ptr<Array> affine(const std::shared_ptr<const Array>& image, const float mx[6], bool crop) {
  gpu::LazyImage lazy(image);
  const int64_t w = lazy.width();
  const int64_t h = lazy.height();
  int64_t tw = w, th = h;
  if (!crop) {
    tw = static_cast<int64_t>(w * std::fabs(mx[0]) + h * std::fabs(mx[1]));
    th = static_cast<int64_t>(h * std::fabs(mx[3]) + w * std::fabs(mx[4]));
  }
  lazy.affine(mx, tw, th);
  return lazy.materialise();
}

std::shared_ptr<Array> rotate(const std::shared_ptr<const Array>& image, double angle, bool crop) {
  const float pi = static_cast<float>(std::atan(1.0) * 4);
  const float radians = static_cast<float>(angle * pi / 180.);
  const float c = std::cos(radians);
  const float s = std::sin(radians);
  const float mx[6] = {c, s, 0, -s, c, 0};
  return affine(image, mx, crop);
}

std::shared_ptr<Array> hflip(const std::shared_ptr<const Array>& image) {
  gpu::LazyImage lazy(image);
  lazy.hflip();
  return lazy.materialise();
}

std::shared_ptr<Array> channel_reduction(const std::shared_ptr<const Array>& image, const float bias, const float multiplier[3]) {
  gpu::LazyImage lazy(image);
  lazy.channel_reduction(bias, multiplier);
  return lazy.materialise();
}

} // namespace image
} // namespace core
} // namespace data
} // namespace mlx
