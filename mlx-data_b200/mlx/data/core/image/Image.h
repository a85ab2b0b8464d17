// Free-function image transforms with the signatures of
// mlx/data/core/image/Image.h:51-72; every one runs on the GPU through the
// library's C ABI and returns a new uint8 [H, W, C] host array.
#pragma once

#include "mlx/data/Array.h"

namespace mlx {
namespace data {
namespace core {
namespace image {

void verify_image(const std::shared_ptr<const Array>& image);

inline int64_t width(const std::shared_ptr<const Array>& image) { return image->shape()[1]; }
inline int64_t height(const std::shared_ptr<const Array>& image) { return image->shape()[0]; }
inline int64_t channels(const std::shared_ptr<const Array>& image) { return image->shape()[2]; }

std::shared_ptr<Array> scale(const std::shared_ptr<const Array>& image, double scale);
std::shared_ptr<Array> resize(const std::shared_ptr<const Array>& image, int64_t dw, int64_t dh);
std::shared_ptr<Array> crop(const std::shared_ptr<const Array>& image, int64_t x, int64_t y, int64_t w, int64_t h);
std::shared_ptr<Array> affine(const std::shared_ptr<const Array>& image, const float mx[6], bool crop);
std::shared_ptr<Array> rotate(const std::shared_ptr<const Array>& image, double angle, bool crop);
std::shared_ptr<Array> hflip(const std::shared_ptr<const Array>& image);
std::shared_ptr<Array> channel_reduction(const std::shared_ptr<const Array>& image, const float bias, const float multiplier[3]);

} // namespace image
} // namespace core
} // namespace data
} // namespace mlx
