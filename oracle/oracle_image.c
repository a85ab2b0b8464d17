/*
 * TEST INFRASTRUCTURE - CPU oracle, never part of the shipped GPU path.
 *
 * Plain C restatement of the per-sample image ops, the batch/pad copy and the
 * uint8 -> float32 cast of mlx-data's image-transform-and-batch path.  Each
 * function names the reference code it follows.  Only tests, the smoke check
 * and the CPU-baseline leg of the benchmark may load this library.
 *
 * Images are [H, W, C] uint8, C-contiguous, exactly the reference's layout
 * (mlx/data/core/image/Image.h:35-49).
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

#include "resize_restatement.h"

#define ORACLE_API __attribute__((visibility("default")))

/* core::image::resize, mlx/data/core/image/ImageTransform.cpp:41-62.
 * Returns 0 on success. */
ORACLE_API int oracle_resize(
    const uint8_t* src, int64_t h, int64_t w, int64_t c,
    uint8_t* dst, int64_t dh, int64_t dw) {
  return mlxd_oracle_resize_u8(src, (int)w, (int)h, dst, (int)dw, (int)dh, (int)c) ? 0 : -1;
}

/* Target size of image_resize_smallest_side: op ImageResizeSmallestSide::apply_image
 * (mlx/data/op/ImageTransform.cpp:78-94) followed by core::image::scale
 * (mlx/data/core/image/ImageTransform.cpp:33-39). */
ORACLE_API void oracle_smallest_side_dims(
    int64_t h, int64_t w, int64_t size, int64_t* dh, int64_t* dw) {
  double scale;
  if (h > w) {
    scale = (double)size / (double)w;
  } else {
    scale = (double)size / (double)h;
  }
  *dw = lround(scale * (double)w);
  *dh = lround(scale * (double)h);
}

/* core::image::crop -> array::sub, mlx/data/core/image/ImageTransform.cpp:64-73
 * and mlx/data/Array.cpp:544-583.  Returns -1 when the window leaves the image. */
ORACLE_API int oracle_crop(
    const uint8_t* src, int64_t h, int64_t w, int64_t c,
    int64_t x, int64_t y, int64_t cw, int64_t ch, uint8_t* dst) {
  if (x < 0 || y < 0 || cw <= 0 || ch <= 0 || x + cw > w || y + ch > h) {
    return -1;
  }
  for (int64_t r = 0; r < ch; r++) {
    memcpy(dst + r * cw * c, src + ((y + r) * w + x) * c, (size_t)(cw * c));
  }
  return 0;
}

/* core::image::hflip, mlx/data/core/image/ImageTransform.cpp:123-140. */
ORACLE_API void oracle_hflip(
    const uint8_t* src, int64_t h, int64_t w, int64_t c, uint8_t* dst) {
  for (int64_t y = 0; y < h; y++) {
    for (int64_t x = 0; x < w; x++) {
      for (int64_t k = 0; k < c; k++) {
        dst[(y * w + x) * c + k] = src[(y * w + (w - x - 1)) * c + k];
      }
    }
  }
}

/* Rotation matrix of core::image::rotate,
 * mlx/data/core/image/ImageTransform.cpp:113-121: pi and the angle in float,
 * cos/sin evaluated in float. */
ORACLE_API void oracle_rotate_matrix(double angle, float mx[6]) {
  const float pi = (float)(atan(1.0) * 4);
  float rangle = (float)(angle * pi / 180.);
  float c = cosf(rangle);
  float s = sinf(rangle);
  mx[0] = c;
  mx[1] = s;
  mx[2] = 0;
  mx[3] = -s;
  mx[4] = c;
  mx[5] = 0;
}

/* core::image::affine, mlx/data/core/image/ImageTransform.cpp:75-111: nearest
 * neighbour, coordinate sums in float then double, truncation toward zero,
 * zero fill outside the source. */
ORACLE_API void oracle_affine(
    const uint8_t* src, int64_t h, int64_t w, int64_t c,
    const float mx[6], int64_t th, int64_t tw, uint8_t* dst) {
  const float twh = (float)(tw / 2.0);
  const float thh = (float)(th / 2.0);
  const float wh = (float)(w / 2.0);
  const float hh = (float)(h / 2.0);
  for (int64_t ty = 0; ty < th; ty++) {
    for (int64_t tx = 0; tx < tw; tx++) {
      float fx = mx[0] * ((float)tx - twh) + mx[1] * ((float)ty - thh) + mx[2];
      float fy = mx[3] * ((float)tx - twh) + mx[4] * ((float)ty - thh) + mx[5];
      int64_t x = (int64_t)((double)fx + 0.5 + (double)wh);
      int64_t y = (int64_t)((double)fy + 0.5 + (double)hh);
      uint8_t* d = dst + (ty * tw + tx) * c;
      if (x < 0 || y < 0 || x >= w || y >= h) {
        memset(d, 0, (size_t)c);
      } else {
        memcpy(d, src + (y * w + x) * c, (size_t)c);
      }
    }
  }
}

/* core::image::channel_reduction, mlx/data/core/image/ImageTransform.cpp:142-182:
 * 16.16 fixed point with truncated coefficients, C int division, clamp. */
ORACLE_API void oracle_channel_reduction(
    const uint8_t* src, int64_t h, int64_t w, float bias, const float m3[3], uint8_t* dst) {
  const int scale = 256 * 256;
  int int_bias = (int)(bias * scale);
  int m[3];
  for (int i = 0; i < 3; i++) {
    m[i] = (int)(m3[i] * scale);
  }
  for (int64_t i = 0; i < h * w; i++) {
    int value = (src[i * 3 + 0] * m[0] + src[i * 3 + 1] * m[1] + src[i * 3 + 2] * m[2] + int_bias) / scale;
    value = value <= 255 ? value : 255;
    value = value >= 0 ? value : 0;
    dst[i] = (uint8_t)value;
  }
}

/* array::batch for uint8 images, mlx/data/Array.cpp:465-498 with
 * core::BatchShape::add (mlx/data/core/BatchShape.cpp:26-45): the slot of every
 * sample is [max_h, max_w, c]; the whole tensor is filled with (uint8)pad and
 * each sample is copied into the top-left corner of its slot. */
ORACLE_API void oracle_batch_pad_u8(
    const uint8_t* const* imgs, const int64_t* hs, const int64_t* ws, int64_t n,
    int64_t c, int64_t max_h, int64_t max_w, double pad, uint8_t* dst) {
  memset(dst, (uint8_t)pad, (size_t)(n * max_h * max_w * c));
  for (int64_t i = 0; i < n; i++) {
    uint8_t* slot = dst + i * max_h * max_w * c;
    for (int64_t y = 0; y < hs[i]; y++) {
      memcpy(slot + y * max_w * c, imgs[i] + y * ws[i] * c, (size_t)(ws[i] * c));
    }
  }
}

/* The cast the reference pipelines run as a Python lambda
 * (README.md:55-57, benchmarks/comparative/caltech101/mlx_data.py:34,46):
 * x.astype(float32) / 255, and with normalisation (x/255 - mean) / std per
 * channel, every step a float32 IEEE operation.  mean == NULL selects the
 * first form.  count is the number of pixels, c the channel count. */
ORACLE_API void oracle_cast_f32(
    const uint8_t* src, int64_t count, int64_t c, const float* mean, const float* std_, float* dst) {
  for (int64_t i = 0; i < count; i++) {
    for (int64_t k = 0; k < c; k++) {
      float v = (float)src[i * c + k] / 255.0f;
      if (mean) {
        float t = v - mean[k];
        v = t / std_[k];
      }
      dst[i * c + k] = v;
    }
  }
}
