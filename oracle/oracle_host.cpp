/*
 * TEST INFRASTRUCTURE - CPU oracle, never part of the shipped GPU path.
 *
 * Host-side restatement of what mlx-data draws and sizes per sample before any
 * pixel is touched: the random generator state, the random crop / area crop /
 * flip draws and the output size of an affine warp.  These depend on the exact
 * behaviour of libstdc++'s <random> distributions and of <cmath> overloads, so
 * they are restated in C++ against the same headers the reference uses.
 */
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <random>

#define ORACLE_API extern "C" __attribute__((visibility("default")))

namespace {
// One generator, as in core::State (mlx/data/core/State.h:14-17); the oracle is
// single-threaded, so the thread-local copy of mlx/data/core/State.cpp:16-22
// is the generator itself.
std::mt19937 g_gen;
} // namespace

/* core::set_state, mlx/data/core/State.cpp:11-14. */
ORACLE_API void oracle_set_state(int64_t seed) {
  g_gen = std::mt19937(seed);
}

/* ImageRandomHFlip::apply_image, mlx/data/op/ImageTransform.cpp:323-332:
 * one float draw in [0, 1), flip when it is <= prob. */
ORACLE_API int oracle_draw_hflip(float prob) {
  std::uniform_real_distribution<float> uniform{0, 1.0};
  return uniform(g_gen) <= prob ? 1 : 0;
}

/* ImageRandomCrop::generate_random_crop_, mlx/data/op/ImageTransform.cpp:135-150:
 * x drawn before y.  Returns -1 when the target exceeds the image. */
ORACLE_API int oracle_draw_random_crop(
    int64_t w, int64_t h, int64_t cw, int64_t ch, int64_t out[4]) {
  if (ch > h || cw > w) {
    return -1;
  }
  std::uniform_int_distribution<int64_t> x_uniform{0, w - cw};
  std::uniform_int_distribution<int64_t> y_uniform{0, h - ch};
  int64_t x = x_uniform(g_gen);
  int64_t y = y_uniform(g_gen);
  out[0] = x;
  out[1] = y;
  out[2] = cw;
  out[3] = ch;
  return 0;
}

/* ImageRandomAreaCrop::generate_random_crop_,
 * mlx/data/op/ImageTransform.cpp:213-280, including its behaviour when every
 * trial is rejected (the last drawn sizes are kept).  out = {tx, ty, tw, th};
 * all zero means "leave the image unchanged" (:282-291). */
ORACLE_API void oracle_draw_area_crop(
    int64_t w, int64_t h, float area_lo, float area_hi, float ratio_lo, float ratio_hi,
    int num_trial, int64_t out[4]) {
  out[0] = out[1] = out[2] = out[3] = 0;
  const float wf = static_cast<float>(w);
  const float hf = static_cast<float>(h);
  float r = wf / hf;
  if (w == 0 || h == 0) {
    return;
  }
  int64_t wmin = std::ceil(std::sqrt(area_lo * ratio_lo) * wf);
  int64_t wmax = std::floor(std::min(std::sqrt(area_hi * ratio_hi) * wf, wf));
  if (wmin > wmax) {
    return;
  }
  std::uniform_int_distribution<int64_t> w_uniform{wmin, wmax};
  int64_t tw = 0;
  int64_t th = 0;
  for (int trial = 0; trial < num_trial; trial++) {
    tw = w_uniform(g_gen);
    int64_t hmin = std::ceil(std::max(1.0f / (r * ratio_hi) * tw, area_lo * wf * hf / tw));
    int64_t hmax = std::floor(
        std::min(std::min(1.0f / (r * ratio_lo) * tw, area_hi * wf * hf / tw), hf));
    if (hmin > hmax) {
      continue;
    }
    std::uniform_int_distribution<int64_t> h_uniform{hmin, hmax};
    th = h_uniform(g_gen);
    float tr = static_cast<float>(tw) / static_cast<float>(th);
    if ((area_lo * w * h > tw * th) || (area_hi * w * h < tw * th)) {
      continue;
    }
    if ((ratio_lo * r > tr) || (ratio_hi * r < tr)) {
      continue;
    }
    if (tw <= 0 || tw > w) {
      continue;
    }
    if (th <= 0 || th > h) {
      continue;
    }
    break;
  }
  if ((tw == 0) || (th == 0)) {
    return;
  }
  std::uniform_int_distribution<int64_t> x_uniform{0, w - tw};
  std::uniform_int_distribution<int64_t> y_uniform{0, h - th};
  int64_t tx = x_uniform(g_gen);
  int64_t ty = y_uniform(g_gen);
  out[0] = tx;
  out[1] = ty;
  out[2] = tw;
  out[3] = th;
}

/* Output size of core::image::affine,
 * mlx/data/core/image/ImageTransform.cpp:80-86: when not cropping, both sizes
 * are int64 * |float| products summed and truncated; the second line pairs h
 * with mx[3] and w with mx[4], which the reference does too. */
ORACLE_API void oracle_affine_dims(
    int64_t h, int64_t w, const float mx[6], int crop, int64_t* th_out, int64_t* tw_out) {
  int64_t tw = w;
  int64_t th = h;
  if (!crop) {
    tw = w * fabs(mx[0]) + h * fabs(mx[1]);
    th = h * fabs(mx[3]) + w * fabs(mx[4]);
  }
  *tw_out = tw;
  *th_out = th;
}
