/*
 * TEST INFRASTRUCTURE - CPU oracle, never part of the shipped GPU path.
 *
 * CPU restatement of the 2-D resize that mlx-data reaches through
 * core::image::resize (mlx/data/core/image/ImageTransform.cpp:41-62), i.e. the
 * call stbir_resize_uint8_linear(in, w, h, 0, out, dw, dh, 0, channels) with
 * both default filters forced to the triangle filter
 * (mlx/data/core/image/ImageTransform.cpp:7-10).
 *
 * The routine itself lives in the third-party header stb_image_resize2.h
 * (nothings/stb, pinned at f0569113c93ad095470c54bf34a17b36646bbbb5 by the
 * reference's CMakeLists.txt:20-24), which the reference does not vendor.
 * PARITY UNPINNED: no golden vector of the reference pins this routine; what is
 * restated here is the published behaviour of a separable triangle-filter
 * resampler with clamp-to-edge sampling, written from its mathematical
 * definition, not from that header.
 *
 * Definition, per axis (n source samples -> m output samples), all in float32:
 *   ratio = n / m                       source samples per output sample
 *   u(o)  = (o + 0.5) * ratio - 0.5     centre of output sample o in source space
 *   fs    = min(1, m / n)               tent is stretched when shrinking
 *   R     = max(1, ratio)               tent radius in source samples
 *   taps  i = ceil(u - R) .. floor(u + R),  k_i = max(0, 1 - |i - u| * fs)
 *   w_i   = k_i / sum(k)                normalised in increasing-i order
 *   a tap outside [0, n-1] reads the nearest edge sample (clamp)
 *   m == n is the identity on that axis.
 * The vertical axis is filtered first into a float32 row, the horizontal axis
 * second.  Each sum is a chain acc = fma(w_i, v_i, acc) from acc = 0 in
 * increasing-i order; the result is (int)(acc + 0.5f) clamped to [0, 255].
 */
#ifndef MLXD_ORACLE_RESIZE_RESTATEMENT_H
#define MLXD_ORACLE_RESIZE_RESTATEMENT_H

#include <math.h>
#include <stdint.h>
#include <stdlib.h>

/* Upper bound on the tap count of any output sample of an n -> m axis. */
static inline int mlxd_oracle_axis_cap(int n, int m) {
  if (n <= m) {
    return 4;
  }
  return 2 * (int)ceilf((float)n / (float)m) + 3;
}

typedef struct {
  int first;   /* un-clamped index of the first tap */
  int count;   /* number of taps */
} mlxd_oracle_span;

/* Tap range and normalised weights of output sample o; weights holds cap
 * floats.  Returns 0 on success, -1 when the tap count exceeds cap. */
static inline int mlxd_oracle_axis_taps(
    int n, int m, int o, int cap, mlxd_oracle_span* span, float* weights) {
  if (n == m) {
    span->first = o;
    span->count = 1;
    weights[0] = 1.0f;
    return 0;
  }
  const float ratio = (float)n / (float)m;
  const float scale = (float)m / (float)n;
  const float fs = scale < 1.0f ? scale : 1.0f;
  const float radius = ratio > 1.0f ? ratio : 1.0f;
  const float u = ((float)o + 0.5f) * ratio - 0.5f;
  const int lo = (int)ceilf(u - radius);
  const int hi = (int)floorf(u + radius);
  const int count = hi - lo + 1;
  if (count > cap || count < 1) {
    return -1;
  }
  float sum = 0.0f;
  for (int k = 0; k < count; k++) {
    float d = (float)(lo + k) - u;
    d = d < 0.0f ? -d : d;
    float v = 1.0f - d * fs;
    v = v > 0.0f ? v : 0.0f;
    weights[k] = v;
    sum = sum + v;
  }
  for (int k = 0; k < count; k++) {
    weights[k] = weights[k] / sum;
  }
  span->first = lo;
  span->count = count;
  return 0;
}

/* acc[x] = fma(w, row[x], acc[x]) over a row of bytes. */
#if defined(__x86_64__)
__attribute__((target("fma,avx2")))
#endif
static void mlxd_oracle_row_fma_hw(float* acc, const uint8_t* row, float w, int len) {
  for (int x = 0; x < len; x++) {
    acc[x] = __builtin_fmaf(w, (float)row[x], acc[x]);
  }
}

static void mlxd_oracle_row_fma_sw(float* acc, const uint8_t* row, float w, int len) {
  for (int x = 0; x < len; x++) {
    acc[x] = fmaf(w, (float)row[x], acc[x]);
  }
}

#if defined(__x86_64__)
__attribute__((target("fma,avx2")))
#endif
static void mlxd_oracle_hpass_hw(
    const float* mid, int w, int c, int dw, const int* first, const int* count,
    const float* weights, int cap, uint8_t* out) {
  for (int ox = 0; ox < dw; ox++) {
    const float* wx = weights + (size_t)ox * cap;
    for (int ch = 0; ch < c; ch++) {
      float acc = 0.0f;
      for (int k = 0; k < count[ox]; k++) {
        int sx = first[ox] + k;
        sx = sx < 0 ? 0 : (sx > w - 1 ? w - 1 : sx);
        acc = __builtin_fmaf(wx[k], mid[(size_t)sx * c + ch], acc);
      }
      float r = acc + 0.5f;
      int q = r < 0.0f ? 0 : (r > 255.0f ? 255 : (int)r);
      out[(size_t)ox * c + ch] = (uint8_t)q;
    }
  }
}

static void mlxd_oracle_hpass_sw(
    const float* mid, int w, int c, int dw, const int* first, const int* count,
    const float* weights, int cap, uint8_t* out) {
  for (int ox = 0; ox < dw; ox++) {
    const float* wx = weights + (size_t)ox * cap;
    for (int ch = 0; ch < c; ch++) {
      float acc = 0.0f;
      for (int k = 0; k < count[ox]; k++) {
        int sx = first[ox] + k;
        sx = sx < 0 ? 0 : (sx > w - 1 ? w - 1 : sx);
        acc = fmaf(wx[k], mid[(size_t)sx * c + ch], acc);
      }
      float r = acc + 0.5f;
      int q = r < 0.0f ? 0 : (r > 255.0f ? 255 : (int)r);
      out[(size_t)ox * c + ch] = (uint8_t)q;
    }
  }
}

/* [h, w, c] u8 -> [dh, dw, c] u8, tightly packed rows.  Returns 1 on success
 * and 0 on failure, the convention of the routine it stands in for. */
static int mlxd_oracle_resize_u8(
    const uint8_t* src, int w, int h, uint8_t* dst, int dw, int dh, int c) {
  if (!src || !dst || w <= 0 || h <= 0 || dw <= 0 || dh <= 0 || c <= 0 || c > 4) {
    return 0;
  }
#if defined(__x86_64__)
  const int hw = __builtin_cpu_supports("fma") && __builtin_cpu_supports("avx2");
#else
  const int hw = 0;
#endif
  const int rowlen = w * c;
  float* mid = (float*)malloc(sizeof(float) * (size_t)rowlen);
  int* first = (int*)malloc(sizeof(int) * (size_t)dw);
  int* count = (int*)malloc(sizeof(int) * (size_t)dw);
  const int capx = mlxd_oracle_axis_cap(w, dw);
  const int capy = mlxd_oracle_axis_cap(h, dh);
  float* weights = (float*)malloc(sizeof(float) * (size_t)dw * capx);
  float* wy = (float*)malloc(sizeof(float) * (size_t)capy);
  int ok = mid && first && count && weights && wy;
  for (int ox = 0; ok && ox < dw; ox++) {
    mlxd_oracle_span s;
    if (mlxd_oracle_axis_taps(w, dw, ox, capx, &s, weights + (size_t)ox * capx)) {
      ok = 0;
      break;
    }
    first[ox] = s.first;
    count[ox] = s.count;
  }
  for (int oy = 0; ok && oy < dh; oy++) {
    mlxd_oracle_span s;
    if (mlxd_oracle_axis_taps(h, dh, oy, capy, &s, wy)) {
      ok = 0;
      break;
    }
    for (int x = 0; x < rowlen; x++) {
      mid[x] = 0.0f;
    }
    for (int k = 0; k < s.count; k++) {
      int sy = s.first + k;
      sy = sy < 0 ? 0 : (sy > h - 1 ? h - 1 : sy);
      const uint8_t* row = src + (size_t)sy * rowlen;
      if (hw) {
        mlxd_oracle_row_fma_hw(mid, row, wy[k], rowlen);
      } else {
        mlxd_oracle_row_fma_sw(mid, row, wy[k], rowlen);
      }
    }
    uint8_t* out = dst + (size_t)oy * dw * c;
    if (hw) {
      mlxd_oracle_hpass_hw(mid, w, c, dw, first, count, weights, capx, out);
    } else {
      mlxd_oracle_hpass_sw(mid, w, c, dw, first, count, weights, capx, out);
    }
  }
  free(mid);
  free(first);
  free(count);
  free(weights);
  free(wy);
  return ok;
}

#endif /* MLXD_ORACLE_RESIZE_RESTATEMENT_H */
