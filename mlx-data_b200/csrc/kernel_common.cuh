// Device helpers shared by the two kernels of the library.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "fused_batch.h"

namespace mlxd {

__device__ __forceinline__ int clampi(int v, int lo, int hi) {
  return v < lo ? lo : (v > hi ? hi : v);
}

// Geometry of one axis of a triangle-filter resize, n source -> m output
// samples.  Every step is one correctly rounded float32 operation in a fixed
// order (no contraction), so host and device agree bit for bit:
//   ratio = n / m, u(o) = (o + 0.5) * ratio - 0.5, radius = max(1, ratio),
//   taps i = ceil(u - radius) .. floor(u + radius),
//   k_i = max(0, 1 - |i - u| * min(1, m / n)), w_i = k_i / sum(k).
struct Axis {
  float ratio, fs, radius;
  bool identity;
};

__device__ __forceinline__ Axis make_axis(int n, int m) {
  Axis a;
  a.identity = n == m;
  a.ratio = __fdiv_rn((float)n, (float)m);
  const float scale = __fdiv_rn((float)m, (float)n);
  a.fs = scale < 1.0f ? scale : 1.0f;
  a.radius = a.ratio > 1.0f ? a.ratio : 1.0f;
  return a;
}

__device__ __forceinline__ float axis_center(const Axis& a, int o) {
  return __fsub_rn(__fmul_rn(__fadd_rn((float)o, 0.5f), a.ratio), 0.5f);
}

// Un-clamped first and last tap of output sample o.
__device__ __forceinline__ void axis_range(const Axis& a, int o, int& lo, int& hi) {
  if (a.identity) {
    lo = hi = o;
    return;
  }
  const float u = axis_center(a, o);
  lo = (int)ceilf(__fsub_rn(u, a.radius));
  hi = (int)floorf(__fadd_rn(u, a.radius));
}

// Un-normalised tent value of source sample i for the output centred at u.
__device__ __forceinline__ float axis_tent(const Axis& a, float u, int i) {
  const float d = fabsf(__fsub_rn((float)i, u));
  const float v = __fsub_rn(1.0f, __fmul_rn(d, a.fs));
  return v > 0.0f ? v : 0.0f;
}

// Tap range and normalised weights of output sample o; at most cap taps.
__device__ __forceinline__ void axis_taps(
    int n, int m, int o, int cap, int& first, int& count, float* w) {
  if (n == m) {
    first = o;
    count = 1;
    w[0] = 1.0f;
    return;
  }
  const Axis a = make_axis(n, m);
  const float u = axis_center(a, o);
  int lo, hi;
  axis_range(a, o, lo, hi);
  int cnt = hi - lo + 1;
  cnt = cnt > cap ? cap : cnt;
  float sum = 0.0f;
  for (int k = 0; k < cnt; k++) {
    const float v = axis_tent(a, u, lo + k);
    w[k] = v;
    sum = __fadd_rn(sum, v);
  }
  for (int k = 0; k < cnt; k++) {
    w[k] = __fdiv_rn(w[k], sum);
  }
  first = lo;
  count = cnt;
}

__device__ __forceinline__ int quantise(float acc) {
  const float r = __fadd_rn(acc, 0.5f);
  return r < 0.0f ? 0 : (r > 255.0f ? 255 : (int)r);
}

template <int CO>
__device__ __forceinline__ float pad_pick(const float (&padf)[4], int m) {
  if (CO == 1) {
    return padf[0];
  }
  float v = padf[0];
  v = m == 1 ? padf[1] : v;
  v = m == 2 ? padf[2] : v;
  if (CO > 3) {
    v = m == 3 ? padf[3] : v;
  }
  return v;
}

// Pad value (already cast) into the rectangle [ya, yb) x [xa, xb) of a slot
// with CO channels, 16-byte stores wherever the row segment allows.
//
// When the row pitch is a multiple of 16 bytes every row of the rectangle
// starts at the same offset within a 16-byte unit, so a thread works out its
// column position and its four values once and walks down the rows with
// nothing but stores; the CTA's threads are dealt over (column position, row
// phase) so that narrow rectangles still use all of them.
template <int CO>
__device__ __forceinline__ void fill_rect_f32(
    float* base, int slot_w, int ya, int yb, int xa, int xb, const float (&padf)[4]) {
  if (ya >= yb || xa >= xb) {
    return;
  }
  const int L = (xb - xa) * CO;
  const int ny = yb - ya;
  const size_t row_floats = (size_t)slot_w * CO;
  float* row0 = base + ((size_t)ya * slot_w + xa) * CO;
  if ((row_floats & 3) == 0) {
    const int mis = (int)((reinterpret_cast<uintptr_t>(row0) >> 2) & 3);
    int head = (4 - mis) & 3;
    head = head > L ? L : head;
    const int nvec = (L - head) >> 2;
    if (nvec > 0) {
      const int lanes_q = nvec >= kThreads ? kThreads : nvec;
      const int phases = kThreads / lanes_q;
      const int r0 = (int)threadIdx.x / lanes_q;
      if (r0 < phases) {
        for (int q = (int)threadIdx.x - r0 * lanes_q; q < nvec; q += lanes_q) {
          const int j = head + 4 * q;
          const int m = j % CO;
          const float4 v = make_float4(
              pad_pick<CO>(padf, m), pad_pick<CO>(padf, (m + 1) % CO), pad_pick<CO>(padf, (m + 2) % CO),
              pad_pick<CO>(padf, (m + 3) % CO));
          float* p = row0 + (size_t)r0 * row_floats + j;
          for (int ry = r0; ry < ny; ry += phases, p += (size_t)phases * row_floats) {
            *reinterpret_cast<float4*>(p) = v;
          }
        }
      }
    }
    // the few floats before the first and after the last aligned unit of each row
    const int tail = head + 4 * nvec;
    const int loose = head + (L - tail);
    for (int i = threadIdx.x; i < ny * loose; i += kThreads) {
      const int ry = i / loose;
      const int k = i - ry * loose;
      const int j = k < head ? k : tail + (k - head);
      row0[(size_t)ry * row_floats + j] = pad_pick<CO>(padf, j % CO);
    }
    return;
  }
  const int Q = ((L + 3) >> 2) + 2;
  for (int i = threadIdx.x; i < ny * Q; i += kThreads) {
    const int ry = i / Q;
    const int q = i - ry * Q;
    float* rowp = row0 + (size_t)ry * row_floats;
    const int mis = (int)((reinterpret_cast<uintptr_t>(rowp) >> 2) & 3);
    int head = (4 - mis) & 3;
    head = head > L ? L : head;
    const int nvec = (L - head) >> 2;
    if (q == 0) {
      for (int j = 0; j < head; j++) {
        rowp[j] = pad_pick<CO>(padf, j % CO);
      }
    } else if (q <= nvec) {
      const int j = head + 4 * (q - 1);
      const int m = j % CO;
      *reinterpret_cast<float4*>(rowp + j) = make_float4(
          pad_pick<CO>(padf, m), pad_pick<CO>(padf, (m + 1) % CO), pad_pick<CO>(padf, (m + 2) % CO),
          pad_pick<CO>(padf, (m + 3) % CO));
    } else if (q == nvec + 1) {
      for (int j = head + 4 * nvec; j < L; j++) {
        rowp[j] = pad_pick<CO>(padf, j % CO);
      }
    }
  }
}

// The same for a uint8 slot: every byte of the padding is the pad pixel, so the
// aligned middle of every row goes out as 16-byte stores of one pattern.
template <int CO>
__device__ __forceinline__ void fill_rect_u8(
    uint8_t* base, int slot_w, int ya, int yb, int xa, int xb, int pad_px) {
  if (ya >= yb || xa >= xb) {
    return;
  }
  const int L = (xb - xa) * CO;
  const int ny = yb - ya;
  const size_t row_bytes = (size_t)slot_w * CO;
  const unsigned w = (unsigned)(pad_px & 0xff) * 0x01010101u;
  const uint4 v = make_uint4(w, w, w, w);
  for (int ry = (int)threadIdx.x >> 5; ry < ny; ry += kThreads >> 5) {     // a warp per row
    uint8_t* rowp = base + (size_t)(ya + ry) * row_bytes + (size_t)xa * CO;
    const int mis = (int)(reinterpret_cast<uintptr_t>(rowp) & 15);
    int head = (16 - mis) & 15;
    head = head > L ? L : head;
    const int nvec = (L - head) >> 4;
    const int lane = (int)threadIdx.x & 31;
    for (int q = lane; q < nvec; q += 32) {
      *reinterpret_cast<uint4*>(rowp + head + 16 * q) = v;
    }
    const int tail = head + 16 * nvec;
    for (int k = lane; k < head + (L - tail); k += 32) {
      rowp[k < head ? k : tail + (k - head)] = (uint8_t)pad_px;
    }
  }
}

} // namespace mlxd
