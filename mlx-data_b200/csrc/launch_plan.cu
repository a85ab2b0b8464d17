// Host side of a launch: which kernels run it, and the planner's bounds on
// what one resize pass needs on chip.  The kernels themselves are in
// fused_fast.cu.
//
// Reference behaviour the kernels reproduce (paths inside mlx-data):
//   resize             mlx/data/core/image/ImageTransform.cpp:41-62 (triangle filter, clamp to edge)
//   crop               mlx/data/core/image/ImageTransform.cpp:64-73, mlx/data/Array.cpp:544-583
//   affine / rotate    mlx/data/core/image/ImageTransform.cpp:75-121
//   hflip              mlx/data/core/image/ImageTransform.cpp:123-140
//   channel_reduction  mlx/data/core/image/ImageTransform.cpp:142-182
//   batch + pad        mlx/data/Array.cpp:465-498, mlx/data/core/BatchShape.cpp:26-45
//   cast               README.md:55-57 (x.astype(float32) / 255 and its normalised form)
#include <cmath>

#include "fused_batch.h"

namespace mlxd {

cudaError_t launch_fused_batch(const LaunchParams& p, cudaStream_t stream) {
  return launch_fused_fast(p, stream);
}

void choose_kernel(LaunchParams& p, const PassNeed& need, const DevSample* host_samples, int n) {
  (void)need;
  // The rows below a sample's post window are one contiguous run of its slot;
  // when those runs are at least an eighth of the batch they get a linear fill
  // of their own (pad_fill_kernel), which writes at memory speed.
  p.pad_apart = 0;
  p.direct = 0;
  for (int i = 0; i < n; i++) {
    if (host_samples[i].mode == kModeResizeDirect) {
      p.direct = 1;
    }
  }
  if (n > 0) {
    unsigned long long rows = 0, below = 0;
    for (int i = 0; i < n; i++) {
      const int h = host_samples[i].slot_h;
      const int ph = host_samples[i].post_h < h ? host_samples[i].post_h : h;
      const int first = ((ph + kTileH - 1) / kTileH) * kTileH;
      rows += (unsigned long long)h;
      below += (unsigned long long)(first < h ? h - first : 0);
    }
    p.pad_apart = below * 8 >= rows ? 1 : 0;
  }
}

AxisPlan plan_axis(int32_t n_src, int32_t n_dst, int32_t sub) {
  AxisPlan a;
  if (n_src <= n_dst) {
    a.cap = 4;
    a.extent = sub + 4;
    return a;
  }
  // Output o reads taps ceil(u - R) .. floor(u + R) with u = (o + 0.5) * ratio - 0.5
  // and R = ratio: at most floor(2R) + 1 of them, and `sub` consecutive
  // outputs span at most (sub - 1) * ratio + 2R + 1 source samples.  One more
  // of each covers the float32 rounding of u and R in the kernel.
  const double ratio = (double)n_src / (double)n_dst;
  a.cap = (int32_t)std::floor(2.0 * ratio) + 2;
  a.extent = (int32_t)std::ceil((double)(sub - 1) * ratio + 2.0 * ratio) + 2;
  return a;
}

PassNeed plan_pass(
    const AxisPlan& ay, const AxisPlan& ax, int32_t sub_h, int32_t sub_w, int32_t pre_h, int32_t pre_w, int32_t channels,
    bool& fits) {
  const long long rows = ay.extent < pre_h ? ay.extent : pre_h;
  const long long cols = ax.extent < pre_w ? ax.extent : pre_w;
  const long long wbytes = cols * channels;
  const long long pitch = (wbytes + 49 + 15) & ~15LL;
  const long long src = rows * pitch;
  // every plane is padded by up to 7 columns on either side and one slot is
  // skipped after every eight columns
  const long long pad = (7 + channels - 1) / channels;
  const long long pslots = (cols + 2 * pad) + (cols + 2 * pad) / 8 + 1;
  const long long mid4 = ((sub_h + 3) / 4) * channels * pslots;   // one set of planes per group of four rows
  const long long wts = (long long)sub_h * ay.cap + (long long)sub_w * ax.cap;
  fits = src <= kSrcTileBytes && mid4 * 4 <= kMidFloats && wts <= kWeightFloats && rows <= kMaxStagedRows;
  PassNeed n;
  n.src_bytes = (int32_t)src;
  n.mid_float4s = (int32_t)mid4;
  n.weight_floats = (int32_t)wts;
  n.u_cap = (int32_t)(ay.extent < pre_h + 2 * ay.cap ? ay.extent : pre_h + 2 * ay.cap);
  return n;
}

} // namespace mlxd
