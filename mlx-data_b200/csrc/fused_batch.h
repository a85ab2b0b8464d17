// Device-side layout of one fused batch launch: the per-sample programs the
// kernel executes and the launch-wide parameters.  Host code fills these from
// the public descriptors (include/mlxd_b200.h) after validating them.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace mlxd {

constexpr int kTileH = 16;    // output rows per CTA
constexpr int kTileW = 64;    // output pixels per row per CTA
constexpr int kThreads = 256;

// Upper bounds on the shared memory one resize pass may ask for.  The planner
// shrinks the pass (sub_h x sub_w outputs) until its footprint fits; a launch
// then allocates only the largest need among its samples.
constexpr int kSrcTileBytes = 48 * 1024;   // staged source footprint, uint8
constexpr int kMidFloats = 12 * 1024;      // vertically filtered values, float32
constexpr int kWeightFloats = 2 * 1024;    // tap weights of both axes
constexpr int kMaxStagedRows = 192;        // source rows per pass

// kModeResizeDirect: a resize whose tap footprint does not fit the on-chip
// passes at any pass size (shrink ratios of about 60 and more); every output
// pixel is then filtered straight from global memory by resize_direct_kernel.
enum Mode : int32_t { kModeCopy = 0, kModeResize = 1, kModeAffine = 2, kModeResizeDirect = 3 };

// One sample's program.  Coordinates name four nested images:
//   source [src_h, src_w] -> pre window [pre_h, pre_w] (+mirror)
//   -> geometric output [geom_h, geom_w] -> post window [post_h, post_w] (+mirror)
// and the post window lands in the top-left corner of the slot [slot_h, slot_w].
struct __align__(16) DevSample {
  const uint8_t* src;
  void* dst;
  int32_t src_h, src_w;
  int32_t pre_x, pre_y, pre_w, pre_h;
  int32_t geom_w, geom_h;
  int32_t post_x, post_y, post_w, post_h;
  int32_t slot_h, slot_w;
  int32_t mode;
  int32_t pre_flip, post_flip;
  int32_t sub_h, sub_w;   // resize: geometric-output rows / columns filtered per pass
  int32_t cap_y, cap_x;   // resize: tap-count bound per axis
  float mx[6];
  int32_t r0_staged;      // host use: first source row held by the staged copy
  // resize, float32 kernel: this sample's own shared-memory needs.  A CTA lays
  // its shared memory out from these, so a launch is sized by the largest sum
  // over its samples, not by the sum of the largest parts.
  int32_t need_src, need_mid4;
  int32_t need_wts_ucap;  // weight floats in the low 16 bits, u_cap above
};

struct LaunchParams {
  const DevSample* samples;
  int32_t n;
  int32_t tiles_y, tiles_x;   // tile grid of the largest slot
  int32_t c_in;               // channels of every source
  int32_t c_out;              // 1 when gray, else c_in
  int32_t gray;
  int32_t gray_m[3];
  int32_t gray_bias;
  int32_t out_f32;
  const float* lut;           // [c_out][256] cast table, device
  int32_t pad_px;             // pad value as a pixel
  int32_t* status;            // device word, non-zero once a self-check failed
  // shared memory of the resize passes (0 when no sample resizes)
  int32_t src_tile_bytes;
  int32_t mid_float4s;
  int32_t weight_floats;
  int32_t u_cap;              // bound on the source rows feeding four adjacent output rows
  int32_t band_tiles;         // float32 kernel: tiles per CTA along a row band (set at launch)
  int32_t bands_x;            // float32 kernel: CTAs per row band
  int32_t fast_smem_bytes;    // float32 kernel: dynamic shared memory of the launch
  int32_t pad_apart;          // float32 kernel: the rows below each post window are written by pad_fill_kernel
  int32_t direct;             // some sample is kModeResizeDirect: resize_direct_kernel runs after the band kernel
  int32_t starve_wait;        // test hook: the first pass of every band expects 16 bytes that no copy delivers
};

// Shared-memory need of one resize pass, from the planner's conservative bounds.
struct PassNeed {
  int32_t src_bytes;
  int32_t mid_float4s;
  int32_t weight_floats;
  int32_t u_cap;
  int64_t sum_bytes;          // largest per-sample sum of the parts that grow with the pass (pass_bytes)
  int64_t fast_smem_bytes;    // float32 kernel: largest per-sample shared-memory layout
};

// Dynamic shared memory of the float32 kernel for a sample with these needs
// (c_out channels in the cast table).
size_t fused_fast_layout_bytes(int c_out, int u_cap, int weight_floats, int mid_float4s, int src_tile_bytes);

// Launch the band kernel that fits the parameters (float32, float32 after the
// channel reduction, uint8, two channels), preceded by pad_fill_kernel when
// p.pad_apart is set.
cudaError_t launch_fused_batch(const LaunchParams& p, cudaStream_t stream);
cudaError_t launch_fused_fast(const LaunchParams& p, cudaStream_t stream);

// Decide whether a ragged batch's padding gets a launch of its own; call after
// the planner filled `need` and the host copy of the sample table.
void choose_kernel(LaunchParams& p, const PassNeed& need, const DevSample* host_samples, int n);

// Conservative per-axis bounds used by the host planner.
struct AxisPlan {
  int32_t cap;      // tap-count bound
  int32_t extent;   // bound on source samples touched by `sub` outputs
};
AxisPlan plan_axis(int32_t n_src, int32_t n_dst, int32_t sub);

// Bound on the shared memory of a pass over sub_h x sub_w outputs of an axis
// pair; `fits` tells whether it respects the limits above.
PassNeed plan_pass(
    const AxisPlan& ay, const AxisPlan& ax, int32_t sub_h, int32_t sub_w, int32_t pre_h, int32_t pre_w, int32_t channels,
    bool& fits);

} // namespace mlxd
