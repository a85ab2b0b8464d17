// Bridge between the C++ pipeline and the CUDA library's C ABI
// (include/mlxd_b200.h): the process-wide context, page-locked Array storage,
// and LazyImage - an image described by a source array plus the op chain
// still to be run on it, so that a whole batch becomes one kernel launch.
#pragma once

#include <cstdint>
#include <memory>
#include <condition_variable>
#include <mutex>
#include <map>
#include <utility>
#include <vector>

#include "mlx/data/Array.h"
#include "mlxd_b200.h"

namespace mlx {
namespace data {
namespace gpu {

// The uint8 -> float32 cast fused after batching: x / divisor, optionally
// (x / divisor - mean[c]) / std[c] - numpy's float32 arithmetic for
// x.astype("float32") / 255 and its normalised form.
struct CastSpec {
  float divisor = 255.0f;
  bool normalise = false;
  float mean[4] = {0, 0, 0, 0};
  float std_[4] = {1, 1, 1, 1};
};

// Axis-aligned window of an image, optionally mirrored left-right.
struct Window {
  int64_t x = 0, y = 0, w = 0, h = 0;
  bool flip = false;
  // Crop the (possibly mirrored) window in its own coordinates.
  void crop(int64_t cx, int64_t cy, int64_t cw, int64_t ch);
};

// Where a batch node leaves its results and on which stream it may queue work.
// A node copies the process-wide defaults when it is built and keeps its copy:
// placement is a property of a pipeline, later changes of the defaults do not
// reach pipelines that already exist.
struct Placement {
  bool device_output = false;   // leave batches in GPU memory instead of page-locked host memory
  void* stream = nullptr;       // caller-owned CUDA stream for all-GPU work
  bool use_stream = false;
};

class LazyImage {
 public:
  // Checks that src looks like an image the way core::image::verify_image does.
  explicit LazyImage(const std::shared_ptr<const Array>& src);

  int64_t width() const;
  int64_t height() const;
  int64_t channels() const { return gray_ ? 1 : channels_; }
  int64_t source_channels() const { return channels_; }
  bool is_gray() const { return gray_; }
  // True while no op has been folded in: the result is the source itself.
  bool untouched() const { return untouched_; }
  const std::shared_ptr<const Array>& source() const { return src_; }
  // The same program on another source of the same shape (the frames of a clip).
  LazyImage with_source(const std::shared_ptr<const Array>& src) const;

  // Every op returns false when it cannot join the program already recorded
  // (a second geometric op, a geometric op after the channel reduction, any
  // op after an extension); the caller then materialises and starts a new
  // LazyImage.
  bool crop(int64_t x, int64_t y, int64_t w, int64_t h);
  bool hflip();
  bool resize(int64_t dw, int64_t dh);
  bool affine(const float mx[6], int64_t tw, int64_t th);
  bool channel_reduction(float bias, const float m[3]);

  // Explicit padding at the end of the rows (dim 0) or columns (dim 1):
  // `amount` more of them holding `value`.  Nothing is computed for it - the
  // image only claims a larger rectangle of its batch slot, which the kernel
  // fills with the batch's pad value; so the batch node checks that the two
  // values agree (extension_matches) and materialises the image when not.
  // False for another dimension, a value that is no uint8, or a second value.
  bool pad_end(int dim, int64_t amount, double value);
  bool extended() const { return ext_w_ > 0 || ext_h_ > 0; }
  bool extension_matches(double batch_pad_value) const;

  void describe(mlxd_sample_desc& d) const;
  void gray_params(int32_t m[3], int32_t& bias) const;

  // Run the recorded program now: a uint8 [h, w, channels()] array.
  std::shared_ptr<Array> materialise() const;

 private:
  std::shared_ptr<const Array> src_;
  int64_t channels_ = 0;
  Window pre_, post_;
  int geom_ = MLXD_GEOM_NONE;
  int64_t geom_w_ = 0, geom_h_ = 0;
  float mx_[6] = {0, 0, 0, 0, 0, 0};
  bool gray_ = false;
  int32_t gray_m_[3] = {0, 0, 0};
  int32_t gray_bias_ = 0;
  bool untouched_ = true;
  int64_t ext_w_ = 0, ext_h_ = 0;   // columns / rows claimed beyond the program's output
  int ext_value_ = 0;
};

class Runtime {
 public:
  static Runtime& get();

  // Choose the CUDA device before the first GPU call (default: environment
  // MLXD_DEVICE, then LOCAL_RANK, then 0).
  static void set_device(int device);
  static int device();

  // Keep the calling thread - and every thread it starts afterwards, the
  // pipeline's workers included - on the CPUs of the NUMA node the selected
  // GPU hangs off, so that page-locked blocks are allocated in that node's
  // memory and copies do not cross the socket interconnect.  Call it before the
  // first pipeline is built.  Returns {node, cpus kept}; {-1, 0} and no change
  // when the node cannot be read (no sysfs entry, single-node machine).
  static std::pair<int, int> bind_host_threads_to_device_node();
  // The same for a PCI address ("0000:1b:00.0", any case) looked up under a
  // sysfs tree; the tests point it at a made-up tree.
  static std::pair<int, int> bind_host_threads_to_node_of(const std::string& pci_bus_id, const std::string& sysfs);

  mlxd_ctx* ctx();
  // Check a lane out for one call in flight (blocks while all are busy) and
  // hand it back afterwards.
  int acquire_lane();
  void release_lane(int lane);
  void check(int rc) const;

  // Array whose storage is page-locked host memory from a recycling pool.
  std::shared_ptr<Array> pinned_array(ArrayType type, const std::vector<int64_t>& shape);
  // Array whose storage is memory of the context's GPU, from a recycling pool.
  // `queued_on`, when given, is the caller-owned stream on which work that
  // writes (and later reads) the block is queued without being waited for:
  // the block goes back to the pool tagged with it, and whoever takes it for
  // another stream waits for that stream first.
  std::shared_ptr<Array> device_array(
      ArrayType type, const std::vector<int64_t>& shape, const void* const* queued_on = nullptr);

  // Where batch() and cast() leave their results: host (default, what
  // mlx-data does) or the GPU's memory, for consumers that train on that GPU.
  void set_device_output(bool on);
  bool device_output() const { return placement().device_output; }
  // The defaults a batch node built now would take.
  Placement placement() const;
  // Resizing a 4-channel image.  mlx-data hands such images to its resize
  // library as RGBA, which weights the colour channels by alpha while it
  // filters; the kernels here filter the four channels independently of one
  // another, so the results differ wherever alpha varies.  The resize ops
  // therefore refuse 4-channel images unless the caller has accepted the
  // independent filtering here.
  static void set_rgba_resize_independent(bool accept);
  static bool rgba_resize_independent();
  // Launch on a caller-owned CUDA stream instead of the lanes.  Only used for
  // work whose sources and result are all in GPU memory; such calls return
  // without waiting and the result is ordered on that stream.
  void set_stream(void* cuda_stream, bool enabled);

  // One fused launch: every image's program, batch + pad, optional cast.
  // Result is [N, max_h, max_w, C] uint8, or float32 when cast is given.
  std::shared_ptr<Array> batch(
      const std::vector<LazyImage>& images, double pad_value, const CastSpec* cast, const Placement& where);

  // Cast an existing uint8 array (any shape, last dimension = channels <= 4).
  std::shared_ptr<Array> cast(const std::shared_ptr<const Array>& arr, const CastSpec& spec);

  ~Runtime();

 private:
  Runtime() = default;
  struct Block {
    void* p;
    bool tagged;      // last used by work queued on `stream` that nobody waited for
    void* stream;
  };
  struct Pool {
    std::multimap<size_t, Block> blocks;
    size_t bytes = 0;
    size_t limit = size_t(16) << 30;
  };
  bool pool_take(Pool& pool, size_t bytes, size_t& held, Block& out);
  bool pool_give(Pool& pool, const Block& b, size_t bytes);
  std::shared_ptr<Array> pooled_array(
      ArrayType type, const std::vector<int64_t>& shape, bool on_device, const void* const* queued_on);
  Pool device_pool_;
  Placement defaults_;          // guarded by mu_

  mutable std::mutex mu_;
  mlxd_ctx* ctx_ = nullptr;
  int n_lanes_ = 8;
  std::vector<int> free_lanes_;
  bool lanes_ready_ = false;
  std::condition_variable lane_cv_;
  Pool pinned_pool_;
};

} // namespace gpu
} // namespace data
} // namespace mlx
