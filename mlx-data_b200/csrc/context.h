// Host-side state behind the C ABI: the context, its lanes and the code that
// turns public descriptors into a launch.
#pragma once

#include <cuda_runtime.h>

#include <atomic>
#include <map>
#include <mutex>
#include <shared_mutex>
#include <string>
#include <vector>

#include "../../include/mlxd_b200.h"
#include "fused_batch.h"

namespace mlxd {

const std::string& error_text();
void set_error(const std::string& msg);
int fail(int code, const std::string& msg);
int fail_cuda(cudaError_t e, const char* what);

#define MLXD_CUDA(call)                       \
  do {                                        \
    cudaError_t e__ = (call);                 \
    if (e__ != cudaSuccess) {                 \
      return ::mlxd::fail_cuda(e__, #call);   \
    }                                         \
  } while (0)

// Makes `device` current for the life of the object and puts the caller's
// device back afterwards: an entry point of this library never leaves the
// calling thread on another device than it came with.
struct DeviceGuard {
  int prev = -1;
  bool switched = false;
  cudaError_t err = cudaSuccess;
  explicit DeviceGuard(int device) {
    err = cudaGetDevice(&prev);
    if (err == cudaSuccess && prev != device) {
      err = cudaSetDevice(device);
      switched = err == cudaSuccess;
    }
  }
  ~DeviceGuard() {
    if (switched) {
      cudaSetDevice(prev);
    }
  }
  DeviceGuard(const DeviceGuard&) = delete;
  DeviceGuard& operator=(const DeviceGuard&) = delete;
};

#define MLXD_ON_DEVICE(device)                                  \
  ::mlxd::DeviceGuard device_guard__(device);                   \
  if (device_guard__.err != cudaSuccess) {                      \
    return ::mlxd::fail_cuda(device_guard__.err, "cudaSetDevice"); \
  }

// Grow-only device or pinned-host buffer.
struct Arena {
  void* ptr = nullptr;
  size_t cap = 0;
};

constexpr int kDescSlots = 4;

struct Lane {
  cudaStream_t stream = nullptr;
  cudaEvent_t done = nullptr;
  Arena d_src;                        // staged sources
  Arena h_src;                        // page-locked bounce block for sources in ordinary host memory
  cudaEvent_t src_copied = nullptr;   // the bounce block has left for the device
  Arena d_out;                        // batch written by the kernel when dst is host memory
  Arena d_desc[kDescSlots];           // DevSample tables
  Arena h_desc[kDescSlots];           // their pinned images
  cudaEvent_t desc_copied[kDescSlots] = {};
  cudaEvent_t k_begin[kDescSlots] = {};   // timing events around the kernel of each slot
  cudaEvent_t k_end[kDescSlots] = {};
  cudaEvent_t in_begin[kDescSlots] = {};  // around the host-to-device stage (gather kernel or copies)
  cudaEvent_t out_end[kDescSlots] = {};   // after the device-to-host copy of the batch (k_end is its start)
  bool k_pending[kDescSlots] = {};        // recorded, not yet added to the statistics
  bool in_timed[kDescSlots] = {};
  bool out_timed[kDescSlots] = {};
  int next_slot = 0;
  int32_t* d_status = nullptr;        // this lane's word of the context's status block
  int32_t* h_status = nullptr;        // pinned copy of the device status word
  std::mutex mu;                      // one caller at a time per lane
};

struct LutKey {
  int32_t c_out, normalise;
  uint32_t divisor_bits;
  uint32_t mean_bits[4];
  uint32_t std_bits[4];
  bool operator<(const LutKey& o) const;
};

} // namespace mlxd

struct mlxd_ctx {
  int device = 0;
  std::vector<mlxd::Lane*> lanes;     // n_lanes user lanes + one private lane for the synchronous ops
  int n_user_lanes = 0;
  int32_t* d_status = nullptr;        // one self-check word per lane, 64 bytes apart
  std::mutex lut_mu;
  std::map<mlxd::LutKey, float*> luts;   // at most mlxd::kMaxCastTables entries, see LutUse
  std::shared_mutex lut_users;           // shared: a launch being prepared holds a table pointer; exclusive: emptying the cache
  std::atomic<uint64_t> batches{0}, samples{0}, launches{0}, h2d{0}, d2h{0}, reserved{0};
  std::atomic<uint64_t> kernel_ns{0}, timed_launches{0};
  std::atomic<uint64_t> h2d_ns{0}, d2h_ns{0}, host_stage_ns{0};
  std::atomic<uint64_t> algo_src{0}, algo_dst{0};
  std::atomic<int> timing{0};
};

namespace mlxd {

// Validate descriptors and build the device programs (src/dst pointers are
// filled by the caller).  Returns MLXD_OK or an error with the message set.
int plan_samples(
    const mlxd_sample_desc* samples, int n, const mlxd_batch_desc* b,
    std::vector<DevSample>& out, PassNeed& need);

// One sample of plan_samples; `need` accumulates the shared-memory bounds.
// One rectangle of a host source that gather.cu packs into device memory:
// `rows` rows of `row_bytes` bytes, `src_pitch` apart at the source (a pointer
// the GPU can dereference), tightly packed at `dst`.  `first_row` is the number
// of rows of all earlier pieces of the launch.
struct GatherPiece {
  const uint8_t* src;
  uint8_t* dst;
  uint64_t src_pitch;
  uint32_t rows, row_bytes;
  uint32_t first_row, pad_;
};
// Blocks handed out by mlxd_pinned_alloc, with the address the GPU uses for
// them.  pinned_registry_lookup returns the device-side pointer for a host
// pointer inside a registered block, nullptr otherwise.
void pinned_registry_add(void* host, size_t bytes, void* device_side);
void pinned_registry_remove(void* host);
const uint8_t* pinned_registry_lookup(const void* host);

cudaError_t launch_gather_rows(const GatherPiece* table_dev, int n, uint32_t total_rows, cudaStream_t stream);

int plan_one_sample(
    const mlxd_sample_desc& d, int i, const mlxd_batch_desc* b, DevSample& out, PassNeed& need, long long pass_budget);
// plan_samples into caller-owned storage of n entries.
int plan_into(const mlxd_sample_desc* samples, int n, const mlxd_batch_desc* b, DevSample* out, PassNeed& need);

// The cast table of a batch descriptor: table[c * 256 + v], c < c_out.
void compute_cast_table(const mlxd_batch_desc* b, int c_out, float* table);

// Launch-wide parameters (cast table included) from a batch descriptor.
int prepare_launch(mlxd_ctx* ctx, const mlxd_batch_desc* b, int n, LaunchParams& p);

// Device cast table for a batch descriptor (cached per context).
int get_lut(mlxd_ctx* ctx, const mlxd_batch_desc* b, int c_out, const float** lut);

// The cache of cast tables is bounded: a caller that changes mean/std on every
// call would otherwise grow it for ever.  Every entry point that prepares a
// launch holds a LutUse from before prepare_launch() until its kernel is
// queued.  Constructing one first empties a full cache - with the exclusive
// lock, so no other thread sits between "has a table pointer" and "kernel
// queued", and after the device has drained, so no queued kernel reads a
// freed table.
constexpr size_t kMaxCastTables = 256;   // 4 KB each at most
class LutUse {
 public:
  explicit LutUse(mlxd_ctx* ctx);
 private:
  std::shared_lock<std::shared_mutex> hold_;
};

// Part of a sample's source that its chain can read: rows [r0, r1), columns
// [c0, c1); `margin` widens a filter footprint by that many source samples.
void needed_region(const DevSample& s, int margin, int32_t& r0, int32_t& r1, int32_t& c0, int32_t& c1);

int arena_reserve(mlxd_ctx* ctx, Arena& a, size_t bytes, bool pinned, cudaStream_t stream_to_drain);

int enqueue_on_lane(
    mlxd_ctx* ctx, Lane& lane, const mlxd_sample_desc* samples, int n, const mlxd_batch_desc* batch,
    const std::vector<void*>* per_sample_dst);

int wait_lane(mlxd_ctx* ctx, Lane& lane, int timeout_ms);

// Add the elapsed time of a finished, timed slot to the statistics.  With
// `block` the call waits for the slot's kernel; otherwise unfinished slots
// stay pending.
void harvest_timing(mlxd_ctx* ctx, Lane& lane, int slot, bool block);

} // namespace mlxd
