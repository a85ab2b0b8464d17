// Context, lanes, descriptor planning and the enqueue path of the C ABI.
#include "context.h"

#include <map>

#include <atomic>
#include <chrono>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <thread>

namespace mlxd {

namespace {
thread_local std::string g_error;
}

const std::string& error_text() {
  return g_error;
}

void set_error(const std::string& msg) {
  g_error = msg;
}

int fail(int code, const std::string& msg) {
  g_error = msg;
  return code;
}

int fail_cuda(cudaError_t e, const char* what) {
  g_error = std::string(what) + ": " + cudaGetErrorString(e);
  return e == cudaErrorMemoryAllocation ? MLXD_ERR_NOMEM : MLXD_ERR_CUDA;
}

bool LutKey::operator<(const LutKey& o) const {
  return std::memcmp(this, &o, sizeof(LutKey)) < 0;
}

namespace {
struct PinnedBlock {
  size_t bytes;
  intptr_t device_delta;   // device-side address minus host address
};
std::mutex g_pinned_mu;
std::map<uintptr_t, PinnedBlock> g_pinned;
}  // namespace

void pinned_registry_add(void* host, size_t bytes, void* device_side) {
  std::lock_guard<std::mutex> g(g_pinned_mu);
  g_pinned[reinterpret_cast<uintptr_t>(host)] =
      PinnedBlock{bytes, static_cast<intptr_t>(reinterpret_cast<uintptr_t>(device_side) - reinterpret_cast<uintptr_t>(host))};
}

void pinned_registry_remove(void* host) {
  std::lock_guard<std::mutex> g(g_pinned_mu);
  g_pinned.erase(reinterpret_cast<uintptr_t>(host));
}

const uint8_t* pinned_registry_lookup(const void* host) {
  const uintptr_t a = reinterpret_cast<uintptr_t>(host);
  std::lock_guard<std::mutex> g(g_pinned_mu);
  auto it = g_pinned.upper_bound(a);
  if (it == g_pinned.begin()) {
    return nullptr;
  }
  --it;
  if (a >= it->first + it->second.bytes) {
    return nullptr;
  }
  return reinterpret_cast<const uint8_t*>(a + it->second.device_delta);
}

int arena_reserve(mlxd_ctx* ctx, Arena& a, size_t bytes, bool pinned, cudaStream_t stream_to_drain) {
  if (bytes <= a.cap) {
    return MLXD_OK;
  }
  // Work already queued may still read the old block.
  if (stream_to_drain) {
    MLXD_CUDA(cudaStreamSynchronize(stream_to_drain));
  }
  size_t want = bytes + bytes / 4;
  want = (want + 4095) & ~(size_t)4095;
  void* p = nullptr;
  if (pinned) {
    MLXD_CUDA(cudaHostAlloc(&p, want, cudaHostAllocDefault));
    if (a.ptr) {
      cudaFreeHost(a.ptr);
    }
  } else {
    if (a.ptr) {
      cudaFree(a.ptr);
      ctx->reserved -= a.cap;
      a.ptr = nullptr;
      a.cap = 0;
    }
    MLXD_CUDA(cudaMalloc(&p, want));
    ctx->reserved += want;
  }
  a.ptr = p;
  a.cap = want;
  return MLXD_OK;
}

// "sample <i>: <what>" as the thread's error text.  Only failing calls come
// here, so a call that succeeds builds no string at all.
static int bad_sample(int i, const char* what) {
  return fail(MLXD_ERR_INVALID, "sample " + std::to_string(i) + ": " + what);
}

static int check_sample(const mlxd_sample_desc& d, int i, const mlxd_batch_desc* b, int slot_h, int slot_w) {
  if (!d.src) {
    return bad_sample(i, "null source");
  }
  if (d.src_h <= 0 || d.src_w <= 0) {
    return bad_sample(i, "image: cannot create image with 0 or negative dimension");
  }
  if (d.pre_w <= 0 || d.pre_h <= 0 || d.pre_x < 0 || d.pre_y < 0 ||
      (int64_t)d.pre_x + d.pre_w > d.src_w || (int64_t)d.pre_y + d.pre_h > d.src_h) {
    return bad_sample(i, "window before the geometric op leaves the source image");
  }
  if (d.geom < MLXD_GEOM_NONE || d.geom > MLXD_GEOM_AFFINE) {
    return bad_sample(i, "unknown geometric op");
  }
  if (d.geom_w <= 0 || d.geom_h <= 0) {
    return bad_sample(i, "image: cannot create image with 0 or negative dimension");
  }
  if (d.geom == MLXD_GEOM_NONE && (d.geom_w != d.pre_w || d.geom_h != d.pre_h)) {
    return bad_sample(i, "geom_w, geom_h must equal pre_w, pre_h without a geometric op");
  }
  if (d.post_w <= 0 || d.post_h <= 0 || d.post_x < 0 || d.post_y < 0 ||
      (int64_t)d.post_x + d.post_w > d.geom_w || (int64_t)d.post_y + d.post_h > d.geom_h) {
    return bad_sample(i, "window after the geometric op leaves its output");
  }
  if (d.post_w > slot_w || d.post_h > slot_h) {
    return bad_sample(i, "result is larger than its slot in the batch");
  }
  if ((int64_t)d.src_h * d.src_w * b->channels >= ((int64_t)1 << 40)) {
    return bad_sample(i, "source image too large");
  }
  return MLXD_OK;
}

// Shared memory of the float32 kernel that grows with the pass (staged source,
// planar buffer, two table sets, vertical weights), and the budget under which
// three CTAs still fit on one SM next to the fixed part (cast table, headers).
static long long pass_bytes(const PassNeed& n) {
  return (long long)n.src_bytes + 16LL * n.mid_float4s + 16LL * n.weight_floats + 256LL * n.u_cap;
}
constexpr long long kPassBudgetBytes = 69 * 1024;

static int plan_resize(DevSample& s, int C, int i, PassNeed& need, long long pass_budget) {
  // First look for the largest pass within the three-CTA budget, not going
  // below 4 x 16 outputs; failing that, take the largest pass that fits at all.
  for (int budgeted = 1; budgeted >= 0; budgeted--) {
    int sub_h = kTileH, sub_w = kTileW;
    for (;;) {
      const AxisPlan ay = plan_axis(s.pre_h, s.geom_h, sub_h);
      const AxisPlan ax = plan_axis(s.pre_w, s.geom_w, sub_w);
      bool fits = false;
      PassNeed n = plan_pass(ay, ax, sub_h, sub_w, s.pre_h, s.pre_w, C, fits);
      // source rows feeding one group of (at most) four adjacent output rows
      n.u_cap = plan_axis(s.pre_h, s.geom_h, std::min(4, sub_h)).extent;
      fits = fits && n.u_cap <= kMaxStagedRows;
      if (budgeted) {
        fits = fits && pass_bytes(n) <= pass_budget;
      }
      if (fits) {
        s.sub_h = sub_h;
        s.sub_w = sub_w;
        s.cap_y = ay.cap;
        s.cap_x = ax.cap;
        need.src_bytes = std::max(need.src_bytes, n.src_bytes);
        need.mid_float4s = std::max(need.mid_float4s, n.mid_float4s);
        need.weight_floats = std::max(need.weight_floats, n.weight_floats);
        need.u_cap = std::max(need.u_cap, n.u_cap);
        // the float32 kernel lays a CTA out from its own sample's needs
        s.need_src = n.src_bytes;
        s.need_mid4 = n.mid_float4s;
        s.need_wts_ucap = n.weight_floats | (n.u_cap << 16);
        need.sum_bytes = std::max<int64_t>(need.sum_bytes, pass_bytes(n));
        need.fast_smem_bytes = std::max<int64_t>(
            need.fast_smem_bytes,
            (int64_t)fused_fast_layout_bytes(C, n.u_cap, n.weight_floats, n.mid_float4s, n.src_bytes));
        return MLXD_OK;
      }
      if (budgeted && sub_h <= 4 && sub_w <= 16) {
        break;
      }
      if (sub_h > 4) {
        sub_h /= 2;
      } else if (sub_w > 8) {
        sub_w /= 2;
      } else if (sub_h > 1) {
        sub_h /= 2;
      } else if (sub_w > 1) {
        sub_w /= 2;
      } else {
        break;
      }
    }
  }
  // No pass size holds the taps of even one output: the sample is filtered
  // pixel by pixel from global memory instead.
  (void)i;
  s.mode = kModeResizeDirect;
  s.cap_y = plan_axis(s.pre_h, s.geom_h, 1).cap;
  s.cap_x = plan_axis(s.pre_w, s.geom_w, 1).cap;
  return MLXD_OK;
}

int plan_one_sample(
    const mlxd_sample_desc& d, int i, const mlxd_batch_desc* b, DevSample& out, PassNeed& need, long long pass_budget) {
  {
    int rc = check_sample(d, i, b, b->slot_h, b->slot_w);
    if (rc != MLXD_OK) {
      return rc;
    }
    DevSample s;
    std::memset(&s, 0, sizeof(s));
    s.src = d.src;
    s.src_h = d.src_h;
    s.src_w = d.src_w;
    s.pre_x = d.pre_x;
    s.pre_y = d.pre_y;
    s.pre_w = d.pre_w;
    s.pre_h = d.pre_h;
    s.pre_flip = d.pre_flip ? 1 : 0;
    s.geom_w = d.geom_w;
    s.geom_h = d.geom_h;
    s.post_x = d.post_x;
    s.post_y = d.post_y;
    s.post_w = d.post_w;
    s.post_h = d.post_h;
    s.post_flip = d.post_flip ? 1 : 0;
    s.slot_h = b->slot_h;
    s.slot_w = b->slot_w;
    std::memcpy(s.mx, d.mx, sizeof(s.mx));
    s.sub_h = kTileH;
    s.sub_w = kTileW;
    s.cap_y = s.cap_x = 1;
    if (d.geom == MLXD_GEOM_RESIZE) {
      if (d.pre_w == d.geom_w && d.pre_h == d.geom_h) {
        s.mode = kModeCopy;  // identity on both axes
      } else {
        s.mode = kModeResize;
        rc = plan_resize(s, b->channels, i, need, pass_budget);
        if (rc != MLXD_OK) {
          return rc;
        }
      }
    } else if (d.geom == MLXD_GEOM_AFFINE) {
      s.mode = kModeAffine;
    } else {
      s.mode = kModeCopy;
    }
    if (s.mode == kModeCopy && s.pre_flip) {
      // Without a geometric op the two mirrors compose into one.
      s.pre_flip = 0;
      s.post_flip ^= 1;
      s.post_x = s.geom_w - s.post_x - s.post_w;
    }
    out = s;
  }
  return MLXD_OK;
}

int plan_into(const mlxd_sample_desc* samples, int n, const mlxd_batch_desc* b, DevSample* out, PassNeed& need) {
  // A launch allocates the largest need of every kind over its samples, which
  // may come from different samples.  If the combination misses the three-CTA
  // budget, one try with smaller passes; if that is not enough either, the
  // full-size passes at two CTAs per SM are the better deal.
  const long long budgets[3] = {kPassBudgetBytes, kPassBudgetBytes - 8 * 1024, kPassBudgetBytes};
  for (int k = 0; k < 3; k++) {
    need = PassNeed{0, 0, 0, 0, 0, 0};
    for (int i = 0; i < n; i++) {
      const int rc = plan_one_sample(samples[i], i, b, out[i], need, budgets[k]);
      if (rc != MLXD_OK) {
        return rc;
      }
    }
    // the float32 kernel needs the largest per-sample sum, the generic one the sum of the largest parts
    const bool fast = true;
    if ((fast ? (long long)need.sum_bytes : pass_bytes(need)) <= kPassBudgetBytes) {
      break;
    }
  }
  return MLXD_OK;
}

int plan_samples(
    const mlxd_sample_desc* samples, int n, const mlxd_batch_desc* b,
    std::vector<DevSample>& out, PassNeed& need) {
  out.resize(n);
  return plan_into(samples, n, b, out.data(), need);
}

// Source samples of an n_src -> n_dst axis that outputs [o_lo, o_hi) can read,
// widened by `margin` on both sides and clipped to the axis.
static void axis_span(int64_t n_src, int64_t n_dst, int64_t o_lo, int64_t o_hi, int margin, int64_t& lo, int64_t& hi) {
  if (n_src == n_dst) {
    lo = o_lo;
    hi = o_hi;
  } else {
    const double ratio = (double)n_src / (double)n_dst;
    const double radius = ratio > 1.0 ? ratio : 1.0;
    lo = (int64_t)std::floor((o_lo + 0.5) * ratio - 0.5 - radius) - margin;
    hi = (int64_t)std::ceil((o_hi - 0.5) * ratio - 0.5 + radius) + 1 + margin;
  }
  lo = std::max<int64_t>(lo, 0);
  hi = std::min<int64_t>(hi, n_src);
}

void needed_region(const DevSample& s, int margin, int32_t& r0, int32_t& r1, int32_t& c0, int32_t& c1) {
  int64_t rlo = 0, rhi = s.pre_h, clo = 0, chi = s.pre_w;  // in pre-window coordinates
  if (s.mode == kModeCopy) {
    rlo = s.post_y;
    rhi = (int64_t)s.post_y + s.post_h;
    clo = s.post_x;
    chi = (int64_t)s.post_x + s.post_w;
  } else if (s.mode == kModeResize || s.mode == kModeResizeDirect) {
    axis_span(s.pre_h, s.geom_h, s.post_y, (int64_t)s.post_y + s.post_h, margin, rlo, rhi);
    axis_span(s.pre_w, s.geom_w, s.post_x, (int64_t)s.post_x + s.post_w, margin, clo, chi);
    if (s.pre_flip) {
      const int64_t a = s.pre_w - chi, b = s.pre_w - clo;
      clo = a;
      chi = b;
    }
  }
  r0 = (int32_t)(s.pre_y + rlo);
  r1 = (int32_t)(s.pre_y + rhi);
  c0 = (int32_t)(s.pre_x + clo);
  c1 = (int32_t)(s.pre_x + chi);
}

void compute_cast_table(const mlxd_batch_desc* b, int c_out, float* table) {
  // Every entry is the chain of float32 operations numpy performs:
  // float(v) / divisor, then - mean, then / std.
  for (int c = 0; c < c_out; c++) {
    for (int v = 0; v < 256; v++) {
      volatile float x = (float)v;
      volatile float q = x / b->divisor;
      if (b->normalise) {
        volatile float t = q - b->mean[c];
        q = t / b->std_[c];
      }
      table[(size_t)c * 256 + v] = q;
    }
  }
}

LutUse::LutUse(mlxd_ctx* ctx) {
  bool full;
  {
    std::lock_guard<std::mutex> g(ctx->lut_mu);
    full = ctx->luts.size() >= kMaxCastTables;
  }
  if (full) {
    std::unique_lock<std::shared_mutex> alone(ctx->lut_users);
    std::lock_guard<std::mutex> g(ctx->lut_mu);
    if (ctx->luts.size() >= kMaxCastTables) {
      DeviceGuard on_device(ctx->device);
      cudaDeviceSynchronize();
      for (auto& kv : ctx->luts) {
        cudaFree(kv.second);
      }
      ctx->luts.clear();
    }
  }
  hold_ = std::shared_lock<std::shared_mutex>(ctx->lut_users);
}

int get_lut(mlxd_ctx* ctx, const mlxd_batch_desc* b, int c_out, const float** lut) {
  LutKey key;
  std::memset(&key, 0, sizeof(key));
  key.c_out = c_out;
  key.normalise = b->normalise ? 1 : 0;
  std::memcpy(&key.divisor_bits, &b->divisor, 4);
  if (key.normalise) {
    std::memcpy(key.mean_bits, b->mean, 4 * c_out);
    std::memcpy(key.std_bits, b->std_, 4 * c_out);
  }
  std::lock_guard<std::mutex> g(ctx->lut_mu);
  auto it = ctx->luts.find(key);
  if (it != ctx->luts.end()) {
    *lut = it->second;
    return MLXD_OK;
  }
  std::vector<float> table((size_t)c_out * 256);
  compute_cast_table(b, c_out, table.data());
  float* d = nullptr;
  MLXD_CUDA(cudaMalloc(&d, table.size() * sizeof(float)));
  cudaError_t e = cudaMemcpy(d, table.data(), table.size() * sizeof(float), cudaMemcpyHostToDevice);
  if (e != cudaSuccess) {
    cudaFree(d);
    return fail_cuda(e, "cudaMemcpy(cast table)");
  }
  ctx->luts[key] = d;
  *lut = d;
  return MLXD_OK;
}

int prepare_launch(
    mlxd_ctx* ctx, const mlxd_batch_desc* b, int n, LaunchParams& p) {
  if (b->channels < 1 || b->channels > 4) {
    return fail(MLXD_ERR_INVALID, "image: channels must be 0 < c <= 4");
  }
  if (b->gray && b->channels != 3) {
    return fail(MLXD_ERR_INVALID, "image::channelReduction: expected a 3 channel uint8 array");
  }
  if (b->slot_h <= 0 || b->slot_w <= 0) {
    return fail(MLXD_ERR_INVALID, "batch slot must have positive height and width");
  }
  if (b->out_dtype != MLXD_U8 && b->out_dtype != MLXD_F32) {
    return fail(MLXD_ERR_INVALID, "unknown output dtype");
  }
  std::memset(&p, 0, sizeof(p));
  p.n = n;
  p.tiles_y = (b->slot_h + kTileH - 1) / kTileH;
  p.tiles_x = (b->slot_w + kTileW - 1) / kTileW;
  p.c_in = b->channels;
  p.c_out = b->gray ? 1 : b->channels;
  p.gray = b->gray ? 1 : 0;
  p.gray_m[0] = b->gray_m[0];
  p.gray_m[1] = b->gray_m[1];
  p.gray_m[2] = b->gray_m[2];
  p.gray_bias = b->gray_bias;
  p.out_f32 = b->out_dtype == MLXD_F32;
  p.pad_px = (int32_t)(uint8_t)(int32_t)b->pad_value;
  p.status = ctx->d_status;   // callers point this at their lane's word
  // Test hook (MLXD_TEST_STARVE_WAIT=1, read per launch): the resize bands'
  // first bounded wait runs out, so the path from the kernel's status word to
  // the caller's error code can be exercised without a fault or a hang.
  const char* starve = std::getenv("MLXD_TEST_STARVE_WAIT");
  p.starve_wait = (starve && starve[0] == '1') ? 1 : 0;
  if (p.out_f32) {
    if (!(b->divisor != 0.0f)) {
      return fail(MLXD_ERR_INVALID, "cast divisor must be non-zero");
    }
    int rc = get_lut(ctx, b, p.c_out, &p.lut);
    if (rc != MLXD_OK) {
      return rc;
    }
  }
  return MLXD_OK;
}

// Threads that pack one batch's pageable sources (the caller included):
// MLXD_PACK_THREADS, default 4, at most 32.
static int pack_threads() {
  static const int n = [] {
    const char* v = std::getenv("MLXD_PACK_THREADS");
    const int want = v && *v ? std::atoi(v) : 4;
    return want < 1 ? 1 : (want > 32 ? 32 : want);
  }();
  return n;
}

int enqueue_on_lane(
    mlxd_ctx* ctx, Lane& lane, const mlxd_sample_desc* samples, int n, const mlxd_batch_desc* batch,
    const std::vector<void*>* per_sample_dst) {
  if (!samples || !batch || n < 0) {
    return fail(MLXD_ERR_INVALID, "null descriptor or negative sample count");
  }
  if (n == 0) {
    return MLXD_OK;
  }
  if (!batch->dst && !per_sample_dst) {
    return fail(MLXD_ERR_INVALID, "null batch destination");
  }
  MLXD_ON_DEVICE(ctx->device);
  LutUse table_in_use(ctx);
  LaunchParams p;
  int rc = prepare_launch(ctx, batch, n, p);
  if (rc != MLXD_OK) {
    return rc;
  }
  std::vector<DevSample> dev;
  PassNeed need;
  p.status = lane.d_status;
  rc = plan_samples(samples, n, batch, dev, need);
  if (rc != MLXD_OK) {
    return rc;
  }
  p.src_tile_bytes = need.src_bytes;
  p.mid_float4s = need.mid_float4s;
  p.weight_floats = need.weight_floats;
  p.u_cap = need.u_cap;
  p.fast_smem_bytes = (int32_t)need.fast_smem_bytes;
  choose_kernel(p, need, dev.data(), n);
  const size_t esize = p.out_f32 ? 4 : 1;
  const size_t slot_bytes = (size_t)batch->slot_h * batch->slot_w * p.c_out * esize;
  const size_t out_bytes = slot_bytes * n;
  const bool host_src = batch->src_mem == MLXD_MEM_HOST;
  const bool host_dst = batch->dst_mem == MLXD_MEM_HOST;
  if (per_sample_dst && host_dst) {
    return fail(MLXD_ERR_INVALID, "per-sample destinations must be device memory");
  }

  std::lock_guard<std::mutex> guard(lane.mu);
  const int slot = lane.next_slot;
  lane.next_slot = (slot + 1) % kDescSlots;
  // The pinned descriptor table of this slot may still be in flight.
  MLXD_CUDA(cudaEventSynchronize(lane.desc_copied[slot]));
  harvest_timing(ctx, lane, slot, true);
  // descriptors, then (for host sources) the table of the gather kernel
  const size_t desc_bytes = (sizeof(DevSample) * n + 255) & ~(size_t)255;
  const size_t block_bytes = desc_bytes + sizeof(GatherPiece) * n;
  rc = arena_reserve(ctx, lane.h_desc[slot], block_bytes, true, lane.stream);
  if (rc != MLXD_OK) {
    return rc;
  }
  rc = arena_reserve(ctx, lane.d_desc[slot], block_bytes, false, lane.stream);
  if (rc != MLXD_OK) {
    return rc;
  }

  // Stage host sources: only the rows the chain reads, each block 256-byte aligned.
  struct Piece {
    size_t offset, row_bytes, rows, from_pitch;
    const uint8_t* from;
  };
  std::vector<Piece> pieces;
  size_t stage_bytes = 0;
  uint64_t algo_src = 0;
  for (int i = 0; i < n; i++) {
    int32_t r0, r1, c0, c1;
    needed_region(dev[i], 0, r0, r1, c0, c1);
    algo_src += (uint64_t)(r1 - r0) * (uint64_t)(c1 - c0) * p.c_in;
  }
  ctx->algo_src += algo_src;
  ctx->algo_dst += out_bytes;
  // Page-locked sources that the GPU can address are packed by a kernel that
  // reads exactly the needed rectangles (gather.cu); anything else goes
  // through the copy engines.  MLXD_HOST_GATHER=0 turns the kernel path off.
  bool gather = false;
  std::vector<const uint8_t*> src_dev;
  if (host_src) {
    static const bool gather_enabled = [] {
      const char* v = std::getenv("MLXD_HOST_GATHER");
      return !(v && *v == '0');
    }();
    gather = gather_enabled;
    src_dev.resize(n);
    // sources in blocks from mlxd_pinned_alloc: a table look-up, no driver call
    for (int i = 0; i < n && gather; i++) {
      src_dev[i] = pinned_registry_lookup(samples[i].src);
      gather = src_dev[i] != nullptr;
    }
  }
  bool bounce = false;              // some source lies in ordinary (pageable) host memory
  std::vector<char> direct_copy;    // per sample: page-locked memory the copy engines can read
  unsigned int host_flags = 0;
  if (host_src) {
    pieces.resize(n);
    direct_copy.assign(n, 0);
    for (int i = 0; i < n; i++) {
      int32_t r0, r1, c0, c1;
      needed_region(dev[i], 2, r0, r1, c0, c1);
      // A strided (2-D) copy moves fewer bytes but runs slower per byte than a
      // contiguous one: trim columns only when that drops at least the
      // configured share of every row (MLXD_TRIM_PERCENT, default 60).
      static const int trim_percent = [] {
        const char* v = std::getenv("MLXD_TRIM_PERCENT");
        return v && *v ? std::atoi(v) : 60;
      }();
      // (sources in ordinary host memory are packed by the calling thread into a
      // page-locked block, which drops the columns for free)
      const bool direct = !gather && cudaHostGetFlags(&host_flags, const_cast<uint8_t*>(samples[i].src)) == cudaSuccess;
      if (!gather && !direct) {
        cudaGetLastError();
        bounce = true;
      }
      if (direct && (int64_t)(dev[i].src_w - (c1 - c0)) * 100 < (int64_t)trim_percent * dev[i].src_w) {
        c0 = 0;
        c1 = dev[i].src_w;
      }
      direct_copy[i] = direct;
      // The staged block is an image of its own: rows [r0, r1), columns
      // [c0, c1) of the source, tightly packed.
      pieces[i].offset = stage_bytes;
      pieces[i].row_bytes = (size_t)(c1 - c0) * p.c_in;
      pieces[i].rows = (size_t)(r1 - r0);
      pieces[i].from_pitch = (size_t)dev[i].src_w * p.c_in;
      pieces[i].from = samples[i].src + pieces[i].from_pitch * (size_t)r0 + (size_t)c0 * p.c_in;
      stage_bytes += (pieces[i].row_bytes * pieces[i].rows + 255) & ~(size_t)255;
      dev[i].src_w = c1 - c0;
      dev[i].pre_x -= c0;
      dev[i].r0_staged = r0;
    }
    rc = arena_reserve(ctx, lane.d_src, stage_bytes + 256, false, lane.stream);
    if (rc != MLXD_OK) {
      return rc;
    }
    for (int i = 0; i < n; i++) {
      // Base of a virtual image whose rows from r0 on are the staged block.
      dev[i].src = static_cast<const uint8_t*>(lane.d_src.ptr) + pieces[i].offset -
          pieces[i].row_bytes * (size_t)dev[i].r0_staged;
    }
  }
  uint8_t* out_base = static_cast<uint8_t*>(batch->dst);
  if (host_dst) {
    rc = arena_reserve(ctx, lane.d_out, out_bytes, false, lane.stream);
    if (rc != MLXD_OK) {
      return rc;
    }
    out_base = static_cast<uint8_t*>(lane.d_out.ptr);
  }
  for (int i = 0; i < n; i++) {
    dev[i].dst = per_sample_dst ? (*per_sample_dst)[i] : static_cast<void*>(out_base + slot_bytes * i);
  }

  std::memcpy(lane.h_desc[slot].ptr, dev.data(), sizeof(DevSample) * n);
  size_t upload = sizeof(DevSample) * n;
  uint32_t gather_rows = 0;
  if (gather) {
    GatherPiece* gp = reinterpret_cast<GatherPiece*>(static_cast<uint8_t*>(lane.h_desc[slot].ptr) + desc_bytes);
    for (int i = 0; i < n; i++) {
      gp[i].src = src_dev[i] + (pieces[i].from - samples[i].src);
      gp[i].dst = static_cast<uint8_t*>(lane.d_src.ptr) + pieces[i].offset;
      gp[i].src_pitch = pieces[i].from_pitch;
      gp[i].rows = (uint32_t)pieces[i].rows;
      gp[i].row_bytes = (uint32_t)pieces[i].row_bytes;
      gp[i].first_row = gather_rows;
      gp[i].pad_ = 0;
      gather_rows += (uint32_t)pieces[i].rows;
    }
    upload = block_bytes;
  }
  MLXD_CUDA(cudaMemcpyAsync(lane.d_desc[slot].ptr, lane.h_desc[slot].ptr, upload, cudaMemcpyHostToDevice, lane.stream));
  MLXD_CUDA(cudaEventRecord(lane.desc_copied[slot], lane.stream));
  const bool timed = ctx->timing.load() != 0;
  lane.in_timed[slot] = false;
  lane.out_timed[slot] = false;
  if (bounce) {
    // Pack the rectangles of the pageable sources into the lane's page-locked
    // block (the calling thread does the copying), then one copy for all of
    // them.  The block may still be feeding the previous batch of this lane.
    rc = arena_reserve(ctx, lane.h_src, stage_bytes + 256, true, lane.stream);
    if (rc != MLXD_OK) {
      return rc;
    }
    MLXD_CUDA(cudaEventSynchronize(lane.src_copied));
    const auto t0 = std::chrono::steady_clock::now();
    // The calling thread and up to pack_threads - 1 helpers started for this
    // batch take samples off a shared counter; packing is plain row copies.
    std::atomic<int> next{0};
    uint8_t* const block = static_cast<uint8_t*>(lane.h_src.ptr);
    auto pack = [&]() {
      for (int i = next.fetch_add(1); i < n; i = next.fetch_add(1)) {
        if (direct_copy[i]) {
          continue;
        }
        uint8_t* to = block + pieces[i].offset;
        const uint8_t* from = pieces[i].from;
        if (pieces[i].row_bytes == pieces[i].from_pitch) {
          std::memcpy(to, from, pieces[i].row_bytes * pieces[i].rows);
        } else {
          for (size_t r = 0; r < pieces[i].rows; r++) {
            std::memcpy(to + r * pieces[i].row_bytes, from + r * pieces[i].from_pitch, pieces[i].row_bytes);
          }
        }
      }
    };
    const int helpers = stage_bytes >= (size_t(8) << 20) ? std::min(pack_threads() - 1, n - 1) : 0;
    std::vector<std::thread> crew;
    crew.reserve(helpers > 0 ? helpers : 0);
    for (int t = 0; t < helpers; t++) {
      crew.emplace_back(pack);
    }
    pack();
    for (auto& th : crew) {
      th.join();
    }
    ctx->host_stage_ns += (uint64_t)std::chrono::duration_cast<std::chrono::nanoseconds>(
        std::chrono::steady_clock::now() - t0).count();
  }
  if (timed && host_src) {
    MLXD_CUDA(cudaEventRecord(lane.in_begin[slot], lane.stream));
    lane.in_timed[slot] = true;
  }
  if (gather) {
    const GatherPiece* gd =
        reinterpret_cast<const GatherPiece*>(static_cast<const uint8_t*>(lane.d_desc[slot].ptr) + desc_bytes);
    MLXD_CUDA(launch_gather_rows(gd, n, gather_rows, lane.stream));
    ctx->launches += 1;
    uint64_t moved = 0;
    for (int i = 0; i < n; i++) {
      moved += (uint64_t)pieces[i].row_bytes * pieces[i].rows;
    }
    ctx->h2d += moved;
  } else if (host_src) {
    bool all_bounced = true;
    for (int i = 0; i < n; i++) {
      all_bounced = all_bounced && !direct_copy[i];
    }
    if (all_bounced) {
      MLXD_CUDA(cudaMemcpyAsync(lane.d_src.ptr, lane.h_src.ptr, stage_bytes, cudaMemcpyHostToDevice, lane.stream));
    } else {
      for (int i = 0; i < n; i++) {
        uint8_t* to = static_cast<uint8_t*>(lane.d_src.ptr) + pieces[i].offset;
        const size_t bytes = pieces[i].row_bytes * pieces[i].rows;
        if (!direct_copy[i]) {
          MLXD_CUDA(cudaMemcpyAsync(
              to, static_cast<uint8_t*>(lane.h_src.ptr) + pieces[i].offset, bytes, cudaMemcpyHostToDevice, lane.stream));
        } else if (pieces[i].row_bytes == pieces[i].from_pitch) {
          MLXD_CUDA(cudaMemcpyAsync(to, pieces[i].from, bytes, cudaMemcpyHostToDevice, lane.stream));
        } else {
          MLXD_CUDA(cudaMemcpy2DAsync(
              to, pieces[i].row_bytes, pieces[i].from, pieces[i].from_pitch, pieces[i].row_bytes, pieces[i].rows,
              cudaMemcpyHostToDevice, lane.stream));
        }
      }
    }
    if (bounce) {
      MLXD_CUDA(cudaEventRecord(lane.src_copied, lane.stream));
    }
    ctx->h2d += stage_bytes;
  }
  p.samples = static_cast<const DevSample*>(lane.d_desc[slot].ptr);
  if (timed) {
    MLXD_CUDA(cudaEventRecord(lane.k_begin[slot], lane.stream));
  }
  MLXD_CUDA(launch_fused_batch(p, lane.stream));
  if (timed) {
    MLXD_CUDA(cudaEventRecord(lane.k_end[slot], lane.stream));
    lane.k_pending[slot] = true;
  }
  if (host_dst) {
    MLXD_CUDA(cudaMemcpyAsync(batch->dst, lane.d_out.ptr, out_bytes, cudaMemcpyDeviceToHost, lane.stream));
    ctx->d2h += out_bytes;
    if (timed) {
      MLXD_CUDA(cudaEventRecord(lane.out_end[slot], lane.stream));
      lane.out_timed[slot] = true;
    }
  }
  MLXD_CUDA(cudaMemcpyAsync(lane.h_status, lane.d_status, sizeof(int32_t), cudaMemcpyDeviceToHost, lane.stream));
  MLXD_CUDA(cudaEventRecord(lane.done, lane.stream));
  ctx->batches += 1;
  ctx->samples += n;
  ctx->launches += 1;
  return MLXD_OK;
}

void harvest_timing(mlxd_ctx* ctx, Lane& lane, int slot, bool block) {
  if (!lane.k_pending[slot]) {
    return;
  }
  if (block) {
    if (cudaEventSynchronize(lane.k_end[slot]) != cudaSuccess) {
      return;
    }
  } else if (cudaEventQuery(lane.k_end[slot]) != cudaSuccess) {
    return;
  }
  if (lane.out_timed[slot]) {
    const cudaError_t oe = block ? cudaEventSynchronize(lane.out_end[slot]) : cudaEventQuery(lane.out_end[slot]);
    if (oe != cudaSuccess) {
      return;
    }
  }
  float ms = 0.0f;
  if (cudaEventElapsedTime(&ms, lane.k_begin[slot], lane.k_end[slot]) == cudaSuccess) {
    ctx->kernel_ns += (uint64_t)((double)ms * 1e6);
    ctx->timed_launches += 1;
  }
  if (lane.in_timed[slot] && cudaEventElapsedTime(&ms, lane.in_begin[slot], lane.k_begin[slot]) == cudaSuccess) {
    ctx->h2d_ns += (uint64_t)((double)ms * 1e6);
  }
  if (lane.out_timed[slot] && cudaEventElapsedTime(&ms, lane.k_end[slot], lane.out_end[slot]) == cudaSuccess) {
    ctx->d2h_ns += (uint64_t)((double)ms * 1e6);
  }
  lane.in_timed[slot] = false;
  lane.out_timed[slot] = false;
  lane.k_pending[slot] = false;
}

int wait_lane(mlxd_ctx* ctx, Lane& lane, int timeout_ms) {
  MLXD_ON_DEVICE(ctx->device);
  const auto start = std::chrono::steady_clock::now();
  if (timeout_ms < 0) {
    // no deadline: block in the driver instead of polling it from every lane
    MLXD_CUDA(cudaEventSynchronize(lane.done));
  }
  for (;;) {
    cudaError_t e = cudaEventQuery(lane.done);
    if (e == cudaSuccess) {
      break;
    }
    if (e != cudaErrorNotReady) {
      return fail_cuda(e, "cudaEventQuery(lane)");
    }
    if (timeout_ms >= 0) {
      const auto el = std::chrono::duration_cast<std::chrono::milliseconds>(
          std::chrono::steady_clock::now() - start).count();
      if (el >= timeout_ms) {
        return fail(MLXD_ERR_TIMEOUT, "lane still busy after " + std::to_string(timeout_ms) + " ms");
      }
    }
    std::this_thread::sleep_for(std::chrono::microseconds(20));
  }
  {
    std::lock_guard<std::mutex> guard(lane.mu);
    for (int s = 0; s < kDescSlots; s++) {
      harvest_timing(ctx, lane, s, false);
    }
  }
  if (*lane.h_status != 0) {
    // Reported once: the word is cleared so that later batches on this lane
    // start clean (other lanes have words of their own).
    const int32_t seen = *lane.h_status;
    *lane.h_status = 0;
    cudaMemsetAsync(lane.d_status, 0, sizeof(int32_t), lane.stream);
    return fail(MLXD_ERR_DEVICE, "kernel self-check failed (status " + std::to_string(seen) + ")");
  }
  return MLXD_OK;
}

} // namespace mlxd
