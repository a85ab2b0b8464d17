// extern "C" entry points declared in include/mlxd_b200.h.
#include <cstring>
#include <new>

#include "context.h"

using namespace mlxd;

namespace {

thread_local std::string g_last;

// int32 words between the self-check words of two lanes
constexpr size_t kStatusStride = 16;

void destroy_lane(Lane* l) {
  if (!l) {
    return;
  }
  if (l->stream) {
    cudaStreamSynchronize(l->stream);
  }
  for (int s = 0; s < kDescSlots; s++) {
    if (l->d_desc[s].ptr) cudaFree(l->d_desc[s].ptr);
    if (l->h_desc[s].ptr) cudaFreeHost(l->h_desc[s].ptr);
    if (l->desc_copied[s]) cudaEventDestroy(l->desc_copied[s]);
    if (l->k_begin[s]) cudaEventDestroy(l->k_begin[s]);
    if (l->k_end[s]) cudaEventDestroy(l->k_end[s]);
    if (l->in_begin[s]) cudaEventDestroy(l->in_begin[s]);
    if (l->out_end[s]) cudaEventDestroy(l->out_end[s]);
  }
  if (l->src_copied) cudaEventDestroy(l->src_copied);
  if (l->h_src.ptr) cudaFreeHost(l->h_src.ptr);
  if (l->d_src.ptr) cudaFree(l->d_src.ptr);
  if (l->d_out.ptr) cudaFree(l->d_out.ptr);
  if (l->h_status) cudaFreeHost(l->h_status);
  if (l->done) cudaEventDestroy(l->done);
  if (l->stream) cudaStreamDestroy(l->stream);
  delete l;
}

int make_lane(Lane** out) {
  Lane* l = new (std::nothrow) Lane();
  if (!l) {
    return fail(MLXD_ERR_NOMEM, "out of host memory");
  }
  cudaError_t e = cudaStreamCreateWithFlags(&l->stream, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaEventCreateWithFlags(&l->done, cudaEventDisableTiming | cudaEventBlockingSync);
  if (e == cudaSuccess) e = cudaEventCreateWithFlags(&l->src_copied, cudaEventDisableTiming);
  for (int s = 0; s < kDescSlots && e == cudaSuccess; s++) {
    e = cudaEventCreateWithFlags(&l->desc_copied[s], cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreate(&l->k_begin[s]);
    if (e == cudaSuccess) e = cudaEventCreate(&l->k_end[s]);
    if (e == cudaSuccess) e = cudaEventCreate(&l->in_begin[s]);
    if (e == cudaSuccess) e = cudaEventCreate(&l->out_end[s]);
  }
  if (e == cudaSuccess) e = cudaHostAlloc(reinterpret_cast<void**>(&l->h_status), sizeof(int32_t), cudaHostAllocDefault);
  if (e != cudaSuccess) {
    destroy_lane(l);
    return fail_cuda(e, "lane setup");
  }
  *l->h_status = 0;
  *out = l;
  return MLXD_OK;
}

// Synchronous run of one launch on the context's private lane.
int run_sync(mlxd_ctx* ctx, const mlxd_sample_desc* s, int n, const mlxd_batch_desc* b) {
  Lane& lane = *ctx->lanes[ctx->n_user_lanes];
  int rc = enqueue_on_lane(ctx, lane, s, n, b, nullptr);
  if (rc != MLXD_OK) {
    return rc;
  }
  return wait_lane(ctx, lane, -1);
}

mlxd_sample_desc whole_image(const uint8_t* src, int h, int w) {
  mlxd_sample_desc d;
  std::memset(&d, 0, sizeof(d));
  d.src = src;
  d.src_h = h;
  d.src_w = w;
  d.pre_w = w;
  d.pre_h = h;
  d.geom = MLXD_GEOM_NONE;
  d.geom_w = w;
  d.geom_h = h;
  d.post_w = w;
  d.post_h = h;
  return d;
}

mlxd_batch_desc u8_batch(void* dst, int slot_h, int slot_w, int c) {
  mlxd_batch_desc b;
  std::memset(&b, 0, sizeof(b));
  b.dst = dst;
  b.slot_h = slot_h;
  b.slot_w = slot_w;
  b.channels = c;
  b.out_dtype = MLXD_U8;
  b.divisor = 1.0f;
  b.src_mem = MLXD_MEM_HOST;
  b.dst_mem = MLXD_MEM_HOST;
  return b;
}

} // namespace

extern "C" {

int mlxd_ctx_create(int device, int n_lanes, mlxd_ctx** out) {
  if (!out || n_lanes < 1 || n_lanes > 256) {
    return fail(MLXD_ERR_INVALID, "mlxd_ctx_create: need an output pointer and 1..256 lanes");
  }
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess) {
    return fail_cuda(e, "cudaGetDeviceCount");
  }
  if (device < 0 || device >= count) {
    return fail(MLXD_ERR_INVALID, "mlxd_ctx_create: no such CUDA device");
  }
  MLXD_ON_DEVICE(device);
  mlxd_ctx* ctx = new (std::nothrow) mlxd_ctx();
  if (!ctx) {
    return fail(MLXD_ERR_NOMEM, "out of host memory");
  }
  ctx->device = device;
  ctx->n_user_lanes = n_lanes;
  const size_t status_bytes = (size_t)(n_lanes + 2) * kStatusStride * sizeof(int32_t);
  e = cudaMalloc(reinterpret_cast<void**>(&ctx->d_status), status_bytes);
  if (e == cudaSuccess) e = cudaMemset(ctx->d_status, 0, status_bytes);
  if (e != cudaSuccess) {
    mlxd_ctx_destroy(ctx);
    return fail_cuda(e, "status word");
  }
  // user lanes, then one private lane for the synchronous ops and one whose
  // descriptor ring serves launches on caller streams
  for (int i = 0; i < n_lanes + 2; i++) {
    Lane* l = nullptr;
    int rc = make_lane(&l);
    if (rc != MLXD_OK) {
      mlxd_ctx_destroy(ctx);
      return rc;
    }
    l->d_status = ctx->d_status + (size_t)i * kStatusStride;
    ctx->lanes.push_back(l);
  }
  *out = ctx;
  return MLXD_OK;
}

void mlxd_ctx_destroy(mlxd_ctx* ctx) {
  if (!ctx) {
    return;
  }
  DeviceGuard on_device(ctx->device);
  for (Lane* l : ctx->lanes) {
    destroy_lane(l);
  }
  for (auto& kv : ctx->luts) {
    cudaFree(kv.second);
  }
  if (ctx->d_status) {
    cudaFree(ctx->d_status);
  }
  delete ctx;
}

int mlxd_device_pci_bus_id(int device, char* out, size_t len) {
  if (!out || len < 16) {
    return fail(MLXD_ERR_INVALID, "mlxd_device_pci_bus_id: buffer of at least 16 bytes expected");
  }
  MLXD_CUDA(cudaDeviceGetPCIBusId(out, (int)len, device));
  return MLXD_OK;
}

const char* mlxd_last_error(void) {
  g_last = error_text();
  return g_last.c_str();
}

void* mlxd_pinned_alloc(size_t bytes) {
  void* p = nullptr;
  if (bytes == 0) {
    bytes = 1;
  }
  cudaError_t e = cudaHostAlloc(&p, bytes, cudaHostAllocPortable | cudaHostAllocMapped);
  if (e != cudaSuccess) {
    fail_cuda(e, "cudaHostAlloc");
    return nullptr;
  }
  // Remember the block: sources inside it can be read by the gather kernel.
  void* dp = nullptr;
  if (cudaHostGetDevicePointer(&dp, p, 0) == cudaSuccess && dp != nullptr) {
    mlxd::pinned_registry_add(p, bytes, dp);
  } else {
    cudaGetLastError();
  }
  return p;
}

void mlxd_pinned_free(void* p) {
  if (p) {
    mlxd::pinned_registry_remove(p);
    cudaFreeHost(p);
  }
}

void* mlxd_device_alloc(mlxd_ctx* ctx, size_t bytes) {
  if (!ctx) {
    fail(MLXD_ERR_INVALID, "mlxd_device_alloc: null context");
    return nullptr;
  }
  void* p = nullptr;
  DeviceGuard on_device(ctx->device);
  cudaError_t e = on_device.err;
  if (e == cudaSuccess) e = cudaMalloc(&p, bytes == 0 ? 1 : bytes);
  if (e != cudaSuccess) {
    fail_cuda(e, "cudaMalloc");
    return nullptr;
  }
  return p;
}

void mlxd_device_free(mlxd_ctx* ctx, void* p) {
  if (ctx && p) {
    DeviceGuard on_device(ctx->device);
    cudaFree(p);
  }
}

int mlxd_ctx_set_timing(mlxd_ctx* ctx, int on) {
  if (!ctx) {
    return fail(MLXD_ERR_INVALID, "mlxd_ctx_set_timing: null context");
  }
  ctx->timing.store(on ? 1 : 0);
  return MLXD_OK;
}

int mlxd_fused_batch(
    mlxd_ctx* ctx, int lane, const mlxd_sample_desc* samples, int n, const mlxd_batch_desc* batch) {
  if (!ctx || lane < 0 || lane >= ctx->n_user_lanes) {
    return fail(MLXD_ERR_INVALID, "mlxd_fused_batch: bad context or lane index");
  }
  return enqueue_on_lane(ctx, *ctx->lanes[lane], samples, n, batch, nullptr);
}

int mlxd_batch_wait(mlxd_ctx* ctx, int lane, int timeout_ms) {
  if (!ctx || lane < 0 || lane >= ctx->n_user_lanes) {
    return fail(MLXD_ERR_INVALID, "mlxd_batch_wait: bad context or lane index");
  }
  return wait_lane(ctx, *ctx->lanes[lane], timeout_ms);
}

int mlxd_fused_batch_on_stream(
    mlxd_ctx* ctx, void* cuda_stream, const mlxd_sample_desc* samples, int n, const mlxd_batch_desc* batch) {
  if (!ctx || !samples || !batch || n < 0) {
    return fail(MLXD_ERR_INVALID, "mlxd_fused_batch_on_stream: null argument");
  }
  if (n == 0) {
    return MLXD_OK;
  }
  if (batch->src_mem != MLXD_MEM_DEVICE || batch->dst_mem != MLXD_MEM_DEVICE || !batch->dst) {
    return fail(MLXD_ERR_INVALID, "mlxd_fused_batch_on_stream: sources and destination must be device memory");
  }
  MLXD_ON_DEVICE(ctx->device);
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  // validate + plan
  std::vector<DevSample> dev;
  PassNeed need;
  mlxd_batch_desc b = *batch;
  Lane& ring = *ctx->lanes[ctx->n_user_lanes + 1];
  LutUse table_in_use(ctx);
  LaunchParams p;
  int rc = prepare_launch(ctx, &b, n, p);
  if (rc != MLXD_OK) {
    return rc;
  }
  p.status = ring.d_status;
  rc = plan_samples(samples, n, &b, dev, need);
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
  const size_t slot_bytes = (size_t)b.slot_h * b.slot_w * p.c_out * esize;
  uint64_t algo_src = 0;
  for (int i = 0; i < n; i++) {
    dev[i].dst = static_cast<uint8_t*>(b.dst) + slot_bytes * i;
    int32_t r0, r1, c0, c1;
    needed_region(dev[i], 0, r0, r1, c0, c1);
    algo_src += (uint64_t)(r1 - r0) * (uint64_t)(c1 - c0) * p.c_in;
  }
  ctx->algo_src += algo_src;
  ctx->algo_dst += slot_bytes * n;
  std::lock_guard<std::mutex> guard(ring.mu);
  const int slot = ring.next_slot;
  ring.next_slot = (slot + 1) % kDescSlots;
  // Here the slot's event is recorded after the kernel, so a finished wait
  // means neither the copy nor the kernel still needs the tables.
  MLXD_CUDA(cudaEventSynchronize(ring.desc_copied[slot]));
  harvest_timing(ctx, ring, slot, true);
  rc = arena_reserve(ctx, ring.h_desc[slot], sizeof(DevSample) * n, true, nullptr);
  if (rc != MLXD_OK) {
    return rc;
  }
  rc = arena_reserve(ctx, ring.d_desc[slot], sizeof(DevSample) * n, false, nullptr);
  if (rc != MLXD_OK) {
    return rc;
  }
  std::memcpy(ring.h_desc[slot].ptr, dev.data(), sizeof(DevSample) * n);
  MLXD_CUDA(cudaMemcpyAsync(
      ring.d_desc[slot].ptr, ring.h_desc[slot].ptr, sizeof(DevSample) * n, cudaMemcpyHostToDevice, stream));
  p.samples = static_cast<const DevSample*>(ring.d_desc[slot].ptr);
  const bool timed = ctx->timing.load() != 0;
  if (timed) {
    MLXD_CUDA(cudaEventRecord(ring.k_begin[slot], stream));
  }
  MLXD_CUDA(launch_fused_batch(p, stream));
  if (timed) {
    MLXD_CUDA(cudaEventRecord(ring.k_end[slot], stream));
    ring.k_pending[slot] = true;
  }
  MLXD_CUDA(cudaEventRecord(ring.desc_copied[slot], stream));
  ctx->batches += 1;
  ctx->samples += n;
  ctx->launches += 1;
  return MLXD_OK;
}

int mlxd_stream_status(mlxd_ctx* ctx, void* cuda_stream, int32_t* status) {
  if (!ctx) {
    return fail(MLXD_ERR_INVALID, "mlxd_stream_status: null context");
  }
  MLXD_ON_DEVICE(ctx->device);
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  Lane& ring = *ctx->lanes[ctx->n_user_lanes + 1];
  std::lock_guard<std::mutex> guard(ring.mu);
  MLXD_CUDA(cudaMemcpyAsync(ring.h_status, ring.d_status, sizeof(int32_t), cudaMemcpyDeviceToHost, stream));
  MLXD_CUDA(cudaStreamSynchronize(stream));
  const int32_t seen = *ring.h_status;
  if (status) {
    *status = seen;
  }
  if (seen != 0) {
    *ring.h_status = 0;
    MLXD_CUDA(cudaMemsetAsync(ring.d_status, 0, sizeof(int32_t), stream));
    return fail(MLXD_ERR_DEVICE, "kernel self-check failed (status " + std::to_string(seen) + ")");
  }
  return MLXD_OK;
}

int mlxd_image_resize(mlxd_ctx* ctx, const uint8_t* src, int h, int w, int c, uint8_t* dst, int dh, int dw) {
  if (!ctx || !src || !dst) {
    return fail(MLXD_ERR_INVALID, "mlxd_image_resize: null argument");
  }
  if (dh <= 0 || dw <= 0) {
    return fail(MLXD_ERR_INVALID, "image: cannot create image with 0 or negative dimension");
  }
  mlxd_sample_desc d = whole_image(src, h, w);
  d.geom = MLXD_GEOM_RESIZE;
  d.geom_w = dw;
  d.geom_h = dh;
  d.post_w = dw;
  d.post_h = dh;
  mlxd_batch_desc b = u8_batch(dst, dh, dw, c);
  return run_sync(ctx, &d, 1, &b);
}

int mlxd_image_crop(
    mlxd_ctx* ctx, const uint8_t* src, int h, int w, int c, int x, int y, int cw, int ch, uint8_t* dst) {
  if (!ctx || !src || !dst) {
    return fail(MLXD_ERR_INVALID, "mlxd_image_crop: null argument");
  }
  mlxd_sample_desc d = whole_image(src, h, w);
  d.post_x = x;
  d.post_y = y;
  d.post_w = cw;
  d.post_h = ch;
  mlxd_batch_desc b = u8_batch(dst, ch, cw, c);
  return run_sync(ctx, &d, 1, &b);
}

int mlxd_image_hflip(mlxd_ctx* ctx, const uint8_t* src, int h, int w, int c, uint8_t* dst) {
  if (!ctx || !src || !dst) {
    return fail(MLXD_ERR_INVALID, "mlxd_image_hflip: null argument");
  }
  mlxd_sample_desc d = whole_image(src, h, w);
  d.post_flip = 1;
  mlxd_batch_desc b = u8_batch(dst, h, w, c);
  return run_sync(ctx, &d, 1, &b);
}

int mlxd_image_affine(
    mlxd_ctx* ctx, const uint8_t* src, int h, int w, int c, const float mx[6], int th, int tw, uint8_t* dst) {
  if (!ctx || !src || !dst || !mx) {
    return fail(MLXD_ERR_INVALID, "mlxd_image_affine: null argument");
  }
  if (th <= 0 || tw <= 0) {
    return fail(MLXD_ERR_INVALID, "image: cannot create image with 0 or negative dimension");
  }
  mlxd_sample_desc d = whole_image(src, h, w);
  d.geom = MLXD_GEOM_AFFINE;
  d.geom_w = tw;
  d.geom_h = th;
  d.post_w = tw;
  d.post_h = th;
  std::memcpy(d.mx, mx, sizeof(d.mx));
  mlxd_batch_desc b = u8_batch(dst, th, tw, c);
  return run_sync(ctx, &d, 1, &b);
}

int mlxd_image_channel_reduction(
    mlxd_ctx* ctx, const uint8_t* src, int h, int w, const int32_t m_fixed[3], int32_t bias_fixed, uint8_t* dst) {
  if (!ctx || !src || !dst || !m_fixed) {
    return fail(MLXD_ERR_INVALID, "mlxd_image_channel_reduction: null argument");
  }
  mlxd_sample_desc d = whole_image(src, h, w);
  mlxd_batch_desc b = u8_batch(dst, h, w, 3);
  b.gray = 1;
  b.gray_m[0] = m_fixed[0];
  b.gray_m[1] = m_fixed[1];
  b.gray_m[2] = m_fixed[2];
  b.gray_bias = bias_fixed;
  return run_sync(ctx, &d, 1, &b);
}

int mlxd_batch_pad(
    mlxd_ctx* ctx, const uint8_t* const* srcs, const int32_t* hs, const int32_t* ws, int n, int c,
    int slot_h, int slot_w, double pad_value, uint8_t* dst) {
  if (!ctx || !srcs || !hs || !ws || !dst || n < 0) {
    return fail(MLXD_ERR_INVALID, "mlxd_batch_pad: null argument");
  }
  std::vector<mlxd_sample_desc> d((size_t)n);
  for (int i = 0; i < n; i++) {
    d[i] = whole_image(srcs[i], hs[i], ws[i]);
  }
  mlxd_batch_desc b = u8_batch(dst, slot_h, slot_w, c);
  b.pad_value = pad_value;
  return run_sync(ctx, d.data(), n, &b);
}

int mlxd_cast_scale_normalise(
    mlxd_ctx* ctx, const uint8_t* src, int64_t count, int c, float divisor,
    const float* mean, const float* std_, float* dst) {
  if (!ctx || !src || !dst || count < 0 || c < 1 || c > 4) {
    return fail(MLXD_ERR_INVALID, "mlxd_cast_scale_normalise: bad argument");
  }
  if ((mean == nullptr) != (std_ == nullptr)) {
    return fail(MLXD_ERR_INVALID, "mlxd_cast_scale_normalise: mean and std come together");
  }
  // The pixel run is cast as a [rows, 4096] image followed by one short row.
  const int64_t kRow = 4096;
  const int64_t rows = count / kRow;
  const int64_t rem = count - rows * kRow;
  if (rows > 0x7fffffff) {
    return fail(MLXD_ERR_INVALID, "mlxd_cast_scale_normalise: too many pixels");
  }
  for (int part = 0; part < 2; part++) {
    const int h = part == 0 ? (int)rows : 1;
    const int w = part == 0 ? (int)kRow : (int)rem;
    if (h == 0 || w == 0) {
      continue;
    }
    const int64_t off = part == 0 ? 0 : rows * kRow * c;
    mlxd_sample_desc d = whole_image(src + off, h, w);
    mlxd_batch_desc b = u8_batch(dst + off, h, w, c);
    b.out_dtype = MLXD_F32;
    b.divisor = divisor;
    if (mean) {
      b.normalise = 1;
      for (int k = 0; k < c; k++) {
        b.mean[k] = mean[k];
        b.std_[k] = std_[k];
      }
    }
    int rc = run_sync(ctx, &d, 1, &b);
    if (rc != MLXD_OK) {
      return rc;
    }
  }
  return MLXD_OK;
}

int mlxd_stats_get(mlxd_ctx* ctx, mlxd_stats* out) {
  if (!ctx || !out) {
    return fail(MLXD_ERR_INVALID, "mlxd_stats_get: null argument");
  }
  // launches on caller streams are harvested here, once they have finished
  {
    Lane& ring = *ctx->lanes[ctx->n_user_lanes + 1];
    std::lock_guard<std::mutex> guard(ring.mu);
    for (int s = 0; s < kDescSlots; s++) {
      harvest_timing(ctx, ring, s, false);
    }
  }
  out->algo_src_bytes = ctx->algo_src.load();
  out->algo_dst_bytes = ctx->algo_dst.load();
  out->kernel_ns = ctx->kernel_ns.load();
  out->timed_launches = ctx->timed_launches.load();
  out->batches = ctx->batches.load();
  out->samples = ctx->samples.load();
  out->kernel_launches = ctx->launches.load();
  out->h2d_bytes = ctx->h2d.load();
  out->d2h_bytes = ctx->d2h.load();
  out->device_bytes_reserved = ctx->reserved.load();
  out->h2d_ns = ctx->h2d_ns.load();
  out->d2h_ns = ctx->d2h_ns.load();
  out->host_stage_ns = ctx->host_stage_ns.load();
  return MLXD_OK;
}

} // extern "C"
