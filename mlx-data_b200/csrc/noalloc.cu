// mlxd_fused_batch_noalloc: the fused batch for callers that must not allocate.
//
// Some hosts of this library run where a CUDA allocation is not an option: a
// data-loading plug-in called from inside a training step whose memory pool
// owns the whole GPU, a real-time service that forbids allocator calls after
// start-up, a process that is already close to its memory limit.  The regular
// entry points keep descriptor tables, the cast table and a status word in
// memory they allocate on demand; this one keeps them in a fixed array that is
// part of the library image, so a call allocates nothing, on the device or on
// the host.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <mutex>

#include "context.h"

using namespace mlxd;

namespace {

constexpr int kMaxSamples = MLXD_NOALLOC_MAX_SAMPLES;
constexpr size_t kTableBytes = sizeof(DevSample) * kMaxSamples;
constexpr size_t kLutBytes = 4 * 256 * sizeof(float);
constexpr size_t kStatusOffset = kTableBytes + kLutBytes;
constexpr size_t kScratchBytes = kStatusOffset + 256;

// Scratch of the entry point: descriptor table, cast table, status word.
// Every GPU that loads the library holds these bytes until the process exits.
static __device__ __align__(256) unsigned char g_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mu;
unsigned char* g_scratch_addr[kMaxDevices] = {};

// Device address of g_scratch on `device`, which must be the current device.
// In host code the array's name is only a handle; the address a kernel can use
// comes from cudaGetSymbolAddress, once per device.
int scratch_for(int device, unsigned char** out) {
  std::lock_guard<std::mutex> g(g_setup_mu);
  if (!g_scratch_addr[device]) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_scratch);
    if (e != cudaSuccess) {
      return fail_cuda(e, "cudaGetSymbolAddress(scratch)");
    }
    g_scratch_addr[device] = static_cast<unsigned char*>(p);
  }
  *out = g_scratch_addr[device];
  return MLXD_OK;
}

}  // namespace

extern "C" int mlxd_fused_batch_noalloc(
    int device, void* cuda_stream, const mlxd_sample_desc* samples, int n, const mlxd_batch_desc* batch) {
  if (!samples || !batch || n < 0) {
    return fail(MLXD_ERR_INVALID, "mlxd_fused_batch_noalloc: null descriptor or negative sample count");
  }
  if (n > kMaxSamples) {
    char msg[160];
    snprintf(msg, sizeof(msg),
             "mlxd_fused_batch_noalloc: at most %d samples per call (got %d); split the batch or use "
             "mlxd_fused_batch_on_stream", kMaxSamples, n);
    return fail(MLXD_ERR_INVALID, msg);
  }
  if (device < 0 || device >= kMaxDevices) {
    return fail(MLXD_ERR_INVALID, "mlxd_fused_batch_noalloc: device index out of range");
  }
  if (n == 0) {
    return MLXD_OK;
  }
  if (batch->src_mem != MLXD_MEM_DEVICE || batch->dst_mem != MLXD_MEM_DEVICE || !batch->dst) {
    return fail(MLXD_ERR_INVALID, "mlxd_fused_batch_noalloc: sources and destination must be device memory");
  }
  if (batch->channels < 1 || batch->channels > 4) {
    return fail(MLXD_ERR_INVALID, "image: channels must be 0 < c <= 4");
  }
  if (batch->gray && batch->channels != 3) {
    return fail(MLXD_ERR_INVALID, "image::channelReduction: expected a 3 channel uint8 array");
  }
  if (batch->slot_h <= 0 || batch->slot_w <= 0) {
    return fail(MLXD_ERR_INVALID, "batch slot must have positive height and width");
  }
  if (batch->out_dtype != MLXD_U8 && batch->out_dtype != MLXD_F32) {
    return fail(MLXD_ERR_INVALID, "unknown output dtype");
  }
  if (batch->out_dtype == MLXD_F32 && !(batch->divisor != 0.0f)) {
    return fail(MLXD_ERR_INVALID, "cast divisor must be non-zero");
  }
  MLXD_ON_DEVICE(device);
  unsigned char* scratch = nullptr;
  int rc = scratch_for(device, &scratch);
  if (rc != MLXD_OK) {
    return rc;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);

  // Host images of the tables: fixed storage in the library image (neither heap
  // nor lazily allocated thread-local memory), one caller at a time.
  static DevSample table[kMaxSamples];
  static float lut[4 * 256];
  static std::mutex table_mu;
  std::lock_guard<std::mutex> table_guard(table_mu);

  LaunchParams p;
  std::memset(&p, 0, sizeof(p));
  p.n = n;
  p.tiles_y = (batch->slot_h + kTileH - 1) / kTileH;
  p.tiles_x = (batch->slot_w + kTileW - 1) / kTileW;
  p.c_in = batch->channels;
  p.c_out = batch->gray ? 1 : batch->channels;
  p.gray = batch->gray ? 1 : 0;
  p.gray_m[0] = batch->gray_m[0];
  p.gray_m[1] = batch->gray_m[1];
  p.gray_m[2] = batch->gray_m[2];
  p.gray_bias = batch->gray_bias;
  p.out_f32 = batch->out_dtype == MLXD_F32;
  p.pad_px = (int32_t)(uint8_t)(int32_t)batch->pad_value;
  p.samples = reinterpret_cast<const DevSample*>(scratch);
  p.lut = reinterpret_cast<const float*>(scratch + kTableBytes);
  p.status = reinterpret_cast<int32_t*>(scratch + kStatusOffset);

  PassNeed need = PassNeed{0, 0, 0, 0, 0, 0};
  const size_t esize = p.out_f32 ? 4 : 1;
  const size_t slot_bytes = (size_t)batch->slot_h * batch->slot_w * p.c_out * esize;
  rc = plan_into(samples, n, batch, table, need);
  if (rc != MLXD_OK) {
    return rc;
  }
  for (int i = 0; i < n; i++) {
    table[i].dst = static_cast<uint8_t*>(batch->dst) + slot_bytes * i;
  }
  p.src_tile_bytes = need.src_bytes;
  p.mid_float4s = need.mid_float4s;
  p.weight_floats = need.weight_floats;
  p.u_cap = need.u_cap;
  p.fast_smem_bytes = (int32_t)need.fast_smem_bytes;
  choose_kernel(p, need, table, n);

  // The scratch keeps whatever the previous call left.  Its status word is
  // read back first (the kernel of the previous call is ahead of this copy on
  // the stream), then cleared; the tables are overwritten up to what this call
  // reads.
  static int32_t previous_status;
  previous_status = 0;
  MLXD_CUDA(cudaMemcpyAsync(&previous_status, scratch + kStatusOffset, sizeof(int32_t), cudaMemcpyDeviceToHost, stream));
  MLXD_CUDA(cudaMemsetAsync(scratch + kStatusOffset, 0, 256, stream));
  MLXD_CUDA(cudaMemcpyAsync(scratch, table, sizeof(DevSample) * n, cudaMemcpyHostToDevice, stream));
  if (p.out_f32) {
    compute_cast_table(batch, p.c_out, lut);
    MLXD_CUDA(cudaMemcpyAsync(
        scratch + kTableBytes, lut, (size_t)p.c_out * 256 * sizeof(float), cudaMemcpyHostToDevice, stream));
  }
  // the host tables are reused by the next call: let the copies finish
  MLXD_CUDA(cudaStreamSynchronize(stream));
  if (previous_status != 0) {
    // Nothing is launched: the caller learns here that the batch written by
    // the call before this one is not to be trusted.
    char msg[96];
    snprintf(msg, sizeof(msg), "the previous call's kernel failed a self-check (status %d); this call ran nothing",
             (int)previous_status);
    return fail(MLXD_ERR_DEVICE, msg);
  }
  MLXD_CUDA(launch_fused_batch(p, stream));
  return MLXD_OK;
}

extern "C" int mlxd_noalloc_status(int device, void* cuda_stream, int32_t* status) {
  if (device < 0 || device >= kMaxDevices) {
    return fail(MLXD_ERR_INVALID, "mlxd_noalloc_status: device index out of range");
  }
  MLXD_ON_DEVICE(device);
  unsigned char* scratch = nullptr;
  int rc = scratch_for(device, &scratch);
  if (rc != MLXD_OK) {
    return rc;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  static int32_t seen;
  static std::mutex seen_mu;
  std::lock_guard<std::mutex> g(seen_mu);
  seen = 0;
  MLXD_CUDA(cudaMemcpyAsync(&seen, scratch + kStatusOffset, sizeof(int32_t), cudaMemcpyDeviceToHost, stream));
  MLXD_CUDA(cudaStreamSynchronize(stream));
  if (status) {
    *status = seen;
  }
  if (seen != 0) {
    MLXD_CUDA(cudaMemsetAsync(scratch + kStatusOffset, 0, 256, stream));
    char msg[64];
    snprintf(msg, sizeof(msg), "kernel self-check failed (status %d)", (int)seen);
    return fail(MLXD_ERR_DEVICE, msg);
  }
  return MLXD_OK;
}
