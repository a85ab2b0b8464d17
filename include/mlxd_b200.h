/*
 * C ABI of the B200 image-transform-and-batch library (libmlxd_b200.so).
 *
 * mlx-data has no C ABI of its own: its boundary for this path is a set of C++
 * virtuals (op::ImageTransformOp::apply_image, stream::Batch::next,
 * core::merge_batch).  The entry points below are what those virtuals bind to
 * when the path runs on the GPU; each one names the reference interface it
 * replaces.  Plain pointers and sizes only, an int status on every call, no
 * exceptions and no C++ or torch types cross this boundary.
 *
 * Images are [H, W, C] uint8, C-contiguous (mlx/data/core/image/Image.h:35-49),
 * 1 <= C <= 4.  A batch is [N, slot_h, slot_w, C_out], C-contiguous.
 */
#ifndef MLXD_B200_H
#define MLXD_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MLXD_API __attribute__((visibility("default")))

typedef struct mlxd_ctx mlxd_ctx;

enum mlxd_status {
  MLXD_OK = 0,
  MLXD_ERR_INVALID = 1,     /* bad argument; mlxd_last_error() says which */
  MLXD_ERR_CUDA = 2,        /* a CUDA call failed; message carries its text */
  MLXD_ERR_NOMEM = 3,       /* host or device allocation failed */
  MLXD_ERR_TIMEOUT = 4,     /* mlxd_batch_wait ran out of time; work still queued */
  MLXD_ERR_UNSUPPORTED = 5, /* a shape the device code cannot run (kept for callers; nothing returns it now) */
  MLXD_ERR_DEVICE = 6       /* the kernel recorded a failed self-check */
};

enum mlxd_geom {
  MLXD_GEOM_NONE = 0,
  MLXD_GEOM_RESIZE = 1, /* core::image::resize, mlx/data/core/image/ImageTransform.cpp:41-62 */
  MLXD_GEOM_AFFINE = 2  /* core::image::affine, mlx/data/core/image/ImageTransform.cpp:75-111 */
};

enum mlxd_dtype { MLXD_U8 = 0, MLXD_F32 = 1 };
enum mlxd_mem { MLXD_MEM_HOST = 0, MLXD_MEM_DEVICE = 1 };

/*
 * One sample's op chain, already reduced by the caller to the canonical order
 *   source -> window+mirror -> one geometric op -> window+mirror -> [gray] -> slot.
 * It stands for a run of op::ImageTransformOp::apply_image calls
 * (mlx/data/op/ImageTransform.cpp:78-369) on one key of one sample:
 *   pre_*   crops (core::image::crop, ImageTransform.cpp:64-73) and horizontal
 *           flips (core::image::hflip, :123-140) that come before the geometric op;
 *   geom    image_resize / image_resize_smallest_side (target size in geom_w,
 *           geom_h) or image_rotate (matrix in mx, output size in geom_w, geom_h,
 *           both computed by the caller exactly as :80-86 and :113-121 do);
 *   post_*  crops and flips after it.
 * With geom == NONE the geometric output is the pre window itself and
 * geom_w, geom_h must equal pre_w, pre_h.  Random parameters (crop rectangles,
 * flip decisions) are drawn by the caller on the host.
 *
 * Resize with 4 channels: the reference passes the channel count to its resize
 * library as the pixel layout (ImageTransform.cpp:49-58), and layout 4 is
 * RGBA, whose colour channels are weighted by alpha while filtering.  The
 * kernels behind this struct filter every channel independently, also for
 * C == 4, so a 4-channel resize differs from the reference wherever alpha
 * varies.  The pipeline layer above this ABI refuses such resizes unless the
 * caller opted in; at this level the caller is expected to know.
 */
typedef struct mlxd_sample_desc {
  const uint8_t* src; /* [src_h, src_w, C] */
  int32_t src_h, src_w;
  int32_t pre_x, pre_y, pre_w, pre_h;
  int32_t pre_flip;
  int32_t geom;
  int32_t geom_w, geom_h;
  float mx[6];
  int32_t post_x, post_y, post_w, post_h;
  int32_t post_flip;
  int32_t reserved;
} mlxd_sample_desc;

/*
 * The batch the samples are written into: array::batch
 * (mlx/data/Array.cpp:465-498) with core::BatchShape (mlx/data/core/BatchShape.cpp:26-45)
 * followed by the cast that reference pipelines run as a Python lambda
 * (README.md:55-57): x.astype(float32) / 255, optionally (x/255 - mean) / std.
 * Sample i occupies slot i; its post window sits in the slot's top-left corner
 * and the rest of the slot holds the pad value (cast like every other pixel).
 */
typedef struct mlxd_batch_desc {
  void* dst;           /* [n, slot_h, slot_w, C_out] of out_dtype */
  int32_t slot_h, slot_w;
  int32_t channels;    /* C of every source image */
  int32_t gray;        /* 1: core::image::channel_reduction (ImageTransform.cpp:142-182) after the post window; C_out = 1 */
  int32_t gray_m[3];   /* its 16.16 fixed-point multipliers, (int)(coef * 65536) */
  int32_t gray_bias;   /* (int)(bias * 65536) */
  int32_t out_dtype;   /* MLXD_U8: raw bytes; MLXD_F32: cast below */
  int32_t normalise;   /* 0: x / divisor; 1: (x / divisor - mean[c]) / std[c] */
  float divisor;       /* 255 for the usual cast; 1 gives a plain astype */
  float mean[4];
  float std_[4];
  double pad_value;    /* batch pad value, converted to uint8 like Array::fill (mlx/data/Array.cpp:123-134) */
  int32_t src_mem;     /* mlxd_mem of every sample's src */
  int32_t dst_mem;     /* mlxd_mem of dst */
} mlxd_batch_desc;

typedef struct mlxd_stats {
  uint64_t batches;        /* fused launches issued */
  uint64_t samples;
  uint64_t kernel_launches;
  uint64_t h2d_bytes;
  uint64_t d2h_bytes;
  uint64_t device_bytes_reserved; /* staging + output arenas currently held */
  uint64_t kernel_ns;             /* summed device time of the timed launches (CUDA events around each kernel) */
  uint64_t timed_launches;        /* launches included in kernel_ns; 0 unless timing is on */
  uint64_t algo_src_bytes;        /* summed source footprints: the uint8 source rectangle each sample's chain can read */
  uint64_t algo_dst_bytes;        /* summed batch tensor bytes written, padding included */
  uint64_t h2d_ns;                /* timed launches: device time of the host-to-device stage (gather kernel or copies) */
  uint64_t d2h_ns;                /* timed launches: device time of the batch's copy back to the host */
  uint64_t host_stage_ns;         /* host time spent copying sources from ordinary memory into page-locked blocks */
} mlxd_stats;

/* Context: one device, n_lanes independent lanes.  A lane owns a CUDA stream, a
 * device staging arena and an output arena; calls on one lane are stream
 * ordered, different lanes overlap.  Replaces the role of core::ThreadPool
 * workers under stream::Prefetch (mlx/data/stream/Prefetch.cpp:29-56): one
 * prefetch worker drives one lane. */
MLXD_API int mlxd_ctx_create(int device, int n_lanes, mlxd_ctx** out);
MLXD_API void mlxd_ctx_destroy(mlxd_ctx* ctx);

/* Text of the last error raised on the calling thread. */
MLXD_API const char* mlxd_last_error(void);

/* Page-locked host memory for sample and batch storage; backs Array storage
 * through the external-storage constructor (mlx/data/Array.h:28-31).  The
 * blocks are mapped into the GPU's address space and remembered: when every
 * source of a host-fed mlxd_fused_batch lies in such blocks, a kernel reads
 * just the rectangle each chain needs over the bus (for a centre crop of a
 * 1080 x 1920 frame that is 57 % of the bytes a row-contiguous copy moves);
 * page-locked memory that did not come from here goes through the copy engines,
 * and sources in ordinary (pageable) memory are first packed - needed rectangle
 * only - into a page-locked block of the lane by the calling thread and up to
 * MLXD_PACK_THREADS - 1 helpers (default 4 threads in all), then copied once
 * per batch.  MLXD_HOST_GATHER=0 in the environment turns the kernel path off. */
MLXD_API void* mlxd_pinned_alloc(size_t bytes);
MLXD_API void mlxd_pinned_free(void* p);

/* PCI address of a CUDA device as "dddd:bb:dd.f" (NUL-terminated, len >= 16):
 * the name of its directory under /sys/bus/pci/devices, where a host finds the
 * NUMA node its loader threads and page-locked pools belong on.  (No
 * counterpart in the reference.) */
MLXD_API int mlxd_device_pci_bus_id(int device, char* out, size_t len);

/* Device memory on the context's GPU, for sources and batches that stay in
 * HBM (no counterpart in the reference, which is host-only).  NULL on failure. */
MLXD_API void* mlxd_device_alloc(mlxd_ctx* ctx, size_t bytes);
MLXD_API void mlxd_device_free(mlxd_ctx* ctx, void* p);

/* Bracket every fused kernel with CUDA events on the stream it is launched on
 * and add the elapsed device time to mlxd_stats.kernel_ns (off by default). */
MLXD_API int mlxd_ctx_set_timing(mlxd_ctx* ctx, int on);

/* The fused batch for callers that cannot allocate.  It has no counterpart in
 * the reference.  Who needs it: a loader plug-in that runs inside a training
 * step whose framework has handed the whole GPU to its own memory pool, a
 * service that bans allocator calls once it is warm, a process sitting at its
 * memory limit - for them a cudaMalloc (or a pinned-host allocation) in the
 * data path is a failure or a stall, and the other entry points do allocate:
 * descriptor tables, the cast table and a status word, on demand.  Here those
 * live in a fixed array inside the library image, so the call allocates
 * nothing on the device or the host, and needs no context.
 *
 * Same meaning as mlxd_fused_batch_on_stream: sources and destination are
 * device memory (batch->src_mem == batch->dst_mem == MLXD_MEM_DEVICE), the
 * kernel is queued on the caller's CUDA stream, the descriptors are read
 * before the call returns.  Limits and rules:
 *  - at most MLXD_NOALLOC_MAX_SAMPLES samples per call; more is refused with
 *    MLXD_ERR_INVALID (split the batch, or use the allocating entry point);
 *  - the array (about 0.15 MB) is held by every GPU that loads the library
 *    until the process exits;
 *  - the first call on a device looks up the array's device address; make
 *    that first call before any stream capture;
 *  - every call waits on the host until the stream has drained (its small
 *    tables are copied from fixed host storage that the next call reuses), so
 *    the host blocks behind whatever is queued on that stream before it;
 *  - the stream must belong to `device`; the calling thread's current device
 *    is the same after the call as before it;
 *  - all calls share the one array, which keeps the previous call's contents
 *    (the call clears what must start at zero): two calls whose kernels can
 *    overlap on the GPU - different streams, or different host threads - race;
 *    order them on one stream;
 *  - the kernel's self-check word (a bounded wait that ran out, a shared-memory
 *    bound) is read back at the start of the NEXT call on the same stream,
 *    which then returns MLXD_ERR_DEVICE and launches nothing; after the last
 *    call of a run ask mlxd_noalloc_status. */
#define MLXD_NOALLOC_MAX_SAMPLES 1024
MLXD_API int mlxd_fused_batch_noalloc(
    int device, void* cuda_stream, const mlxd_sample_desc* samples, int n, const mlxd_batch_desc* batch);

/* Self-check word of the most recent mlxd_fused_batch_noalloc kernel on this
 * device, read from the same fixed array (no allocation; no counterpart in the
 * reference).  Waits for `cuda_stream`, stores the word in *status (0 = clean),
 * clears it, and returns MLXD_ERR_DEVICE when it was set. */
MLXD_API int mlxd_noalloc_status(int device, void* cuda_stream, int32_t* status);

/* Enqueue one fused batch on a lane and return: host sources are copied to the
 * device (only the rows the chain reads), one kernel writes every slot, and a
 * host dst is copied back.  Replaces stream::Batch::next -> core::merge_batch
 * (mlx/data/stream/Batch.cpp:25-39, mlx/data/core/Utils.cpp:209-252) together
 * with the per-sample op calls listed at mlxd_sample_desc.  Host memory must
 * stay untouched until mlxd_batch_wait returns MLXD_OK. */
MLXD_API int mlxd_fused_batch(
    mlxd_ctx* ctx, int lane, const mlxd_sample_desc* samples, int n, const mlxd_batch_desc* batch);

/* Wait for everything queued on a lane, at most timeout_ms (< 0: no limit).
 * Replaces future.get() in stream::Prefetch::next (mlx/data/stream/Prefetch.cpp:43-53). */
MLXD_API int mlxd_batch_wait(mlxd_ctx* ctx, int lane, int timeout_ms);

/* Same work for device-resident sources and destination, launched on the
 * caller's CUDA stream (a cudaStream_t passed as void*; NULL is the default
 * stream).  Nothing is copied except the descriptors. */
MLXD_API int mlxd_fused_batch_on_stream(
    mlxd_ctx* ctx, void* cuda_stream, const mlxd_sample_desc* samples, int n, const mlxd_batch_desc* batch);

/* Self-check word of the kernels launched by mlxd_fused_batch_on_stream: waits
 * for `cuda_stream`, stores the word in *status (0 = clean; bit 1/2: a pass
 * larger than the planned shared memory, 4: a bounded wait on a bulk copy ran
 * out, 8: more filter rows than planned), clears it, and returns
 * MLXD_ERR_DEVICE when it was set.  The lanes of mlxd_fused_batch report the
 * same word through mlxd_batch_wait.  No counterpart in the reference, whose
 * CPU ops throw where they stand. */
MLXD_API int mlxd_stream_status(mlxd_ctx* ctx, void* cuda_stream, int32_t* status);

/* One entry per named op, host buffers in and out, synchronous; for chains
 * that cannot be fused (a host callback between two ops).  Each runs the same
 * kernel with a one-stage program. */
/* core::image::resize, mlx/data/core/image/ImageTransform.cpp:41-62
 * (c == 4: channels filtered independently, see mlxd_sample_desc) */
MLXD_API int mlxd_image_resize(
    mlxd_ctx* ctx, const uint8_t* src, int h, int w, int c, uint8_t* dst, int dh, int dw);
/* core::image::crop, mlx/data/core/image/ImageTransform.cpp:64-73 */
MLXD_API int mlxd_image_crop(
    mlxd_ctx* ctx, const uint8_t* src, int h, int w, int c, int x, int y, int cw, int ch, uint8_t* dst);
/* core::image::hflip, mlx/data/core/image/ImageTransform.cpp:123-140 */
MLXD_API int mlxd_image_hflip(mlxd_ctx* ctx, const uint8_t* src, int h, int w, int c, uint8_t* dst);
/* core::image::affine, mlx/data/core/image/ImageTransform.cpp:75-111; th, tw as computed at :80-86 */
MLXD_API int mlxd_image_affine(
    mlxd_ctx* ctx, const uint8_t* src, int h, int w, int c, const float mx[6], int th, int tw, uint8_t* dst);
/* core::image::channel_reduction, mlx/data/core/image/ImageTransform.cpp:142-182 */
MLXD_API int mlxd_image_channel_reduction(
    mlxd_ctx* ctx, const uint8_t* src, int h, int w, const int32_t m_fixed[3], int32_t bias_fixed, uint8_t* dst);
/* array::batch for uint8 images, mlx/data/Array.cpp:465-498 */
MLXD_API int mlxd_batch_pad(
    mlxd_ctx* ctx, const uint8_t* const* srcs, const int32_t* hs, const int32_t* ws, int n, int c,
    int slot_h, int slot_w, double pad_value, uint8_t* dst);
/* the float32 cast of README.md:55-57; count pixels of c channels */
MLXD_API int mlxd_cast_scale_normalise(
    mlxd_ctx* ctx, const uint8_t* src, int64_t count, int c, float divisor,
    const float* mean, const float* std_, float* dst);

MLXD_API int mlxd_stats_get(mlxd_ctx* ctx, mlxd_stats* out);

#ifdef __cplusplus
}
#endif
#endif /* MLXD_B200_H */
