// One kernel per batch: every CTA owns a kTileH x kTileW tile of one sample's
// slot in the batch tensor, evaluates that sample's op chain for the tile
// (window/mirror -> resize or nearest-neighbour affine -> window/mirror ->
// optional gray), quantises to uint8 exactly where mlx-data materialises a
// uint8 image between ops, and writes the cast float32 (or raw uint8) values,
// pad included, straight into the batch tensor.
//
// Reference behaviour reproduced here (paths inside mlx-data):
//   resize             mlx/data/core/image/ImageTransform.cpp:41-62 (triangle filter, clamp to edge)
//   crop               mlx/data/core/image/ImageTransform.cpp:64-73, mlx/data/Array.cpp:544-583
//   affine / rotate    mlx/data/core/image/ImageTransform.cpp:75-121
//   hflip              mlx/data/core/image/ImageTransform.cpp:123-140
//   channel_reduction  mlx/data/core/image/ImageTransform.cpp:142-182
//   batch + pad        mlx/data/Array.cpp:465-498, mlx/data/core/BatchShape.cpp:26-45
//   cast               README.md:55-57 (x.astype(float32) / 255 and its normalised form)
#include "fused_batch.h"

#include "kernel_common.cuh"

namespace mlxd {
namespace {

struct SmemLayout {
  float* lut;
  uint8_t* outq;
  int* vfirst;
  int* vcount;
  int* hfirst;
  int* hcount;
  int2* urow;
  float4* uw;
  int* ucount;
  uint64_t* bar;
  float* wts;
  float* mid;
  uint8_t* srct;
};

__host__ __device__ inline size_t align16(size_t v) {
  return (v + 15) & ~(size_t)15;
}

__device__ __forceinline__ SmemLayout carve(unsigned char* base, const LaunchParams& p) {
  SmemLayout l;
  size_t off = 0;
  l.lut = reinterpret_cast<float*>(base + off);
  off += (size_t)p.c_out * 256 * sizeof(float);
  l.outq = base + off;
  off += kTileH * kTileW * 4;
  l.vfirst = reinterpret_cast<int*>(base + off);
  off += kTileH * sizeof(int);
  l.vcount = reinterpret_cast<int*>(base + off);
  off += kTileH * sizeof(int);
  l.hfirst = reinterpret_cast<int*>(base + off);
  off += kTileW * sizeof(int);
  l.hcount = reinterpret_cast<int*>(base + off);
  off += kTileW * sizeof(int);
  l.uw = reinterpret_cast<float4*>(base + off);
  off += (size_t)4 * p.u_cap * sizeof(float4);
  l.urow = reinterpret_cast<int2*>(base + off);
  off += (size_t)4 * p.u_cap * sizeof(int2);
  l.ucount = reinterpret_cast<int*>(base + off);
  off += 16;
  l.bar = reinterpret_cast<uint64_t*>(base + off);
  off += 16;
  l.wts = reinterpret_cast<float*>(base + off);
  off = align16(off + (size_t)p.weight_floats * sizeof(float));
  l.mid = reinterpret_cast<float*>(base + off);
  off = align16(off + (size_t)p.mid_float4s * 16);
  l.srct = base + off;
  return l;
}

// Pad value (already cast) into the rectangle [ya, yb) x [xa, xb) of a slot,
// 16-byte stores wherever the row segment allows.
__device__ void fill_rect_f32(
    float* base, int slot_w, int co, int ya, int yb, int xa, int xb, const float* padf) {
  if (ya >= yb || xa >= xb) {
    return;
  }
  const int L = (xb - xa) * co;
  const int Q = ((L + 3) >> 2) + 2;
  const int ny = yb - ya;
  for (int i = threadIdx.x; i < ny * Q; i += kThreads) {
    const int ry = i / Q;
    const int q = i - ry * Q;
    float* rowp = base + ((size_t)(ya + ry) * slot_w + xa) * co;
    const int mis = (int)((reinterpret_cast<uintptr_t>(rowp) >> 2) & 3);
    int head = (4 - mis) & 3;
    head = head > L ? L : head;
    const int nvec = (L - head) >> 2;
    if (q == 0) {
      for (int j = 0; j < head; j++) {
        rowp[j] = padf[j % co];
      }
    } else if (q <= nvec) {
      const int j = head + 4 * (q - 1);
      const int m = j % co;
      *reinterpret_cast<float4*>(rowp + j) =
          make_float4(padf[m], padf[(m + 1) % co], padf[(m + 2) % co], padf[(m + 3) % co]);
    } else if (q == nvec + 1) {
      for (int j = head + 4 * nvec; j < L; j++) {
        rowp[j] = padf[j % co];
      }
    }
  }
}

__device__ void fill_rect_u8(
    uint8_t* base, int slot_w, int co, int ya, int yb, int xa, int xb, int pad_px) {
  if (ya >= yb || xa >= xb) {
    return;
  }
  const int L = (xb - xa) * co;
  const int ny = yb - ya;
  for (int i = threadIdx.x; i < ny * L; i += kThreads) {
    const int ry = i / L;
    const int j = i - ry * L;
    base[((size_t)(ya + ry) * slot_w + xa) * co + j] = (uint8_t)pad_px;
  }
}

// Generic resize of the geometric-output rectangle [gy_lo, gy_hi) x
// [gx_lo, gx_hi) into outq (uint8), sub_h x sub_w outputs per pass.  Handles
// every channel count, mirrored sources and uint8 destinations; the common
// float32 case runs fast::resize_pass instead.
__device__ void resize_region(
    const DevSample& s, const LaunchParams& p, const SmemLayout& sm,
    int y0, int x0, int gy_lo, int gy_hi, int gx_lo, int gx_hi) {
  const int tid = threadIdx.x;
  const int C = p.c_in;
  float* wv = sm.wts;
  float* wh = sm.wts + s.sub_h * s.cap_y;
  for (int by = gy_lo; by < gy_hi; by += s.sub_h) {
    for (int bx = gx_lo; bx < gx_hi; bx += s.sub_w) {
      const int nr = min(s.sub_h, gy_hi - by);
      const int nc = min(s.sub_w, gx_hi - bx);
      for (int i = tid; i < nr + nc; i += kThreads) {
        if (i < nr) {
          axis_taps(s.pre_h, s.geom_h, by + i, s.cap_y, sm.vfirst[i], sm.vcount[i], wv + i * s.cap_y);
        } else {
          const int j = i - nr;
          axis_taps(s.pre_w, s.geom_w, bx + j, s.cap_x, sm.hfirst[j], sm.hcount[j], wh + j * s.cap_x);
        }
      }
      __syncthreads();
      const int rlo = clampi(sm.vfirst[0], 0, s.pre_h - 1);
      const int rhi = clampi(sm.vfirst[nr - 1] + sm.vcount[nr - 1] - 1, 0, s.pre_h - 1);
      const int clo = clampi(sm.hfirst[0], 0, s.pre_w - 1);
      const int chi = clampi(sm.hfirst[nc - 1] + sm.hcount[nc - 1] - 1, 0, s.pre_w - 1);
      const int rows = rhi - rlo + 1;
      const int wbytes = (chi - clo + 1) * C;
      const int pitch = (wbytes + 3) & ~3;
      const int nwords = pitch >> 2;
      if (rows * pitch > p.src_tile_bytes || nr * pitch > p.mid_float4s * 4) {
        // The host planner sizes sub_h, sub_w so this cannot happen; record it
        // instead of overrunning shared memory.
        if (tid == 0) {
          atomicOr(p.status, 1);
        }
        __syncthreads();
        continue;
      }
      if (!s.pre_flip) {
        uint32_t* srcw = reinterpret_cast<uint32_t*>(sm.srct);
        for (int i = tid; i < rows * nwords; i += kThreads) {
          const int r = i / nwords;
          const int j = i - r * nwords;
          const size_t g = ((size_t)(s.pre_y + rlo + r) * s.src_w + (s.pre_x + clo)) * C + 4 * j;
          const uintptr_t a = reinterpret_cast<uintptr_t>(s.src + g);
          const unsigned mis = (unsigned)(a & 3);
          const uint32_t* wa = reinterpret_cast<const uint32_t*>(a - mis);
          const int need = min(4, wbytes - 4 * j);
          const uint32_t lo = __ldg(wa);
          uint32_t hi = 0;
          if (mis != 0 && (int)(4 - mis) < need) {
            hi = __ldg(wa + 1);
          }
          srcw[i] = __funnelshift_r(lo, hi, mis * 8);
        }
      } else {
        for (int i = tid; i < rows * wbytes; i += kThreads) {
          const int r = i / wbytes;
          const int j = i - r * wbytes;
          const int px = j / C;
          const int ch = j - px * C;
          const int sx = s.pre_x + s.pre_w - 1 - (clo + px);
          sm.srct[r * pitch + j] = __ldg(s.src + ((size_t)(s.pre_y + rlo + r) * s.src_w + sx) * C + ch);
        }
      }
      __syncthreads();
      {
        const uint32_t* srcw = reinterpret_cast<const uint32_t*>(sm.srct);
        for (int i = tid; i < nr * nwords; i += kThreads) {
          const int r = i / nwords;
          const int g = i - r * nwords;
          const int f = sm.vfirst[r];
          const int cnt = sm.vcount[r];
          const float* w = wv + r * s.cap_y;
          float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
          for (int k = 0; k < cnt; k++) {
            const int sr = clampi(f + k, 0, s.pre_h - 1) - rlo;
            const uint32_t word = srcw[sr * nwords + g];
            const float wk = w[k];
            a0 = __fmaf_rn(wk, (float)(word & 0xffu), a0);
            a1 = __fmaf_rn(wk, (float)((word >> 8) & 0xffu), a1);
            a2 = __fmaf_rn(wk, (float)((word >> 16) & 0xffu), a2);
            a3 = __fmaf_rn(wk, (float)(word >> 24), a3);
          }
          *reinterpret_cast<float4*>(sm.mid + r * pitch + 4 * g) = make_float4(a0, a1, a2, a3);
        }
      }
      __syncthreads();
      for (int i = tid; i < nr * nc * C; i += kThreads) {
        const int r = i / (nc * C);
        const int rem = i - r * nc * C;
        const int x = rem / C;
        const int ch = rem - x * C;
        const int f = sm.hfirst[x];
        const int cnt = sm.hcount[x];
        const float* w = wh + x * s.cap_x;
        const float* row = sm.mid + r * pitch + ch;
        float acc = 0.0f;
        for (int k = 0; k < cnt; k++) {
          const int col = clampi(f + k, 0, s.pre_w - 1) - clo;
          acc = __fmaf_rn(w[k], row[col * C], acc);
        }
        int px = bx + x - s.post_x;
        if (s.post_flip) {
          px = s.post_w - 1 - px;
        }
        const int oy = by + r - s.post_y - y0;
        sm.outq[(oy * kTileW + (px - x0)) * C + ch] = (uint8_t)quantise(acc);
      }
      __syncthreads();
    }
  }
}

__global__ void __launch_bounds__(kThreads, 2) fused_batch_kernel(const LaunchParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const SmemLayout sm = carve(smem_raw, p);
  const int tid = threadIdx.x;

  unsigned t = blockIdx.x;
  const int tx = t % p.tiles_x;
  t /= p.tiles_x;
  const int ty = t % p.tiles_y;
  const int n = t / p.tiles_y;
  if (n >= p.n) {
    return;
  }
  const DevSample s = p.samples[n];
  const int y0 = ty * kTileH;
  const int x0 = tx * kTileW;
  if (y0 >= s.slot_h || x0 >= s.slot_w) {
    return;
  }
  const int y1 = min(y0 + kTileH, s.slot_h);
  const int x1 = min(x0 + kTileW, s.slot_w);
  const int vy1 = min(y1, s.post_h);
  const int vx1 = min(x1, s.post_w);
  const bool has_valid = (y0 < vy1) && (x0 < vx1);
  const int C = p.c_in;
  const int co = p.c_out;

  float padf[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  if (p.out_f32) {
    for (int c = 0; c < co; c++) {
      padf[c] = __ldg(p.lut + c * 256 + p.pad_px);
    }
  }
  if (!has_valid) {
    if (p.out_f32) {
      fill_rect_f32(reinterpret_cast<float*>(s.dst), s.slot_w, co, y0, y1, x0, x1, padf);
    } else {
      fill_rect_u8(reinterpret_cast<uint8_t*>(s.dst), s.slot_w, co, y0, y1, x0, x1, p.pad_px);
    }
    return;
  }

  if (p.out_f32) {
    for (int i = tid; i < co * 256; i += kThreads) {
      sm.lut[i] = __ldg(p.lut + i);
    }
  }
  const int nvy = vy1 - y0;
  const int nvx = vx1 - x0;
  if (s.mode == kModeResize) {
    int gx_lo, gx_hi;
    if (!s.post_flip) {
      gx_lo = s.post_x + x0;
      gx_hi = s.post_x + vx1;
    } else {
      gx_lo = s.post_x + s.post_w - vx1;
      gx_hi = s.post_x + s.post_w - x0;
    }
    resize_region(s, p, sm, y0, x0, s.post_y + y0, s.post_y + vy1, gx_lo, gx_hi);
  } else if (s.mode == kModeAffine) {
    // Nearest-neighbour warp.  The coordinate is built from float products
    // and float sums, then two double additions, then truncation toward
    // zero - the evaluation order of the reference expression - and no
    // multiply-add is contracted.
    const float twh = (float)((double)s.geom_w / 2.0);
    const float thh = (float)((double)s.geom_h / 2.0);
    const float wh = (float)((double)s.pre_w / 2.0);
    const float hh = (float)((double)s.pre_h / 2.0);
    for (int i = tid; i < nvy * nvx; i += kThreads) {
      const int ry = i / nvx;
      const int rx = i - ry * nvx;
      const int px = s.post_flip ? (s.post_w - 1 - (x0 + rx)) : (x0 + rx);
      const float dxf = __fsub_rn((float)(long long)(s.post_x + px), twh);
      const float dyf = __fsub_rn((float)(long long)(s.post_y + y0 + ry), thh);
      const float fx = __fadd_rn(__fadd_rn(__fmul_rn(s.mx[0], dxf), __fmul_rn(s.mx[1], dyf)), s.mx[2]);
      const float fy = __fadd_rn(__fadd_rn(__fmul_rn(s.mx[3], dxf), __fmul_rn(s.mx[4], dyf)), s.mx[5]);
      const long long ax = (long long)__dadd_rn(__dadd_rn((double)fx, 0.5), (double)wh);
      const long long ay = (long long)__dadd_rn(__dadd_rn((double)fy, 0.5), (double)hh);
      uint8_t* q = sm.outq + (ry * kTileW + rx) * C;
      if (ax < 0 || ay < 0 || ax >= s.pre_w || ay >= s.pre_h) {
        for (int ch = 0; ch < C; ch++) {
          q[ch] = 0;
        }
      } else {
        const int sx = s.pre_x + (s.pre_flip ? (s.pre_w - 1 - (int)ax) : (int)ax);
        const int sy = s.pre_y + (int)ay;
        const uint8_t* g = s.src + ((size_t)sy * s.src_w + sx) * C;
        for (int ch = 0; ch < C; ch++) {
          q[ch] = __ldg(g + ch);
        }
      }
    }
  } else {
    const int rowlen = nvx * C;
    for (int i = tid; i < nvy * rowlen; i += kThreads) {
      const int ry = i / rowlen;
      const int j = i - ry * rowlen;
      const int rx = j / C;
      const int ch = j - rx * C;
      const int px = s.post_flip ? (s.post_w - 1 - (x0 + rx)) : (x0 + rx);
      const int gx = s.post_x + px;
      const int gy = s.post_y + y0 + ry;
      const int sx = s.pre_x + (s.pre_flip ? (s.pre_w - 1 - gx) : gx);
      const int sy = s.pre_y + gy;
      sm.outq[(ry * kTileW + rx) * C + ch] = __ldg(s.src + ((size_t)sy * s.src_w + sx) * C + ch);
    }
  }
  __syncthreads();

  // ---- write the tile: cast values, pad outside the post window -------------
  const int ny = y1 - y0;
  const int L = (x1 - x0) * co;
  auto pixel = [&](int ry, int j) -> int {
    const int rx = j / co;
    const int ch = j - rx * co;
    if ((y0 + ry) < s.post_h && (x0 + rx) < s.post_w) {
      const uint8_t* q = sm.outq + (ry * kTileW + rx) * C;
      if (p.gray) {
        int v = ((int)q[0] * p.gray_m[0] + (int)q[1] * p.gray_m[1] + (int)q[2] * p.gray_m[2] + p.gray_bias) / 65536;
        v = v <= 255 ? v : 255;
        v = v >= 0 ? v : 0;
        return v;
      }
      return q[ch];
    }
    return p.pad_px;
  };
  if (p.out_f32) {
    const float* lut = sm.lut;
    auto value = [&](int ry, int j) -> float {
      const int ch = j % co;
      return lut[ch * 256 + pixel(ry, j)];
    };
    float* base = reinterpret_cast<float*>(s.dst);
    const int Q = ((L + 3) >> 2) + 2;
    for (int i = tid; i < ny * Q; i += kThreads) {
      const int ry = i / Q;
      const int q = i - ry * Q;
      float* rowp = base + ((size_t)(y0 + ry) * s.slot_w + x0) * co;
      const int mis = (int)((reinterpret_cast<uintptr_t>(rowp) >> 2) & 3);
      int head = (4 - mis) & 3;
      head = head > L ? L : head;
      const int nvec = (L - head) >> 2;
      if (q == 0) {
        for (int j = 0; j < head; j++) {
          rowp[j] = value(ry, j);
        }
      } else if (q <= nvec) {
        const int j = head + 4 * (q - 1);
        *reinterpret_cast<float4*>(rowp + j) =
            make_float4(value(ry, j), value(ry, j + 1), value(ry, j + 2), value(ry, j + 3));
      } else if (q == nvec + 1) {
        for (int j = head + 4 * nvec; j < L; j++) {
          rowp[j] = value(ry, j);
        }
      }
    }
  } else {
    uint8_t* base = reinterpret_cast<uint8_t*>(s.dst);
    for (int i = tid; i < ny * L; i += kThreads) {
      const int ry = i / L;
      const int j = i - ry * L;
      base[((size_t)(y0 + ry) * s.slot_w + x0) * co + j] = (uint8_t)pixel(ry, j);
    }
  }
}

} // namespace

size_t fused_batch_smem_bytes(const LaunchParams& p) {
  size_t off = (size_t)p.c_out * 256 * sizeof(float) + kTileH * kTileW * 4 + 2 * kTileH * sizeof(int) +
      2 * kTileW * sizeof(int) + (size_t)4 * p.u_cap * (sizeof(float4) + sizeof(int2)) + 16 + 16;
  off = align16(off + (size_t)p.weight_floats * sizeof(float));
  off = align16(off + (size_t)p.mid_float4s * 16);
  off += (size_t)p.src_tile_bytes;
  return off + 16;
}

cudaError_t launch_fused_batch(const LaunchParams& p, cudaStream_t stream) {
  if (p.use_fast) {
    return launch_fused_fast(p, stream);
  }
  const size_t smem = fused_batch_smem_bytes(p);
  static thread_local int configured_device = -1;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    return e;
  }
  if (configured_device != dev) {
    LaunchParams worst = p;
    worst.c_out = 4;
    worst.weight_floats = kWeightFloats;
    worst.mid_float4s = kMidFloats / 4;
    worst.src_tile_bytes = kSrcTileBytes;
    worst.u_cap = kMaxStagedRows;
    e = cudaFuncSetAttribute(
        fused_batch_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fused_batch_smem_bytes(worst));
    if (e != cudaSuccess) {
      return e;
    }
    configured_device = dev;
  }
  const unsigned long long blocks = (unsigned long long)p.n * p.tiles_y * p.tiles_x;
  if (blocks == 0) {
    return cudaSuccess;
  }
  if (blocks > 0x7fffffffULL) {
    return cudaErrorInvalidConfiguration;
  }
  fused_batch_kernel<<<(unsigned)blocks, kThreads, smem, stream>>>(p);
  return cudaGetLastError();
}

void choose_kernel(LaunchParams& p, const PassNeed& need, const DevSample* host_samples, int n) {
  const bool channels_ok = p.c_in == 1 || p.c_in == 3 || p.c_in == 4;
  p.use_fast = (channels_ok && !need.needs_generic) ? 1 : 0;
  // The rows below a sample's post window are one contiguous run of its slot;
  // when those runs are at least an eighth of the batch they get a linear fill
  // of their own (pad_fill_kernel), which writes at memory speed.
  p.pad_apart = 0;
  if (p.use_fast && n > 0) {
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
  const int r = (n_src + n_dst - 1) / n_dst;  // ceil of the shrink ratio
  a.cap = 2 * r + 3;
  const long long span = ((long long)sub * n_src + n_dst - 1) / n_dst;
  a.extent = (int32_t)(span + 2 * r + 3);
  return a;
}

PassNeed plan_pass(
    const AxisPlan& ay, const AxisPlan& ax, int32_t sub_h, int32_t sub_w, int32_t pre_h, int32_t pre_w, int32_t channels,
    bool& fits) {
  const long long rows = ay.extent < pre_h ? ay.extent : pre_h;
  const long long cols = ax.extent < pre_w ? ax.extent : pre_w;
  const long long wbytes = cols * channels;
  const long long pitch = (wbytes + 49 + 15) & ~15LL;   // covers both staging layouts
  const long long nwords = (wbytes + 6) / 4 + 1;
  const long long src = rows * pitch;
  // the float32 kernel pads every plane by up to 7 columns on either side and
  // skips one slot after every eight columns
  const long long pad = (7 + channels - 1) / channels;
  const long long pslots = (cols + 2 * pad) + (cols + 2 * pad) / 8 + 1;
  const long long mid4_fast = ((sub_h + 3) / 4) * channels * pslots;   // one set of planes per group of four rows
  const long long mid4 = 16 * nwords > mid4_fast ? 16 * nwords : mid4_fast;
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
