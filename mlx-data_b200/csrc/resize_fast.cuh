// Fast path of the fused kernel for resize samples whose output is float32:
// the source footprint of a tile is staged in shared memory with bulk
// asynchronous copies (cp.async.bulk, one per source row, completion on an
// mbarrier), filtered vertically four output rows at a time into a transposed
// float4 buffer, filtered horizontally four rows per thread, quantised, cast
// through the table and stored straight into the batch tensor.
//
// The arithmetic is that of the generic path in fused_batch.cu: every output
// is a chain acc = fma(w_k, v_k, acc) from 0 in increasing tap order, vertical
// axis first, quantised as (int)(acc + 0.5) clamped to [0, 255].
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "fused_batch.h"

namespace mlxd {
namespace fast {

constexpr int kMaxRows = 192;          // staged source rows per pass
constexpr unsigned kSpinLimit = 1u << 22;

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, unsigned bytes) {
  asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile(
      "{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(smem_addr(bar))
      : "memory");
}

// Bounded wait for the phase with the given parity.  Returns false when the
// limit was reached; the caller records that and goes on without hanging.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, unsigned parity) {
  const uint32_t a = smem_addr(bar);
  for (unsigned i = 0; i < kSpinLimit; i++) {
    unsigned done;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(a), "r"(parity)
        : "memory");
    if (done) {
      return true;
    }
  }
  return false;
}

// 16-byte aligned global -> shared bulk copy, bytes a multiple of 16.
__device__ __forceinline__ void bulk_copy(void* dst_smem, const void* src_gmem, unsigned bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_addr(dst_smem)),
      "l"(src_gmem), "r"(bytes), "r"(smem_addr(bar))
      : "memory");
}

__device__ __forceinline__ void fence_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// Byte `B` of a word as float, exactly: place it in the mantissa of 2^23, subtract 2^23.
template <int B>
__device__ __forceinline__ float byte_to_float(uint32_t word) {
  return __fsub_rn(__uint_as_float(__byte_perm(word, 0x4B000000u, 0x7540u + B)), 8388608.0f);
}

// Column j of the vertically filtered buffer lives in float4 slot swz(j): the
// four columns of a source word are rotated by the word index so that both the
// writer (one thread per word) and the reader hit distinct banks.
__device__ __forceinline__ int swz(int j) {
  return (j & ~3) | ((j ^ (j >> 3)) & 3);
}

struct Layout {
  float* lut;
  int* vfirst;
  int* vcount;
  int* hfirst;
  int* hcount;
  int2* rowinfo;    // per staged row: {word index of the row's first word, funnel shift in bits}
  float* wts;
  float4* mid;
  uint8_t* srct;
  uint64_t* bar;
};

template <int C>
__device__ __forceinline__ int clampi(int v, int lo, int hi) {
  return v < lo ? lo : (v > hi ? hi : v);
}

// One pass: geometric-output rows [by, by+nr) x columns [bx, bx+nc) of a
// resize sample (nr <= kTileH, nc <= kTileW), written to the batch tensor.
template <int C>
__device__ void resize_pass(
    const DevSample& s, const LaunchParams& p, const Layout& sm, unsigned& parity,
    int by, int bx, int nr, int nc) {
  const int tid = threadIdx.x;
  float* wv = sm.wts;
  float* wh = sm.wts + s.sub_h * s.cap_y;

  // ---- tap tables ----------------------------------------------------------
  for (int i = tid; i < nr + nc; i += kThreads) {
    if (i < nr) {
      axis_taps(s.pre_h, s.geom_h, by + i, s.cap_y, sm.vfirst[i], sm.vcount[i], wv + i * s.cap_y);
    } else {
      const int j = i - nr;
      axis_taps(s.pre_w, s.geom_w, bx + j, s.cap_x, sm.hfirst[j], sm.hcount[j], wh + j * s.cap_x);
    }
  }
  __syncthreads();
  const int rlo = clampi<C>(sm.vfirst[0], 0, s.pre_h - 1);
  const int rhi = clampi<C>(sm.vfirst[nr - 1] + sm.vcount[nr - 1] - 1, 0, s.pre_h - 1);
  const int clo = clampi<C>(sm.hfirst[0], 0, s.pre_w - 1);
  const int chi = clampi<C>(sm.hfirst[nc - 1] + sm.hcount[nc - 1] - 1, 0, s.pre_w - 1);
  const int rows = rhi - rlo + 1;
  const int wbytes = (chi - clo + 1) * C;
  const size_t src_pitch = (size_t)s.src_w * C;
  const uint8_t* g0 = s.src + ((size_t)(s.pre_y + rlo) * s.src_w + (s.pre_x + clo)) * C;
  const int phase0 = (int)(reinterpret_cast<uintptr_t>(g0) & 15);
  const int common = phase0 & 3;
  const int pitch_s = (wbytes + 15 + 15 + 4 + 15) & ~15;   // staged row pitch, bytes
  const int nwords = (common + wbytes + 3) >> 2;
  if (rows > kMaxRows || rows * pitch_s > p.src_tile_bytes || nwords * 4 * 4 > p.mid_float4s) {
    if (tid == 0) {
      atomicOr(p.status, 2);
    }
    __syncthreads();
    return;
  }

  // ---- stage the footprint: one bulk copy per source row -----------------------
  if (tid < rows) {
    const uintptr_t ga = reinterpret_cast<uintptr_t>(g0) + (size_t)tid * src_pitch;
    const int phase = (int)(ga & 15);
    const unsigned len = (unsigned)((phase + wbytes + 15) & ~15);
    sm.rowinfo[tid] = make_int2((tid * pitch_s + phase - common) >> 2, ((phase - common) & 3) * 8);
    mbar_expect_tx(sm.bar, len);
    bulk_copy(sm.srct + tid * pitch_s, reinterpret_cast<const void*>(ga - phase), len, sm.bar);
  }
  __syncthreads();
  if (tid == 0) {
    mbar_arrive(sm.bar);
  }
  if (!mbar_wait(sm.bar, parity)) {
    atomicOr(p.status, 4);
  }
  parity ^= 1;

  // ---- vertical filter: thread = (source word, group of four output rows) -----
  {
    const uint32_t* srcw = reinterpret_cast<const uint32_t*>(sm.srct);
    const int ncols = nwords * 4;
    for (int rg = tid >> 7; rg * 4 < nr; rg += kThreads >> 7) {
      for (int g = tid & 127; g < nwords; g += 128) {
        float a[4][4];
#pragma unroll
        for (int r = 0; r < 4; r++) {
          a[r][0] = a[r][1] = a[r][2] = a[r][3] = 0.0f;
        }
#pragma unroll
        for (int r = 0; r < 4; r++) {
          const int o = rg * 4 + r;
          if (o < nr) {
            const int f = sm.vfirst[o];
            const int cnt = sm.vcount[o];
            const float* w = wv + o * s.cap_y;
            for (int k = 0; k < cnt; k++) {
              const int sr = clampi<C>(f + k, 0, s.pre_h - 1) - rlo;
              const int2 ri = sm.rowinfo[sr];
              uint32_t word = srcw[ri.x + g];
              if (ri.y) {
                word = __funnelshift_r(word, srcw[ri.x + g + 1], ri.y);
              }
              const float wk = w[k];
              a[r][0] = __fmaf_rn(wk, byte_to_float<0>(word), a[r][0]);
              a[r][1] = __fmaf_rn(wk, byte_to_float<1>(word), a[r][1]);
              a[r][2] = __fmaf_rn(wk, byte_to_float<2>(word), a[r][2]);
              a[r][3] = __fmaf_rn(wk, byte_to_float<3>(word), a[r][3]);
            }
          }
        }
        float4* out = sm.mid + rg * ncols + g * 4;
        const int rot = (g >> 1) & 3;
#pragma unroll
        for (int b = 0; b < 4; b++) {
          out[b ^ rot] = make_float4(a[0][b], a[1][b], a[2][b], a[3][b]);
        }
      }
    }
  }
  __syncthreads();

  // ---- horizontal filter: thread = (output column, channel, group of four rows) ----
  {
    const int ncols = nwords * 4;
    const int per_rg = nc * C;
    const int ngroups = (nr + 3) >> 2;
    float* base = reinterpret_cast<float*>(s.dst);
    for (int item = tid; item < ngroups * per_rg; item += kThreads) {
      const int rg = item / per_rg;
      const int rem = item - rg * per_rg;
      const int x = rem / C;
      const int ch = rem - x * C;
      const int f = sm.hfirst[x];
      const int cnt = sm.hcount[x];
      const float* w = wh + x * s.cap_x;
      const float4* row = sm.mid + rg * ncols;
      float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      for (int k = 0; k < cnt; k++) {
        const int col = clampi<C>(f + k, 0, s.pre_w - 1) - clo;
        const float4 v = row[swz(common + col * C + ch)];
        const float wk = w[k];
        acc.x = __fmaf_rn(wk, v.x, acc.x);
        acc.y = __fmaf_rn(wk, v.y, acc.y);
        acc.z = __fmaf_rn(wk, v.z, acc.z);
        acc.w = __fmaf_rn(wk, v.w, acc.w);
      }
      int px = bx + x - s.post_x;
      if (s.post_flip) {
        px = s.post_w - 1 - px;
      }
      const int oy = by + rg * 4 - s.post_y;
      const float* lut = sm.lut + ch * 256;
      float* dst = base + ((size_t)oy * s.slot_w + px) * C + ch;
      const size_t row_stride = (size_t)s.slot_w * C;
      const int left = nr - rg * 4;
      dst[0] = lut[quantise(acc.x)];
      if (left > 1) dst[row_stride] = lut[quantise(acc.y)];
      if (left > 2) dst[2 * row_stride] = lut[quantise(acc.z)];
      if (left > 3) dst[3 * row_stride] = lut[quantise(acc.w)];
    }
  }
  __syncthreads();
  // the staging buffer is about to be rewritten by the async proxy
  fence_async_smem();
}

} // namespace fast
} // namespace mlxd
