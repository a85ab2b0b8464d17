// The float32-output kernel: one CTA per kTileH x kTileW tile of one sample's
// slot.  Resize tiles stage their source footprint in shared memory with bulk
// asynchronous copies (cp.async.bulk, one per source row, completion on an
// mbarrier) issued before anything else, filter vertically four output rows
// per thread into planar float4 columns, filter horizontally four rows per
// thread, quantise, cast through the table and store straight into the batch
// tensor.  Copy and nearest-neighbour affine tiles read their source through
// the read-only path; pad-only tiles are plain 16-byte stores.
//
// The arithmetic is that of the generic kernel in fused_batch.cu: every resize
// output is a chain acc = fma(w_k, v_k, acc) from 0 in increasing tap order,
// vertical axis first, quantised as (int)(acc + 0.5) clamped to [0, 255].  The
// vertical pass walks the union of the source rows of its four output rows; a
// row that is not a tap of one of them enters that output with weight 0, which
// leaves its accumulator unchanged, so every chain is the same.
#include "fused_batch.h"
#include "kernel_common.cuh"

namespace mlxd {
namespace {

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

// d = a * b + d on two float lanes with one instruction (each lane is an IEEE
// fused multiply-add, identical to two fmaf calls).
__device__ __forceinline__ void ffma2(float& d0, float& d1, float a0, float a1, float b0, float b1) {
  asm("{\n\t.reg .b64 ra, rb, rc;\n\t"
      "mov.b64 ra, {%2, %3};\n\t"
      "mov.b64 rb, {%4, %5};\n\t"
      "mov.b64 rc, {%0, %1};\n\t"
      "fma.rn.f32x2 rc, ra, rb, rc;\n\t"
      "mov.b64 {%0, %1}, rc;\n\t}"
      : "+f"(d0), "+f"(d1)
      : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}

// Two bytes of a word as floats, exactly: each byte is placed in the mantissa
// of 2^23 and 2^23 is subtracted (one packed add for both).
template <int B0, int B1>
__device__ __forceinline__ void bytes_to_float2(uint32_t word, float& f0, float& f1) {
  const float x0 = __uint_as_float(__byte_perm(word, 0x4B000000u, 0x7540u + B0));
  const float x1 = __uint_as_float(__byte_perm(word, 0x4B000000u, 0x7540u + B1));
  asm("{\n\t.reg .b64 ra, rb, rc;\n\t"
      "mov.b64 ra, {%2, %3};\n\t"
      "mov.b64 rb, {%4, %4};\n\t"
      "add.rn.f32x2 rc, ra, rb;\n\t"
      "mov.b64 {%0, %1}, rc;\n\t}"
      : "=f"(f0), "=f"(f1)
      : "f"(x0), "f"(x1), "f"(-8388608.0f));
}

// (int)(acc + 0.5) clamped to [0, 255]: the float-to-uint8 conversion truncates
// toward zero and saturates at both ends, which is that clamp.
__device__ __forceinline__ unsigned quantise_sat(float acc) {
  unsigned q;
  asm("cvt.rzi.u8.f32 %0, %1;" : "=r"(q) : "f"(__fadd_rn(acc, 0.5f)));
  return q;
}

// Tables that change from pass to pass (a pass = one run of output columns of
// the band); two sets, so the next pass's tables are built while the current
// pass is still filtering horizontally.
struct PassTables {
  int* hfirst;      // [kTileW]
  int* hcount;      // [kTileW]
  float* wh;        // [kTileW][cap_x]
  int2* urow;       // [4][u_cap]  {word index of the staged row, funnel shift in bits}
};

struct Smem {
  float* lut;       // [c][256]
  PassTables tab[2];
  float4* uw;       // [4][u_cap]  weight of a union row in each of the group's four outputs
  int* ucount;      // [4]
  uint64_t* bar;
  float4* mid;      // [4][C][ncols]
  uint8_t* srct;
};

__host__ __device__ inline size_t align16(size_t v) {
  return (v + 15) & ~(size_t)15;
}

__host__ __device__ inline size_t smem_layout(const LaunchParams& p, unsigned char* base, Smem* out) {
  Smem sm;
  size_t off = 0;
  sm.lut = reinterpret_cast<float*>(base + off);
  off += (size_t)p.c_out * 256 * sizeof(float);
  for (int k = 0; k < 2; k++) {
    sm.tab[k].hfirst = reinterpret_cast<int*>(base + off);
    off += kTileW * sizeof(int);
    sm.tab[k].hcount = reinterpret_cast<int*>(base + off);
    off += kTileW * sizeof(int);
    sm.tab[k].urow = reinterpret_cast<int2*>(base + off);
    off += (size_t)4 * p.u_cap * sizeof(int2);
    sm.tab[k].wh = reinterpret_cast<float*>(base + off);   // (w, w) pairs
    off = align16(off + (size_t)p.weight_floats * 2 * sizeof(float));
  }
  sm.uw = reinterpret_cast<float4*>(base + off);
  off += (size_t)4 * p.u_cap * 2 * sizeof(float4);
  sm.ucount = reinterpret_cast<int*>(base + off);
  off += 16;
  sm.bar = reinterpret_cast<uint64_t*>(base + off);
  off += 16;
  sm.mid = reinterpret_cast<float4*>(base + off);
  off = align16(off + (size_t)p.mid_float4s * 16);
  sm.srct = base + off;
  off += (size_t)p.src_tile_bytes;
  if (out) {
    *out = sm;
  }
  return off + 16;
}

// Source footprint of one pass, computed identically by every thread.
struct PassGeom {
  int bx, nc;          // first geometric-output column and column count
  int clo, ncols;      // first source column staged, columns staged
  int wbytes, pitch_s, nwords, common;
  bool edge_x;
  const uint8_t* g0;   // source byte of (first staged row, first staged column)
};

template <int C>
__device__ __forceinline__ PassGeom pass_geom(const DevSample& s, const Axis& ax, int rlo, int bx, int nc) {
  PassGeom g;
  g.bx = bx;
  g.nc = nc;
  int f0, l0, f1, l1;
  axis_range(ax, bx, f0, l0);
  axis_range(ax, bx + nc - 1, f1, l1);
  g.clo = clampi(f0, 0, s.pre_w - 1);
  const int chi = clampi(l1, 0, s.pre_w - 1);
  g.edge_x = f0 < 0 || l1 > s.pre_w - 1;
  g.ncols = chi - g.clo + 1;
  g.wbytes = g.ncols * C;
  g.g0 = s.src + ((size_t)(s.pre_y + rlo) * s.src_w + (s.pre_x + g.clo)) * C;
  g.common = (int)(reinterpret_cast<uintptr_t>(g.g0) & 3);
  g.pitch_s = (g.wbytes + 15 + 15 + 4 + 15) & ~15;
  g.nwords = (g.common + g.wbytes + 3) >> 2;
  return g;
}

// Issue the bulk copies of a pass (threads < rows) and build its tables
// (threads 0..nc-1 the horizontal taps, the others the staged-row addresses of
// the vertical union).
template <int C>
__device__ __forceinline__ void start_pass(
    const DevSample& s, const LaunchParams& p, const Smem& sm, const PassTables& tab, const PassGeom& g,
    const Axis& ay, const Axis& ax, int by, int nr, int rlo, int rows) {
  const int tid = threadIdx.x;
  const size_t src_pitch = (size_t)s.src_w * C;
  if (tid < rows) {
    const uintptr_t ga = reinterpret_cast<uintptr_t>(g.g0) + (size_t)tid * src_pitch;
    const int phase = (int)(ga & 15);
    const unsigned len = (unsigned)((phase + g.wbytes + 15) & ~15);
    mbar_expect_tx(sm.bar, len);
    bulk_copy(sm.srct + tid * g.pitch_s, reinterpret_cast<const void*>(ga - phase), len, sm.bar);
  }
  // horizontal taps: one thread per output column (the last warps, which issue
  // no copies); every weight is stored twice, side by side, so the packed
  // multiply-add reads its (w, w) operand with one 64-bit load
  {
    const int x = tid - (kThreads - kTileW);
    if (x >= 0 && x < g.nc) {
      int lo, hi;
      axis_range(ax, g.bx + x, lo, hi);
      int cnt = hi - lo + 1;
      cnt = cnt > s.cap_x ? s.cap_x : cnt;
      tab.hfirst[x] = lo;
      tab.hcount[x] = cnt;
      float2* w2 = reinterpret_cast<float2*>(tab.wh) + x * s.cap_x;
      if (ax.identity) {
        w2[0] = make_float2(1.0f, 1.0f);
      } else {
        const float c = axis_center(ax, g.bx + x);
        float sum = 0.0f;
        for (int k = 0; k < cnt; k++) {
          const float v = axis_tent(ax, c, lo + k);
          w2[k].x = v;
          sum = __fadd_rn(sum, v);
        }
        for (int k = 0; k < cnt; k++) {
          const float w = __fdiv_rn(w2[k].x, sum);
          w2[k] = make_float2(w, w);
        }
      }
    }
  }
  const int ngroups = (nr + 3) >> 2;
  for (int i = tid; i < ngroups * p.u_cap; i += kThreads) {
    const int rg = i / p.u_cap;
    const int e = i - rg * p.u_cap;
    if (e < sm.ucount[rg]) {
      int lo, hi;
      axis_range(ay, by + rg * 4, lo, hi);
      const int sr = clampi(lo + e, 0, s.pre_h - 1) - rlo;
      const int phase = (int)((reinterpret_cast<uintptr_t>(g.g0) + (size_t)sr * src_pitch) & 15);
      tab.urow[i] = make_int2((sr * g.pitch_s + phase - g.common) >> 2, ((phase - g.common) & 3) * 8);
    }
  }
}

// Geometric-output rows [by, by+nr) (nr <= kTileH) x columns [gx_lo, gx_hi) of
// a resize sample, sub_w columns per pass, written to the batch tensor.  The
// copies of pass t+1 are in flight while pass t filters horizontally.
template <int C>
__device__ void resize_rows(
    const DevSample& s, const LaunchParams& p, const Smem& sm, unsigned& parity, bool& first_use,
    int by, int nr, int gx_lo, int gx_hi) {
  const int tid = threadIdx.x;
  const Axis ay = make_axis(s.pre_h, s.geom_h);
  const Axis ax = make_axis(s.pre_w, s.geom_w);
  int t0, t1, t2, t3;
  axis_range(ay, by, t0, t1);
  axis_range(ay, by + nr - 1, t2, t3);
  const int rlo = clampi(t0, 0, s.pre_h - 1);
  const int rhi = clampi(t3, 0, s.pre_h - 1);
  const int rows = rhi - rlo + 1;
  const int ngroups = (nr + 3) >> 2;
  if (rows > kMaxStagedRows || rows > kThreads) {
    if (tid == 0) {
      atomicOr(p.status, 2);
    }
    return;
  }
  if (!first_use) {
    // every thread is done with the previous rows' tables and buffers
    __syncthreads();
    fence_async_smem();
  }
  first_use = false;

  // ---- vertical union weights of every group of four output rows ---------------
  for (int i = tid; i < ngroups * p.u_cap; i += kThreads) {
    const int rg = i / p.u_cap;
    const int e = i - rg * p.u_cap;
    const int o0 = by + rg * 4;
    const int on = min(4, nr - rg * 4);
    int lo[4], hi[4];
#pragma unroll
    for (int r = 0; r < 4; r++) {
      axis_range(ay, o0 + (r < on ? r : on - 1), lo[r], hi[r]);
    }
    const int ufirst = lo[0];
    const int ulast = hi[3];   // rows past the group's end repeat its last row
    const int u = ufirst + e;
    if (e == 0) {
      int cnt = ulast - ufirst + 1;
      if (cnt > p.u_cap) {
        cnt = p.u_cap;
        atomicOr(p.status, 8);
      }
      sm.ucount[rg] = cnt;
    }
    if (u <= ulast) {
      float w4[4];
#pragma unroll
      for (int r = 0; r < 4; r++) {
        float w = 0.0f;
        if (r < on && u >= lo[r] && u <= hi[r]) {
          if (ay.identity) {
            w = 1.0f;
          } else {
            const float c = axis_center(ay, o0 + r);
            float sum = 0.0f;
            for (int k = lo[r]; k <= hi[r]; k++) {
              sum = __fadd_rn(sum, axis_tent(ay, c, k));
            }
            w = __fdiv_rn(axis_tent(ay, c, u), sum);
          }
        }
        w4[r] = w;
      }
      sm.uw[2 * i] = make_float4(w4[0], w4[0], w4[1], w4[1]);
      sm.uw[2 * i + 1] = make_float4(w4[2], w4[2], w4[3], w4[3]);
    }
  }
  __syncthreads();   // ucount is read by start_pass

  PassGeom cur = pass_geom<C>(s, ax, rlo, gx_lo, min(s.sub_w, gx_hi - gx_lo));
  if (rows * cur.pitch_s > p.src_tile_bytes || 4 * C * cur.ncols > p.mid_float4s) {
    if (tid == 0) {
      atomicOr(p.status, 2);
    }
    return;
  }
  start_pass<C>(s, p, sm, sm.tab[0], cur, ay, ax, by, nr, rlo, rows);
  __syncthreads();
  if (tid == 0) {
    mbar_arrive(sm.bar);
  }

  float* base = reinterpret_cast<float*>(s.dst);
  const size_t row_stride = (size_t)s.slot_w * C;
  int it = 0;
  for (;;) {
    const PassTables tab = (it & 1) ? sm.tab[1] : sm.tab[0];
    const PassTables tab_next = (it & 1) ? sm.tab[0] : sm.tab[1];
    if (!mbar_wait(sm.bar, parity)) {
      atomicOr(p.status, 4);
    }
    parity ^= 1;

    // ---- vertical filter: thread = (source word, group of four output rows) -----
    {
      const uint32_t* srcw = reinterpret_cast<const uint32_t*>(sm.srct);
      // every thread owns one source word (four byte columns) and walks the row
      // groups with a stride of two; where its columns land in the planar
      // buffer does not depend on the group
      for (int g = tid & 127; g < cur.nwords; g += 128) {
        int off0, off1, off2, off3;
        {
          const int jb = 4 * g - cur.common;
          int j = jb;
          off0 = (j >= 0 && j < cur.wbytes) ? (j % C) * cur.ncols + j / C : -1;
          j = jb + 1;
          off1 = (j >= 0 && j < cur.wbytes) ? (j % C) * cur.ncols + j / C : -1;
          j = jb + 2;
          off2 = (j >= 0 && j < cur.wbytes) ? (j % C) * cur.ncols + j / C : -1;
          j = jb + 3;
          off3 = (j >= 0 && j < cur.wbytes) ? (j % C) * cur.ncols + j / C : -1;
        }
        for (int rg = tid >> 7; rg < ngroups; rg += kThreads >> 7) {
          const int cnt = sm.ucount[rg];
          const int2* urow = tab.urow + rg * p.u_cap;
          const float4* uw = sm.uw + 2 * rg * p.u_cap;
          float a00 = 0.f, a01 = 0.f, a02 = 0.f, a03 = 0.f;
          float a10 = 0.f, a11 = 0.f, a12 = 0.f, a13 = 0.f;
          float a20 = 0.f, a21 = 0.f, a22 = 0.f, a23 = 0.f;
          float a30 = 0.f, a31 = 0.f, a32 = 0.f, a33 = 0.f;
          for (int e = 0; e < cnt; e++) {
            const int2 ri = urow[e];
            const float4 wa = uw[2 * e];       // (w0, w0, w1, w1)
            const float4 wb = uw[2 * e + 1];   // (w2, w2, w3, w3)
            uint32_t word = srcw[ri.x + g];
            if (ri.y) {
              word = __funnelshift_r(word, srcw[ri.x + g + 1], ri.y);
            }
            float v0, v1, v2, v3;
            bytes_to_float2<0, 1>(word, v0, v1);
            bytes_to_float2<2, 3>(word, v2, v3);
            ffma2(a00, a01, v0, v1, wa.x, wa.y);
            ffma2(a02, a03, v2, v3, wa.x, wa.y);
            ffma2(a10, a11, v0, v1, wa.z, wa.w);
            ffma2(a12, a13, v2, v3, wa.z, wa.w);
            ffma2(a20, a21, v0, v1, wb.x, wb.y);
            ffma2(a22, a23, v2, v3, wb.x, wb.y);
            ffma2(a30, a31, v0, v1, wb.z, wb.w);
            ffma2(a32, a33, v2, v3, wb.z, wb.w);
          }
          // planar store: column (px, ch) of group rg -> mid[(rg * C + ch) * ncols + px]
          float4* plane = sm.mid + rg * C * cur.ncols;
          if (off0 >= 0) plane[off0] = make_float4(a00, a10, a20, a30);
          if (off1 >= 0) plane[off1] = make_float4(a01, a11, a21, a31);
          if (off2 >= 0) plane[off2] = make_float4(a02, a12, a22, a32);
          if (off3 >= 0) plane[off3] = make_float4(a03, a13, a23, a33);
        }
      }
    }
    __syncthreads();   // the staging buffer is free, the columns are complete

    // ---- start the next pass: copies fly while this one filters horizontally ------
    const int next_bx = cur.bx + s.sub_w;
    const bool more = next_bx < gx_hi;
    PassGeom nxt = cur;
    if (more) {
      nxt = pass_geom<C>(s, ax, rlo, next_bx, min(s.sub_w, gx_hi - next_bx));
      if (rows * nxt.pitch_s > p.src_tile_bytes || 4 * C * nxt.ncols > p.mid_float4s) {
        if (tid == 0) {
          atomicOr(p.status, 2);
        }
        return;
      }
      fence_async_smem();
      start_pass<C>(s, p, sm, tab_next, nxt, ay, ax, by, nr, rlo, rows);
    }

    // ---- horizontal filter: thread = (output column, channel, group of four rows) ----
    {
      const int per_rg = cur.nc * C;
      for (int item = tid; item < ngroups * per_rg; item += kThreads) {
        int rg, rem;
        if (cur.nc == kTileW) {
          rg = item / (kTileW * C);
          rem = item - rg * (kTileW * C);
        } else {
          rg = item / per_rg;
          rem = item - rg * per_rg;
        }
        const int x = rem / C;
        const int ch = rem - x * C;
        const int f = tab.hfirst[x];
        const int cnt = tab.hcount[x];
        const float2* w = reinterpret_cast<const float2*>(tab.wh) + x * s.cap_x;
        const float4* col = sm.mid + (rg * C + ch) * cur.ncols;
        float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
        if (!cur.edge_x) {
          const float4* c0 = col + (f - cur.clo);
          for (int k = 0; k < cnt; k++) {
            const float4 v = c0[k];
            const float2 wk = w[k];
            ffma2(a0, a1, v.x, v.y, wk.x, wk.y);
            ffma2(a2, a3, v.z, v.w, wk.x, wk.y);
          }
        } else {
          for (int k = 0; k < cnt; k++) {
            const float4 v = col[clampi(f + k, 0, s.pre_w - 1) - cur.clo];
            const float2 wk = w[k];
            ffma2(a0, a1, v.x, v.y, wk.x, wk.y);
            ffma2(a2, a3, v.z, v.w, wk.x, wk.y);
          }
        }
        int px = cur.bx + x - s.post_x;
        if (s.post_flip) {
          px = s.post_w - 1 - px;
        }
        const int oy = by + rg * 4 - s.post_y;
        const float* lut = sm.lut + ch * 256;
        float* dst = base + ((size_t)oy * s.slot_w + px) * C + ch;
        const int left = nr - rg * 4;
        dst[0] = lut[quantise_sat(a0)];
        if (left > 1) dst[row_stride] = lut[quantise_sat(a1)];
        if (left > 2) dst[2 * row_stride] = lut[quantise_sat(a2)];
        if (left > 3) dst[3 * row_stride] = lut[quantise_sat(a3)];
      }
    }
    if (!more) {
      break;
    }
    __syncthreads();   // the columns are free, the next pass's tables are complete
    if (tid == 0) {
      mbar_arrive(sm.bar);
    }
    cur = nxt;
    it++;
  }
}

// Copy (crop / flip / batch only) and nearest-neighbour affine: one thread per
// output pixel of rows [y0, vy1) x columns [xa, xb), source bytes through the
// read-only path.
template <int C>
__device__ void gather_rows(const DevSample& s, const LaunchParams& p, int y0, int vy1, int xa, int xb) {
  const int nvx = xb - xa;
  const int nvy = vy1 - y0;
  float* base = reinterpret_cast<float*>(s.dst);
  const float twh = (float)((double)s.geom_w / 2.0);
  const float thh = (float)((double)s.geom_h / 2.0);
  const float wh = (float)((double)s.pre_w / 2.0);
  const float hh = (float)((double)s.pre_h / 2.0);
  for (int ry = 0; ry < nvy; ry++) {
    const int gy = s.post_y + y0 + ry;
    for (int rx = threadIdx.x; rx < nvx; rx += kThreads) {
      const int px = s.post_flip ? (s.post_w - 1 - (xa + rx)) : (xa + rx);
      const int gx = s.post_x + px;
      int sx = gx, sy = gy;
      bool inside = true;
      if (s.mode == kModeAffine) {
        // The coordinate is built from float products and float sums, then two
        // double additions, then truncation toward zero - the evaluation order
        // of the reference expression - and no multiply-add is contracted.
        const float dxf = __fsub_rn((float)(long long)gx, twh);
        const float dyf = __fsub_rn((float)(long long)gy, thh);
        const float fx = __fadd_rn(__fadd_rn(__fmul_rn(s.mx[0], dxf), __fmul_rn(s.mx[1], dyf)), s.mx[2]);
        const float fy = __fadd_rn(__fadd_rn(__fmul_rn(s.mx[3], dxf), __fmul_rn(s.mx[4], dyf)), s.mx[5]);
        const long long ax = (long long)__dadd_rn(__dadd_rn((double)fx, 0.5), (double)wh);
        const long long ay = (long long)__dadd_rn(__dadd_rn((double)fy, 0.5), (double)hh);
        inside = !(ax < 0 || ay < 0 || ax >= s.pre_w || ay >= s.pre_h);
        sx = (int)ax;
        sy = (int)ay;
      }
      float* dst = base + ((size_t)(y0 + ry) * s.slot_w + (xa + rx)) * C;
      if (inside) {
        const int ix = s.pre_x + (s.pre_flip ? (s.pre_w - 1 - sx) : sx);
        const uint8_t* g = s.src + ((size_t)(s.pre_y + sy) * s.src_w + ix) * C;
#pragma unroll
        for (int ch = 0; ch < C; ch++) {
          dst[ch] = __ldg(p.lut + ch * 256 + __ldg(g + ch));
        }
      } else {
#pragma unroll
        for (int ch = 0; ch < C; ch++) {
          dst[ch] = __ldg(p.lut + ch * 256);
        }
      }
    }
  }
}

// One CTA: rows [y0, y0 + kTileH) of one slot, columns of p.band_tiles tiles.
template <int C>
__device__ void run_band(const LaunchParams& p, unsigned char* smem_raw) {
  unsigned t = blockIdx.x;
  const int tb = t % p.bands_x;
  t /= p.bands_x;
  const int ty = t % p.tiles_y;
  const int n = t / p.tiles_y;
  if (n >= p.n) {
    return;
  }
  const DevSample s = p.samples[n];
  const int y0 = ty * kTileH;
  const int x0 = tb * p.band_tiles * kTileW;
  if (y0 >= s.slot_h || x0 >= s.slot_w) {
    return;
  }
  const int y1 = min(y0 + kTileH, s.slot_h);
  const int x1 = min(x0 + p.band_tiles * kTileW, s.slot_w);
  const int vy1 = min(y1, s.post_h);
  const int vx1 = min(x1, s.post_w);
  const bool has_valid = (y0 < vy1) && (x0 < vx1);
  float padf[4];
#pragma unroll
  for (int c = 0; c < 4; c++) {
    padf[c] = c < C ? __ldg(p.lut + c * 256 + p.pad_px) : 0.0f;
  }
  float* out = reinterpret_cast<float*>(s.dst);
  if (!has_valid) {
    fill_rect_f32<C>(out, s.slot_w, y0, y1, x0, x1, padf);
    return;
  }
  if (s.mode == kModeResize) {
    Smem sm;
    smem_layout(p, smem_raw, &sm);
    if (threadIdx.x == 0) {
      mbar_init(sm.bar, 1);
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (int i = threadIdx.x; i < C * 256; i += kThreads) {
      sm.lut[i] = __ldg(p.lut + i);
    }
    __syncthreads();
    int gx_lo, gx_hi;
    if (!s.post_flip) {
      gx_lo = s.post_x + x0;
      gx_hi = s.post_x + vx1;
    } else {
      gx_lo = s.post_x + s.post_w - vx1;
      gx_hi = s.post_x + s.post_w - x0;
    }
    unsigned parity = 0;
    bool first_use = true;
    for (int by = s.post_y + y0; by < s.post_y + vy1; by += s.sub_h) {
      resize_rows<C>(s, p, sm, parity, first_use, by, min(s.sub_h, s.post_y + vy1 - by), gx_lo, gx_hi);
    }
  } else {
    gather_rows<C>(s, p, y0, vy1, x0, vx1);
  }
  // pad the part of the band outside the post window
  fill_rect_f32<C>(out, s.slot_w, vy1, y1, x0, x1, padf);
  fill_rect_f32<C>(out, s.slot_w, y0, vy1, vx1, x1, padf);
}

__global__ void __launch_bounds__(kThreads, 3) fused_fast_kernel(const LaunchParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  if (p.c_in == 3) {
    run_band<3>(p, smem_raw);
  } else if (p.c_in == 1) {
    run_band<1>(p, smem_raw);
  } else {
    run_band<4>(p, smem_raw);
  }
}

} // namespace

size_t fused_fast_smem_bytes(const LaunchParams& p) {
  if (p.src_tile_bytes == 0) {
    return 0;   // no sample resizes: nothing is staged
  }
  return smem_layout(p, nullptr, nullptr);
}

cudaError_t launch_fused_fast(const LaunchParams& p_in, cudaStream_t stream) {
  static thread_local int configured_device = -1;
  static thread_local int sm_count = 0;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    return e;
  }
  if (configured_device != dev) {
    LaunchParams worst = p_in;
    worst.c_out = 4;
    worst.weight_floats = kWeightFloats;
    worst.mid_float4s = kMidFloats / 4;
    worst.src_tile_bytes = kSrcTileBytes;
    worst.u_cap = kMaxStagedRows;
    e = cudaFuncSetAttribute(
        fused_fast_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_layout(worst, nullptr, nullptr));
    if (e != cudaSuccess) {
      return e;
    }
    e = cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) {
      return e;
    }
    configured_device = dev;
  }
  LaunchParams p = p_in;
  // Tiles per CTA along a row band: as many as keeps about eight waves of CTAs
  // on the device (3 CTAs per SM), at most 8.
  const long long tiles = (long long)p.n * p.tiles_y * p.tiles_x;
  const long long want_ctas = (long long)sm_count * 3 * 8;
  int band = (int)(tiles / (want_ctas > 0 ? want_ctas : 1));
  band = band < 1 ? 1 : (band > 8 ? 8 : band);
  band = band > p.tiles_x ? p.tiles_x : band;
  p.band_tiles = band;
  p.bands_x = (p.tiles_x + band - 1) / band;
  const unsigned long long blocks = (unsigned long long)p.n * p.tiles_y * p.bands_x;
  if (blocks == 0) {
    return cudaSuccess;
  }
  if (blocks > 0x7fffffffULL) {
    return cudaErrorInvalidConfiguration;
  }
  fused_fast_kernel<<<(unsigned)blocks, kThreads, fused_fast_smem_bytes(p), stream>>>(p);
  return cudaGetLastError();
}

} // namespace mlxd
