// The kernels that run every launch (float32 batches, float32 batches after the
// channel reduction, two-channel float32 batches, uint8 batches; one entry point
// each, the same code): one CTA per band of up to eight kTileH x kTileW tiles of
// one sample's slot, run as a sequence of passes (sub_h x sub_w outputs each).
// A resize pass stages its source footprint in shared memory with bulk
// asynchronous copies (cp.async.bulk, one per source row, completion on an
// mbarrier, bounded wait; the next pass's copies are issued as soon as the
// vertical filter has consumed the buffer), filters vertically - a thread takes
// eight byte columns into two output rows - into planar float4 columns, filters
// horizontally - a thread takes one output column of four rows over all
// channels - quantises, casts through the table (float32 batches) and stores
// straight into the batch tensor.  Copy and nearest-neighbour affine bands read
// their source through the read-only path, four pixels per thread, and store
// 16 bytes at a time; pad-only bands are plain 16-byte stores, and the rows
// below a sample in a ragged batch go out through a linear fill kernel.  A
// resize whose taps fit no pass size (shrink ratios of about 60 and more) is
// filtered pixel by pixel from global memory by a kernel of its own.
//
// The arithmetic: every resize output is a chain acc = fma(w_k, v_k, acc) from
// 0 in increasing tap order, vertical axis first, quantised as (int)(acc + 0.5)
// clamped to [0, 255].  The vertical pass walks the union of the source rows of
// its two output rows; a row that is not a tap of one of them enters that
// output with weight 0, which leaves its accumulator unchanged, so every chain
// is the same.
#include "fused_batch.h"
#include "kernel_common.cuh"

namespace mlxd {
namespace {

// Polls of an mbarrier before a wait gives up: about a second (a poll that finds
// the phase incomplete returns after a few microseconds), five orders of
// magnitude above what a pass's copies take.
constexpr unsigned kSpinLimit = 1u << 18;

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(unsigned bar, unsigned bytes) {
  asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(unsigned bar) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(bar) : "memory");
}

// Bounded wait for the phase with the given parity.  Returns false when the
// limit was reached; the caller records that and goes on without hanging.
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity) {
  const uint32_t a = bar;
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
__device__ __forceinline__ void bulk_copy(unsigned dst_smem, const void* src_gmem, unsigned bytes, unsigned bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_smem),
      "l"(src_gmem), "r"(bytes), "r"(bar)
      : "memory");
}

// Typed view of a shared-space address.
template <typename T>
__device__ __forceinline__ T* sp(unsigned a) {
  return reinterpret_cast<T*>(__cvta_shared_to_generic(a));
}

__device__ __forceinline__ void fence_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// Two float lanes in one 64-bit register, the operand form of the packed
// instructions; keeping values packed avoids repacking moves around them.
typedef unsigned long long f32x2;

// d = a * b + d on both lanes (each lane is an IEEE fused multiply-add,
// identical to fmaf).
__device__ __forceinline__ void ffma2(f32x2& d, f32x2 a, f32x2 b) {
  asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(d) : "l"(a), "l"(b));
}

__device__ __forceinline__ f32x2 fmul2(f32x2 a, f32x2 b) {
  f32x2 d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

__device__ __forceinline__ f32x2 pack2(float lo, float hi) {
  f32x2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}

__device__ __forceinline__ void unpack2(f32x2 v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}

// Bytes B0 and B1 of a word as two packed floats, exactly: each byte is placed
// in the mantissa of 2^23 and 2^23 is subtracted (one packed add for both).
template <int B0, int B1>
__device__ __forceinline__ f32x2 bytes_to_f32x2(uint32_t word, f32x2 minus_two23) {
  const float x0 = __uint_as_float(__byte_perm(word, 0x4B000000u, 0x7540u + B0));
  const float x1 = __uint_as_float(__byte_perm(word, 0x4B000000u, 0x7540u + B1));
  f32x2 r = pack2(x0, x1);
  asm("add.rn.f32x2 %0, %0, %1;" : "+l"(r) : "l"(minus_two23));
  return r;
}

// (int)(acc + 0.5) clamped to [0, 255]: the float-to-uint8 conversion truncates
// toward zero and saturates at both ends, which is that clamp.
__device__ __forceinline__ unsigned quantise_sat(float acc) {
  unsigned q;
  asm("cvt.rzi.u8.f32 %0, %1;" : "=r"(q) : "f"(__fadd_rn(acc, 0.5f)));
  return q;
}

// Shared-memory loads by 32-bit shared-space address plus a constant offset.
// Spelling the inner loops with these keeps their address arithmetic to the
// pointer increments written out in the loops.
template <int OFF>
__device__ __forceinline__ uint32_t lds_u32(unsigned a) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(a), "n"(OFF));
  return v;
}

template <int OFF>
__device__ __forceinline__ void lds_v2u32(unsigned a, uint32_t& x, uint32_t& y) {
  asm volatile("ld.shared.v2.u32 {%0, %1}, [%2+%3];" : "=r"(x), "=r"(y) : "r"(a), "n"(OFF));
}

template <int OFF>
__device__ __forceinline__ f32x2 lds_u64(unsigned a) {
  f32x2 v;
  asm volatile("ld.shared.u64 %0, [%1+%2];" : "=l"(v) : "r"(a), "n"(OFF));
  return v;
}

template <int OFF>
__device__ __forceinline__ void lds_v2u64(unsigned a, f32x2& x, f32x2& y) {
  asm volatile("ld.shared.v2.u64 {%0, %1}, [%2+%3];" : "=l"(x), "=l"(y) : "r"(a), "n"(OFF));
}

template <int OFF>
__device__ __forceinline__ void sts_v2f32(unsigned a, float x, float y) {
  asm volatile("st.shared.v2.f32 [%0+%1], {%2, %3};" ::"r"(a), "n"(OFF), "f"(x), "f"(y) : "memory");
}

// Columns of padding on either side of every plane of the planar buffer: an
// octet of byte columns may start up to 7 before the first staged byte and end
// up to 7 past the last, and its stores are not bounds-checked.
template <int C>
struct PlanePad {
  static constexpr int value = (7 + C - 1) / C;
};

// Slot of column c (>= 0, padding included) inside its plane: one slot is
// skipped after every eight columns.  Threads of a warp touch columns a fixed
// distance apart - 8/C columns per lane in the vertical pass, the resize ratio
// in the horizontal one - and with 16-byte slots in a row every distance that
// is a multiple of 2 would keep hitting the same banks.
__device__ __forceinline__ int skew(int c) {
  return c + (c >> 3);
}

// Slots per plane for ncols staged columns.
template <int C>
__device__ __forceinline__ int plane_slots(int ncols) {
  return skew(ncols + 2 * PlanePad<C>::value) + 1;
}

// The eight results of one thread of the vertical pass - byte columns j0..j0+7
// of a row pair - go to the planar buffer: byte column j = (px, ch) sits in
// plane ch at slot skew(pad + px).  b[m] is the shared address of column
// j0 + m for m < C and low[m] that column's index modulo 8; column j0 + k =
// j0 + m + C * t is t columns further in the same plane, one slot more when
// it crosses a multiple of eight.  Columns outside the staged row land in the
// padding.
template <int C, int K>
__device__ __forceinline__ void store_column(const unsigned (&b)[C], const int (&low)[C], float x, float y) {
  constexpr int m = K % C;
  constexpr int t = K / C;
  if (t == 0) {
    sts_v2f32<0>(b[m], x, y);
  } else {
    // t <= 7: at most one multiple of eight is crossed
    const unsigned a = b[m] + ((low[m] + t) >= 8 ? 16u : 0u);
    sts_v2f32<16 * t>(a, x, y);
  }
}

template <int C>
__device__ __forceinline__ void store_octet(const unsigned (&b)[C], const int (&low)[C], const f32x2 (&acc)[8]) {
  float lo0, hi0, lo1, hi1;
  unpack2(acc[0], lo0, hi0);
  unpack2(acc[2], lo1, hi1);
  store_column<C, 0>(b, low, lo0, lo1);
  store_column<C, 1>(b, low, hi0, hi1);
  unpack2(acc[1], lo0, hi0);
  unpack2(acc[3], lo1, hi1);
  store_column<C, 2>(b, low, lo0, lo1);
  store_column<C, 3>(b, low, hi0, hi1);
  unpack2(acc[4], lo0, hi0);
  unpack2(acc[6], lo1, hi1);
  store_column<C, 4>(b, low, lo0, lo1);
  store_column<C, 5>(b, low, hi0, hi1);
  unpack2(acc[5], lo0, hi0);
  unpack2(acc[7], lo1, hi1);
  store_column<C, 6>(b, low, lo0, lo1);
  store_column<C, 7>(b, low, hi0, hi1);
}

// Byte offsets and low bits (see store_octet) of the octet that starts at byte
// column j0, relative to the first plane of a group; pslots = slots per plane.
template <int C>
__device__ __forceinline__ void octet_offsets(int j0, int pslots, unsigned (&b)[C], int (&low)[C]) {
  const int q0 = (j0 + 8 * C) / C - 8;
  const int r0 = (j0 + 8 * C) - (q0 + 8) * C;
#pragma unroll
  for (int m = 0; m < C; m++) {
    const int r = r0 + m;
    const int wrap = r >= C ? 1 : 0;
    const int c = PlanePad<C>::value + q0 + wrap;
    low[m] = c & 7;
    b[m] = (unsigned)(((r - wrap * C) * pslots + skew(c)) * 16);
  }
}

// One union row of vertical_taps into the eight accumulators: the two words at
// shared address ra (funnel-shifted by sh when SHIFT), the row's weights at wp.
// FIRST: products instead of multiply-adds onto zero.  Pixels and weights are
// never negative, so the product is the same float, +0 included.
template <bool SHIFT, bool FIRST>
__device__ __forceinline__ void vertical_row(unsigned ra, unsigned sh, unsigned wp, f32x2 minus_two23, f32x2 (&acc)[8]) {
  f32x2 w0, w1;
  lds_v2u64<0>(wp, w0, w1);
  uint32_t wa, wb;
  if (SHIFT) {
    const uint32_t x0 = lds_u32<0>(ra);
    const uint32_t x1 = lds_u32<4>(ra);
    const uint32_t x2 = lds_u32<8>(ra);
    wa = __funnelshift_r(x0, x1, sh);
    wb = __funnelshift_r(x1, x2, sh);
  } else {
    lds_v2u32<0>(ra, wa, wb);
  }
  const f32x2 v0 = bytes_to_f32x2<0, 1>(wa, minus_two23);
  const f32x2 v1 = bytes_to_f32x2<2, 3>(wa, minus_two23);
  const f32x2 v2 = bytes_to_f32x2<0, 1>(wb, minus_two23);
  const f32x2 v3 = bytes_to_f32x2<2, 3>(wb, minus_two23);
  if (FIRST) {
    acc[0] = fmul2(v0, w0);
    acc[1] = fmul2(v1, w0);
    acc[2] = fmul2(v0, w1);
    acc[3] = fmul2(v1, w1);
    acc[4] = fmul2(v2, w0);
    acc[5] = fmul2(v3, w0);
    acc[6] = fmul2(v2, w1);
    acc[7] = fmul2(v3, w1);
  } else {
    ffma2(acc[0], v0, w0);
    ffma2(acc[1], v1, w0);
    ffma2(acc[2], v0, w1);
    ffma2(acc[3], v1, w1);
    ffma2(acc[4], v2, w0);
    ffma2(acc[5], v3, w0);
    ffma2(acc[6], v2, w1);
    ffma2(acc[7], v3, w1);
  }
}

// Vertical taps of eight adjacent byte columns (two source words) into a pair
// of output rows.  acc[4 * h + 2 * r + k] holds, for word h and row r of the
// pair, the byte pair (2k, 2k+1).  up walks the {row address, funnel shift}
// table of the pair's union of source rows, wp its weights (w0,w0,w1,w1); g8 is
// the thread's byte offset in every staged row.  Without SHIFT every staged
// row starts on an 8-byte boundary and the two words come with one load.
template <bool SHIFT>
__device__ __forceinline__ void vertical_taps(unsigned up, unsigned wp, unsigned g8, int cnt, f32x2 (&acc)[8]) {
  const f32x2 minus_two23 = pack2(-8388608.0f, -8388608.0f);
  const unsigned up_end = up + 8u * (unsigned)cnt;
  // The table entry of the next row is fetched while this row is filtered, so
  // a row's loads do not wait for one another.  The entry after the last row
  // is read and dropped: it lies inside the table set whatever cnt is.
  uint32_t ra, sh;
  lds_v2u32<0>(up, ra, sh);
  {
    uint32_t ra_n, sh_n;
    lds_v2u32<8>(up, ra_n, sh_n);
    vertical_row<SHIFT, true>(ra + g8, sh, wp, minus_two23, acc);
    ra = ra_n;
    sh = sh_n;
    up += 8;
    wp += 16;
  }
  while (up != up_end) {
    uint32_t ra_n, sh_n;
    lds_v2u32<8>(up, ra_n, sh_n);
    vertical_row<SHIFT, false>(ra + g8, sh, wp, minus_two23, acc);
    ra = ra_n;
    sh = sh_n;
    up += 8;
    wp += 16;
  }
}

// Channel reduction of one quantised pixel: 16.16 fixed point, truncating
// division, clamped (core::image::channel_reduction,
// mlx/data/core/image/ImageTransform.cpp:159-180).
__device__ __forceinline__ unsigned gray_mix(const LaunchParams& p, unsigned r, unsigned g, unsigned b) {
  int v = ((int)r * p.gray_m[0] + (int)g * p.gray_m[1] + (int)b * p.gray_m[2] + p.gray_bias) / 65536;
  v = v <= 255 ? v : 255;
  v = v >= 0 ? v : 0;
  return (unsigned)v;
}

// One output pixel's C floats; four-channel pixels go out as one 16-byte store
// when the destination allows it.
template <int C>
__device__ __forceinline__ void store_pixel(float* dst, const float (&v)[C], bool vec_ok) {
  if (C == 4 && vec_ok) {
    *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1 % C], v[2 % C], v[3 % C]);
  } else {
#pragma unroll
    for (int c = 0; c < C; c++) {
      dst[c] = v[c];
    }
  }
}

// Shared memory of a CTA, as shared-space byte addresses (32-bit: a struct of
// generic pointers would hold twice the registers across the pass loop).
// There are two sets of the tables that change from pass to pass (a pass = one
// run of output columns of the band), so the next pass's are built while the
// current pass is still filtering horizontally.  One set:
//   +0              int   hfirst[kTileW]
//   +256            int   hcount[kTileW]
//   +512            int2  urow[8][u_cap]  {shared address of the staged row's first word, funnel shift in bits}
//   +wh_off         float2 wh[kTileW][cap_x]  (w, w) pairs
struct Smem {
  unsigned lut;         // float [c][256]
  unsigned tab0;        // first table set
  unsigned tab_stride;  // bytes from one set to the next
  unsigned wh_off;
  unsigned uw;          // float4 [8][u_cap]  (w0,w0,w1,w1): weight of a union row in the two outputs of a row pair
  unsigned ucount;      // int [8]  rows in each row pair's union
  unsigned ufirst;      // int [8]  first (unclamped) source row of each row pair's union
  unsigned bar;
  unsigned mid;         // float4 [4][C][plane_slots]
  unsigned srct;
};

constexpr unsigned kTabHcount = kTileW * 4;
constexpr unsigned kTabUrow = kTileW * 8;

__host__ __device__ inline size_t align16(size_t v) {
  return (v + 15) & ~(size_t)15;
}

// Fills `out` with addresses relative to `base` (the shared-space address of
// the dynamic shared memory) and returns the bytes needed.
// The parts of it whose size depends on the sample.
struct Caps {
  int u_cap, weight_floats, mid_float4s, src_tile_bytes;
};

__host__ __device__ inline size_t smem_layout(int c_out, const Caps& p, unsigned base, Smem* out) {
  Smem sm;
  size_t off = 0;
  sm.lut = base + (unsigned)off;
  off += (size_t)c_out * 256 * sizeof(float);
  sm.tab0 = base + (unsigned)off;
  sm.wh_off = (unsigned)align16(kTabUrow + (size_t)8 * p.u_cap * sizeof(int2));
  sm.tab_stride = (unsigned)align16(sm.wh_off + (size_t)p.weight_floats * 2 * sizeof(float));
  off += 2 * (size_t)sm.tab_stride;
  sm.uw = base + (unsigned)off;
  off += (size_t)8 * p.u_cap * sizeof(float4);
  sm.ucount = base + (unsigned)off;
  off += 32;
  sm.ufirst = base + (unsigned)off;
  off += 32;
  sm.bar = base + (unsigned)off;
  off += 16;
  sm.mid = base + (unsigned)off;
  off = align16(off + (size_t)p.mid_float4s * 16);
  sm.srct = base + (unsigned)off;
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
  int wbytes, pitch_s, npairs, common;
  bool edge_x, shifted;
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
  // f0 .. l1 are columns of the window as the filter sees it; with a mirrored
  // source they are staged from the mirrored positions (the vertical pass does
  // not care, the horizontal pass walks the planes right to left)
  int alo = clampi(f0, 0, s.pre_w - 1);
  int chi = clampi(l1, 0, s.pre_w - 1);
  if (s.pre_flip) {
    const int t = alo;
    alo = s.pre_w - 1 - chi;
    chi = s.pre_w - 1 - t;
  }
  g.clo = alo;
  g.edge_x = f0 < 0 || l1 > s.pre_w - 1;
  g.ncols = chi - g.clo + 1;
  g.wbytes = g.ncols * C;
  g.g0 = s.src + ((size_t)(s.pre_y + rlo) * s.src_w + (s.pre_x + g.clo)) * C;
  // rows whose pitch is a multiple of 8 all start at the same offset within an
  // 8-byte unit, so a thread reads its two words with one aligned load; other
  // sources take the funnel-shift path from 4-byte units
  g.shifted = (((unsigned)s.src_w * C) & 7u) != 0;
  g.common = (int)(reinterpret_cast<uintptr_t>(g.g0) & (g.shifted ? 3 : 7));
  g.pitch_s = (g.wbytes + 15 + 15 + 4 + 15) & ~15;
  g.npairs = (g.common + g.wbytes + 7) >> 3;
  return g;
}

// Issue the bulk copies of a pass (threads < rows) and build its tables
// (the last kTileW threads the horizontal taps, all the staged-row addresses
// of the vertical unions).
template <int C>
__device__ __forceinline__ void start_pass(
    const DevSample& s, const LaunchParams& p, const Caps& caps, const Smem& sm, unsigned tab, const PassGeom& g,
    const Axis& ax, int nr, int rlo, int rows) {
  const int tid = threadIdx.x;
  const size_t src_pitch = (size_t)s.src_w * C;
  if (tid < rows) {
    const uintptr_t ga = reinterpret_cast<uintptr_t>(g.g0) + (size_t)tid * src_pitch;
    const int phase = (int)(ga & 15);
    const unsigned len = (unsigned)((phase + g.wbytes + 15) & ~15);
    mbar_expect_tx(sm.bar, len);
    bulk_copy(sm.srct + (unsigned)(tid * g.pitch_s), reinterpret_cast<const void*>(ga - phase), len, sm.bar);
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
      sp<int>(tab)[x] = lo;
      sp<int>(tab + kTabHcount)[x] = cnt;
      float2* w2 = sp<float2>(tab + sm.wh_off) + x * s.cap_x;
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
  // staged-row addresses: warp rp takes row pair rp (at most kTileH / 2 = 8 of them)
  const int nrp = (nr + 1) >> 1;
  const int rp = tid >> 5;
  if (rp < nrp) {
    const int cnt = sp<int>(sm.ucount)[rp];
    const int first = sp<int>(sm.ufirst)[rp];
    for (int e = tid & 31; e < cnt; e += 32) {
      const int sr = min(clampi(first + e, 0, s.pre_h - 1) - rlo, rows - 1);
      const int phase = (int)((reinterpret_cast<uintptr_t>(g.g0) + (size_t)sr * src_pitch) & 15);
      // aligned sources: boff is a multiple of 8 and the shift is unused
      const int boff = sr * g.pitch_s + phase - g.common;
      sp<int2>(tab + kTabUrow)[rp * caps.u_cap + e] =
          make_int2((int)(sm.srct + (unsigned)(boff & ~3)), (boff & 3) * 8);
    }
  }
}

// Geometric-output rows [by, by+nr) (nr <= kTileH) x columns [gx_lo, gx_hi) of
// a resize sample, sub_w columns per pass, written to the batch tensor.  The
// copies of pass t+1 are in flight while pass t filters horizontally.
template <int C, bool GRAY, bool U8>
__device__ void resize_rows(
    const DevSample& s, const LaunchParams& p, const Caps& caps, const Smem& sm, unsigned& parity, bool& first_use,
    int by, int nr, int gx_lo, int gx_hi) {
  constexpr int CO = GRAY ? 1 : C;   // channels of the batch tensor
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

  // ---- vertical union weights of every pair of output rows ------------------------
  const int nrp = (nr + 1) >> 1;
  for (int i = tid; i < nrp * caps.u_cap; i += kThreads) {
    const int rp = i / caps.u_cap;
    const int e = i - rp * caps.u_cap;
    const int o0 = by + rp * 2;
    const int on = min(2, nr - rp * 2);
    int lo[2], hi[2];
#pragma unroll
    for (int r = 0; r < 2; r++) {
      axis_range(ay, o0 + (r < on ? r : on - 1), lo[r], hi[r]);
    }
    const int ufirst = lo[0];
    const int ulast = hi[1];   // a missing second row repeats the first
    const int u = ufirst + e;
    if (e == 0) {
      int cnt = ulast - ufirst + 1;
      if (cnt > caps.u_cap) {
        cnt = caps.u_cap;
        atomicOr(p.status, 8);
      }
      sp<int>(sm.ucount)[rp] = cnt;
      sp<int>(sm.ufirst)[rp] = ufirst;
    }
    if (u <= ulast) {
      float w2[2];
#pragma unroll
      for (int r = 0; r < 2; r++) {
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
        w2[r] = w;
      }
      sp<float4>(sm.uw)[i] = make_float4(w2[0], w2[0], w2[1], w2[1]);
    }
  }
  __syncthreads();   // ucount is read by start_pass

  PassGeom cur = pass_geom<C>(s, ax, rlo, gx_lo, min(s.sub_w, gx_hi - gx_lo));
  if (rows * cur.pitch_s > caps.src_tile_bytes || ngroups * C * plane_slots<C>(cur.ncols) > caps.mid_float4s) {
    if (tid == 0) {
      atomicOr(p.status, 2);
    }
    return;
  }
  start_pass<C>(s, p, caps, sm, sm.tab0, cur, ax, nr, rlo, rows);
  if (p.starve_wait && tid == 0) {
    mbar_expect_tx(sm.bar, 16);   // test hook: bytes that never arrive, the wait below runs out
  }
  __syncthreads();
  if (tid == 0) {
    mbar_arrive(sm.bar);
  }

  float* base = reinterpret_cast<float*>(s.dst);
  const size_t row_stride = (size_t)s.slot_w * CO;
  const bool vec_ok = (reinterpret_cast<uintptr_t>(base) & 15) == 0;
  int it = 0;
  for (;;) {
    const unsigned tab = sm.tab0 + ((it & 1) ? sm.tab_stride : 0u);
    const unsigned tab_next = sm.tab0 + ((it & 1) ? 0u : sm.tab_stride);
    if (!mbar_wait(sm.bar, parity)) {
      atomicOr(p.status, 4);
    }
    parity ^= 1;

    // ---- vertical filter: thread = (eight byte columns, pair of output rows) --------
    {
      const unsigned urow_base = tab + kTabUrow;
      const unsigned uw_base = sm.uw;
      const int np = cur.npairs;
      const int pslots = plane_slots<C>(cur.ncols);
      const unsigned group_bytes = (unsigned)(C * pslots) * 16u;
      // Two ways to deal the (row pair, column octet) items out.  Blocked: a
      // quarter of the CTA per row pair, 64 octets per round - every warp works
      // on one row pair, so its table loads are broadcasts and the store offsets
      // serve every row pair.  Flat: one sequence over all items, which keeps
      // the warps full when the octet count is far from a multiple of 64.
      const int blocked_slots = ((np + 63) >> 6) * 64 * ((nrp + 3) >> 2) * 4;
      if (4 * np * nrp >= 3 * blocked_slots) {
        for (int g = tid & 63; g < np; g += 64) {
          const int j0 = 8 * g - cur.common;
          unsigned b0[C];
          int low[C];
          octet_offsets<C>(j0, pslots, b0, low);
          for (int rp = tid >> 6; rp < nrp; rp += kThreads >> 6) {
            const int cnt = sp<int>(sm.ucount)[rp];
            f32x2 acc[8];
            if (cur.shifted) {
              vertical_taps<true>(urow_base + rp * caps.u_cap * 8, uw_base + rp * caps.u_cap * 16, 8u * g, cnt, acc);
            } else {
              vertical_taps<false>(urow_base + rp * caps.u_cap * 8, uw_base + rp * caps.u_cap * 16, 8u * g, cnt, acc);
            }
            // the pair's rows are one half of a float4 of its group of four rows
            const unsigned pb = sm.mid + (unsigned)(rp >> 1) * group_bytes + (unsigned)(rp & 1) * 8u;
            unsigned b[C];
#pragma unroll
            for (int m = 0; m < C; m++) {
              b[m] = pb + b0[m];
            }
            store_octet<C>(b, low, acc);
          }
        }
      } else {
        const float inv_np = 1.0f / (float)np;
        for (int i = tid; i < np * nrp; i += kThreads) {
          int rp = (int)((float)i * inv_np);
          rp -= (rp * np > i) ? 1 : 0;
          rp += ((rp + 1) * np <= i) ? 1 : 0;
          const int g = i - rp * np;
          const int cnt = sp<int>(sm.ucount)[rp];
          f32x2 acc[8];
          if (cur.shifted) {
            vertical_taps<true>(urow_base + rp * caps.u_cap * 8, uw_base + rp * caps.u_cap * 16, 8u * g, cnt, acc);
          } else {
            vertical_taps<false>(urow_base + rp * caps.u_cap * 8, uw_base + rp * caps.u_cap * 16, 8u * g, cnt, acc);
          }
          const int j0 = 8 * g - cur.common;
          unsigned b[C];
          int low[C];
          octet_offsets<C>(j0, pslots, b, low);
          const unsigned pb = sm.mid + (unsigned)(rp >> 1) * group_bytes + (unsigned)(rp & 1) * 8u;
#pragma unroll
          for (int m = 0; m < C; m++) {
            b[m] += pb;
          }
          store_octet<C>(b, low, acc);
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
      if (rows * nxt.pitch_s > caps.src_tile_bytes || ngroups * C * plane_slots<C>(nxt.ncols) > caps.mid_float4s) {
        if (tid == 0) {
          atomicOr(p.status, 2);
        }
        return;
      }
      fence_async_smem();
      start_pass<C>(s, p, caps, sm, tab_next, nxt, ax, nr, rlo, rows);
    }

    // ---- horizontal filter: thread = (output column, group of four rows), all channels ----
    {
      const unsigned plane = (unsigned)plane_slots<C>(cur.ncols) * 16u;
      for (int item = tid; item < ngroups * cur.nc; item += kThreads) {
        int rg, x;
        if (cur.nc == kTileW) {
          rg = item / kTileW;
          x = item - rg * kTileW;
        } else {
          rg = item / cur.nc;
          x = item - rg * cur.nc;
        }
        const int f = (int)lds_u32<0>(tab + 4u * (unsigned)x);
        const int cnt = (int)lds_u32<kTabHcount>(tab + 4u * (unsigned)x);
        unsigned wq = tab + sm.wh_off + (unsigned)(x * s.cap_x) * 8u;
        const unsigned wq_end = wq + 8u * (unsigned)cnt;
        const unsigned col_a = sm.mid + (unsigned)(rg * C) * plane;
        f32x2 acc[C][2];   // per channel: rows 0,1 and rows 2,3 of the group
#pragma unroll
        for (int c = 0; c < C; c++) {
          acc[c][0] = 0;
          acc[c][1] = 0;
        }
        unsigned cb[C];   // the group's plane of every channel
#pragma unroll
        for (int c = 0; c < C; c++) {
          cb[c] = col_a + (unsigned)c * plane;
        }
        if (!cur.edge_x) {
          // two copies of the tap loop, so that the usual one keeps its constant step
          if (!s.pre_flip) {
            int col = PlanePad<C>::value + f - cur.clo;
            while (wq != wq_end) {
              const f32x2 wk = lds_u64<0>(wq);
              const unsigned off = (unsigned)skew(col) * 16u;
#pragma unroll
              for (int c = 0; c < C; c++) {
                f32x2 v01, v23;
                lds_v2u64<0>(cb[c] + off, v01, v23);
                ffma2(acc[c][0], v01, wk);
                ffma2(acc[c][1], v23, wk);
              }
              col++;
              wq += 8;
            }
          } else {
            int col = PlanePad<C>::value + (s.pre_w - 1 - f) - cur.clo;
            while (wq != wq_end) {
              const f32x2 wk = lds_u64<0>(wq);
              const unsigned off = (unsigned)skew(col) * 16u;
#pragma unroll
              for (int c = 0; c < C; c++) {
                f32x2 v01, v23;
                lds_v2u64<0>(cb[c] + off, v01, v23);
                ffma2(acc[c][0], v01, wk);
                ffma2(acc[c][1], v23, wk);
              }
              col--;
              wq += 8;
            }
          }
        } else {
          for (int k = 0; wq != wq_end; k++) {
            const f32x2 wk = lds_u64<0>(wq);
            const int seen = clampi(f + k, 0, s.pre_w - 1);
            const unsigned off =
                (unsigned)skew(PlanePad<C>::value + (s.pre_flip ? s.pre_w - 1 - seen : seen) - cur.clo) * 16u;
#pragma unroll
            for (int c = 0; c < C; c++) {
              f32x2 v01, v23;
              lds_v2u64<0>(cb[c] + off, v01, v23);
              ffma2(acc[c][0], v01, wk);
              ffma2(acc[c][1], v23, wk);
            }
            wq += 8;
          }
        }
        int px = cur.bx + x - s.post_x;
        if (s.post_flip) {
          px = s.post_w - 1 - px;
        }
        const int oy = by + rg * 4 - s.post_y;
        const int left = nr - rg * 4;
        if (U8) {
          // uint8 batch: the quantised pixel (or its channel reduction) as it is
          unsigned q[4][C];
#pragma unroll
          for (int c = 0; c < C; c++) {
            float a0, a1, a2, a3;
            unpack2(acc[c][0], a0, a1);
            unpack2(acc[c][1], a2, a3);
            q[0][c] = quantise_sat(a0);
            q[1][c] = quantise_sat(a1);
            q[2][c] = quantise_sat(a2);
            q[3][c] = quantise_sat(a3);
          }
          uint8_t* dst8 = reinterpret_cast<uint8_t*>(s.dst) + ((size_t)oy * s.slot_w + px) * CO;
#pragma unroll
          for (int r = 0; r < 4; r++) {
            if (r < left) {
              if (GRAY) {
                dst8[r * row_stride] = (uint8_t)gray_mix(p, q[r][0], q[r][1 % C], q[r][2 % C]);
              } else {
#pragma unroll
                for (int c = 0; c < C; c++) {
                  dst8[r * row_stride + c] = (uint8_t)q[r][c];
                }
              }
            }
          }
        } else {
        float* dst = base + ((size_t)oy * s.slot_w + px) * CO;
        float out[4][CO];
        if (GRAY) {
          // the resized pixel is quantised first, as the image the reference hands
          // to its channel reduction is; then the fixed-point mix, then the cast
          unsigned q[4][C];
#pragma unroll
          for (int c = 0; c < C; c++) {
            float a0, a1, a2, a3;
            unpack2(acc[c][0], a0, a1);
            unpack2(acc[c][1], a2, a3);
            q[0][c] = quantise_sat(a0);
            q[1][c] = quantise_sat(a1);
            q[2][c] = quantise_sat(a2);
            q[3][c] = quantise_sat(a3);
          }
#pragma unroll
          for (int r = 0; r < 4; r++) {
            out[r][0] = __uint_as_float(lds_u32<0>(sm.lut + 4u * gray_mix(p, q[r][0], q[r][1 % C], q[r][2 % C])));
          }
        } else {
#pragma unroll
          for (int c = 0; c < C; c++) {
            float a0, a1, a2, a3;
            unpack2(acc[c][0], a0, a1);
            unpack2(acc[c][1], a2, a3);
            const unsigned lut = sm.lut + (unsigned)c * 1024u;
            out[0][c % CO] = __uint_as_float(lds_u32<0>(lut + 4u * quantise_sat(a0)));
            out[1][c % CO] = __uint_as_float(lds_u32<0>(lut + 4u * quantise_sat(a1)));
            out[2][c % CO] = __uint_as_float(lds_u32<0>(lut + 4u * quantise_sat(a2)));
            out[3][c % CO] = __uint_as_float(lds_u32<0>(lut + 4u * quantise_sat(a3)));
          }
        }
#pragma unroll
        for (int r = 0; r < 4; r++) {
          if (r < left) {
            store_pixel<CO>(dst + r * row_stride, out[r], vec_ok);
          }
        }
        }
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

// Source pixel of post-window pixel (px, y) of an affine sample: coordinates in
// the pre window, or false when it falls outside it (the output is 0 there).
// The coordinate is built from float products and float sums, then two double
// additions, then truncation toward zero - the evaluation order of the
// reference expression - and no multiply-add is contracted.
__device__ __forceinline__ bool affine_source(
    const DevSample& s, int gx, int gy, float twh, float thh, float wh, float hh, int& sx, int& sy) {
  const float dxf = __fsub_rn((float)(long long)gx, twh);
  const float dyf = __fsub_rn((float)(long long)gy, thh);
  const float fx = __fadd_rn(__fadd_rn(__fmul_rn(s.mx[0], dxf), __fmul_rn(s.mx[1], dyf)), s.mx[2]);
  const float fy = __fadd_rn(__fadd_rn(__fmul_rn(s.mx[3], dxf), __fmul_rn(s.mx[4], dyf)), s.mx[5]);
  const long long ax = (long long)__dadd_rn(__dadd_rn((double)fx, 0.5), (double)wh);
  const long long ay = (long long)__dadd_rn(__dadd_rn((double)fy, 0.5), (double)hh);
  sx = (int)ax;
  sy = (int)ay;
  return !(ax < 0 || ay < 0 || ax >= s.pre_w || ay >= s.pre_h);
}

// Copy (crop / flip / batch only) and nearest-neighbour affine tiles: rows
// [y0, vy1) x columns [xa, xb) of the slot, a thread takes four adjacent pixels
// of a row.  The cast table is read from shared memory (lut_s); the four pixels
// leave as 16-byte stores when the row segment allows it.  Without a geometric
// op the four source pixels are adjacent too and come as aligned words.
template <int C, bool GRAY, bool U8>
__device__ void gather_rows(
    const DevSample& s, const LaunchParams& p, unsigned lut_s, int y0, int vy1, int xa, int xb) {
  constexpr int CO = GRAY ? 1 : C;
  const int nvx = xb - xa;
  const int nvy = vy1 - y0;
  const int quads = (nvx + 3) >> 2;
  float* base = reinterpret_cast<float*>(s.dst);
  const float twh = (float)((double)s.geom_w / 2.0);
  const float thh = (float)((double)s.geom_h / 2.0);
  const float wh = (float)((double)s.pre_w / 2.0);
  const float hh = (float)((double)s.pre_h / 2.0);
  const size_t row_floats = (size_t)s.slot_w * CO;
  const bool vec_ok = (row_floats & 3) == 0 && ((xa * CO) & 3) == 0 && (reinterpret_cast<uintptr_t>(base) & 15) == 0;
  // last 4-byte word of the source image: nothing behind it is read
  const uintptr_t last_word = (reinterpret_cast<uintptr_t>(s.src) + (size_t)s.src_h * s.src_w * C - 1) & ~(uintptr_t)3;
  for (int i = threadIdx.x; i < nvy * quads; i += kThreads) {
    const int ry = i / quads;
    const int q = i - ry * quads;
    const int x_first = xa + 4 * q;
    const int npx = min(4, xb - x_first);
    const int gy = s.post_y + y0 + ry;
    unsigned px[4][C];   // source bytes of the four pixels
    if (s.mode == kModeAffine) {
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const int x = x_first + (j < npx ? j : 0);
        const int gx = s.post_x + (s.post_flip ? (s.post_w - 1 - x) : x);
        int sx, sy;
        const bool inside = affine_source(s, gx, gy, twh, thh, wh, hh, sx, sy);
        const int ix = s.pre_x + (s.pre_flip ? (s.pre_w - 1 - sx) : sx);
        // the pixel's C bytes from the one or two aligned words that hold them
        const uintptr_t g = reinterpret_cast<uintptr_t>(s.src) + ((size_t)(s.pre_y + sy) * s.src_w + ix) * C;
        const uint32_t* w = reinterpret_cast<const uint32_t*>(g & ~(uintptr_t)3);
        const unsigned sh = (unsigned)(g & 3) * 8u;
        const uint32_t w0 = inside ? __ldg(w) : 0u;
        const uint32_t w1 = (inside && (int)(g & 3) + C > 4) ? __ldg(w + 1) : 0u;
        const uint32_t v = __funnelshift_r(w0, w1, sh);
#pragma unroll
        for (int ch = 0; ch < C; ch++) {
          px[j][ch] = (v >> (8 * ch)) & 0xffu;
        }
      }
    } else {
      // pre_flip is folded into post_flip for copies: the source pixels of columns
      // x_first .. x_first + 3 are adjacent, ascending or (mirrored) descending
      const int gx_a = s.post_x + (s.post_flip ? (s.post_w - 1 - x_first) : x_first);
      const int sx_lo = s.pre_x + (s.post_flip ? gx_a - (npx - 1) : gx_a);
      const uintptr_t g =
          reinterpret_cast<uintptr_t>(s.src) + ((size_t)(s.pre_y + gy) * s.src_w + sx_lo) * C;
      const uint32_t* w = reinterpret_cast<const uint32_t*>(g & ~(uintptr_t)3);
      const unsigned sh = (unsigned)(g & 3) * 8u;
      const int need = (int)(g & 3) + npx * C;   // bytes from the first word on
      uint32_t x[C + 1];
#pragma unroll
      for (int k = 0; k < C + 1; k++) {
        const bool take = 4 * k < need && reinterpret_cast<uintptr_t>(w + k) <= last_word;
        x[k] = take ? __ldg(w + k) : 0u;
      }
      uint32_t v[C];   // the 4 * C bytes from g on
#pragma unroll
      for (int k = 0; k < C; k++) {
        v[k] = __funnelshift_r(x[k], x[k + 1], sh);
      }
#pragma unroll
      for (int j = 0; j < 4; j++) {
#pragma unroll
        for (int ch = 0; ch < C; ch++) {
          const int byte = j * C + ch;
          const unsigned val = (v[byte >> 2] >> (8 * (byte & 3))) & 0xffu;
          // mirrored: source pixel j is output pixel npx - 1 - j
          if (!s.post_flip) {
            px[j][ch] = val;
          } else {
#pragma unroll
            for (int o = 0; o < 4; o++) {
              if (o == npx - 1 - j) {
                px[o][ch] = val;
              }
            }
          }
        }
      }
    }
    if (U8) {
      // uint8 batch: the 4 * CO bytes as CO aligned words when the row segment allows it
      unsigned by[4 * CO];
#pragma unroll
      for (int j = 0; j < 4; j++) {
        if (GRAY) {
          by[j] = gray_mix(p, px[j][0], px[j][1 % C], px[j][2 % C]);
        } else {
#pragma unroll
          for (int ch = 0; ch < C; ch++) {
            by[(j * CO + ch) % (4 * CO)] = px[j][ch];
          }
        }
      }
      uint8_t* dst8 = reinterpret_cast<uint8_t*>(s.dst) + ((size_t)(y0 + ry) * s.slot_w + x_first) * CO;
      if (npx == 4 && (reinterpret_cast<uintptr_t>(dst8) & 3) == 0) {
#pragma unroll
        for (int k = 0; k < CO; k++) {
          reinterpret_cast<uint32_t*>(dst8)[k] =
              by[4 * k] | (by[4 * k + 1] << 8) | (by[4 * k + 2] << 16) | (by[4 * k + 3] << 24);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 4; j++) {
          if (j < npx) {
#pragma unroll
            for (int ch = 0; ch < CO; ch++) {
              dst8[j * CO + ch] = (uint8_t)by[j * CO + ch];
            }
          }
        }
      }
    } else {
    float out[4][CO];
#pragma unroll
    for (int j = 0; j < 4; j++) {
      if (GRAY) {
        out[j][0] = __uint_as_float(lds_u32<0>(lut_s + 4u * gray_mix(p, px[j][0], px[j][1 % C], px[j][2 % C])));
      } else {
#pragma unroll
        for (int ch = 0; ch < C; ch++) {
          out[j][ch % CO] = __uint_as_float(lds_u32<0>(lut_s + (unsigned)ch * 1024u + 4u * px[j][ch]));
        }
      }
    }
    float* dst = base + ((size_t)(y0 + ry) * s.slot_w + x_first) * CO;
    if (vec_ok && npx == 4) {
      const float* o = &out[0][0];
#pragma unroll
      for (int k = 0; k < CO; k++) {
        reinterpret_cast<float4*>(dst)[k] = make_float4(o[4 * k], o[4 * k + 1], o[4 * k + 2], o[4 * k + 3]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; j++) {
        if (j < npx) {
#pragma unroll
          for (int ch = 0; ch < CO; ch++) {
            dst[j * CO + ch] = out[j][ch];
          }
        }
      }
    }
    }
  }
}

// One CTA: rows [y0, y0 + kTileH) of one slot, columns of p.band_tiles tiles.
template <int C, bool GRAY, bool U8>
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
  constexpr int CO = GRAY ? 1 : C;
  float padf[4];
#pragma unroll
  for (int c = 0; c < 4; c++) {
    padf[c] = (!U8 && c < CO) ? __ldg(p.lut + c * 256 + p.pad_px) : 0.0f;
  }
  float* out = reinterpret_cast<float*>(s.dst);
  // pad value into a rectangle of the slot, float32 or uint8
  auto pad_rect = [&](int ya, int yb, int xa, int xb) {
    if (U8) {
      fill_rect_u8<CO>(reinterpret_cast<uint8_t*>(s.dst), s.slot_w, ya, yb, xa, xb, p.pad_px);
    } else {
      fill_rect_f32<CO>(out, s.slot_w, ya, yb, xa, xb, padf);
    }
  };
  if (!has_valid) {
    // bands below the post window are pad_fill_kernel's when it runs
    if (!(p.pad_apart && y0 >= s.post_h)) {
      pad_rect(y0, y1, x0, x1);
    }
    return;
  }
  // a resize sample lays the CTA's shared memory out from its own needs
  Caps caps;
  caps.u_cap = s.need_wts_ucap >> 16;
  caps.weight_floats = s.need_wts_ucap & 0xffff;
  caps.mid_float4s = s.need_mid4;
  caps.src_tile_bytes = s.need_src;
  Smem sm;
  smem_layout(p.c_out, caps, smem_addr(smem_raw), &sm);
  if (!U8) {
    for (int i = threadIdx.x; i < CO * 256; i += kThreads) {
      sp<float>(sm.lut)[i] = __ldg(p.lut + i);
    }
  }
  if (s.mode == kModeResize) {
    if (threadIdx.x == 0) {
      mbar_init(sm.bar, 1);
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
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
      resize_rows<C, GRAY, U8>(s, p, caps, sm, parity, first_use, by, min(s.sub_h, s.post_y + vy1 - by), gx_lo, gx_hi);
    }
  } else if (s.mode != kModeResizeDirect) {
    __syncthreads();
    gather_rows<C, GRAY, U8>(s, p, sm.lut, y0, vy1, x0, vx1);
  }
  // (the post window of a kModeResizeDirect sample is resize_direct_kernel's)
  // pad the part of the band outside the post window
  pad_rect(vy1, y1, x0, x1);
  pad_rect(y0, vy1, vx1, x1);
}

__global__ void __launch_bounds__(kThreads, 3) fused_fast_kernel(const LaunchParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  if (p.c_in == 3) {
    run_band<3, false, false>(p, smem_raw);
  } else if (p.c_in == 1) {
    run_band<1, false, false>(p, smem_raw);
  } else {
    run_band<4, false, false>(p, smem_raw);
  }
}

// Two-channel images, float32 batches.  Rare; kept out of the kernel above so
// that its register allocation is decided by the common cases alone.
__global__ void __launch_bounds__(kThreads, 3) fused_fast_c2_kernel(const LaunchParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  run_band<2, false, false>(p, smem_raw);
}

// uint8 batches (no cast): stand-alone ops, images between two geometric ops,
// pipelines that cast on the host.  Kernels of their own for the same reason
// as the channel-reduction one.
__global__ void __launch_bounds__(kThreads, 3) fused_fast_u8_kernel(const LaunchParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  if (p.c_in == 3) {
    if (p.gray) {
      run_band<3, true, true>(p, smem_raw);
    } else {
      run_band<3, false, true>(p, smem_raw);
    }
  } else if (p.c_in == 1) {
    run_band<1, false, true>(p, smem_raw);
  } else if (p.c_in == 2) {
    run_band<2, false, true>(p, smem_raw);
  } else {
    run_band<4, false, true>(p, smem_raw);
  }
}

// The padding below a sample of a ragged batch.  Rows of a slot are contiguous,
// so everything from the first row band that holds no row of the sample's post
// window down to the end of the slot is one contiguous run of floats: written
// here as a linear fill (16-byte stores, consecutive threads on consecutive
// addresses, kPadChunks CTAs per sample), which runs at memory speed - the
// band kernels above, writing 16-row strips, reach about 60 % of that.  The
// strips to the right of the post window stay with the band kernels.
constexpr int kPadChunks = 128;

template <int CO>
__device__ __forceinline__ void pad_below(const LaunchParams& p) {
  const int n = blockIdx.x / kPadChunks;
  const int chunk = blockIdx.x - n * kPadChunks;
  if (n >= p.n) {
    return;
  }
  const DevSample* s = p.samples + n;
  const int slot_h = s->slot_h, slot_w = s->slot_w;
  const int post_h = s->post_h < slot_h ? s->post_h : slot_h;
  const int first_row = ((post_h + kTileH - 1) / kTileH) * kTileH;   // first row of the first band without a valid row
  if (first_row >= slot_h) {
    return;
  }
  float padf[4];
#pragma unroll
  for (int c = 0; c < 4; c++) {
    padf[c] = c < CO ? __ldg(p.lut + c * 256 + p.pad_px) : 0.0f;
  }
  const size_t row_floats = (size_t)slot_w * CO;
  float* run = reinterpret_cast<float*>(s->dst) + (size_t)first_row * row_floats;   // starts on a pixel: channel 0
  const size_t len = (size_t)(slot_h - first_row) * row_floats;
  const size_t mis = (reinterpret_cast<uintptr_t>(run) >> 2) & 3;
  size_t head = (4 - mis) & 3;
  head = head > len ? len : head;
  const size_t nvec = (len - head) >> 2;
  // this CTA's share of the aligned units
  const size_t q0 = nvec * (size_t)chunk / kPadChunks;
  const size_t q1 = nvec * (size_t)(chunk + 1) / kPadChunks;
  for (size_t q = q0 + threadIdx.x; q < q1; q += kThreads) {
    const size_t j = head + 4 * q;
    const int m = (int)(j % CO);
    *reinterpret_cast<float4*>(run + j) = make_float4(
        pad_pick<CO>(padf, m), pad_pick<CO>(padf, (m + 1) % CO), pad_pick<CO>(padf, (m + 2) % CO),
        pad_pick<CO>(padf, (m + 3) % CO));
  }
  if (chunk == 0) {
    // the floats before the first and after the last aligned unit
    const size_t tail = head + 4 * nvec;
    for (size_t k = threadIdx.x; k < head + (len - tail); k += kThreads) {
      const size_t j = k < head ? k : tail + (k - head);
      run[j] = pad_pick<CO>(padf, (int)(j % CO));
    }
  }
}

// The same for a uint8 batch: a linear fill of bytes.
__device__ __forceinline__ void pad_below_u8(const LaunchParams& p) {
  const int n = blockIdx.x / kPadChunks;
  const int chunk = blockIdx.x - n * kPadChunks;
  if (n >= p.n) {
    return;
  }
  const DevSample* s = p.samples + n;
  const int slot_h = s->slot_h, slot_w = s->slot_w;
  const int post_h = s->post_h < slot_h ? s->post_h : slot_h;
  const int first_row = ((post_h + kTileH - 1) / kTileH) * kTileH;
  if (first_row >= slot_h) {
    return;
  }
  const size_t row_bytes = (size_t)slot_w * p.c_out;
  uint8_t* run = reinterpret_cast<uint8_t*>(s->dst) + (size_t)first_row * row_bytes;
  const size_t len = (size_t)(slot_h - first_row) * row_bytes;
  const size_t mis = reinterpret_cast<uintptr_t>(run) & 15;
  size_t head = (16 - mis) & 15;
  head = head > len ? len : head;
  const size_t nvec = (len - head) >> 4;
  const unsigned w = (unsigned)(p.pad_px & 0xff) * 0x01010101u;
  const uint4 v = make_uint4(w, w, w, w);
  const size_t q0 = nvec * (size_t)chunk / kPadChunks;
  const size_t q1 = nvec * (size_t)(chunk + 1) / kPadChunks;
  for (size_t q = q0 + threadIdx.x; q < q1; q += kThreads) {
    *reinterpret_cast<uint4*>(run + head + 16 * q) = v;
  }
  if (chunk == 0) {
    const size_t tail = head + 16 * nvec;
    for (size_t k = threadIdx.x; k < head + (len - tail); k += kThreads) {
      run[k < head ? k : tail + (k - head)] = (uint8_t)p.pad_px;
    }
  }
}

__global__ void __launch_bounds__(kThreads, 6) pad_fill_kernel(const LaunchParams p) {
  if (!p.out_f32) {
    pad_below_u8(p);
    return;
  }
  if (p.c_out == 3) {
    pad_below<3>(p);
  } else if (p.c_out == 1) {
    pad_below<1>(p);
  } else if (p.c_out == 2) {
    pad_below<2>(p);
  } else {
    pad_below<4>(p);
  }
}

// Launches that end in the channel reduction: three channels in, one out.  A
// kernel of its own, so that the usual one's register allocation is not touched.
__global__ void __launch_bounds__(kThreads, 3) fused_fast_gray_kernel(const LaunchParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  run_band<3, true, false>(p, smem_raw);
}

} // namespace

// ---- resizes whose taps do not fit the on-chip passes ---------------------------------
//
// One thread per pixel of the post window, every tap read from global memory.
// The arithmetic is that of the band kernel, value by value: per source column
// the vertical sum (first tap a product, then multiply-adds in tap order, taps
// outside the window reading the clamped row), then the horizontal
// multiply-adds over those sums in tap order onto zero, weights tent / sum
// with the sum taken in tap order.  Such samples are rare and small on the
// output side (a shrink ratio of 60 or more), so nothing is staged or shared.
template <int C>
__device__ void direct_pixel(const DevSample& s, const LaunchParams& p, int ox, int oy) {
  const Axis ay = make_axis(s.pre_h, s.geom_h);
  const Axis ax = make_axis(s.pre_w, s.geom_w);
  const int gy = s.post_y + oy;
  const int gx = s.post_x + (s.post_flip ? s.post_w - 1 - ox : ox);
  int ylo, yhi, xlo, xhi;
  axis_range(ay, gy, ylo, yhi);
  axis_range(ax, gx, xlo, xhi);
  const int cy = yhi - ylo + 1;
  int cx = xhi - xlo + 1;
  cx = cx > s.cap_x ? s.cap_x : cx;
  const float uy = axis_center(ay, gy);
  const float ux = axis_center(ax, gx);
  float sum_y = 0.0f, sum_x = 0.0f;
  if (!ay.identity) {
    for (int k = 0; k < cy; k++) {
      sum_y = __fadd_rn(sum_y, axis_tent(ay, uy, ylo + k));
    }
  }
  if (!ax.identity) {
    for (int j = 0; j < cx; j++) {
      sum_x = __fadd_rn(sum_x, axis_tent(ax, ux, xlo + j));
    }
  }
  float acc_h[C];
#pragma unroll
  for (int c = 0; c < C; c++) {
    acc_h[c] = 0.0f;
  }
  for (int j = 0; j < cx; j++) {
    const float wx = ax.identity ? 1.0f : __fdiv_rn(axis_tent(ax, ux, xlo + j), sum_x);
    const int seen = clampi(xlo + j, 0, s.pre_w - 1);
    const int col = s.pre_x + (s.pre_flip ? s.pre_w - 1 - seen : seen);
    float acc_v[C];
#pragma unroll
    for (int c = 0; c < C; c++) {
      acc_v[c] = 0.0f;
    }
    for (int k = 0; k < cy; k++) {
      const float wy = ay.identity ? 1.0f : __fdiv_rn(axis_tent(ay, uy, ylo + k), sum_y);
      const int row = s.pre_y + clampi(ylo + k, 0, s.pre_h - 1);
      const uint8_t* px = s.src + ((size_t)row * s.src_w + col) * C;
#pragma unroll
      for (int c = 0; c < C; c++) {
        const float v = (float)__ldg(px + c);
        acc_v[c] = k == 0 ? __fmul_rn(v, wy) : __fmaf_rn(v, wy, acc_v[c]);
      }
    }
#pragma unroll
    for (int c = 0; c < C; c++) {
      acc_h[c] = __fmaf_rn(acc_v[c], wx, acc_h[c]);
    }
  }
  unsigned q[C];
#pragma unroll
  for (int c = 0; c < C; c++) {
    q[c] = quantise_sat(acc_h[c]);
  }
  const size_t at = (size_t)oy * s.slot_w + ox;
  if (p.gray) {
    const unsigned g = gray_mix(p, q[0], q[1 % C], q[2 % C]);
    if (p.out_f32) {
      reinterpret_cast<float*>(s.dst)[at] = __ldg(p.lut + g);
    } else {
      reinterpret_cast<uint8_t*>(s.dst)[at] = (uint8_t)g;
    }
  } else {
#pragma unroll
    for (int c = 0; c < C; c++) {
      if (p.out_f32) {
        reinterpret_cast<float*>(s.dst)[at * C + c] = __ldg(p.lut + c * 256 + q[c]);
      } else {
        reinterpret_cast<uint8_t*>(s.dst)[at * C + c] = (uint8_t)q[c];
      }
    }
  }
}

constexpr int kDirectChunks = 64;   // CTAs per sample

__global__ void __launch_bounds__(kThreads) resize_direct_kernel(const LaunchParams p) {
  const DevSample& s = p.samples[blockIdx.y];
  if (s.mode != kModeResizeDirect) {
    return;
  }
  const int vh = s.post_h < s.slot_h ? s.post_h : s.slot_h;
  const int vw = s.post_w < s.slot_w ? s.post_w : s.slot_w;
  const long long count = (long long)vh * vw;
  for (long long i = (long long)blockIdx.x * kThreads + threadIdx.x; i < count; i += (long long)kDirectChunks * kThreads) {
    const int oy = (int)(i / vw);
    const int ox = (int)(i - (long long)oy * vw);
    if (p.c_in == 3) {
      direct_pixel<3>(s, p, ox, oy);
    } else if (p.c_in == 1) {
      direct_pixel<1>(s, p, ox, oy);
    } else if (p.c_in == 2) {
      direct_pixel<2>(s, p, ox, oy);
    } else {
      direct_pixel<4>(s, p, ox, oy);
    }
  }
}

size_t fused_fast_layout_bytes(int c_out, int u_cap, int weight_floats, int mid_float4s, int src_tile_bytes) {
  const Caps caps{u_cap, weight_floats, mid_float4s, src_tile_bytes};
  return smem_layout(c_out, caps, 0u, nullptr);   // without a resize only the cast table
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
    const int most = (int)fused_fast_layout_bytes(4, kMaxStagedRows, kWeightFloats, kMidFloats / 4, kSrcTileBytes);
    e = cudaFuncSetAttribute(fused_fast_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
    if (e != cudaSuccess) {
      return e;
    }
    e = cudaFuncSetAttribute(fused_fast_gray_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
    if (e != cudaSuccess) {
      return e;
    }
    e = cudaFuncSetAttribute(fused_fast_u8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
    if (e != cudaSuccess) {
      return e;
    }
    e = cudaFuncSetAttribute(fused_fast_c2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
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
  // sized by the planner: the largest layout any one sample of the launch needs
  const size_t smem = p.fast_smem_bytes > 0 ? (size_t)p.fast_smem_bytes : fused_fast_layout_bytes(p.c_out, 0, 0, 0, 0);
  if (p.pad_apart) {
    pad_fill_kernel<<<(unsigned)p.n * kPadChunks, kThreads, 0, stream>>>(p);
    const cudaError_t pe = cudaGetLastError();
    if (pe != cudaSuccess) {
      return pe;
    }
  }
  if (!p.out_f32) {
    fused_fast_u8_kernel<<<(unsigned)blocks, kThreads, smem, stream>>>(p);
  } else if (p.c_in == 2) {
    fused_fast_c2_kernel<<<(unsigned)blocks, kThreads, smem, stream>>>(p);
  } else if (p.gray) {
    fused_fast_gray_kernel<<<(unsigned)blocks, kThreads, smem, stream>>>(p);
  } else {
    fused_fast_kernel<<<(unsigned)blocks, kThreads, smem, stream>>>(p);
  }
  if (p.direct) {
    const cudaError_t be = cudaGetLastError();
    if (be != cudaSuccess) {
      return be;
    }
    resize_direct_kernel<<<dim3(kDirectChunks, (unsigned)p.n), kThreads, 0, stream>>>(p);
  }
  return cudaGetLastError();
}

} // namespace mlxd
