#include "mlx/data/core/image/Jpeg.h"

#include <cstring>
#include <vector>

namespace mlx {
namespace data {
namespace core {
namespace image {

namespace {

// Position of the k-th coefficient of the zigzag sequence in an 8 x 8 block.
const unsigned char kZigzag[64] = {0,  1,  8,  16, 9,  2,  3,  10, 17, 24, 32, 25, 18, 11, 4,  5,  12, 19, 26, 33, 40, 48,
                                   41, 34, 27, 20, 13, 6,  7,  14, 21, 28, 35, 42, 49, 56, 57, 50, 43, 36, 29, 22, 15, 23,
                                   30, 37, 44, 51, 58, 59, 52, 45, 38, 31, 39, 46, 53, 60, 61, 54, 47, 55, 62, 63};

struct Huffman {
  bool present = false;
  unsigned char values[256];
  int mincode[17], maxcode[18], valptr[17];
  // codes of at most kLook bits, by their first kLook bits: length << 8 | value, 0 for longer codes
  static constexpr int kLook = 9;
  uint16_t look[1 << kLook];
  // AC tables: when a code and the value bits after it fit in kLook bits, the
  // decoded step at once: value << 8 | zero run << 4 | bits used; 0 otherwise
  int16_t step[1 << kLook];

  // bits[l] = number of codes of length l (1..16), values in code order
  bool build(const unsigned char* bits, const unsigned char* vals, int count) {
    std::memcpy(values, vals, count);
    int code = 0, k = 0;
    for (int l = 1; l <= 16; l++) {
      valptr[l] = k;
      mincode[l] = code;
      code += bits[l];
      k += bits[l];
      maxcode[l] = bits[l] ? code - 1 : -1;
      if (code > (1 << l)) {
        return false;
      }
      code <<= 1;
    }
    maxcode[17] = 0x7fffffff;
    std::memset(look, 0, sizeof(look));
    for (int l = 1; l <= kLook; l++) {
      for (int i = 0; i < bits[l]; i++) {
        const int c = mincode[l] + i;
        const int first = c << (kLook - l);
        for (int fill = 0; fill < (1 << (kLook - l)); fill++) {
          look[first + fill] = static_cast<uint16_t>(l << 8 | values[valptr[l] + i]);
        }
      }
    }
    for (int i = 0; i < (1 << kLook); i++) {
      step[i] = 0;
      const int l = look[i] >> 8, rs = look[i] & 0xff, size = rs & 15;
      if (l && size && l + size <= kLook) {
        int v = (i >> (kLook - l - size)) & ((1 << size) - 1);
        if (v < (1 << (size - 1))) {
          v -= (1 << size) - 1;
        }
        if (v >= -128 && v <= 127) {
          step[i] = static_cast<int16_t>(v * 256 + (rs >> 4) * 16 + l + size);
        }
      }
    }
    present = true;
    return true;
  }
};

struct Component {
  int id = 0, h = 1, v = 1, tq = 0;
  int td = 0, ta = 0;        // tables of the current scan
  int blocks_w = 0, blocks_h = 0;   // padded to whole MCUs
  int64_t dw = 0, dh = 0;    // true size of the (possibly subsampled) plane
  int pred = 0;
  std::vector<unsigned char> plane;   // [blocks_h * 8][blocks_w * 8]
  std::vector<int> coef;              // progressive frames: [blocks_h * blocks_w][64], kept across scans
};

// Entropy-coded segment reader: bytes with FF 00 unstuffed; a marker ends the
// data (further bits read as zero, the way a truncated file is padded).
struct Bits {
  const unsigned char* data;
  size_t size, pos;
  uint64_t acc = 0;   // the next bits, left-aligned; the top `count` of them are valid
  int count = 0;
  bool hit_marker = false;

  void fill() {
    // eight bytes at once when none of them is FF (no stuffing, no marker)
    if (!hit_marker && pos + 8 <= size) {
      uint64_t v = 0;
      for (int i = 0; i < 8; i++) {
        v = v << 8 | data[pos + i];
      }
      const uint64_t x = ~v;
      if (((x - 0x0101010101010101ULL) & ~x & 0x8080808080808080ULL) == 0) {
        const int bytes = (64 - count) >> 3;
        if (bytes > 0) {
          const uint64_t chunk = bytes == 8 ? v : v & ~((uint64_t(1) << (64 - 8 * bytes)) - 1);
          acc |= chunk >> count;
          count += 8 * bytes;
          pos += bytes;
        }
        return;
      }
    }
    while (count <= 56) {
      uint64_t b = 0;
      if (!hit_marker && pos < size) {
        b = data[pos];
        if (b == 0xff) {
          const unsigned next = pos + 1 < size ? data[pos + 1] : 0xd9;
          if (next == 0) {
            pos += 2;
          } else {
            hit_marker = true;
            b = 0;
          }
        } else {
          pos++;
        }
      }
      acc |= b << (56 - count);
      count += 8;
    }
  }
  int get(int n) {
    if (n == 0) {
      return 0;
    }
    if (count < n) {
      fill();
    }
    const int v = static_cast<int>(acc >> (64 - n));
    acc <<= n;
    count -= n;
    return v;
  }
  int peek(int n) {
    if (count < n) {
      fill();
    }
    return static_cast<int>(acc >> (64 - n));
  }
  void skip(int n) {
    acc <<= n;
    count -= n;
  }
  void restart() {
    acc = 0;
    count = 0;
    hit_marker = false;
  }
};

int decode_symbol(Bits& b, const Huffman& t) {
  const unsigned hit = t.look[b.peek(Huffman::kLook)];
  if (hit) {
    b.skip(hit >> 8);
    return hit & 0xff;
  }
  int code = b.get(Huffman::kLook);
  for (int l = Huffman::kLook + 1; l <= 16; l++) {
    code = (code << 1) | b.get(1);
    if (t.maxcode[l] >= 0 && code <= t.maxcode[l] && code >= t.mincode[l]) {
      return t.values[t.valptr[l] + code - t.mincode[l]];
    }
  }
  return -1;
}

int extend(int v, int bits) {
  return v < (1 << (bits - 1)) ? v - (1 << bits) + 1 : v;
}

// ---- inverse DCT: Loeffler-Ligtenberg-Moschytz, 13-bit constants, two passes ----
constexpr int kConstBits = 13, kPass1Bits = 2;
constexpr int64_t F0_298 = 2446, F0_390 = 3196, F0_541 = 4433, F0_765 = 6270, F0_899 = 7373, F1_175 = 9633,
                  F1_501 = 12299, F1_847 = 15137, F1_961 = 16069, F2_053 = 16819, F2_562 = 20995, F3_072 = 25172;

inline int64_t descale(int64_t x, int n) {
  return (x + (int64_t(1) << (n - 1))) >> n;
}

inline void idct_1d(const int64_t in[8], int64_t out[8], int shift) {
  // even part
  int64_t z2 = in[2], z3 = in[6];
  int64_t z1 = (z2 + z3) * F0_541;
  const int64_t tmp2 = z1 - z3 * F1_847;
  const int64_t tmp3 = z1 + z2 * F0_765;
  const int64_t tmp0 = (in[0] + in[4]) * (int64_t(1) << kConstBits);
  const int64_t tmp1 = (in[0] - in[4]) * (int64_t(1) << kConstBits);
  const int64_t tmp10 = tmp0 + tmp3, tmp13 = tmp0 - tmp3, tmp11 = tmp1 + tmp2, tmp12 = tmp1 - tmp2;
  // odd part
  int64_t t0 = in[7], t1 = in[5], t2 = in[3], t3 = in[1];
  z1 = t0 + t3;
  z2 = t1 + t2;
  z3 = t0 + t2;
  int64_t z4 = t1 + t3;
  const int64_t z5 = (z3 + z4) * F1_175;
  t0 *= F0_298;
  t1 *= F2_053;
  t2 *= F3_072;
  t3 *= F1_501;
  z1 *= -F0_899;
  z2 *= -F2_562;
  z3 = z3 * -F1_961 + z5;
  z4 = z4 * -F0_390 + z5;
  t0 += z1 + z3;
  t1 += z2 + z4;
  t2 += z2 + z3;
  t3 += z1 + z4;
  out[0] = descale(tmp10 + t3, shift);
  out[7] = descale(tmp10 - t3, shift);
  out[1] = descale(tmp11 + t2, shift);
  out[6] = descale(tmp11 - t2, shift);
  out[2] = descale(tmp12 + t1, shift);
  out[5] = descale(tmp12 - t1, shift);
  out[3] = descale(tmp13 + t0, shift);
  out[4] = descale(tmp13 - t0, shift);
}

void idct_block(const int coef[64], const uint16_t* q, unsigned char* dst, size_t pitch) {
  int64_t ws[64];
  for (int c = 0; c < 8; c++) {
    int64_t in[8], out[8];
    if ((coef[8 + c] | coef[16 + c] | coef[24 + c] | coef[32 + c] | coef[40 + c] | coef[48 + c] | coef[56 + c]) == 0) {
      // a column with only its DC term: the transform of a constant, exactly dc * 4 after the first descaling
      const int64_t dcv = static_cast<int64_t>(coef[c]) * q[c] * (1 << kPass1Bits);
      for (int r = 0; r < 8; r++) {
        ws[r * 8 + c] = dcv;
      }
      continue;
    }
    for (int r = 0; r < 8; r++) {
      in[r] = static_cast<int64_t>(coef[r * 8 + c]) * q[r * 8 + c];
    }
    idct_1d(in, out, kConstBits - kPass1Bits);
    for (int r = 0; r < 8; r++) {
      ws[r * 8 + c] = out[r];
    }
  }
  for (int r = 0; r < 8; r++) {
    int64_t out[8];
    const int64_t* w = ws + r * 8;
    if ((w[1] | w[2] | w[3] | w[4] | w[5] | w[6] | w[7]) == 0) {
      // a row with only its first term is constant: the same value the full transform gives
      int64_t v = descale(w[0] * (int64_t(1) << kConstBits), kConstBits + kPass1Bits + 3) + 128;
      v = v < 0 ? 0 : (v > 255 ? 255 : v);
      std::memset(dst + r * pitch, static_cast<int>(v), 8);
      continue;
    }
    idct_1d(w, out, kConstBits + kPass1Bits + 3);
    for (int c = 0; c < 8; c++) {
      const int64_t v = out[c] + 128;
      dst[r * pitch + c] = static_cast<unsigned char>(v < 0 ? 0 : (v > 255 ? 255 : v));
    }
  }
}

struct Decoder {
  const unsigned char* data;
  size_t size;
  std::string why;
  uint16_t qt[4][64];
  bool qt_present[4] = {false, false, false, false};
  Huffman dc[4], ac[4];
  Component comp[4];
  int ncomp = 0;
  int64_t width = 0, height = 0;
  int hmax = 1, vmax = 1;
  int64_t mcux = 0, mcuy = 0;
  int restart_interval = 0;
  bool saw_jfif = false, saw_adobe = false;
  int adobe_transform = 0;
  bool have_frame = false;
  bool progressive = false;
  int ss = 0, se = 63, ah = 0, al = 0;   // spectral band and bit position of the current scan
  int eobrun = 0;                        // blocks still covered by an end-of-band run

  bool fail(const std::string& w) {
    why = w;
    return false;
  }

  bool read_dqt(size_t at, size_t end) {
    while (at < end) {
      const int pq = data[at] >> 4, tq = data[at] & 15;
      at++;
      if (tq > 3 || pq > 1 || at + 64 * (pq + 1) > end) {
        return fail("bad quantisation table");
      }
      for (int k = 0; k < 64; k++) {
        const unsigned v = pq ? (data[at] << 8 | data[at + 1]) : data[at];
        at += pq + 1;
        qt[tq][kZigzag[k]] = static_cast<uint16_t>(v);
      }
      qt_present[tq] = true;
    }
    return true;
  }

  bool read_dht(size_t at, size_t end) {
    while (at < end) {
      const int tc = data[at] >> 4, th = data[at] & 15;
      at++;
      if (tc > 1 || th > 3 || at + 16 > end) {
        return fail("bad Huffman table");
      }
      unsigned char bits[17] = {0};
      int count = 0;
      for (int l = 1; l <= 16; l++) {
        bits[l] = data[at + l - 1];
        count += bits[l];
      }
      at += 16;
      if (count > 256 || at + count > end) {
        return fail("bad Huffman table");
      }
      if (!(tc ? ac[th] : dc[th]).build(bits, data + at, count)) {
        return fail("bad Huffman table");
      }
      at += count;
    }
    return true;
  }

  bool read_sof(size_t at, size_t end) {
    if (end - at < 6 || data[at] != 8) {
      return fail("only 8-bit samples are read (a 12-bit file?)");
    }
    height = data[at + 1] << 8 | data[at + 2];
    width = data[at + 3] << 8 | data[at + 4];
    ncomp = data[at + 5];
    if (width <= 0 || height <= 0) {
      return fail("image size missing from the frame header");
    }
    if ((ncomp != 1 && ncomp != 3 && ncomp != 4) || end - at < static_cast<size_t>(6 + 3 * ncomp)) {
      return fail("bad frame header");
    }
    hmax = vmax = 1;
    for (int i = 0; i < ncomp; i++) {
      const unsigned char* c = data + at + 6 + 3 * i;
      comp[i].id = c[0];
      comp[i].h = c[1] >> 4;
      comp[i].v = c[1] & 15;
      comp[i].tq = c[2];
      if (comp[i].h < 1 || comp[i].v < 1 || comp[i].h > 4 || comp[i].v > 4 || comp[i].tq > 3) {
        return fail("bad frame header");
      }
      hmax = comp[i].h > hmax ? comp[i].h : hmax;
      vmax = comp[i].v > vmax ? comp[i].v : vmax;
    }
    if (ncomp == 1) {
      // a lone component is never interleaved: its sampling factors mean nothing
      comp[0].h = comp[0].v = hmax = vmax = 1;
    }
    mcux = (width + 8 * hmax - 1) / (8 * hmax);
    mcuy = (height + 8 * vmax - 1) / (8 * vmax);
    for (int i = 0; i < ncomp; i++) {
      Component& c = comp[i];
      const int eh = hmax / c.h, ev = vmax / c.v;
      if (eh * c.h != hmax || ev * c.v != vmax || eh > 2 || ev > 2) {
        return fail("sampling factors other than 1 and 2 are not read");
      }
      c.blocks_w = static_cast<int>(mcux) * c.h;
      c.blocks_h = static_cast<int>(mcuy) * c.v;
      c.dw = (width * c.h + hmax - 1) / hmax;
      c.dh = (height * c.v + vmax - 1) / vmax;
      c.plane.assign(static_cast<size_t>(c.blocks_w) * 8 * c.blocks_h * 8, 0);
      if (progressive) {
        c.coef.assign(static_cast<size_t>(c.blocks_w) * c.blocks_h * 64, 0);
      }
    }
    have_frame = true;
    return true;
  }

  // One block of a progressive scan (T.81 annex G): the scan carries either the
  // DC terms or one band of AC terms, either their high bits (first pass, value
  // shifted left by al) or one more bit each (refinement).
  bool progressive_block(Bits& b, Component& c) {
    if (bx >= c.blocks_w || by >= c.blocks_h) {
      return fail("corrupt entropy-coded data");
    }
    int* coef = c.coef.data() + (static_cast<size_t>(by) * c.blocks_w + bx) * 64;
    if (ss == 0) {
      if (ah == 0) {
        const int t = decode_symbol(b, dc[c.td]);
        if (t < 0 || t > 11) {
          return fail("corrupt entropy-coded data");
        }
        c.pred += t ? extend(b.get(t), t) : 0;
        coef[0] = c.pred * (1 << al);
      } else if (b.get(1)) {
        coef[0] |= 1 << al;
      }
      return true;
    }
    const int p1 = 1 << al, m1 = -(1 << al);
    int k = ss;
    if (ah == 0) {
      if (eobrun > 0) {
        eobrun--;
        return true;
      }
      while (k <= se) {
        const int rs = decode_symbol(b, ac[c.ta]);
        if (rs < 0) {
          return fail("corrupt entropy-coded data");
        }
        const int r = rs >> 4, s = rs & 15;
        if (s == 0) {
          if (r < 15) {
            eobrun = (1 << r) - 1;
            if (r) {
              eobrun += b.get(r);
            }
            break;
          }
          k += 16;
          continue;
        }
        k += r;
        if (k > se) {
          return fail("corrupt entropy-coded data");
        }
        coef[kZigzag[k]] = extend(b.get(s), s) * (1 << al);
        k++;
      }
      return true;
    }
    // refinement of a band: known non-zero terms get one more bit each, new terms are +-1 << al
    auto refine = [&](int& v) {
      if (b.get(1) && (v & p1) == 0) {
        v += v >= 0 ? p1 : m1;
      }
    };
    if (eobrun == 0) {
      for (; k <= se; k++) {
        const int rs = decode_symbol(b, ac[c.ta]);
        if (rs < 0) {
          return fail("corrupt entropy-coded data");
        }
        int r = rs >> 4;
        const int s = rs & 15;
        int value = 0;
        if (s) {
          value = b.get(1) ? p1 : m1;
        } else if (r != 15) {
          eobrun = 1 << r;
          if (r) {
            eobrun += b.get(r);
          }
          break;
        }
        while (k <= se) {
          int& v = coef[kZigzag[k]];
          if (v != 0) {
            refine(v);
          } else if (--r < 0) {
            break;
          }
          k++;
        }
        if (s && k <= se) {
          coef[kZigzag[k]] = value;
        }
      }
    }
    if (eobrun > 0) {
      for (; k <= se; k++) {
        int& v = coef[kZigzag[k]];
        if (v != 0) {
          refine(v);
        }
      }
      eobrun--;
    }
    return true;
  }

  // After the last scan of a progressive frame: every block through the inverse DCT.
  void finish_progressive() {
    for (int i = 0; i < ncomp; i++) {
      Component& c = comp[i];
      const size_t pitch = static_cast<size_t>(c.blocks_w) * 8;
      for (int y = 0; y < c.blocks_h; y++) {
        for (int x = 0; x < c.blocks_w; x++) {
          idct_block(c.coef.data() + (static_cast<size_t>(y) * c.blocks_w + x) * 64, qt[c.tq],
                     c.plane.data() + static_cast<size_t>(y) * 8 * pitch + static_cast<size_t>(x) * 8, pitch);
        }
      }
    }
  }

  bool decode_block(Bits& b, Component& c) {
    if (progressive) {
      return progressive_block(b, c);
    }
    int coef[64] = {0};
    const int t = decode_symbol(b, dc[c.td]);
    if (t < 0 || t > 11) {
      return fail("corrupt entropy-coded data");
    }
    c.pred += t ? extend(b.get(t), t) : 0;
    coef[0] = c.pred;
    const Huffman& act = ac[c.ta];
    for (int k = 1; k < 64;) {
      const int quick = act.step[b.peek(Huffman::kLook)];
      if (quick) {
        k += (quick >> 4) & 15;
        if (k > 63) {
          return fail("corrupt entropy-coded data");
        }
        coef[kZigzag[k++]] = quick >> 8;
        b.skip(quick & 15);
        continue;
      }
      const int rs = decode_symbol(b, act);
      if (rs < 0) {
        return fail("corrupt entropy-coded data");
      }
      const int r = rs >> 4, s = rs & 15;
      if (s == 0) {
        if (r != 15) {
          break;
        }
        k += 16;
        continue;
      }
      k += r;
      if (k > 63) {
        return fail("corrupt entropy-coded data");
      }
      coef[kZigzag[k]] = extend(b.get(s), s);
      k++;
    }
    // a baseline block is complete after its one visit: inverse DCT into its place
    const size_t pitch = static_cast<size_t>(c.blocks_w) * 8;
    if (bx < c.blocks_w && by < c.blocks_h) {
      idct_block(coef, qt[c.tq], c.plane.data() + static_cast<size_t>(by) * 8 * pitch + static_cast<size_t>(bx) * 8, pitch);
    }
    return true;
  }

  int bx = 0, by = 0;   // block being decoded, in blocks of its component

  // Scan header at `at`; the entropy-coded data follows.  Returns the position
  // after the scan's data (at the next marker) through `next`.
  bool read_scan(size_t at, size_t end, size_t& next) {
    if (!have_frame) {
      return fail("scan before the frame header");
    }
    const int ns = data[at];
    if (ns < 1 || ns > ncomp || end - at < static_cast<size_t>(1 + 2 * ns + 3)) {
      return fail("bad scan header");
    }
    Component* sc[4];
    for (int i = 0; i < ns; i++) {
      const int id = data[at + 1 + 2 * i], tables = data[at + 2 + 2 * i];
      sc[i] = nullptr;
      for (int j = 0; j < ncomp; j++) {
        if (comp[j].id == id) {
          sc[i] = &comp[j];
        }
      }
      if (!sc[i]) {
        return fail("scan names an unknown component");
      }
      sc[i]->td = tables >> 4;
      sc[i]->ta = tables & 15;
      sc[i]->pred = 0;
    }
    ss = data[at + 1 + 2 * ns];
    se = data[at + 2 + 2 * ns];
    ah = data[at + 3 + 2 * ns] >> 4;
    al = data[at + 3 + 2 * ns] & 15;
    eobrun = 0;
    if (!progressive) {
      ss = 0;
      se = 63;
      ah = al = 0;
    } else if (ss > se || se > 63 || al > 13 || (ss == 0 && se != 0) || (ss > 0 && ns != 1)) {
      return fail("bad progressive scan header");
    }
    for (int i = 0; i < ns; i++) {
      const bool needs_dc = ss == 0 && ah == 0, needs_ac = !progressive || ss > 0;
      if (sc[i]->td > 3 || sc[i]->ta > 3 || (needs_dc && !dc[sc[i]->td].present) ||
          (needs_ac && !ac[sc[i]->ta].present) || !qt_present[sc[i]->tq]) {
        return fail("scan uses a table the file does not define");
      }
    }
    Bits b{data, size, end};
    int64_t units_x, units_y;
    if (ns == 1) {
      units_x = (sc[0]->dw + 7) / 8;
      units_y = (sc[0]->dh + 7) / 8;
    } else {
      units_x = mcux;
      units_y = mcuy;
    }
    int64_t until_restart = restart_interval;
    int expect_rst = 0;
    for (int64_t my = 0; my < units_y; my++) {
      for (int64_t mx = 0; mx < units_x; mx++) {
        if (restart_interval && until_restart == 0) {
          // byte-align, then the restart marker
          b.restart();
          size_t p = b.pos;
          while (p + 1 < size && !(data[p] == 0xff && data[p + 1] >= 0xd0 && data[p + 1] <= 0xd7)) {
            p++;
          }
          if (p + 1 >= size || data[p + 1] != 0xd0 + expect_rst) {
            return fail("restart marker missing");
          }
          b.pos = p + 2;
          expect_rst = (expect_rst + 1) & 7;
          until_restart = restart_interval;
          for (int i = 0; i < ns; i++) {
            sc[i]->pred = 0;
          }
          eobrun = 0;
        }
        if (ns == 1) {
          bx = static_cast<int>(mx);
          by = static_cast<int>(my);
          if (!decode_block(b, *sc[0])) {
            return false;
          }
        } else {
          for (int i = 0; i < ns; i++) {
            for (int v = 0; v < sc[i]->v; v++) {
              for (int h = 0; h < sc[i]->h; h++) {
                bx = static_cast<int>(mx) * sc[i]->h + h;
                by = static_cast<int>(my) * sc[i]->v + v;
                if (!decode_block(b, *sc[i])) {
                  return false;
                }
              }
            }
          }
        }
        until_restart--;
      }
    }
    // the next marker follows the scan's last byte
    size_t p = b.pos;
    while (p + 1 < size && !(data[p] == 0xff && data[p + 1] != 0 && !(data[p + 1] >= 0xd0 && data[p + 1] <= 0xd7))) {
      p++;
    }
    next = p;
    return true;
  }

  // Walks the markers; with `header_only` stops at the frame header.
  bool run(bool header_only) {
    if (!jpeg_signature(data, size)) {
      return fail("not a JPEG file");
    }
    size_t at = 2;
    int scans = 0;
    while (at + 1 < size) {
      if (data[at] != 0xff) {
        at++;
        continue;
      }
      const unsigned m = data[at + 1];
      at += 2;
      if (m == 0xff) {
        at--;
        continue;
      }
      if (m == 0xd8 || m == 0x01 || (m >= 0xd0 && m <= 0xd7) || m == 0x00) {
        continue;
      }
      if (m == 0xd9) {
        break;
      }
      if (at + 2 > size) {
        return fail("file cut short");
      }
      const size_t len = data[at] << 8 | data[at + 1];
      if (len < 2 || at + len > size) {
        return fail("marker segment runs past the end of the file");
      }
      const size_t body = at + 2, end = at + len;
      switch (m) {
        case 0xc0:
        case 0xc1:
        case 0xc2:
          progressive = m == 0xc2;
          if (have_frame) {
            return fail("more than one frame header");
          }
          if (!read_sof(body, end)) {
            return false;
          }
          if (header_only) {
            return true;
          }
          break;
        case 0xc3: case 0xc5: case 0xc6: case 0xc7: case 0xc9: case 0xca: case 0xcb: case 0xcd: case 0xce: case 0xcf:
          return fail("lossless, hierarchical and arithmetic-coded JPEG files are not read");
        case 0xc4:
          if (!read_dht(body, end)) {
            return false;
          }
          break;
        case 0xdb:
          if (!read_dqt(body, end)) {
            return false;
          }
          break;
        case 0xdd:
          if (len >= 4) {
            restart_interval = data[body] << 8 | data[body + 1];
          }
          break;
        case 0xe0:
          if (len >= 7 && std::memcmp(data + body, "JFIF", 5) == 0) {
            saw_jfif = true;
          }
          break;
        case 0xee:
          if (len >= 14 && std::memcmp(data + body, "Adobe", 5) == 0) {
            saw_adobe = true;
            adobe_transform = data[body + 11];
          }
          break;
        case 0xda: {
          size_t next = end;
          if (!read_scan(body, end, next)) {
            return false;
          }
          scans++;
          at = next;
          continue;
        }
        default:
          break;
      }
      at = end;
    }
    if (!have_frame) {
      return fail("no frame header");
    }
    if (!header_only && scans == 0) {
      return fail("no image data");
    }
    if (!header_only && progressive) {
      finish_progressive();
    }
    return true;
  }

  // Four components: CMYK as stored, or - when the Adobe marker says so - YCCK,
  // whose first three are converted like YCbCr and then inverted.
  bool is_ycck() const {
    return ncomp == 4 && saw_adobe && adobe_transform == 2;
  }

  bool is_rgb() const {
    if (ncomp != 3) {
      return false;
    }
    if (saw_jfif) {
      return false;
    }
    if (saw_adobe) {
      return adobe_transform == 0;
    }
    return comp[0].id == 'R' && comp[1].id == 'G' && comp[2].id == 'B';
  }
};

// Loops the compiler can vectorise get an AVX2 clone beside the baseline one;
// the dynamic loader picks at start-up.
#if defined(__x86_64__) && defined(__GNUC__) && !defined(__clang__)
#define MLXD_CLONES __attribute__((target_clones("avx2", "default")))
#else
#define MLXD_CLONES
#endif

// Horizontal 2:1 triangle filter of n samples into 2n outputs (n >= 3):
// out[2x] = (3 in[x] + in[x-1] + 1) >> 2, out[2x+1] = (3 in[x] + in[x+1] + 2) >> 2, edges copied.
MLXD_CLONES void h2v1_row(const unsigned char* __restrict in, int64_t n, unsigned char* __restrict out) {
  out[0] = in[0];
  out[1] = static_cast<unsigned char>((3 * in[0] + in[1] + 2) >> 2);
  for (int64_t x = 1; x < n - 1; x++) {
    out[2 * x] = static_cast<unsigned char>((3 * in[x] + in[x - 1] + 1) >> 2);
    out[2 * x + 1] = static_cast<unsigned char>((3 * in[x] + in[x + 1] + 2) >> 2);
  }
  out[2 * n - 2] = static_cast<unsigned char>((3 * in[n - 1] + in[n - 2] + 1) >> 2);
  out[2 * n - 1] = in[n - 1];
}

// Both directions at once: col[x] = 3 near[x] + far[x], then
// out[2x] = (3 col[x] + col[x-1] + 8) >> 4, out[2x+1] = (3 col[x] + col[x+1] + 7) >> 4.
MLXD_CLONES void h2v2_row(const unsigned char* __restrict near, const unsigned char* __restrict far, int64_t n,
                          int* __restrict col, unsigned char* __restrict out) {
  for (int64_t x = 0; x < n; x++) {
    col[x] = 3 * near[x] + far[x];
  }
  out[0] = static_cast<unsigned char>((col[0] * 4 + 8) >> 4);
  out[1] = static_cast<unsigned char>((col[0] * 3 + col[1] + 7) >> 4);
  for (int64_t x = 1; x < n - 1; x++) {
    out[2 * x] = static_cast<unsigned char>((col[x] * 3 + col[x - 1] + 8) >> 4);
    out[2 * x + 1] = static_cast<unsigned char>((col[x] * 3 + col[x + 1] + 7) >> 4);
  }
  out[2 * n - 2] = static_cast<unsigned char>((col[n - 1] * 3 + col[n - 2] + 8) >> 4);
  out[2 * n - 1] = static_cast<unsigned char>((col[n - 1] * 4 + 7) >> 4);
}

MLXD_CLONES void h1v2_row(const unsigned char* __restrict near, const unsigned char* __restrict far, int64_t n, int bias,
                          unsigned char* __restrict out) {
  for (int64_t x = 0; x < n; x++) {
    out[x] = static_cast<unsigned char>((3 * near[x] + far[x] + bias) >> 2);
  }
}

// One output row (full resolution, `width` samples, room for one more) of a
// component whose plane is subsampled by (eh, ev): triangle filter, the nearer
// sample weighted 3:1, edges repeated; the rounding biases alternate between
// neighbouring outputs.
void upsampled_row(const Component& c, int eh, int ev, int64_t y, int64_t width, std::vector<int>& tmp, unsigned char* dst) {
  const size_t pitch = static_cast<size_t>(c.blocks_w) * 8;
  const int64_t n = c.dw;
  if (eh == 1 && ev == 1) {
    std::memcpy(dst, c.plane.data() + static_cast<size_t>(y) * pitch, static_cast<size_t>(width));
    return;
  }
  // planes of one or two columns are doubled without a filter, as libjpeg does
  if (eh == 2 && n <= 2) {
    const unsigned char* in = c.plane.data() + static_cast<size_t>(ev == 2 ? y >> 1 : y) * pitch;
    for (int64_t x = 0; x < width; x++) {
      dst[x] = in[x >> 1];
    }
    return;
  }
  if (ev == 1) {
    h2v1_row(c.plane.data() + static_cast<size_t>(y) * pitch, n, dst);   // 2n >= width outputs
    return;
  }
  // two output rows per input row: the upper one leans on the row above, the lower on the row below
  const int64_t iy = y >> 1;
  const bool lower = (y & 1) != 0;
  int64_t ny = lower ? iy + 1 : iy - 1;
  ny = ny < 0 ? 0 : (ny > c.dh - 1 ? c.dh - 1 : ny);
  const unsigned char* in0 = c.plane.data() + static_cast<size_t>(iy) * pitch;
  const unsigned char* in1 = c.plane.data() + static_cast<size_t>(ny) * pitch;
  if (eh == 1) {
    h1v2_row(in0, in1, width, lower ? 2 : 1, dst);
    return;
  }
  tmp.resize(static_cast<size_t>(n));
  h2v2_row(in0, in1, n, tmp.data(), dst);
}

// YCbCr -> RGB with 16 fractional bits (1.40200, 0.34414, 0.71414, 1.77200),
// the products rounded as libjpeg's tables are.
MLXD_CLONES void ycc_row(const unsigned char* __restrict yy, const unsigned char* __restrict cb,
                         const unsigned char* __restrict cr, int64_t w, unsigned char* __restrict o) {
  for (int64_t x = 0; x < w; x++) {
    const int y0 = yy[x], u = cb[x] - 128, v = cr[x] - 128;
    int rr = y0 + ((91881 * v + 32768) >> 16);
    int gg = y0 + ((-22554 * u + 32768 - 46802 * v) >> 16);
    int bb = y0 + ((116130 * u + 32768) >> 16);
    rr = rr < 0 ? 0 : (rr > 255 ? 255 : rr);
    gg = gg < 0 ? 0 : (gg > 255 ? 255 : gg);
    bb = bb < 0 ? 0 : (bb > 255 ? 255 : bb);
    o[3 * x] = static_cast<unsigned char>(rr);
    o[3 * x + 1] = static_cast<unsigned char>(gg);
    o[3 * x + 2] = static_cast<unsigned char>(bb);
  }
}

inline unsigned char clamp8(int v) {
  return static_cast<unsigned char>(v < 0 ? 0 : (v > 255 ? 255 : v));
}

} // namespace

bool jpeg_signature(const unsigned char* data, size_t size) {
  return size >= 3 && data[0] == 0xff && data[1] == 0xd8 && data[2] == 0xff;
}

bool jpeg_header(const unsigned char* data, size_t size, JpegHeader& h, std::string& why) {
  Decoder d;
  d.data = data;
  d.size = size;
  if (!d.run(true)) {
    why = d.why;
    return false;
  }
  h.width = d.width;
  h.height = d.height;
  h.components = d.ncomp;
  return true;
}

bool jpeg_decode(const unsigned char* data, size_t size, unsigned char* out, std::string& why) {
  Decoder d;
  d.data = data;
  d.size = size;
  if (!d.run(false)) {
    why = d.why;
    return false;
  }
  const int64_t w = d.width, h = d.height;
  if (d.ncomp == 1) {
    const Component& c = d.comp[0];
    const size_t pitch = static_cast<size_t>(c.blocks_w) * 8;
    for (int64_t y = 0; y < h; y++) {
      const unsigned char* in = c.plane.data() + static_cast<size_t>(y) * pitch;
      unsigned char* o = out + static_cast<size_t>(y) * w * 3;
      for (int64_t x = 0; x < w; x++) {
        o[3 * x] = o[3 * x + 1] = o[3 * x + 2] = in[x];
      }
    }
    return true;
  }
  // four components: the reference keeps the first three of libjpeg's CMYK output
  const bool rgb = d.is_rgb() || (d.ncomp == 4 && !d.is_ycck());
  const bool invert = d.is_ycck();
  std::vector<unsigned char> rows[3];
  std::vector<int> tmp;
  for (int i = 0; i < 3; i++) {
    rows[i].resize(static_cast<size_t>(w) + 2);   // a doubled row may be one sample longer than the image
  }
  for (int64_t y = 0; y < h; y++) {
    for (int i = 0; i < 3; i++) {
      const Component& c = d.comp[i];
      const int eh = d.hmax / c.h, ev = d.vmax / c.v;
      upsampled_row(c, eh, ev, y, w, tmp, rows[i].data());
    }
    unsigned char* o = out + static_cast<size_t>(y) * w * 3;
    if (rgb) {
      for (int64_t x = 0; x < w; x++) {
        o[3 * x] = rows[0][x];
        o[3 * x + 1] = rows[1][x];
        o[3 * x + 2] = rows[2][x];
      }
    } else {
      ycc_row(rows[0].data(), rows[1].data(), rows[2].data(), w, o);
      if (invert) {
        for (int64_t x = 0; x < 3 * w; x++) {
          o[x] = static_cast<unsigned char>(255 - o[x]);
        }
      }
    }
  }
  return true;
}

} // namespace image
} // namespace core
} // namespace data
} // namespace mlx
