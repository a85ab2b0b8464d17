#include "mlx/data/core/image/Png.h"

#include <zlib.h>

#include <cstdlib>
#include <cstring>
#include <utility>
#include <vector>

namespace mlx {
namespace data {
namespace core {
namespace image {

namespace {

const unsigned char kSignature[8] = {0x89, 'P', 'N', 'G', 0x0d, 0x0a, 0x1a, 0x0a};

uint32_t be32(const unsigned char* p) {
  return (uint32_t(p[0]) << 24) | (uint32_t(p[1]) << 16) | (uint32_t(p[2]) << 8) | uint32_t(p[3]);
}

int samples_per_pixel(int color) {
  switch (color) {
    case 0: return 1;
    case 2: return 3;
    case 3: return 1;
    case 4: return 2;
    default: return 4;
  }
}

// Bytes of one scanline of `pixels` pixels, without its filter byte.
size_t line_bytes(int64_t pixels, int bits_per_pixel) {
  return (static_cast<size_t>(pixels) * bits_per_pixel + 7) / 8;
}

// The seven Adam7 passes: first column / row and the step between them.
const int kPassX0[7] = {0, 4, 0, 2, 0, 1, 0};
const int kPassY0[7] = {0, 0, 4, 0, 2, 0, 1};
const int kPassDx[7] = {8, 8, 4, 4, 2, 2, 1};
const int kPassDy[7] = {8, 8, 8, 4, 4, 2, 2};

struct Chunks {
  const unsigned char* plte = nullptr;
  size_t plte_entries = 0;
  std::vector<std::pair<const unsigned char*, size_t>> idat;
};

bool walk_chunks(const unsigned char* data, size_t size, Chunks& c, std::string& why) {
  size_t at = 8;
  bool ended = false;
  while (!ended && at + 12 <= size) {
    const size_t len = be32(data + at);
    const unsigned char* type = data + at + 4;
    const unsigned char* body = data + at + 8;
    if (len > size - at - 12) {
      why = "chunk runs past the end of the file";
      return false;
    }
    if (std::memcmp(type, "PLTE", 4) == 0) {
      if (len % 3 != 0 || len > 768) {
        why = "bad PLTE chunk";
        return false;
      }
      c.plte = body;
      c.plte_entries = len / 3;
    } else if (std::memcmp(type, "IDAT", 4) == 0) {
      c.idat.emplace_back(body, len);
    } else if (std::memcmp(type, "IEND", 4) == 0) {
      ended = true;
    }
    at += 12 + len;
  }
  if (c.idat.empty()) {
    why = "no image data";
    return false;
  }
  return true;
}

bool inflate_all(const Chunks& c, std::vector<unsigned char>& raw, std::string& why) {
  z_stream z;
  std::memset(&z, 0, sizeof(z));
  if (inflateInit(&z) != Z_OK) {
    why = "zlib would not start";
    return false;
  }
  z.next_out = raw.data();
  z.avail_out = static_cast<uInt>(raw.size());
  int rc = Z_OK;
  for (size_t i = 0; i < c.idat.size() && rc != Z_STREAM_END; i++) {
    z.next_in = const_cast<unsigned char*>(c.idat[i].first);
    z.avail_in = static_cast<uInt>(c.idat[i].second);
    while (z.avail_in > 0 && rc != Z_STREAM_END) {
      rc = inflate(&z, Z_NO_FLUSH);
      if (rc != Z_OK && rc != Z_STREAM_END) {
        // Z_BUF_ERROR with a full output buffer: more data than the image holds, which is ignored
        if (rc == Z_BUF_ERROR && z.avail_out == 0) {
          rc = Z_STREAM_END;
          break;
        }
        inflateEnd(&z);
        why = "corrupt compressed data";
        return false;
      }
      if (z.avail_out == 0) {
        rc = Z_STREAM_END;
      }
    }
  }
  const bool full = z.avail_out == 0;
  inflateEnd(&z);
  if (!full) {
    why = "not enough pixel data";
    return false;
  }
  return true;
}

int paeth(int a, int b, int c) {
  const int p = a + b - c;
  const int pa = std::abs(p - a), pb = std::abs(p - b), pc = std::abs(p - c);
  if (pa <= pb && pa <= pc) {
    return a;
  }
  return pb <= pc ? b : c;
}

// Undo the scanline filters of `rows` lines of `bytes` bytes each (every line
// preceded by its filter byte), in place.  `unit` is the filter's pixel
// distance in bytes.
bool unfilter(unsigned char* lines, size_t bytes, int64_t rows, int unit, std::string& why) {
  const unsigned char* prev = nullptr;
  for (int64_t y = 0; y < rows; y++) {
    unsigned char* line = lines + static_cast<size_t>(y) * (bytes + 1);
    const int filter = line[0];
    unsigned char* cur = line + 1;
    switch (filter) {
      case 0:
        break;
      case 1:
        for (size_t i = unit; i < bytes; i++) {
          cur[i] = static_cast<unsigned char>(cur[i] + cur[i - unit]);
        }
        break;
      case 2:
        if (prev) {
          for (size_t i = 0; i < bytes; i++) {
            cur[i] = static_cast<unsigned char>(cur[i] + prev[i]);
          }
        }
        break;
      case 3:
        for (size_t i = 0; i < bytes; i++) {
          const int left = i >= static_cast<size_t>(unit) ? cur[i - unit] : 0;
          const int up = prev ? prev[i] : 0;
          cur[i] = static_cast<unsigned char>(cur[i] + ((left + up) >> 1));
        }
        break;
      case 4:
        for (size_t i = 0; i < bytes; i++) {
          const int left = i >= static_cast<size_t>(unit) ? cur[i - unit] : 0;
          const int up = prev ? prev[i] : 0;
          const int corner = (prev && i >= static_cast<size_t>(unit)) ? prev[i - unit] : 0;
          cur[i] = static_cast<unsigned char>(cur[i] + paeth(left, up, corner));
        }
        break;
      default:
        why = "unknown scanline filter";
        return false;
    }
    prev = cur;
  }
  return true;
}

// Pixels of one unfiltered scanline into the output image: `count` pixels to
// columns x0, x0 + dx, ... of row `dst_row` ([width * out_channels] bytes).
void emit_line(
    const unsigned char* line, int64_t count, const PngHeader& h, const Chunks& c, unsigned char* dst_row, int x0,
    int dx) {
  const int oc = h.out_channels;
  const int spp = samples_per_pixel(h.color);
  if (h.depth == 8 && dx == 1 && (h.color == 0 || h.color == 2 || h.color == 4)) {
    std::memcpy(dst_row, line, static_cast<size_t>(count) * spp);   // the file's bytes are the pixels
    return;
  }
  for (int64_t i = 0; i < count; i++) {
    unsigned s[4] = {0, 0, 0, 0};
    if (h.depth == 8) {
      for (int k = 0; k < spp; k++) {
        s[k] = line[i * spp + k];
      }
    } else if (h.depth == 16) {
      for (int k = 0; k < spp; k++) {
        s[k] = line[(i * spp + k) * 2];   // the high byte of a big-endian sample
      }
    } else {
      const int64_t bit = i * h.depth;
      s[0] = (line[bit >> 3] >> (8 - h.depth - (bit & 7))) & ((1u << h.depth) - 1u);
      if (h.color == 0) {
        s[0] *= h.depth == 1 ? 255u : (h.depth == 2 ? 85u : 17u);
      }
    }
    unsigned char* px = dst_row + (static_cast<size_t>(x0) + static_cast<size_t>(i) * dx) * oc;
    if (h.color == 3) {
      const unsigned char* e = s[0] < c.plte_entries ? c.plte + 3 * s[0] : nullptr;
      px[0] = e ? e[0] : 0;
      px[1] = e ? e[1] : 0;
      px[2] = e ? e[2] : 0;
    } else {
      for (int k = 0; k < oc; k++) {
        px[k] = static_cast<unsigned char>(s[k]);
      }
    }
  }
}

} // namespace

bool png_signature(const unsigned char* data, size_t size) {
  return size >= 8 && std::memcmp(data, kSignature, 8) == 0;
}

bool png_header(const unsigned char* data, size_t size, PngHeader& h, std::string& why) {
  if (!png_signature(data, size)) {
    why = "not a PNG file";
    return false;
  }
  if (size < 8 + 12 + 13 || be32(data + 8) != 13 || std::memcmp(data + 12, "IHDR", 4) != 0) {
    why = "the first chunk is not IHDR";
    return false;
  }
  const unsigned char* p = data + 16;
  h.width = be32(p);
  h.height = be32(p + 4);
  h.depth = p[8];
  h.color = p[9];
  h.interlace = p[12];
  if (h.width <= 0 || h.height <= 0 || h.width > (1 << 24) || h.height > (1 << 24)) {
    why = "image size out of range";
    return false;
  }
  const int d = h.depth;
  bool ok = false;
  switch (h.color) {
    case 0: ok = d == 1 || d == 2 || d == 4 || d == 8 || d == 16; break;
    case 3: ok = d == 1 || d == 2 || d == 4 || d == 8; break;
    case 2:
    case 4:
    case 6: ok = d == 8 || d == 16; break;
    default: ok = false;
  }
  if (!ok || p[10] != 0 || p[11] != 0 || h.interlace > 1) {
    why = "unsupported colour type, bit depth, compression, filter or interlace method";
    return false;
  }
  h.out_channels = h.color == 0 ? 1 : (h.color == 4 ? 2 : 3);
  return true;
}

bool png_decode(const unsigned char* data, size_t size, const PngHeader& h, unsigned char* out, std::string& why) {
  Chunks c;
  if (!walk_chunks(data, size, c, why)) {
    return false;
  }
  if (h.color == 3 && c.plte == nullptr) {
    why = "palette image without a PLTE chunk";
    return false;
  }
  const int bits = samples_per_pixel(h.color) * h.depth;
  const int unit = bits >= 8 ? bits / 8 : 1;
  const size_t out_pitch = static_cast<size_t>(h.width) * h.out_channels;

  size_t raw_size = 0;
  if (!h.interlace) {
    raw_size = static_cast<size_t>(h.height) * (1 + line_bytes(h.width, bits));
  } else {
    for (int p = 0; p < 7; p++) {
      const int64_t pw = (h.width - kPassX0[p] + kPassDx[p] - 1) / kPassDx[p];
      const int64_t ph = (h.height - kPassY0[p] + kPassDy[p] - 1) / kPassDy[p];
      if (pw > 0 && ph > 0) {
        raw_size += static_cast<size_t>(ph) * (1 + line_bytes(pw, bits));
      }
    }
  }
  std::vector<unsigned char> raw(raw_size);
  if (!inflate_all(c, raw, why)) {
    return false;
  }

  if (!h.interlace) {
    const size_t bytes = line_bytes(h.width, bits);
    if (!unfilter(raw.data(), bytes, h.height, unit, why)) {
      return false;
    }
    for (int64_t y = 0; y < h.height; y++) {
      emit_line(raw.data() + static_cast<size_t>(y) * (bytes + 1) + 1, h.width, h, c, out + y * out_pitch, 0, 1);
    }
    return true;
  }
  size_t at = 0;
  for (int p = 0; p < 7; p++) {
    const int64_t pw = (h.width - kPassX0[p] + kPassDx[p] - 1) / kPassDx[p];
    const int64_t ph = (h.height - kPassY0[p] + kPassDy[p] - 1) / kPassDy[p];
    if (pw <= 0 || ph <= 0) {
      continue;
    }
    const size_t bytes = line_bytes(pw, bits);
    if (!unfilter(raw.data() + at, bytes, ph, unit, why)) {
      return false;
    }
    for (int64_t y = 0; y < ph; y++) {
      const int64_t row = kPassY0[p] + y * kPassDy[p];
      emit_line(raw.data() + at + static_cast<size_t>(y) * (bytes + 1) + 1, pw, h, c, out + row * out_pitch, kPassX0[p],
                kPassDx[p]);
    }
    at += static_cast<size_t>(ph) * (bytes + 1);
  }
  return true;
}

} // namespace image
} // namespace core
} // namespace data
} // namespace mlx
