// PNG decoding for load_image, written from the PNG specification (chunk
// layout, the five scanline filters, Adam7 interlacing) over zlib's inflate.
//
// The reference decodes PNG through stb_image (core/image/ImageSTBI.cpp:14-58):
// it asks the file for its channel count and loads with
// required_channels = min(channels, 3).  For a PNG that means
//   grey -> [H, W, 1]; grey + alpha -> [H, W, 2]; RGB -> [H, W, 3];
//   RGBA -> [H, W, 3] (alpha dropped); palette -> [H, W, 3] (with or without
//   a tRNS chunk); a tRNS colour key on grey or RGB changes nothing.
// PNG is lossless, so 8-bit pixel values are fixed by the format.  What stb
// does beyond that - 16-bit samples reduced to their high byte, 1/2/4-bit grey
// scaled to 0..255 (x255, x85, x17), no gamma or colour-profile handling, CRCs
// not verified - follows its documented behaviour; stb_image is not available
// here, so those three conversions are unpinned.
#pragma once

#include <cstddef>
#include <cstdint>
#include <string>

namespace mlx {
namespace data {
namespace core {
namespace image {

struct PngHeader {
  int64_t width = 0, height = 0;
  int depth = 0;        // bits per sample: 1, 2, 4, 8, 16
  int color = 0;        // PNG colour type: 0 grey, 2 RGB, 3 palette, 4 grey+alpha, 6 RGBA
  int interlace = 0;    // 0 none, 1 Adam7
  int out_channels = 0; // channels of the decoded array (see above)
};

// True when the bytes start with the PNG signature.
bool png_signature(const unsigned char* data, size_t size);

// Reads IHDR; false (with `why`) when the bytes are no PNG this decoder reads.
bool png_header(const unsigned char* data, size_t size, PngHeader& h, std::string& why);

// Decodes the whole file into out[height * width * out_channels]; false (with
// `why`) on a malformed file.  `out` may be page-locked memory: it is written
// once, front to back for non-interlaced files.
bool png_decode(const unsigned char* data, size_t size, const PngHeader& h, unsigned char* out, std::string& why);

} // namespace image
} // namespace core
} // namespace data
} // namespace mlx
