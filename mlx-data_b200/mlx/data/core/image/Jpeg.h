// JPEG decoding for load_image, written from the JPEG standard (ITU T.81:
// markers, Huffman-coded sequential and progressive DCT scans, restart
// intervals) and the JFIF colour convention.
//
// The reference decodes JPEG with libjpeg-turbo at its default settings
// (core/image/ImageJPEG.cpp:99-146): the accurate integer inverse DCT, "fancy"
// (triangle-filter) chroma upsampling, YCbCr -> RGB in 16-bit fixed point, and
// it always returns three channels - a grey file has its one channel copied
// to all three.  The arithmetic here follows those published methods step by
// step (Loeffler-Ligtenberg-Moschytz IDCT with 13-bit constants and the two
// descaling shifts, 3:1 triangle upsampling with the alternating rounding
// biases, the JFIF conversion with 16 fractional bits), so that the pixels are
// the same integers; tests/test_jpeg_cpu.py holds it to Pillow's decoder,
// which is libjpeg-turbo with the same defaults.
//
// Read here: 8-bit baseline, extended-sequential and progressive Huffman files
// (SOF0, SOF1, SOF2) with one component (grey) or three (YCbCr, or RGB when an
// Adobe marker says so), luma sampled 1x1, 2x1, 1x2 or 2x2 against 1x1 chroma,
// interleaved or not, with or without restart markers.  A progressive file is
// decoded from all its scans (spectral selection and successive
// approximation), then transformed once.  Four-component files give the first
// three channels of libjpeg's CMYK output, as the reference keeps them: the
// stored C, M, Y, or for Adobe YCCK files the converted and inverted ones.
// Arithmetic-coded, lossless and 12-bit files are refused by name.  Luma sampled 1x2
// ("4:4:0") is filtered vertically by the same 3:1 rule; Pillow writes no such
// file, so that one case is not pinned.
#pragma once

#include <cstddef>
#include <cstdint>
#include <string>

namespace mlx {
namespace data {
namespace core {
namespace image {

struct JpegHeader {
  int64_t width = 0, height = 0;
  int components = 0;   // in the file: 1, 3 or 4
};

// True when the bytes start with the JPEG signature (FF D8 FF).
bool jpeg_signature(const unsigned char* data, size_t size);

// Reads up to the frame header; false (with `why`) when the file is not one
// this decoder reads.
bool jpeg_header(const unsigned char* data, size_t size, JpegHeader& h, std::string& why);

// Decodes into out[height * width * 3] (RGB); false (with `why`) on a
// malformed or unsupported file.
bool jpeg_decode(const unsigned char* data, size_t size, unsigned char* out, std::string& why);

} // namespace image
} // namespace core
} // namespace data
} // namespace mlx
