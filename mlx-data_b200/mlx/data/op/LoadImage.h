// load_image (mlx/data/op/LoadImage.cpp:11-50): the array at ikey holds a file
// name (int8 characters, joined to `prefix`) or, with from_memory, the file's
// bytes; the result is the image as uint8 [H, W, C], or with `info` the int64
// pair {width, height}.
//
// What this build decodes: JPEG, baseline and progressive (core/image/Jpeg.h: the arithmetic
// of libjpeg-turbo's defaults, always three channels as in
// core/image/ImageJPEG.cpp:99-146), PNG (core/image/Png.h: every colour type
// and bit depth, interlaced or not, with the channel policy of the reference's
// stb path) and binary PNM (P5 grey, P6 colour, maxval <= 255), whose pixels
// are the file's bytes.  The reference uses libjpeg-turbo and stb_image
// (core/image/ImageIO.cpp, ImageJPEG.cpp, ImageSTBI.cpp); neither library is
// available here, so the decoders are this library's own, and what they do
// not read (arithmetic-coded and 12-bit JPEG, the other stb formats) is refused by
// name rather than guessed at.  As in the reference's stb path a grey PNG or
// PNM stays one channel (ImageSTBI.cpp:14-33).
//
// The point of the op here is where the pixels land: they are read from the
// file (or copied from the buffer) straight into a page-locked block of the
// runtime's staging pool, the memory the GPU reads sample rectangles from
// directly - no intermediate host image, no second copy before the transfer.
#pragma once

#include <cstdio>
#include <cstring>
#include <filesystem>
#include <stdexcept>
#include <string>
#include <vector>

#include "mlx/data/core/image/Jpeg.h"
#include "mlx/data/core/image/Png.h"
#include "mlx/data/gpu/Runtime.h"
#include "mlx/data/op/KeyTransform.h"

namespace mlx {
namespace data {
namespace op {

class LoadImage : public KeyTransformOp {
 public:
  LoadImage(const std::string& ikey, const std::string& prefix = "", bool info = false,
            const std::string& format = "RGB", bool from_memory = false, const std::string& okey = "")
      : KeyTransformOp(ikey, okey), prefix_(prefix), info_(info), from_memory_(from_memory) {
    (void)format;  // ignored by the reference too
  }

  // Header of a binary PNM: sizes, channel count and where the pixels start.
  struct Header {
    int64_t width = 0, height = 0, channels = 0;
    size_t pixels_at = 0;
  };

  // Parses "P5|P6 <width> <height> <maxval>" with '#' comments; false when the
  // bytes are no binary PNM this build reads.
  static bool parse_header(const unsigned char* data, size_t size, Header& h) {
    size_t at = 0;
    auto token = [&](std::string& out) {
      for (;;) {
        while (at < size && (data[at] == ' ' || data[at] == '\t' || data[at] == '\n' || data[at] == '\r')) {
          at++;
        }
        if (at < size && data[at] == '#') {
          while (at < size && data[at] != '\n') {
            at++;
          }
          continue;
        }
        break;
      }
      out.clear();
      while (at < size && !(data[at] == ' ' || data[at] == '\t' || data[at] == '\n' || data[at] == '\r')) {
        out.push_back(static_cast<char>(data[at++]));
      }
      return !out.empty();
    };
    auto number = [](const std::string& t, int64_t& v) {
      if (t.empty() || t.size() > 9) {
        return false;
      }
      v = 0;
      for (char c : t) {
        if (c < '0' || c > '9') {
          return false;
        }
        v = v * 10 + (c - '0');
      }
      return true;
    };
    std::string t;
    if (!token(t) || (t != "P5" && t != "P6")) {
      return false;
    }
    h.channels = t == "P5" ? 1 : 3;
    int64_t maxval = 0;
    if (!token(t) || !number(t, h.width) || !token(t) || !number(t, h.height) || !token(t) || !number(t, maxval)) {
      return false;
    }
    if (h.width <= 0 || h.height <= 0 || maxval <= 0 || maxval > 255 || at >= size) {
      return false;
    }
    h.pixels_at = at + 1;  // exactly one white-space byte separates header and pixels
    return true;
  }

  std::shared_ptr<Array> apply_key(const std::shared_ptr<const Array>& src) const override {
    if (from_memory_) {
      const auto* bytes = static_cast<const unsigned char*>(src->data());
      const size_t size = static_cast<size_t>(src->size()) * src->itemsize();
      if (core::image::png_signature(bytes, size)) {
        return png(bytes, size, "stream");
      }
      if (core::image::jpeg_signature(bytes, size)) {
        return jpeg(bytes, size, "stream");
      }
      Header h;
      if (!parse_header(bytes, size, h)) {
        return refuse("stream");
      }
      if (info_) {
        return std::make_shared<Array>(std::vector<int64_t>{h.width, h.height});
      }
      const size_t need = static_cast<size_t>(h.width) * h.height * h.channels;
      if (size - h.pixels_at < need) {
        throw std::runtime_error("LoadImage: unable to load image <stream> (pixel data cut short)");
      }
      auto out = landing(h);
      std::memcpy(out->data(), bytes + h.pixels_at, need);
      return out;
    }
    if (src->type() != ArrayType::Int8) {
      throw std::runtime_error("LoadImage: char array (int8) expected");
    }
    std::filesystem::path path = prefix_;
    path /= std::string(static_cast<const char*>(src->data()), static_cast<size_t>(src->size()));
    FILE* f = std::fopen(path.c_str(), "rb");
    if (!f) {
      throw std::runtime_error("LoadImage: unable to load image <" + path.string() + ">");
    }
    unsigned char head[512];
    const size_t got = std::fread(head, 1, sizeof(head), f);
    if (core::image::png_signature(head, got) || core::image::jpeg_signature(head, got)) {
      // a compressed file is read whole; its pixels are decoded into the page-locked block
      std::vector<unsigned char> file(head, head + got);
      unsigned char chunk[1 << 16];
      size_t n;
      while ((n = std::fread(chunk, 1, sizeof(chunk), f)) > 0) {
        file.insert(file.end(), chunk, chunk + n);
      }
      std::fclose(f);
      return core::image::png_signature(head, got) ? png(file.data(), file.size(), path.string())
                                                   : jpeg(file.data(), file.size(), path.string());
    }
    Header h;
    if (!parse_header(head, got, h)) {
      std::fclose(f);
      return refuse(path.string());
    }
    if (info_) {
      std::fclose(f);
      return std::make_shared<Array>(std::vector<int64_t>{h.width, h.height});
    }
    const size_t need = static_cast<size_t>(h.width) * h.height * h.channels;
    std::shared_ptr<Array> out;
    try {
      out = landing(h);
    } catch (...) {
      std::fclose(f);
      throw;
    }
    // the file's pixel bytes go straight into the page-locked block
    const bool ok = std::fseek(f, static_cast<long>(h.pixels_at), SEEK_SET) == 0 &&
        std::fread(out->data(), 1, need, f) == need;
    std::fclose(f);
    if (!ok) {
      throw std::runtime_error("LoadImage: unable to load image <" + path.string() + "> (pixel data cut short)");
    }
    return out;
  }

 private:
  std::shared_ptr<Array> png(const unsigned char* bytes, size_t size, const std::string& what) const {
    core::image::PngHeader h;
    std::string why;
    if (!core::image::png_header(bytes, size, h, why)) {
      throw std::runtime_error("LoadImage: unable to load image <" + what + "> (" + why + ")");
    }
    if (info_) {
      return std::make_shared<Array>(std::vector<int64_t>{h.width, h.height});
    }
    auto out = gpu::Runtime::get().pinned_array(UInt8, {h.height, h.width, h.out_channels});
    if (!core::image::png_decode(bytes, size, h, static_cast<unsigned char*>(out->data()), why)) {
      throw std::runtime_error("LoadImage: unable to load image <" + what + "> (" + why + ")");
    }
    return out;
  }
  std::shared_ptr<Array> jpeg(const unsigned char* bytes, size_t size, const std::string& what) const {
    core::image::JpegHeader h;
    std::string why;
    if (!core::image::jpeg_header(bytes, size, h, why)) {
      throw std::runtime_error("LoadImage: unable to load image <" + what + "> (" + why + ")");
    }
    if (info_) {
      return std::make_shared<Array>(std::vector<int64_t>{h.width, h.height});
    }
    auto out = gpu::Runtime::get().pinned_array(UInt8, {h.height, h.width, 3});
    if (!core::image::jpeg_decode(bytes, size, static_cast<unsigned char*>(out->data()), why)) {
      throw std::runtime_error("LoadImage: unable to load image <" + what + "> (" + why + ")");
    }
    return out;
  }
  static std::shared_ptr<Array> landing(const Header& h) {
    return gpu::Runtime::get().pinned_array(UInt8, {h.height, h.width, h.channels});
  }
  [[noreturn]] static std::shared_ptr<Array> refuse(const std::string& what) {
    throw std::runtime_error(
        "LoadImage: unable to load image <" + what +
        ">: this build reads JPEG, PNG and binary PNM (P5, P6) - libjpeg-turbo and stb_image, which "
        "mlx-data decodes with, are not available here");
  }

  std::string prefix_;
  bool info_;
  bool from_memory_;
};

} // namespace op
} // namespace data
} // namespace mlx
