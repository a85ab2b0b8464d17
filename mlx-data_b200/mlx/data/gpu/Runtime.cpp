#include "mlx/data/gpu/Runtime.h"

#include <sched.h>

#include <atomic>
#include <cctype>
#include <cstdio>

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <stdexcept>
#include <string>

namespace mlx {
namespace data {
namespace gpu {

namespace {
int g_device = -1;

int env_int(const char* name, int fallback) {
  const char* v = std::getenv(name);
  if (!v || !*v) {
    return fallback;
  }
  return std::atoi(v);
}

int32_t to_i32(int64_t v, const char* what) {
  if (v < 0 || v > 0x7fffffffLL) {
    throw std::runtime_error(std::string("image: ") + what + " out of range");
  }
  return static_cast<int32_t>(v);
}
} // namespace

// ---------------------------------------------------------------- Window
void Window::crop(int64_t cx, int64_t cy, int64_t cw, int64_t ch) {
  // Same checks as array::sub on the materialised image.
  if (cx < 0 || cy < 0 || cx >= w || cy >= h) {
    throw std::runtime_error("Array: sub: offset out of bound");
  }
  if (cx + cw > w || cy + ch > h) {
    throw std::runtime_error("Array: sub: shape out of bound");
  }
  x += flip ? (w - cx - cw) : cx;
  y += cy;
  w = cw;
  h = ch;
}

// ---------------------------------------------------------------- LazyImage
LazyImage::LazyImage(const std::shared_ptr<const Array>& src) : src_(src) {
  if (src->ndim() != 3) {
    throw std::runtime_error("verifyImage: image must be 3 dimension Array (HWC)");
  }
  channels_ = src->shape(2);
  if (channels_ == 0 || channels_ > 4) {
    throw std::runtime_error("verifyImage: channels must be 0 <= c <= 4");
  }
  pre_.w = src->shape(1);
  pre_.h = src->shape(0);
  geom_w_ = pre_.w;
  geom_h_ = pre_.h;
  post_ = Window{0, 0, pre_.w, pre_.h, false};
}

LazyImage LazyImage::with_source(const std::shared_ptr<const Array>& src) const {
  if (src->ndim() != 3 || src->shape(0) != src_->shape(0) || src->shape(1) != src_->shape(1) ||
      src->shape(2) != src_->shape(2)) {
    throw std::runtime_error("LazyImage: a program moves only to a source of the same shape");
  }
  LazyImage out(*this);
  out.src_ = src;
  return out;
}

int64_t LazyImage::width() const {
  return post_.w + ext_w_;
}

int64_t LazyImage::height() const {
  return post_.h + ext_h_;
}

bool LazyImage::pad_end(int dim, int64_t amount, double value) {
  if ((dim != 0 && dim != 1) || amount < 0) {
    return false;
  }
  if (src_->type() != UInt8 || !(value >= 0.0 && value <= 255.0) || value != std::floor(value)) {
    return false;
  }
  const int v = static_cast<int>(value);
  if (extended() && v != ext_value_) {
    return false;
  }
  if (amount == 0) {
    return true;
  }
  (dim == 0 ? ext_h_ : ext_w_) += amount;
  ext_value_ = v;
  untouched_ = false;
  return true;
}

bool LazyImage::extension_matches(double batch_pad_value) const {
  return !extended() || static_cast<int>(static_cast<uint8_t>(static_cast<int32_t>(batch_pad_value))) == ext_value_;
}

bool LazyImage::crop(int64_t x, int64_t y, int64_t w, int64_t h) {
  if (extended()) {
    return false;
  }
  if (w <= 0 || h <= 0) {
    throw std::runtime_error("image: cannot create image with 0 or negative dimension");
  }
  if (geom_ == MLXD_GEOM_NONE) {
    pre_.crop(x, y, w, h);
    geom_w_ = pre_.w;
    geom_h_ = pre_.h;
    post_ = Window{0, 0, pre_.w, pre_.h, false};
  } else {
    post_.crop(x, y, w, h);
  }
  untouched_ = false;
  return true;
}

bool LazyImage::hflip() {
  if (extended()) {
    return false;
  }
  if (geom_ == MLXD_GEOM_NONE) {
    pre_.flip = !pre_.flip;
  } else {
    post_.flip = !post_.flip;
  }
  untouched_ = false;
  return true;
}

bool LazyImage::resize(int64_t dw, int64_t dh) {
  if (geom_ != MLXD_GEOM_NONE || gray_ || extended()) {
    return false;
  }
  if (src_->type() != UInt8) {
    throw std::invalid_argument("image must be of type UInt8");
  }
  if (channels_ == 4 && !Runtime::rgba_resize_independent()) {
    throw std::runtime_error(
        "image resize: 4-channel images are filtered channel by channel here, while mlx-data weights colour by "
        "alpha (RGBA layout of its resize library); call core.set_rgba_resize_independent(True) to accept that");
  }
  if (dh <= 0 || dw <= 0) {
    throw std::runtime_error("image: cannot create image with 0 or negative dimension");
  }
  geom_ = MLXD_GEOM_RESIZE;
  geom_w_ = dw;
  geom_h_ = dh;
  post_ = Window{0, 0, dw, dh, false};
  untouched_ = false;
  return true;
}

bool LazyImage::affine(const float mx[6], int64_t tw, int64_t th) {
  if (geom_ != MLXD_GEOM_NONE || gray_ || extended()) {
    return false;
  }
  if (src_->type() != UInt8) {
    throw std::invalid_argument("image must be of type UInt8");
  }
  if (th <= 0 || tw <= 0) {
    throw std::runtime_error("image: cannot create image with 0 or negative dimension");
  }
  geom_ = MLXD_GEOM_AFFINE;
  geom_w_ = tw;
  geom_h_ = th;
  std::memcpy(mx_, mx, sizeof(mx_));
  post_ = Window{0, 0, tw, th, false};
  untouched_ = false;
  return true;
}

bool LazyImage::channel_reduction(float bias, const float m[3]) {
  if (extended()) {
    return false;
  }
  if (channels() != 3) {
    throw std::runtime_error("image::channelReduction: expected a 3 channel uint8 array");
  }
  if (src_->type() != UInt8) {
    throw std::invalid_argument("image must be of type UInt8");
  }
  // 16.16 fixed point, truncated: float coefficient times the int scale
  // (mlx/data/core/image/ImageTransform.cpp:159-164).
  const int scale = 256 * 256;
  gray_bias_ = static_cast<int>(bias * scale);
  for (int i = 0; i < 3; i++) {
    gray_m_[i] = static_cast<int>(m[i] * scale);
  }
  gray_ = true;
  untouched_ = false;
  return true;
}

void LazyImage::gray_params(int32_t m[3], int32_t& bias) const {
  std::memcpy(m, gray_m_, sizeof(gray_m_));
  bias = gray_bias_;
}

void LazyImage::describe(mlxd_sample_desc& d) const {
  std::memset(&d, 0, sizeof(d));
  d.src = static_cast<const uint8_t*>(src_->data());
  d.src_h = to_i32(src_->shape(0), "height");
  d.src_w = to_i32(src_->shape(1), "width");
  d.pre_x = to_i32(pre_.x, "crop offset");
  d.pre_y = to_i32(pre_.y, "crop offset");
  d.pre_w = to_i32(pre_.w, "crop width");
  d.pre_h = to_i32(pre_.h, "crop height");
  d.pre_flip = pre_.flip ? 1 : 0;
  d.geom = geom_;
  d.geom_w = to_i32(geom_w_, "target width");
  d.geom_h = to_i32(geom_h_, "target height");
  std::memcpy(d.mx, mx_, sizeof(mx_));
  d.post_x = to_i32(post_.x, "crop offset");
  d.post_y = to_i32(post_.y, "crop offset");
  d.post_w = to_i32(post_.w, "crop width");
  d.post_h = to_i32(post_.h, "crop height");
  d.post_flip = post_.flip ? 1 : 0;
}

std::shared_ptr<Array> LazyImage::materialise() const {
  std::vector<LazyImage> one{*this};
  // an image between two ops lives in host memory, like every op result of the reference;
  // the slot of this batch of one is the image with its extension, filled with the extension's value
  auto batched = Runtime::get().batch(one, static_cast<double>(ext_value_), nullptr, Placement());
  // drop the leading batch dimension; storage is shared
  return std::make_shared<Array>(
      batched->type(), std::vector<int64_t>{batched->shape(1), batched->shape(2), batched->shape(3)},
      batched->storage());
}

// ---------------------------------------------------------------- Runtime
Runtime& Runtime::get() {
  static Runtime* rt = new Runtime();  // never destroyed: arrays may outlive static teardown
  return *rt;
}

void Runtime::set_device(int device) {
  g_device = device;
}

int Runtime::device() {
  if (g_device < 0) {
    g_device = env_int("MLXD_DEVICE", env_int("LOCAL_RANK", 0));
  }
  return g_device;
}

std::pair<int, int> Runtime::bind_host_threads_to_device_node() {
  char bus[32] = {0};
  if (mlxd_device_pci_bus_id(device(), bus, sizeof(bus)) != MLXD_OK) {
    return {-1, 0};
  }
  return bind_host_threads_to_node_of(bus, "/sys");
}

std::pair<int, int> Runtime::bind_host_threads_to_node_of(const std::string& pci_bus_id, const std::string& sysfs) {
  std::string bus = pci_bus_id;
  for (auto& c : bus) {
    c = static_cast<char>(std::tolower(static_cast<unsigned char>(c)));
  }
  auto first_line = [](const std::string& path, std::string& line) {
    FILE* f = std::fopen(path.c_str(), "r");
    if (!f) {
      return false;
    }
    char buf[4096];
    const bool ok = std::fgets(buf, sizeof(buf), f) != nullptr;
    std::fclose(f);
    if (ok) {
      line = buf;
      while (!line.empty() && (line.back() == '\n' || line.back() == ' ')) {
        line.pop_back();
      }
    }
    return ok && !line.empty();
  };
  std::string text;
  if (!first_line(sysfs + "/bus/pci/devices/" + bus + "/numa_node", text)) {
    return {-1, 0};
  }
  const int node = std::atoi(text.c_str());
  if (node < 0) {
    return {-1, 0};
  }
  // "0-15,64-79": the node's CPUs, intersected with what this process may use
  std::string list;
  if (!first_line(sysfs + "/devices/system/node/node" + std::to_string(node) + "/cpulist", list)) {
    return {-1, 0};
  }
  cpu_set_t allowed, want;
  CPU_ZERO(&allowed);
  CPU_ZERO(&want);
  if (sched_getaffinity(0, sizeof(allowed), &allowed) != 0) {
    return {-1, 0};
  }
  int kept = 0;
  size_t at = 0;
  while (at < list.size()) {
    size_t end = list.find(',', at);
    if (end == std::string::npos) {
      end = list.size();
    }
    const std::string part = list.substr(at, end - at);
    const size_t dash = part.find('-');
    const int lo = std::atoi(part.c_str());
    const int hi = dash == std::string::npos ? lo : std::atoi(part.c_str() + dash + 1);
    for (int c = lo; c <= hi && c < CPU_SETSIZE; c++) {
      if (c >= 0 && CPU_ISSET(c, &allowed)) {
        CPU_SET(c, &want);
        kept++;
      }
    }
    at = end + 1;
  }
  if (kept == 0 || sched_setaffinity(0, sizeof(want), &want) != 0) {
    return {node, 0};
  }
  return {node, kept};
}

void Runtime::check(int rc) const {
  if (rc == MLXD_OK) {
    return;
  }
  const std::string msg = mlxd_last_error();
  if (rc == MLXD_ERR_INVALID) {
    throw std::runtime_error(msg);
  }
  throw std::runtime_error("mlx-data GPU path: " + msg);
}

mlxd_ctx* Runtime::ctx() {
  std::lock_guard<std::mutex> g(mu_);
  if (!ctx_) {
    n_lanes_ = std::max(1, env_int("MLXD_LANES", 8));
    pinned_pool_.limit = static_cast<size_t>(env_int("MLXD_PINNED_POOL_GIB", 16)) << 30;
    device_pool_.limit = static_cast<size_t>(env_int("MLXD_DEVICE_POOL_GIB", 32)) << 30;
    mlxd_ctx* c = nullptr;
    const int rc = mlxd_ctx_create(device(), n_lanes_, &c);
    if (rc != MLXD_OK) {
      throw std::runtime_error(
          std::string("mlx-data GPU path: cannot create a CUDA context (there is no CPU fallback): ") +
          mlxd_last_error());
    }
    ctx_ = c;
  }
  return ctx_;
}

int Runtime::acquire_lane() {
  ctx();
  std::unique_lock<std::mutex> lk(mu_);
  if (!lanes_ready_) {
    for (int i = n_lanes_ - 1; i >= 0; i--) {
      free_lanes_.push_back(i);
    }
    lanes_ready_ = true;
  }
  lane_cv_.wait(lk, [this] { return !free_lanes_.empty(); });
  // the lane released last is taken first: its staging buffers are already as
  // large as the work in flight needs
  const int ln = free_lanes_.back();
  free_lanes_.pop_back();
  return ln;
}

void Runtime::release_lane(int ln) {
  {
    std::lock_guard<std::mutex> g(mu_);
    free_lanes_.push_back(ln);
  }
  lane_cv_.notify_one();
}

Runtime::~Runtime() {}

namespace {
std::atomic<bool> g_rgba_independent{false};
}

void Runtime::set_rgba_resize_independent(bool accept) {
  g_rgba_independent.store(accept);
}

bool Runtime::rgba_resize_independent() {
  return g_rgba_independent.load();
}

void Runtime::set_device_output(bool on) {
  std::lock_guard<std::mutex> g(mu_);
  defaults_.device_output = on;
}

void Runtime::set_stream(void* cuda_stream, bool enabled) {
  std::lock_guard<std::mutex> g(mu_);
  defaults_.stream = cuda_stream;
  defaults_.use_stream = enabled;
}

Placement Runtime::placement() const {
  std::lock_guard<std::mutex> g(mu_);
  return defaults_;
}

bool Runtime::pool_take(Pool& pool, size_t bytes, size_t& held, Block& out) {
  std::lock_guard<std::mutex> g(mu_);
  auto it = pool.blocks.lower_bound(bytes);
  // Reuse the smallest free block that is large enough: at most 25 % larger
  // than asked for - or up to four times for requests of 64 MiB and more,
  // where a new allocation (and the release of an old one) costs milliseconds
  // and the batches of one pipeline differ in size by such factors.
  const size_t slack = bytes >= (size_t(64) << 20) ? 3 * bytes : bytes / 4;
  if (it != pool.blocks.end() && it->first <= bytes + slack) {
    out = it->second;
    held = it->first;
    pool.bytes -= it->first;
    pool.blocks.erase(it);
    return true;
  }
  return false;
}

bool Runtime::pool_give(Pool& pool, const Block& b, size_t bytes) {
  std::lock_guard<std::mutex> g(mu_);
  if (pool.bytes + bytes <= pool.limit) {
    pool.blocks.emplace(bytes, b);
    pool.bytes += bytes;
    return true;
  }
  return false;
}

std::shared_ptr<Array> Runtime::pooled_array(
    ArrayType type, const std::vector<int64_t>& shape, bool on_device, const void* const* queued_on) {
  mlxd_ctx* c = ctx();
  int64_t n = array_type_size(type);
  for (auto d : shape) {
    n *= d;
  }
  size_t bytes = static_cast<size_t>(std::max<int64_t>(n, 1));
  bytes = (bytes + 4095) & ~size_t(4095);
  Pool& pool = on_device ? device_pool_ : pinned_pool_;
  size_t held = bytes;  // a recycled block goes back under the size it was allocated with
  Block blk{nullptr, false, nullptr};
  if (pool_take(pool, bytes, held, blk)) {
    // Work queued on a caller's stream may still use the block (the kernel
    // that filled it, the caller's consumers queued before it was dropped).
    // The same stream orders itself; anyone else waits for that stream.
    if (blk.tagged && !(queued_on && *queued_on == blk.stream)) {
      int32_t word = 0;
      const int rc = mlxd_stream_status(c, blk.stream, &word);
      if (rc != MLXD_OK) {
        pool_give(pool, blk, held);
        check(rc);
      }
    }
  } else {
    blk.p = on_device ? mlxd_device_alloc(c, bytes) : mlxd_pinned_alloc(bytes);
    if (!blk.p) {
      throw std::runtime_error(std::string("mlx-data GPU path: ") + mlxd_last_error());
    }
  }
  Runtime* self = this;
  const Block back{blk.p, queued_on != nullptr, queued_on ? const_cast<void*>(*queued_on) : nullptr};
  std::shared_ptr<void> storage(blk.p, [self, held, on_device, c, back](void* q) {
    Pool& to = on_device ? self->device_pool_ : self->pinned_pool_;
    if (!self->pool_give(to, back, held)) {
      if (on_device) {
        mlxd_device_free(c, q);   // cudaFree waits for the device
      } else {
        mlxd_pinned_free(q);
      }
    }
  });
  return std::make_shared<Array>(type, shape, storage, on_device ? device() : -1);
}

std::shared_ptr<Array> Runtime::pinned_array(ArrayType type, const std::vector<int64_t>& shape) {
  return pooled_array(type, shape, false, nullptr);
}

std::shared_ptr<Array> Runtime::device_array(
    ArrayType type, const std::vector<int64_t>& shape, const void* const* queued_on) {
  return pooled_array(type, shape, true, queued_on);
}

std::shared_ptr<Array> Runtime::batch(
    const std::vector<LazyImage>& images, double pad_value, const CastSpec* cast, const Placement& where) {
  if (images.empty()) {
    throw std::runtime_error("Array: cannot batch an empty list of arrays");
  }
  const int n = static_cast<int>(images.size());
  const LazyImage& first = images.front();
  int64_t max_h = 0, max_w = 0;
  int on_device = 0;
  std::vector<mlxd_sample_desc> descs(images.size());
  for (int i = 0; i < n; i++) {
    const LazyImage& im = images[i];
    if (im.source()->type() != UInt8) {
      throw std::invalid_argument("image must be of type UInt8");
    }
    if (im.source_channels() != first.source_channels() || im.is_gray() != first.is_gray()) {
      throw std::runtime_error("BatchShape: batched arrays expected to have consistent shapes");
    }
    on_device += im.source()->device() >= 0 ? 1 : 0;
    im.describe(descs[i]);
    max_h = std::max(max_h, im.height());
    max_w = std::max(max_w, im.width());
  }
  if (on_device != 0 && on_device != n) {
    throw std::runtime_error("batch: a batch cannot mix host and GPU-resident images");
  }
  const bool src_dev = on_device == n;
  const bool dst_dev = where.device_output;
  mlxd_batch_desc b;
  std::memset(&b, 0, sizeof(b));
  b.slot_h = to_i32(max_h, "height");
  b.slot_w = to_i32(max_w, "width");
  b.channels = static_cast<int32_t>(first.source_channels());
  if (first.is_gray()) {
    b.gray = 1;
    first.gray_params(b.gray_m, b.gray_bias);
  }
  b.pad_value = pad_value;
  b.src_mem = src_dev ? MLXD_MEM_DEVICE : MLXD_MEM_HOST;
  b.dst_mem = dst_dev ? MLXD_MEM_DEVICE : MLXD_MEM_HOST;
  b.divisor = 1.0f;
  ArrayType out_type = UInt8;
  if (cast) {
    out_type = Float;
    b.out_dtype = MLXD_F32;
    b.divisor = cast->divisor;
    b.normalise = cast->normalise ? 1 : 0;
    std::memcpy(b.mean, cast->mean, sizeof(b.mean));
    std::memcpy(b.std_, cast->std_, sizeof(b.std_));
  }
  const std::vector<int64_t> shape{n, max_h, max_w, first.channels()};
  const bool on_callers_stream = src_dev && dst_dev && where.use_stream;
  const void* callers_stream = where.stream;
  auto out = dst_dev ? device_array(out_type, shape, on_callers_stream ? &callers_stream : nullptr)
                     : pinned_array(out_type, shape);
  b.dst = out->data();
  mlxd_ctx* c = ctx();
  if (on_callers_stream) {
    // everything stays on the GPU: queue on the caller's stream and return
    check(mlxd_fused_batch_on_stream(c, where.stream, descs.data(), n, &b));
    return out;
  }
  // one lane per call in flight, whatever thread makes the call
  const int ln = acquire_lane();
  int rc = mlxd_fused_batch(c, ln, descs.data(), n, &b);
  if (rc == MLXD_OK) {
    rc = mlxd_batch_wait(c, ln, -1);
  }
  release_lane(ln);
  check(rc);
  return out;
}

std::shared_ptr<Array> Runtime::cast(const std::shared_ptr<const Array>& arr, const CastSpec& spec) {
  if (arr->type() != UInt8) {
    throw std::invalid_argument("cast: array must be of type UInt8");
  }
  if (arr->ndim() < 1 || arr->shape(arr->ndim() - 1) < 1 || arr->shape(arr->ndim() - 1) > 4) {
    throw std::runtime_error("cast: the last dimension must hold 1 to 4 channels");
  }
  arr->require_host("cast of a stand-alone array");
  const int c = static_cast<int>(arr->shape(arr->ndim() - 1));
  auto out = pinned_array(Float, arr->shape());
  if (arr->size() == 0) {
    return out;
  }
  check(mlxd_cast_scale_normalise(
      ctx(), static_cast<const uint8_t*>(arr->data()), arr->size() / c, c, spec.divisor,
      spec.normalise ? spec.mean : nullptr, spec.normalise ? spec.std_ : nullptr,
      static_cast<float*>(out->data())));
  return out;
}

} // namespace gpu
} // namespace data
} // namespace mlx
