#include "mlx/data/Array.h"

#include <algorithm>
#include <cstdlib>

namespace mlx {
namespace data {

int64_t array_type_size(ArrayType t) {
  switch (t) {
    case UInt8:
    case Int8:
      return 1;
    case Int32:
    case Float:
      return 4;
    case Int64:
    case Double:
      return 8;
    case Any:
      return 0;
  }
  throw std::runtime_error("Array: internal error: unknown type");
}

namespace {

int64_t count(const std::vector<int64_t>& shape) {
  int64_t n = 1;
  for (auto d : shape) {
    n *= d;
  }
  return n;
}

// Row-major element strides of a shape.
std::vector<int64_t> strides_of(const std::vector<int64_t>& shape) {
  std::vector<int64_t> st(shape.size(), 1);
  for (int d = static_cast<int>(shape.size()) - 2; d >= 0; d--) {
    st[d] = st[d + 1] * shape[d + 1];
  }
  return st;
}

// Copy the block `extent` found at `src_off` inside an array of shape
// `src_shape` to `dst_off` inside an array of shape `dst_shape`; the innermost
// dimension moves as one memcpy per row.
void copy_block(
    char* dst, const std::vector<int64_t>& dst_shape, const std::vector<int64_t>& dst_off,
    const char* src, const std::vector<int64_t>& src_shape, const std::vector<int64_t>& src_off,
    const std::vector<int64_t>& extent, int64_t itemsize) {
  const int nd = static_cast<int>(extent.size());
  if (nd == 0) {
    std::memcpy(dst, src, itemsize);
    return;
  }
  if (count(extent) == 0) {
    return;
  }
  const auto ds = strides_of(dst_shape);
  const auto ss = strides_of(src_shape);
  int64_t d0 = 0, s0 = 0;
  for (int d = 0; d < nd; d++) {
    d0 += dst_off[d] * ds[d];
    s0 += src_off[d] * ss[d];
  }
  const int64_t row = extent[nd - 1] * itemsize;
  std::vector<int64_t> idx(nd, 0);
  for (;;) {
    int64_t di = d0, si = s0;
    for (int d = 0; d < nd - 1; d++) {
      di += idx[d] * ds[d];
      si += idx[d] * ss[d];
    }
    std::memcpy(dst + di * itemsize, src + si * itemsize, row);
    int d = nd - 2;
    while (d >= 0 && ++idx[d] == extent[d]) {
      idx[d--] = 0;
    }
    if (d < 0) {
      break;
    }
  }
}

template <class T>
void fill_as(void* p, int64_t n, double value) {
  T* q = static_cast<T*>(p);
  const T v = static_cast<T>(value);
  std::fill(q, q + n, v);
}

} // namespace

Array::Array(ArrayType type, const std::vector<int64_t>& shape, std::shared_ptr<void> data, int device)
    : type_(type), shape_(shape), data_(std::move(data)), itemsize_(array_type_size(type)), device_(device) {
  if (type_ == Any && size() != 0) {
    throw std::runtime_error("Array: cannot create a tensor of undetermined type");
  }
}

void Array::require_host(const char* what) const {
  if (device_ >= 0) {
    throw std::runtime_error(std::string("Array: ") + what + " needs host memory, but the array lives on GPU " +
                             std::to_string(device_));
  }
}

Array::Array(ArrayType type, const std::vector<int64_t>& shape)
    : type_(type), shape_(shape), itemsize_(array_type_size(type)) {
  if (type_ == Any && size() != 0) {
    throw std::runtime_error("Array: cannot create a tensor of undetermined type");
  }
  const int64_t bytes = size() * itemsize_;
  if (bytes > 0) {
    void* p = std::malloc(static_cast<size_t>(bytes));
    if (!p) {
      throw std::bad_alloc();
    }
    data_ = std::shared_ptr<void>(p, std::free);
  }
}

Array::Array(const std::shared_ptr<const Array>& src)
    : type_(src->type_), shape_(src->shape_), data_(src->data_), itemsize_(src->itemsize_), device_(src->device_) {}

Array::Array(const std::string& str) : Array(std::string_view(str)) {}

Array::Array(std::string_view str) : Array(Int8, std::vector<int64_t>{static_cast<int64_t>(str.size())}) {
  if (!str.empty()) {
    std::memcpy(data_.get(), str.data(), str.size());
  }
}

int64_t Array::size() const {
  return count(shape_);
}

void Array::fill(double value) {
  require_host("fill");
  const int64_t n = size();
  switch (type_) {
    case UInt8:
      return fill_as<unsigned char>(data_.get(), n, value);
    case Int8:
      return fill_as<char>(data_.get(), n, value);
    case Int32:
      return fill_as<int32_t>(data_.get(), n, value);
    case Int64:
      return fill_as<int64_t>(data_.get(), n, value);
    case Float:
      return fill_as<float>(data_.get(), n, value);
    case Double:
      return fill_as<double>(data_.get(), n, value);
    default:
      throw std::runtime_error("Array: internal error: unsupported type");
  }
}

int Array::checkdim(int dim) const {
  const int nd = ndim();
  if (dim < 0) {
    dim += nd;
  }
  if (dim < 0 || dim >= nd) {
    throw std::runtime_error("Array: dimension out of bound");
  }
  return dim;
}

void Array::squeeze(const std::vector<int>& dims) {
  std::vector<bool> drop(shape_.size(), false);
  if (dims.empty()) {
    for (size_t i = 0; i < shape_.size(); i++) {
      drop[i] = shape_[i] == 1;
    }
  } else {
    for (int dim : dims) {
      dim = checkdim(dim);
      if (shape_[dim] != 1) {
        throw std::runtime_error("Array: cannot squeeze a non-singleton dimension");
      }
      drop[dim] = true;
    }
  }
  std::vector<int64_t> kept;
  for (size_t i = 0; i < shape_.size(); i++) {
    if (!drop[i]) {
      kept.push_back(shape_[i]);
    }
  }
  shape_ = kept;
}

void Array::reshape(const std::vector<int64_t>& shape) {
  std::vector<int64_t> ns = shape;
  int infer = -1;
  int64_t known = 1;
  for (size_t d = 0; d < ns.size(); d++) {
    if (ns[d] < 0) {
      if (infer >= 0) {
        throw std::runtime_error("Array: can infer only one dimension");
      }
      infer = static_cast<int>(d);
    } else {
      known *= ns[d];
    }
  }
  const int64_t total = size();
  if (infer >= 0) {
    if (known == 0 || total % known != 0) {
      throw std::runtime_error("Array: cannot infer dimension: incompatible shape provided");
    }
    ns[infer] = total / known;
    known *= ns[infer];
  }
  if (known != total) {
    throw std::runtime_error("Array: incompatible shape provided");
  }
  shape_ = ns;
}

namespace array {

std::shared_ptr<Array> clone(const std::shared_ptr<const Array>& arr) {
  arr->require_host("clone");
  auto res = std::make_shared<Array>(arr->type(), arr->shape());
  if (arr->size() > 0) {
    std::memcpy(res->data(), arr->data(), static_cast<size_t>(arr->size() * arr->itemsize()));
  }
  return res;
}

std::shared_ptr<Array> reshape(const std::shared_ptr<const Array>& arr, const std::vector<int64_t>& shape) {
  auto res = std::make_shared<Array>(arr);
  res->reshape(shape);
  return res;
}

std::shared_ptr<Array> squeeze(const std::shared_ptr<const Array>& arr, const std::vector<int>& dims) {
  auto res = std::make_shared<Array>(arr);
  res->squeeze(dims);
  return res;
}

std::shared_ptr<Array> pad(const std::shared_ptr<const Array>& arr, int dim, int64_t lpad, int64_t rpad, double value) {
  if (lpad == 0 && rpad == 0) {
    return std::make_shared<Array>(arr);
  }
  if (lpad < 0 || rpad < 0) {
    throw std::runtime_error("Array: pad must be positive");
  }
  arr->require_host("pad");
  if (dim < 0 || dim >= arr->ndim()) {
    throw std::runtime_error("Array: dim out of range");
  }
  auto shape = arr->shape();
  shape[dim] += lpad + rpad;
  auto res = std::make_shared<Array>(arr->type(), shape);
  res->fill(value);
  std::vector<int64_t> zero(shape.size(), 0), off(shape.size(), 0);
  off[dim] = lpad;
  copy_block(
      static_cast<char*>(res->data()), shape, off, static_cast<const char*>(arr->data()), arr->shape(), zero,
      arr->shape(), arr->itemsize());
  return res;
}

std::shared_ptr<Array> slice(const std::shared_ptr<const Array>& arr, int index0) {
  if (arr->ndim() == 0) {
    throw std::runtime_error("Array: cannot slice a scalar");
  }
  if (index0 < 0 || index0 >= arr->shape(0)) {
    throw std::runtime_error("Array: slice index out of bound");
  }
  std::vector<int64_t> shape(arr->shape().begin() + 1, arr->shape().end());
  const int64_t step = count(shape) * arr->itemsize();
  // aliasing constructor: the view keeps the parent's storage alive
  std::shared_ptr<void> view(arr->storage(), static_cast<char*>(arr->data()) + step * index0);
  return std::make_shared<Array>(arr->type(), shape, view, arr->device());
}

void copy(const std::shared_ptr<Array>& dst, const std::shared_ptr<const Array>& src) {
  if (dst->type() != src->type() || dst->shape() != src->shape()) {
    throw std::runtime_error("Array: copy expects arrays of the same type and shape");
  }
  dst->require_host("copy");
  src->require_host("copy");
  if (src->size() > 0) {
    std::memcpy(dst->data(), src->data(), static_cast<size_t>(src->size() * src->itemsize()));
  }
}

std::shared_ptr<Array> batch(const std::vector<std::shared_ptr<Array>>& arrs, double pad_value) {
  if (arrs.empty()) {
    throw std::runtime_error("Array: cannot batch an empty list of arrays");
  }
  const auto type = arrs.front()->type();
  const int nd = arrs.front()->ndim();
  std::vector<int64_t> shape(nd + 1, 0);
  shape[0] = static_cast<int64_t>(arrs.size());
  for (auto& a : arrs) {
    if (a->type() != type) {
      throw std::runtime_error("Array: unexpected different types of arrays in batch");
    }
    a->require_host("batch");
    if (a->ndim() != nd) {
      throw std::runtime_error("BatchShape: batched arrays expected to have consistent shapes");
    }
    for (int d = 0; d < nd; d++) {
      shape[d + 1] = std::max(shape[d + 1], a->shape(d));
    }
  }
  auto res = std::make_shared<Array>(type, shape);
  res->fill(pad_value);
  std::vector<int64_t> off(nd + 1, 0), zero(nd + 1, 0);
  for (size_t i = 0; i < arrs.size(); i++) {
    std::vector<int64_t> ext(nd + 1, 1);
    std::copy(arrs[i]->shape().begin(), arrs[i]->shape().end(), ext.begin() + 1);
    off[0] = static_cast<int64_t>(i);
    copy_block(
        static_cast<char*>(res->data()), shape, off, static_cast<const char*>(arrs[i]->data()), ext, zero, ext,
        res->itemsize());
  }
  return res;
}

std::shared_ptr<Array> batch(const std::vector<std::shared_ptr<Array>>& arrs, int dim, double pad_value) {
  if (arrs.empty()) {
    throw std::runtime_error("Array: cannot batch an empty list of arrays");
  }
  const auto type = arrs.front()->type();
  const int nd = arrs.front()->ndim();
  if (dim < 0) {
    dim += nd;
  }
  if (dim < 0 || dim >= nd) {
    throw std::runtime_error("BatchShape: dimension out of bound");
  }
  std::vector<int64_t> shape(nd, 0);
  for (auto& a : arrs) {
    if (a->type() != type) {
      throw std::runtime_error("Array: unexpected different types of arrays in batch");
    }
    a->require_host("batch");
    if (a->ndim() != nd) {
      throw std::runtime_error("BatchShape: batched arrays expected to have consistent shapes");
    }
    for (int d = 0; d < nd; d++) {
      shape[d] = d == dim ? shape[d] + a->shape(d) : std::max(shape[d], a->shape(d));
    }
  }
  auto res = std::make_shared<Array>(type, shape);
  res->fill(pad_value);
  std::vector<int64_t> off(nd, 0), zero(nd, 0);
  for (auto& a : arrs) {
    copy_block(
        static_cast<char*>(res->data()), shape, off, static_cast<const char*>(a->data()), a->shape(), zero,
        a->shape(), res->itemsize());
    off[dim] += a->shape(dim);
  }
  return res;
}

std::shared_ptr<Array> sub(const std::shared_ptr<const Array>& arr, std::vector<int64_t> offset, std::vector<int64_t> shape) {
  if (arr->ndim() != static_cast<int>(offset.size())) {
    throw std::runtime_error("Array: sub: array and offset dim mismatch");
  }
  if (arr->ndim() != static_cast<int>(shape.size())) {
    throw std::runtime_error("Array: sub: array and shape dim mismatch");
  }
  for (int d = 0; d < arr->ndim(); d++) {
    if (offset[d] < 0 || offset[d] >= arr->shape(d)) {
      throw std::runtime_error("Array: sub: offset out of bound");
    }
    if (shape[d] < 0) {
      shape[d] = arr->shape(d);
    }
    if (offset[d] + shape[d] > arr->shape(d)) {
      throw std::runtime_error("Array: sub: shape out of bound");
    }
  }
  arr->require_host("sub");
  auto res = std::make_shared<Array>(arr->type(), shape);
  std::vector<int64_t> zero(shape.size(), 0);
  copy_block(
      static_cast<char*>(res->data()), shape, zero, static_cast<const char*>(arr->data()), arr->shape(), offset,
      shape, arr->itemsize());
  return res;
}

} // namespace array
} // namespace data
} // namespace mlx
