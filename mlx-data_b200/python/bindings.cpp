// pybind11 module `_c`: the Python face of the C++ pipeline, with the class,
// method and keyword names of mlx-data's bindings (python/src/wrap_stream.cpp,
// wrap_buffer.cpp, wrap_dataset.h, wrap_core.cpp) for the ops on the
// image-transform-and-batch path.  Arrays cross the boundary without a copy in
// both directions; every call into the pipeline releases the GIL and Python
// callbacks take it back.
#include <pybind11/functional.h>
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <optional>
#include <sstream>

#include "mlx/data/Buffer.h"
#include "mlx/data/Stream.h"
#include "mlx/data/core/State.h"
#include "mlx/data/core/image/Jpeg.h"
#include "mlx/data/core/image/Png.h"
#include "mlx/data/gpu/Runtime.h"

namespace py = pybind11;
using namespace mlx::data;

namespace {

// Delete pipeline objects without the GIL: their destructors may join worker
// threads that are waiting for it.
template <class T>
struct ReleaseGilDeleter {
  void operator()(T* p) const {
    py::gil_scoped_release nogil;
    delete p;
  }
};

ArrayType dtype_to_type(const py::dtype& dt) {
  const char kind = dt.kind();
  const auto size = dt.itemsize();
  if (kind == 'u' && size == 1) return UInt8;
  if ((kind == 'i' && size == 1) || kind == 'S') return Int8;
  if (kind == 'i' && size == 4) return Int32;
  if (kind == 'i' && size == 8) return Int64;
  if (kind == 'f' && size == 4) return Float;
  if (kind == 'f' && size == 8) return Double;
  throw std::invalid_argument(
      "[to_array] Unsupported dtype " + std::string(py::str(dt)) +
      " (uint8, int8, int32, int64, float32 and float64 are accepted)");
}

// numpy -> Array, sharing memory.  The Array holds a reference to the numpy
// object and drops it under the GIL.
std::shared_ptr<Array> wrap_numpy(py::array a) {
  if (!(a.flags() & py::array::c_style)) {
    throw std::runtime_error("[to_array] Contiguous array expected -- use numpy.ascontiguousarray()");
  }
  const ArrayType type = dtype_to_type(a.dtype());
  std::vector<int64_t> shape(a.shape(), a.shape() + a.ndim());
  if (a.dtype().kind() == 'S') {
    shape.push_back(a.dtype().itemsize());
  }
  PyObject* keep = a.inc_ref().ptr();
  std::shared_ptr<void> storage(const_cast<void*>(a.data()), [keep](void*) {
    py::gil_scoped_acquire gil;
    Py_DECREF(keep);
  });
  return std::make_shared<Array>(type, shape, storage);
}

// A GPU-resident array as Python sees it: shape, dtype and the CUDA array
// interface, which torch.as_tensor / cupy.asarray consume without a copy.
struct PyDeviceArray {
  std::shared_ptr<const Array> a;
};

const char* typestr_of(ArrayType t) {
  switch (t) {
    case Int8: return "|i1";
    case UInt8: return "|u1";
    case Int32: return "<i4";
    case Int64: return "<i8";
    case Float: return "<f4";
    case Double: return "<f8";
    default: throw std::runtime_error("internal error: unknown type");
  }
}

// Object exposing __cuda_array_interface__ (a torch CUDA tensor, a cupy array)
// -> Array that shares its GPU memory and keeps the object alive.
std::shared_ptr<Array> wrap_cuda(py::handle obj) {
  py::dict iface = obj.attr("__cuda_array_interface__").cast<py::dict>();
  if (iface.contains("strides") && !iface["strides"].is_none()) {
    throw std::runtime_error("[to_array] Contiguous GPU array expected -- call .contiguous() first");
  }
  const std::string typestr = iface["typestr"].cast<std::string>();
  const py::dtype dt(typestr);
  const ArrayType type = dtype_to_type(dt);
  const auto shape = iface["shape"].cast<std::vector<int64_t>>();
  const auto data = iface["data"].cast<py::tuple>();
  void* ptr = reinterpret_cast<void*>(data[0].cast<uintptr_t>());
  PyObject* keep = obj.inc_ref().ptr();
  std::shared_ptr<void> storage(ptr, [keep](void*) {
    py::gil_scoped_acquire gil;
    Py_DECREF(keep);
  });
  return std::make_shared<Array>(type, shape, storage, gpu::Runtime::device());
}

py::object to_python(const std::shared_ptr<const Array>& a);

std::shared_ptr<Array> to_array(py::handle obj) {
  if (py::isinstance<PyDeviceArray>(obj)) {
    return std::make_shared<Array>(obj.cast<PyDeviceArray&>().a);
  }
  if (py::hasattr(obj, "__cuda_array_interface__")) {
    return wrap_cuda(obj);
  }
  if (py::isinstance<py::array>(obj)) {
    return wrap_numpy(py::reinterpret_borrow<py::array>(obj));
  }
  if (py::isinstance<py::bool_>(obj) || py::isinstance<py::int_>(obj)) {
    return std::make_shared<Array>(obj.cast<int64_t>());
  }
  if (py::isinstance<py::float_>(obj)) {
    return std::make_shared<Array>(obj.cast<double>());
  }
  if (py::isinstance<py::bytes>(obj)) {
    return std::make_shared<Array>(obj.cast<std::string>());
  }
  if (py::isinstance<py::str>(obj)) {
    throw std::invalid_argument(
        "[to_array] Cannot convert strings to arrays. Please encode them as bytes first.");
  }
  // anything else: let numpy interpret it, then copy (the temporary is ours)
  py::array converted;
  try {
    converted = py::array::ensure(obj, py::array::c_style);
  } catch (...) {
    converted = py::array();
  }
  if (!converted || converted.dtype().kind() == 'O') {
    PyErr_Clear();
    throw std::invalid_argument(
        "[to_array] Cannot convert type " + std::string(py::str(py::type::of(obj))) +
        " to an array. Use a numpy array, a python buffer or scalar.");
  }
  return array::clone(wrap_numpy(converted));
}

py::array to_numpy(const std::shared_ptr<const Array>& a) {
  if (!a) {
    throw std::runtime_error("Stream: empty value in sample");
  }
  const char* fmt = nullptr;
  switch (a->type()) {
    case Int8: fmt = "i1"; break;
    case UInt8: fmt = "u1"; break;
    case Int32: fmt = "i4"; break;
    case Int64: fmt = "i8"; break;
    case Float: fmt = "f4"; break;
    case Double: fmt = "f8"; break;
    default: throw std::runtime_error("internal error: unknown type");
  }
  // the capsule owns one shared_ptr and so keeps the storage alive
  auto* holder = new std::shared_ptr<const Array>(a);
  py::capsule owner(holder, [](void* p) { delete static_cast<std::shared_ptr<const Array>*>(p); });
  std::vector<py::ssize_t> shape(a->shape().begin(), a->shape().end());
  std::vector<py::ssize_t> strides(shape.size());
  py::ssize_t step = static_cast<py::ssize_t>(a->itemsize());
  for (int d = static_cast<int>(shape.size()) - 1; d >= 0; d--) {
    strides[d] = step;
    step *= shape[d];
  }
  return py::array(py::dtype(fmt), shape, strides, a->data(), owner);
}

py::object to_python(const std::shared_ptr<const Array>& a) {
  if (a && a->device() >= 0) {
    return py::cast(PyDeviceArray{a});
  }
  return to_numpy(a);
}

py::dict to_py_sample(const Sample& s) {
  py::dict d;
  for (auto& kv : s) {
    d[py::str(kv.first)] = to_python(kv.second);
  }
  return d;
}

Sample to_sample(const py::dict& d) {
  Sample s;
  for (auto item : d) {
    s[item.first.cast<std::string>()] = to_array(item.second);
  }
  return s;
}

gpu::CastSpec make_cast(const std::string& dtype, double scale, const std::optional<std::vector<float>>& mean,
                        const std::optional<std::vector<float>>& std_) {
  if (dtype != "float32") {
    throw std::invalid_argument("key_cast: only dtype=\"float32\" is available");
  }
  if (mean.has_value() != std_.has_value()) {
    throw std::invalid_argument("key_cast: mean and std must be given together");
  }
  gpu::CastSpec spec;
  spec.divisor = static_cast<float>(scale);
  if (mean) {
    if (mean->size() != std_->size() || mean->empty() || mean->size() > 4) {
      throw std::invalid_argument("key_cast: mean and std need one value per channel (1 to 4)");
    }
    spec.normalise = true;
    for (size_t i = 0; i < 4; i++) {
      // a single value applies to every channel
      spec.mean[i] = (*mean)[mean->size() == 1 ? 0 : std::min(i, mean->size() - 1)];
      spec.std_[i] = (*std_)[std_->size() == 1 ? 0 : std::min(i, std_->size() - 1)];
    }
  }
  return spec;
}

template <class T, class PyClass>
void bind_ops(PyClass& c) {
  using nogil = py::call_guard<py::gil_scoped_release>;
  const char* okd = "output_key";
  // an int or a list of ints
  auto ints = [](py::object o) {
    std::vector<int64_t> v;
    if (py::isinstance<py::int_>(o)) {
      v.push_back(o.cast<int64_t>());
    } else {
      v = o.cast<std::vector<int64_t>>();
    }
    return v;
  };
  c.def("slice",
        [ints](const T& self, const std::string& ikey, py::object dims, py::object starts, py::object ends,
               const std::string& okey) {
          const auto d = ints(dims);
          auto s = ints(starts), e = ints(ends);
          py::gil_scoped_release release;
          return self.slice(ikey, std::vector<int>(d.begin(), d.end()), std::move(s), std::move(e), okey);
        },
        py::arg("ikey"), py::arg("dims"), py::arg("starts"), py::arg("ends"), py::arg(okd) = "",
        "Keep ``[starts, ends)`` along ``dims`` of the array at ``ikey`` (ints or equally long lists).");
  c.def("random_slice",
        [ints](const T& self, const std::string& ikey, py::object dims, py::object sizes, const std::string& okey) {
          const auto d = ints(dims);
          auto s = ints(sizes);
          py::gil_scoped_release release;
          return self.random_slice(ikey, std::vector<int>(d.begin(), d.end()), std::move(s), okey);
        },
        py::arg("ikey"), py::arg("dims"), py::arg("sizes"), py::arg(okd) = "",
        "Keep a window of ``sizes`` along ``dims`` at a uniformly random offset.");
  c.def("slice_if",
        [ints](const T& self, bool cond, const std::string& ikey, py::object dims, py::object starts, py::object ends,
               const std::string& okey) {
          const auto d = ints(dims);
          auto s = ints(starts), e = ints(ends);
          py::gil_scoped_release release;
          return self.slice_if(cond, ikey, std::vector<int>(d.begin(), d.end()), std::move(s), std::move(e), okey);
        },
        py::arg("cond"), py::arg("ikey"), py::arg("dims"), py::arg("starts"), py::arg("ends"), py::arg(okd) = "");
  c.def("random_slice_if",
        [ints](const T& self, bool cond, const std::string& ikey, py::object dims, py::object sizes,
               const std::string& okey) {
          const auto d = ints(dims);
          auto s = ints(sizes);
          py::gil_scoped_release release;
          return self.random_slice_if(cond, ikey, std::vector<int>(d.begin(), d.end()), std::move(s), okey);
        },
        py::arg("cond"), py::arg("ikey"), py::arg("dims"), py::arg("sizes"), py::arg(okd) = "");
  c.def("pad", &T::pad, nogil(), py::arg("key"), py::arg("dim"), py::arg("lpad"), py::arg("rpad"),
        py::arg("pad_value"), py::arg(okd) = "", "Pad the array at ``key`` along ``dim`` on both sides.");
  c.def("pad_if", &T::pad_if, nogil(), py::arg("cond"), py::arg("key"), py::arg("dim"), py::arg("lpad"),
        py::arg("rpad"), py::arg("pad_value"), py::arg(okd) = "");
  c.def("pad_to_multiple", &T::pad_to_multiple, nogil(), py::arg("key"), py::arg("dim"), py::arg("pad_multiple"),
        py::arg("pad_value"), py::arg(okd) = "", "Pad the end of ``dim`` up to a multiple of ``pad_multiple``.");
  c.def("pad_to_multiple_if", &T::pad_to_multiple_if, nogil(), py::arg("cond"), py::arg("key"), py::arg("dim"),
        py::arg("pad_multiple"), py::arg("pad_value"), py::arg(okd) = "");
  c.def("pad_to_size",
        [](const T& self, const std::string& key, int dim, py::object size, double pad_value, const std::string& okey) {
          std::vector<int64_t> sizes;
          if (py::isinstance<py::int_>(size)) {
            sizes.push_back(size.cast<int64_t>());
          } else {
            sizes = size.cast<std::vector<int64_t>>();
          }
          py::gil_scoped_release release;
          return self.pad_to_size(key, dim, sizes, pad_value, okey);
        },
        py::arg("key"), py::arg("dim"), py::arg("size"), py::arg("pad_value"), py::arg(okd) = "",
        "Pad the end of ``dim`` up to ``size`` (or the nearest larger entry of a list of sizes).");
  c.def("pad_to_size_if",
        [](const T& self, bool cond, const std::string& key, int dim, py::object size, double pad_value,
           const std::string& okey) {
          std::vector<int64_t> sizes;
          if (py::isinstance<py::int_>(size)) {
            sizes.push_back(size.cast<int64_t>());
          } else {
            sizes = size.cast<std::vector<int64_t>>();
          }
          py::gil_scoped_release release;
          return self.pad_to_size_if(cond, key, dim, sizes, pad_value, okey);
        },
        py::arg("cond"), py::arg("key"), py::arg("dim"), py::arg("size"), py::arg("pad_value"), py::arg(okd) = "");
  c.def("load_image", &T::load_image, nogil(), py::arg("key"), py::arg("prefix") = "", py::arg("info") = false,
        py::arg("format") = "RGB", py::arg("from_memory") = false, py::arg(okd) = "",
        "Load the image file named by the array at ``key`` (or, with ``from_memory``, held in it) as uint8 "
        "[H, W, C], or with ``info`` its (width, height).  This build decodes binary PNM (P5, P6) only; the "
        "pixels land in page-locked memory that the GPU reads directly.");
  c.def("load_image_if", &T::load_image_if, nogil(), py::arg("cond"), py::arg("key"), py::arg("prefix") = "",
        py::arg("info") = false, py::arg("format") = "RGB", py::arg("from_memory") = false, py::arg(okd) = "");
  c.def("image_center_crop", &T::image_center_crop, nogil(), py::arg("key"), py::arg("w"), py::arg("h"),
        py::arg(okd) = "", "Center crop the image at ``key`` to ``w`` x ``h``.");
  c.def("image_center_crop_if", &T::image_center_crop_if, nogil(), py::arg("cond"), py::arg("key"), py::arg("w"),
        py::arg("h"), py::arg(okd) = "");
  c.def("image_channel_reduction", &T::image_channel_reduction, nogil(), py::arg("key"),
        py::arg("preset") = "default", py::arg(okd) = "",
        "Reduce an RGB image to one channel with a named luma mix (default, rec601, rec709, rec2020, green).");
  c.def("image_channel_reduction_if", &T::image_channel_reduction_if, nogil(), py::arg("cond"), py::arg("key"),
        py::arg("preset") = "default", py::arg(okd) = "");
  c.def("image_random_area_crop", &T::image_random_area_crop, nogil(), py::arg("key"), py::arg("area_range"),
        py::arg("aspect_ratio_range"), py::arg("num_trial") = 10, py::arg(okd) = "",
        "Crop a random rectangle whose area fraction and aspect ratio fall in the given ranges.");
  c.def("image_random_area_crop_if", &T::image_random_area_crop_if, nogil(), py::arg("cond"), py::arg("key"),
        py::arg("area_range"), py::arg("aspect_ratio_range"), py::arg("num_trial") = 10, py::arg(okd) = "");
  c.def("image_random_crop", &T::image_random_crop, nogil(), py::arg("key"), py::arg("w"), py::arg("h"),
        py::arg(okd) = "", "Crop a ``w`` x ``h`` window at a uniformly random position.");
  c.def("image_random_crop_if", &T::image_random_crop_if, nogil(), py::arg("cond"), py::arg("key"), py::arg("w"),
        py::arg("h"), py::arg(okd) = "");
  c.def("image_random_h_flip", &T::image_random_h_flip, nogil(), py::arg("key"), py::arg("prob"),
        py::arg(okd) = "", "Mirror the image left-right with probability ``prob``.");
  c.def("image_random_h_flip_if", &T::image_random_h_flip_if, nogil(), py::arg("cond"), py::arg("key"),
        py::arg("prob"), py::arg(okd) = "");
  c.def("image_resize", &T::image_resize, nogil(), py::arg("key"), py::arg("w"), py::arg("h"), py::arg(okd) = "",
        "Resize the image to ``w`` x ``h`` (triangle filter; may change the aspect ratio).");
  c.def("image_resize_if", &T::image_resize_if, nogil(), py::arg("cond"), py::arg("key"), py::arg("w"),
        py::arg("h"), py::arg(okd) = "");
  c.def("image_resize_smallest_side", &T::image_resize_smallest_side, nogil(), py::arg("key"), py::arg("size"),
        py::arg(okd) = "", "Resize so that the shorter side becomes ``size``, keeping the aspect ratio.");
  c.def("image_resize_smallest_side_if", &T::image_resize_smallest_side_if, nogil(), py::arg("cond"),
        py::arg("key"), py::arg("size"), py::arg(okd) = "");
  c.def("image_rotate", &T::image_rotate, nogil(), py::arg("key"), py::arg("angle"), py::arg("crop") = false,
        py::arg(okd) = "", py::arg("angle_key") = "",
        "Rotate by ``angle`` degrees (nearest neighbour); ``crop`` keeps the input size. With ``angle_key`` "
        "(an addition to mlx-data) the angle is read per sample from the float scalar at that key.");
  c.def("image_rotate_if", &T::image_rotate_if, nogil(), py::arg("cond"), py::arg("key"), py::arg("angle"),
        py::arg("crop") = false, py::arg(okd) = "", py::arg("angle_key") = "");

  auto key_transform = [](const T& ds, const std::string& key, py::function func, const std::string& okey) {
    // the callable is kept in a holder that is released under the GIL
    auto held = std::shared_ptr<py::function>(new py::function(std::move(func)), [](py::function* f) {
      py::gil_scoped_acquire gil;
      delete f;
    });
    auto fn = [held](const std::shared_ptr<const Array>& x) {
      py::gil_scoped_acquire gil;
      return to_array((*held)(to_python(x)));
    };
    py::gil_scoped_release nogil_scope;
    return ds.key_transform(key, fn, okey);
  };
  c.def("key_transform", key_transform, py::arg("key"), py::arg("func"), py::arg(okd) = "",
        "Apply the python function ``func`` to the array at ``key``.");
  c.def("key_transform_if",
        [key_transform](const T& ds, bool cond, const std::string& key, py::function func, const std::string& okey) {
          return cond ? key_transform(ds, key, std::move(func), okey) : T(ds.node());
        },
        py::arg("cond"), py::arg("key"), py::arg("func"), py::arg(okd) = "");

  auto sample_transform = [](const T& ds, py::function func) {
    auto held = std::shared_ptr<py::function>(new py::function(std::move(func)), [](py::function* f) {
      py::gil_scoped_acquire gil;
      delete f;
    });
    auto fn = [held](const Sample& s) {
      py::gil_scoped_acquire gil;
      py::object r = (*held)(to_py_sample(s));
      return to_sample(r.cast<py::dict>());
    };
    py::gil_scoped_release nogil_scope;
    return ds.sample_transform(fn);
  };
  c.def("sample_transform", sample_transform, py::arg("func"),
        "Apply the python function ``func`` to whole samples (dict in, dict out).");
  c.def("sample_transform_if",
        [sample_transform](const T& ds, bool cond, py::function func) {
          return cond ? sample_transform(ds, std::move(func)) : T(ds.node());
        },
        py::arg("cond"), py::arg("func"));

  auto key_cast = [](const T& ds, const std::string& key, const std::string& dtype, double scale,
                     std::optional<std::vector<float>> mean, std::optional<std::vector<float>> std_,
                     const std::string& okey) {
    const gpu::CastSpec spec = make_cast(dtype, scale, mean, std_);
    py::gil_scoped_release nogil_scope;
    return ds.key_cast(key, spec, okey);
  };
  c.def("key_cast", key_cast, py::arg("key"), py::arg("dtype") = "float32", py::arg("scale") = 255.0,
        py::arg("mean") = py::none(), py::arg("std") = py::none(), py::arg(okd) = "",
        R"doc(
        Cast the uint8 array at ``key`` to float32 on the GPU: ``x.astype("float32") / scale`` and,
        with ``mean`` and ``std`` (one value per channel), ``(x / scale - mean) / std`` - the same
        float32 arithmetic as the numpy expressions.  Placed directly after ``batch`` it is fused
        into the batch kernel.  (Not part of mlx-data, where this is a python lambda.)
        )doc");
  c.def("key_cast_if",
        [key_cast](const T& ds, bool cond, const std::string& key, const std::string& dtype, double scale,
                   std::optional<std::vector<float>> mean, std::optional<std::vector<float>> std_,
                   const std::string& okey) {
          return cond ? key_cast(ds, key, dtype, scale, mean, std_, okey) : T(ds.node());
        },
        py::arg("cond"), py::arg("key"), py::arg("dtype") = "float32", py::arg("scale") = 255.0,
        py::arg("mean") = py::none(), py::arg("std") = py::none(), py::arg(okd) = "");
}

struct BufferCursor {
  Buffer buffer;
  int64_t at = 0;
};

// A stream over a python iterable.  It is given the function that makes the
// iterable, not the iterable, so that reset() can start over.  Python objects
// are only touched with the interpreter lock held, which also serialises
// concurrent next() calls.
class PyIterableStream : public stream::Stream {
 public:
  explicit PyIterableStream(py::function factory) : factory_(new py::function(std::move(factory))) {}
  ~PyIterableStream() override {
    py::gil_scoped_acquire gil;
    cursor_.reset();
    factory_.reset();
  }

  Sample next() const override {
    py::gil_scoped_acquire gil;
    if (!cursor_) {
      cursor_.reset(new py::iterator(py::iter((*factory_)())));
    }
    if (*cursor_ == py::iterator::sentinel()) {
      return Sample();
    }
    py::handle item = **cursor_;
    if (!py::isinstance<py::dict>(item)) {
      throw std::invalid_argument("[stream_python_iterable] the iterable must yield dicts of arrays");
    }
    Sample s = to_sample(py::reinterpret_borrow<py::dict>(item));
    ++(*cursor_);
    return s;
  }

  void reset() override {
    py::gil_scoped_acquire gil;
    cursor_.reset();
  }

 private:
  std::unique_ptr<py::function> factory_;
  mutable std::unique_ptr<py::iterator> cursor_;
};

} // namespace

PYBIND11_MODULE(_c, m) {
  m.doc() = "B200-native image-transform-and-batch path with the mlx-data pipeline API";
  using nogil = py::call_guard<py::gil_scoped_release>;
  using MapD = std::unordered_map<std::string, double>;
  using MapI = std::unordered_map<std::string, int>;

  py::class_<PyDeviceArray>(m, "DeviceArray", py::module_local(),
                            "An array in GPU memory. Pass it to torch.as_tensor(x, device=\"cuda\") or "
                            "cupy.asarray(x) to use it without a copy, or call numpy() to fetch it.")
      .def_property_readonly("shape", [](const PyDeviceArray& d) { return py::tuple(py::cast(d.a->shape())); })
      .def_property_readonly("dtype", [](const PyDeviceArray& d) { return py::dtype(typestr_of(d.a->type())); })
      .def_property_readonly("device", [](const PyDeviceArray& d) { return d.a->device(); })
      .def_property_readonly("nbytes", [](const PyDeviceArray& d) { return d.a->size() * d.a->itemsize(); })
      .def_property_readonly("__cuda_array_interface__",
                             [](const PyDeviceArray& d) {
                               py::dict iface;
                               iface["shape"] = py::tuple(py::cast(d.a->shape()));
                               iface["typestr"] = typestr_of(d.a->type());
                               iface["data"] = py::make_tuple(reinterpret_cast<uintptr_t>(d.a->data()), false);
                               iface["version"] = 3;
                               iface["strides"] = py::none();
                               return iface;
                             })
      .def("__repr__", [](const PyDeviceArray& d) {
        std::ostringstream os;
        os << "DeviceArray(shape=(";
        for (size_t i = 0; i < d.a->shape().size(); i++) {
          os << (i ? ", " : "") << d.a->shape()[i];
        }
        os << "), device=" << d.a->device() << ")";
        return os.str();
      });

  py::class_<BufferCursor>(m, "BufferIterator", py::module_local())
      .def("__iter__", [](BufferCursor& c) -> BufferCursor& { return c; })
      .def("__next__", [](BufferCursor& c) {
        Sample s;
        {
          py::gil_scoped_release release;
          if (c.at < c.buffer.size()) {
            s = c.buffer.get(c.at++);
          }
        }
        if (s.empty()) {
          throw py::stop_iteration();
        }
        return to_py_sample(s);
      });

  py::class_<Buffer, std::unique_ptr<Buffer, ReleaseGilDeleter<Buffer>>> buffer(m, "Buffer", py::module_local());
  buffer.def("__iter__", [](Buffer& b) { return BufferCursor{b, 0}; })
      .def("size", &Buffer::size, nogil())
      .def("__len__", &Buffer::size, nogil())
      .def("__getitem__",
           [](const Buffer& b, int64_t idx) {
             Sample s;
             {
               py::gil_scoped_release release;
               if (idx < 0) {
                 idx += b.size();
               }
               s = b.get(idx);
             }
             return to_py_sample(s);
           },
           py::arg("idx"))
      .def("__repr__",
           [](const Buffer& b) {
             std::ostringstream os;
             os << "Buffer(size=" << b.size() << ")";
             return os.str();
           })
      .def("batch",
           [](const Buffer& b, py::object batch_size, const MapD& pad, const MapI& dim) {
             if (py::isinstance<py::int_>(batch_size)) {
               const int64_t n = batch_size.cast<int64_t>();
               py::gil_scoped_release release;
               return b.batch(n, pad, dim);
             }
             const auto sizes = batch_size.cast<std::vector<int64_t>>();
             py::gil_scoped_release release;
             return b.batch(sizes, pad, dim);
           },
           py::arg("batch_size"), py::arg("pad") = MapD(), py::arg("dim") = MapI(),
           "Batch consecutive samples; ``batch_size`` is an int or a list of sizes. Arrays are padded "
           "to the largest shape in the batch with ``pad[key]`` (default 0).")
      .def("dynamic_batch",
           [](const Buffer& b, const std::string& key, const std::optional<Buffer>& size_buffer, int64_t min_data_size,
              int64_t max_data_size, const MapD& pad, const MapI& dim, bool drop_outliers) {
             py::gil_scoped_release release;
             if (size_buffer) {
               return b.dynamic_batch(*size_buffer, key, min_data_size, max_data_size, pad, dim, drop_outliers);
             }
             return b.dynamic_batch(key, min_data_size, max_data_size, pad, dim, drop_outliers);
           },
           py::arg("key"), py::kw_only(), py::arg("size_buffer") = py::none(), py::arg("min_data_size") = -1,
           py::arg("max_data_size") = -1, py::arg("pad") = MapD(), py::arg("dim") = MapI(),
           py::arg("drop_outliers") = false,
           "Batches with about the same number of elements of ``key`` after padding: samples are sorted by "
           "size and grouped so that every padded batch holds between ``min_data_size`` and ``max_data_size`` "
           "elements.")
      .def("ordered_prefetch", &Buffer::ordered_prefetch, nogil(), py::arg("prefetch_size"), py::arg("num_thread"),
           "Fetch samples in background threads, returning them in buffer order.")
      .def("partition", &Buffer::partition, nogil(), py::arg("num_partitions"), py::arg("partition"))
      .def("partition_if", &Buffer::partition_if, nogil(), py::arg("cond"), py::arg("num_partitions"),
           py::arg("partition"))
      .def("perm", &Buffer::perm, nogil(), py::arg("perm"),
           "The samples at the listed indices, in that order (indices may repeat or be left out).")
      .def("shuffle", &Buffer::shuffle, nogil(), "The buffer in a random order (drawn once, here).")
      .def("shuffle_if", &Buffer::shuffle_if, nogil(), py::arg("cond"))
      .def("to_stream", &Buffer::to_stream, nogil());
  bind_ops<Buffer>(buffer);

  auto stream_next = [](Stream& s) {
    Sample res;
    {
      py::gil_scoped_release release;
      res = s.next();
    }
    return to_py_sample(res);
  };
  py::class_<Stream, std::unique_ptr<Stream, ReleaseGilDeleter<Stream>>> stream(m, "Stream", py::module_local());
  stream.def("__iter__", [](Stream& s) { return s; })
      .def("__next__",
           [](Stream& s) {
             Sample res;
             {
               py::gil_scoped_release release;
               res = s.next();
             }
             if (res.empty()) {
               throw py::stop_iteration();
             }
             return to_py_sample(res);
           })
      .def("__call__", stream_next)
      .def("next", stream_next)
      .def("__repr__", [](const Stream&) { return "Stream()"; })
      .def("reset", &Stream::reset, nogil())
      .def("batch", &Stream::batch, nogil(), py::arg("batch_size"), py::arg("pad") = MapD(), py::arg("dim") = MapI())
      .def("dynamic_batch", &Stream::dynamic_batch, nogil(), py::arg("buffer_size"), py::arg("key"), py::kw_only(),
           py::arg("min_data_size") = -1, py::arg("max_data_size") = -1, py::arg("pad") = MapD(),
           py::arg("dim") = MapI(), py::arg("shuffle") = false, py::arg("drop_outliers") = false,
           py::arg("max_skipped_samples") = 1000, py::arg("num_threads") = 1,
           "Batches of about the same number of elements of the array at ``key``: ``buffer_size`` samples are "
           "pulled at a time, ordered by size and cut into batches holding between ``min_data_size`` and "
           "``max_data_size`` elements after padding; samples that fit nowhere (at most "
           "``max_skipped_samples``) join the next pull.")
      .def("repeat", &Stream::repeat, nogil(), py::arg("num_time"),
           "Start the stream over ``num_time`` times before it ends; without end when ``num_time`` <= 0.")
      .def("partition", &Stream::partition, nogil(), py::arg("num_partitions"), py::arg("partition"))
      .def("partition_if", &Stream::partition_if, nogil(), py::arg("cond"), py::arg("num_partitions"),
           py::arg("partition"))
      .def("prefetch", &Stream::prefetch, nogil(), py::arg("prefetch_size"), py::arg("num_threads"))
      .def("prefetch_if", &Stream::prefetch_if, nogil(), py::arg("cond"), py::arg("prefetch_size"),
           py::arg("num_threads"))
      .def("to_buffer", &Stream::to_buffer, nogil());
  bind_ops<Stream>(stream);

  m.def("buffer_from_vector",
        [](const std::vector<py::dict>& data) {
          std::vector<Sample> samples;
          samples.reserve(data.size());
          for (auto& d : data) {
            samples.push_back(to_sample(d));
          }
          py::gil_scoped_release release;
          return buffer_from_vector(std::move(samples));
        },
        py::arg("data"), "Make a buffer from a list of dicts of arrays (numpy arrays are not copied).");

  m.def("stream_python_iterable",
        [](py::function iterable_factory) {
          return Stream(std::make_shared<PyIterableStream>(std::move(iterable_factory)));
        },
        py::arg("iterable_factory"),
        "A stream over the dicts of arrays that ``iterable_factory()`` yields; reset() calls the factory again.");

  py::module core = m.def_submodule("core", "Process-wide state");
  core.def("set_state", &core::set_state, py::arg("seed") = 1234,
           "Seed the random generator used by the random ops.");
  core.def("set_device", &gpu::Runtime::set_device, py::arg("device"),
           "Choose the CUDA device; call before the first op runs.");
  core.def("device", &gpu::Runtime::device);
  core.def("bind_host_threads_to_device_node",
           []() {
             const auto r = gpu::Runtime::bind_host_threads_to_device_node();
             return py::make_tuple(r.first, r.second);
           },
           "Keep this thread, and the threads started from it afterwards (the pipeline's workers), on the CPUs of "
           "the NUMA node the selected GPU is attached to, so page-locked buffers land in that node's memory.  "
           "Call it after set_device and before building pipelines.  Returns (node, cpus kept); (-1, 0) when the "
           "machine does not say.");
  core.def("pinned_empty",
           [](const std::vector<int64_t>& shape, const std::string& dtype) {
             const py::dtype dt(dtype);
             auto arr = gpu::Runtime::get().pinned_array(dtype_to_type(dt), shape);
             return to_numpy(arr);
           },
           py::arg("shape"), py::arg("dtype") = "uint8",
           "A numpy array in page-locked host memory: samples stored in such arrays are copied to the "
           "GPU asynchronously at full PCIe speed.");
  core.def("jpeg_decode",
           [](py::bytes file) {
             const std::string bytes = file;
             const auto* data = reinterpret_cast<const unsigned char*>(bytes.data());
             core::image::JpegHeader h;
             std::string why;
             if (!core::image::jpeg_header(data, bytes.size(), h, why)) {
               throw std::runtime_error("jpeg_decode: " + why);
             }
             py::array_t<uint8_t> out({h.height, h.width, (int64_t)3});
             if (!core::image::jpeg_decode(data, bytes.size(), out.mutable_data(), why)) {
               throw std::runtime_error("jpeg_decode: " + why);
             }
             return out;
           },
           py::arg("file"),
           "The pixels load_image produces for a JPEG file's bytes, as uint8 [H, W, 3] in ordinary "
           "memory (load_image itself decodes into page-locked memory and needs a GPU).");
  core.def("png_decode",
           [](py::bytes file) {
             const std::string bytes = file;
             const auto* data = reinterpret_cast<const unsigned char*>(bytes.data());
             core::image::PngHeader h;
             std::string why;
             if (!core::image::png_header(data, bytes.size(), h, why)) {
               throw std::runtime_error("png_decode: " + why);
             }
             py::array_t<uint8_t> out({h.height, h.width, (int64_t)h.out_channels});
             if (!core::image::png_decode(data, bytes.size(), h, out.mutable_data(), why)) {
               throw std::runtime_error("png_decode: " + why);
             }
             return out;
           },
           py::arg("file"),
           "The pixels load_image produces for a PNG file's bytes, as uint8 [H, W, C] in ordinary memory "
           "(load_image itself decodes into page-locked memory and needs a GPU).");
  core.def("bind_host_threads_to_node_of",
           [](const std::string& pci_bus_id, const std::string& sysfs) {
             const auto r = gpu::Runtime::bind_host_threads_to_node_of(pci_bus_id, sysfs);
             return py::make_tuple(r.first, r.second);
           },
           py::arg("pci_bus_id"), py::arg("sysfs") = "/sys",
           "bind_host_threads_to_device_node for a given PCI address and sysfs tree.");
  core.def("set_rgba_resize_independent", &gpu::Runtime::set_rgba_resize_independent, py::arg("accept"),
           "Resizing 4-channel images: mlx-data weights colour by alpha while filtering, this library filters the "
           "four channels independently, so results differ where alpha varies.  The resize ops refuse 4-channel "
           "images until this is called with True.");
  core.def("set_device_output", [](bool on) { gpu::Runtime::get().set_device_output(on); }, py::arg("on"),
           "Default for batch nodes built from now on: leave batches in GPU memory (returned as DeviceArray) "
           "instead of copying them to the host.  A pipeline keeps the setting it was built with.");
  core.def("set_stream",
           [](uintptr_t stream, bool enabled) {
             gpu::Runtime::get().set_stream(reinterpret_cast<void*>(stream), enabled);
           },
           py::arg("cuda_stream"), py::arg("enabled") = true,
           "Default for batch nodes built from now on: queue GPU-to-GPU work (GPU-resident samples and device "
           "output) on this CUDA stream handle without waiting for it; enabled=False goes back to the internal "
           "lanes.  A pipeline keeps the setting it was built with.  GPU-resident samples must have been "
           "written by work on this stream (or be complete); without a stream set, the internal lanes read "
           "them as they are, so they must be complete before the pipeline pulls them.");
  core.def("stream_status",
           [](uintptr_t stream) {
             int32_t word = 0;
             const int rc = mlxd_stream_status(gpu::Runtime::get().ctx(), reinterpret_cast<void*>(stream), &word);
             if (rc != MLXD_OK && rc != MLXD_ERR_DEVICE) {
               gpu::Runtime::get().check(rc);
             }
             return word;
           },
           py::arg("cuda_stream"),
           "Wait for the stream and return the self-check word of the kernels queued on it (0 = clean); "
           "reading clears it.");
  core.def("set_timing",
           [](bool on) { gpu::Runtime::get().check(mlxd_ctx_set_timing(gpu::Runtime::get().ctx(), on ? 1 : 0)); },
           py::arg("on"), "Time every fused kernel with CUDA events; totals appear in stats().");
  core.def("stats", []() {
    mlxd_stats s;
    gpu::Runtime::get().check(mlxd_stats_get(gpu::Runtime::get().ctx(), &s));
    py::dict d;
    d["batches"] = s.batches;
    d["samples"] = s.samples;
    d["kernel_launches"] = s.kernel_launches;
    d["h2d_bytes"] = s.h2d_bytes;
    d["d2h_bytes"] = s.d2h_bytes;
    d["device_bytes_reserved"] = s.device_bytes_reserved;
    d["kernel_ns"] = s.kernel_ns;
    d["timed_launches"] = s.timed_launches;
    d["algo_src_bytes"] = s.algo_src_bytes;
    d["algo_dst_bytes"] = s.algo_dst_bytes;
    d["h2d_ns"] = s.h2d_ns;
    d["d2h_ns"] = s.d2h_ns;
    d["host_stage_ns"] = s.host_stage_ns;
    return d;
  });
}
