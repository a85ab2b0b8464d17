"""TEST INFRASTRUCTURE - Python face of the CPU oracle (never shipped, never timed as the product).

Thin ctypes wrappers over ``liboracle_mlxd.so`` (built by ``make -C oracle oracle``)
plus a small chain runner that applies a list of ops the way a single-threaded
mlx-data stream does: per sample, op after op, then batch, then the cast.
The order of random draws follows mlx/data/op/ImageTransform.cpp (one generator,
draws in op order per sample, samples in stream order).
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle_mlxd.so")

_i64 = ctypes.c_int64
_u8p = ctypes.POINTER(ctypes.c_uint8)
_f32p = ctypes.POINTER(ctypes.c_float)
_i64p = ctypes.POINTER(ctypes.c_int64)

PRESETS = {
    # mlx/data/op/ImageTransform.cpp:384-404
    "default": (0.0, (0.299, 0.587, 0.114)),
    "rec601": (0.0, (0.299, 0.587, 0.114)),
    "rec709": (0.0, (0.2126, 0.7152, 0.0722)),
    "rec2020": (0.0, (0.2627, 0.678, 0.0593)),
    "green": (0.0, (0.0, 1.0, 0.0)),
}


def build():
    """Compile the C/C++ restatement (a few seconds)."""
    subprocess.check_call(["make", "-s", "-C", _HERE, "oracle"])


def _load():
    if not os.path.exists(_LIB_PATH):
        build()
    return ctypes.CDLL(_LIB_PATH)


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = _load()
        _lib.oracle_resize.restype = ctypes.c_int
    return _lib


def _p8(a):
    return a.ctypes.data_as(_u8p)


def _img(a):
    a = np.ascontiguousarray(a)
    assert a.dtype == np.uint8 and a.ndim == 3, (a.dtype, a.shape)
    return a


def resize(img, dw, dh):
    img = _img(img)
    h, w, c = img.shape
    out = np.empty((dh, dw, c), np.uint8)
    if lib().oracle_resize(_p8(img), _i64(h), _i64(w), _i64(c), _p8(out), _i64(dh), _i64(dw)) != 0:
        raise RuntimeError("image::resize: could not resize image")
    return out


def smallest_side_dims(h, w, size):
    dh, dw = _i64(), _i64()
    lib().oracle_smallest_side_dims(_i64(h), _i64(w), _i64(size), ctypes.byref(dh), ctypes.byref(dw))
    return dh.value, dw.value


def resize_smallest_side(img, size):
    dh, dw = smallest_side_dims(img.shape[0], img.shape[1], size)
    return resize(img, dw, dh)


def crop(img, x, y, w, h):
    img = _img(img)
    out = np.empty((h, w, img.shape[2]), np.uint8)
    rc = lib().oracle_crop(_p8(img), _i64(img.shape[0]), _i64(img.shape[1]), _i64(img.shape[2]),
                           _i64(x), _i64(y), _i64(w), _i64(h), _p8(out))
    if rc != 0:
        raise RuntimeError("crop out of bound")
    return out


def center_crop(img, w, h):
    ih, iw = img.shape[:2]
    if h > ih or w > iw:
        raise RuntimeError("ImageCenterCrop: target image size larger than input image")
    return crop(img, (iw - w) // 2, (ih - h) // 2, w, h)


def hflip(img):
    img = _img(img)
    out = np.empty_like(img)
    lib().oracle_hflip(_p8(img), _i64(img.shape[0]), _i64(img.shape[1]), _i64(img.shape[2]), _p8(out))
    return out


def rotate_matrix(angle):
    mx = (ctypes.c_float * 6)()
    lib().oracle_rotate_matrix(ctypes.c_double(angle), mx)
    return mx


def affine(img, mx, crop_):
    img = _img(img)
    h, w, c = img.shape
    th, tw = _i64(), _i64()
    lib().oracle_affine_dims(_i64(h), _i64(w), mx, ctypes.c_int(1 if crop_ else 0),
                             ctypes.byref(th), ctypes.byref(tw))
    out = np.empty((th.value, tw.value, c), np.uint8)
    lib().oracle_affine(_p8(img), _i64(h), _i64(w), _i64(c), mx, th, tw, _p8(out))
    return out


def rotate(img, angle, crop_=False):
    return affine(img, rotate_matrix(angle), crop_)


def channel_reduction(img, preset="default"):
    img = _img(img)
    if img.shape[2] != 3:
        raise RuntimeError("image::channelReduction: expected a 3 channel uint8 array")
    bias, m = PRESETS[preset]
    out = np.empty((img.shape[0], img.shape[1], 1), np.uint8)
    lib().oracle_channel_reduction(_p8(img), _i64(img.shape[0]), _i64(img.shape[1]),
                                   ctypes.c_float(bias), (ctypes.c_float * 3)(*m), _p8(out))
    return out


def batch_pad(imgs, pad=0.0):
    imgs = [_img(a) for a in imgs]
    n = len(imgs)
    c = imgs[0].shape[2]
    mh = max(a.shape[0] for a in imgs)
    mw = max(a.shape[1] for a in imgs)
    out = np.empty((n, mh, mw, c), np.uint8)
    ptrs = (_u8p * n)(*[_p8(a) for a in imgs])
    hs = (_i64 * n)(*[a.shape[0] for a in imgs])
    ws = (_i64 * n)(*[a.shape[1] for a in imgs])
    lib().oracle_batch_pad_u8(ptrs, hs, ws, _i64(n), _i64(c), _i64(mh), _i64(mw),
                              ctypes.c_double(pad), _p8(out))
    return out


def cast_f32(x, mean=None, std=None):
    x = np.ascontiguousarray(x)
    c = x.shape[-1]
    out = np.empty(x.shape, np.float32)
    if mean is None:
        mp = sp = None
    else:
        mean = np.ascontiguousarray(mean, np.float32)
        std = np.ascontiguousarray(std, np.float32)
        mp, sp = mean.ctypes.data_as(_f32p), std.ctypes.data_as(_f32p)
    lib().oracle_cast_f32(_p8(x), _i64(x.size // c), _i64(c), mp, sp, out.ctypes.data_as(_f32p))
    return out


def set_state(seed):
    lib().oracle_set_state(_i64(seed))


def draw_hflip(prob):
    return bool(lib().oracle_draw_hflip(ctypes.c_float(prob)))


def draw_random_crop(w, h, cw, ch):
    out = (_i64 * 4)()
    if lib().oracle_draw_random_crop(_i64(w), _i64(h), _i64(cw), _i64(ch), out) != 0:
        raise RuntimeError("ImageRandomCrop: target image size larger than input image")
    return tuple(out)


def draw_area_crop(w, h, area_range, ratio_range, num_trial=10):
    out = (_i64 * 4)()
    lib().oracle_draw_area_crop(_i64(w), _i64(h), ctypes.c_float(area_range[0]), ctypes.c_float(area_range[1]),
                                ctypes.c_float(ratio_range[0]), ctypes.c_float(ratio_range[1]),
                                ctypes.c_int(num_trial), out)
    return tuple(out)


def apply_op(sample, op):
    """Apply one op spec ``(method_name, kwargs)`` to a dict sample; names and
    keyword arguments are those of the reference's Python methods
    (python/src/wrap_dataset.h:83-362).  ``image_rotate`` also accepts
    ``angle_key``: the name of a float scalar in the sample holding that
    sample's angle (the reference op takes one fixed angle per op instance)."""
    name, kw = op
    key = kw["key"]
    okey = kw.get("output_key") or key
    img = sample[key]
    if name == "image_resize":
        out = resize(img, kw["w"], kw["h"])
    elif name == "image_resize_smallest_side":
        if kw["size"] <= 0:
            raise RuntimeError("ImageResizeSmallestSide: illegal target size: %d" % kw["size"])
        out = resize_smallest_side(img, kw["size"])
    elif name == "image_center_crop":
        out = center_crop(img, kw["w"], kw["h"])
    elif name == "image_random_crop":
        x, y, w, h = draw_random_crop(img.shape[1], img.shape[0], kw["w"], kw["h"])
        out = crop(img, x, y, w, h)
    elif name == "image_random_area_crop":
        x, y, w, h = draw_area_crop(img.shape[1], img.shape[0], kw["area_range"],
                                    kw["aspect_ratio_range"], kw.get("num_trial", 10))
        out = img if (w == 0 or h == 0) else crop(img, x, y, w, h)
    elif name == "image_random_h_flip":
        out = hflip(img) if draw_hflip(kw["prob"]) else img
    elif name == "image_rotate":
        angle = float(sample[kw["angle_key"]]) if "angle_key" in kw else kw["angle"]
        out = rotate(img, angle, kw.get("crop", False))
    elif name == "image_channel_reduction":
        out = channel_reduction(img, kw.get("preset", "default"))
    else:
        raise ValueError(name)
    res = dict(sample)
    res[okey] = out
    return res


def run_chain(samples, ops, batch_size, pad=None, cast=None):
    """Single-threaded stream semantics: every sample through every op, then
    batches of ``batch_size`` (short last batch kept, mlx/data/stream/Batch.cpp:25-39),
    then the cast on the keys named in ``cast`` = {key: None | (mean, std)}."""
    pad = pad or {}
    cast = cast or {}
    batches = []
    cur = []

    def flush():
        if not cur:
            return
        out = {}
        for k in cur[0].keys():
            vals = [s[k] for s in cur]
            if isinstance(vals[0], np.ndarray) and vals[0].ndim == 3 and vals[0].dtype == np.uint8:
                b = batch_pad(vals, pad.get(k, 0.0))
                if k in cast:
                    ms = cast[k]
                    b = cast_f32(b) if ms is None else cast_f32(b, ms[0], ms[1])
                out[k] = b
            else:
                out[k] = np.stack([np.asarray(v) for v in vals])
        batches.append(out)
        cur.clear()

    for s in samples:
        for op in ops:
            s = apply_op(s, op)
        cur.append(s)
        if len(cur) == batch_size:
            flush()
    flush()
    return batches
