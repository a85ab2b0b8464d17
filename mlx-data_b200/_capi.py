"""ctypes binding of the C ABI in include/mlxd_b200.h.

This is the thinnest possible Python face of ``libmlxd_b200.so``: the same
structs, the same entry points, numpy arrays or raw addresses in and out.
There is no CPU implementation behind it - loading fails loudly when the
library has not been built, and every call needs a CUDA device.
"""
import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libmlxd_b200.so")

OK, ERR_INVALID, ERR_CUDA, ERR_NOMEM, ERR_TIMEOUT, ERR_UNSUPPORTED, ERR_DEVICE = range(7)
GEOM_NONE, GEOM_RESIZE, GEOM_AFFINE = 0, 1, 2
U8, F32 = 0, 1
MEM_HOST, MEM_DEVICE = 0, 1


class SampleDesc(ctypes.Structure):
    _fields_ = [
        ("src", ctypes.c_void_p),
        ("src_h", ctypes.c_int32), ("src_w", ctypes.c_int32),
        ("pre_x", ctypes.c_int32), ("pre_y", ctypes.c_int32),
        ("pre_w", ctypes.c_int32), ("pre_h", ctypes.c_int32),
        ("pre_flip", ctypes.c_int32),
        ("geom", ctypes.c_int32),
        ("geom_w", ctypes.c_int32), ("geom_h", ctypes.c_int32),
        ("mx", ctypes.c_float * 6),
        ("post_x", ctypes.c_int32), ("post_y", ctypes.c_int32),
        ("post_w", ctypes.c_int32), ("post_h", ctypes.c_int32),
        ("post_flip", ctypes.c_int32),
        ("reserved", ctypes.c_int32),
    ]


class BatchDesc(ctypes.Structure):
    _fields_ = [
        ("dst", ctypes.c_void_p),
        ("slot_h", ctypes.c_int32), ("slot_w", ctypes.c_int32),
        ("channels", ctypes.c_int32),
        ("gray", ctypes.c_int32),
        ("gray_m", ctypes.c_int32 * 3),
        ("gray_bias", ctypes.c_int32),
        ("out_dtype", ctypes.c_int32),
        ("normalise", ctypes.c_int32),
        ("divisor", ctypes.c_float),
        ("mean", ctypes.c_float * 4),
        ("std_", ctypes.c_float * 4),
        ("pad_value", ctypes.c_double),
        ("src_mem", ctypes.c_int32),
        ("dst_mem", ctypes.c_int32),
    ]


class Stats(ctypes.Structure):
    _fields_ = [(n, ctypes.c_uint64) for n in (
        "batches", "samples", "kernel_launches", "h2d_bytes", "d2h_bytes", "device_bytes_reserved",
        "kernel_ns", "timed_launches", "algo_src_bytes", "algo_dst_bytes", "h2d_ns", "d2h_ns", "host_stage_ns")]


# numpy mirror of SampleDesc so a whole batch of descriptors is one array
SAMPLE_DTYPE = np.dtype([
    ("src", np.uint64), ("src_h", np.int32), ("src_w", np.int32),
    ("pre_x", np.int32), ("pre_y", np.int32), ("pre_w", np.int32), ("pre_h", np.int32),
    ("pre_flip", np.int32), ("geom", np.int32), ("geom_w", np.int32), ("geom_h", np.int32),
    ("mx", np.float32, (6,)),
    ("post_x", np.int32), ("post_y", np.int32), ("post_w", np.int32), ("post_h", np.int32),
    ("post_flip", np.int32), ("reserved", np.int32),
], align=True)
assert SAMPLE_DTYPE.itemsize == ctypes.sizeof(SampleDesc) == 96

EXPORTS = [
    "mlxd_ctx_create", "mlxd_ctx_destroy", "mlxd_last_error", "mlxd_pinned_alloc", "mlxd_pinned_free",
    "mlxd_fused_batch", "mlxd_batch_wait", "mlxd_fused_batch_on_stream", "mlxd_image_resize",
    "mlxd_image_crop", "mlxd_image_hflip", "mlxd_image_affine", "mlxd_image_channel_reduction",
    "mlxd_batch_pad", "mlxd_cast_scale_normalise", "mlxd_stats_get",
    "mlxd_device_alloc", "mlxd_device_free", "mlxd_ctx_set_timing", "mlxd_fused_batch_noalloc",
    "mlxd_noalloc_status", "mlxd_stream_status", "mlxd_device_pci_bus_id",
]
NOALLOC_MAX_SAMPLES = 1024


class MlxdError(RuntimeError):
    def __init__(self, code, text):
        super().__init__("mlxd status %d: %s" % (code, text))
        self.code = code


_lib = None


def load():
    """Load libmlxd_b200.so; raises if it has not been built (there is no fallback)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            "libmlxd_b200.so is missing at %s - build it with `make -C %s` "
            "(this package has no CPU path)" % (LIB_PATH, os.path.join(_HERE, "csrc")))
    lib = ctypes.CDLL(LIB_PATH)
    vp, i32, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64
    lib.mlxd_ctx_create.argtypes = [i32, i32, ctypes.POINTER(vp)]
    lib.mlxd_ctx_destroy.argtypes = [vp]
    lib.mlxd_ctx_destroy.restype = None
    lib.mlxd_last_error.restype = ctypes.c_char_p
    lib.mlxd_pinned_alloc.argtypes = [ctypes.c_size_t]
    lib.mlxd_pinned_alloc.restype = vp
    lib.mlxd_pinned_free.argtypes = [vp]
    lib.mlxd_pinned_free.restype = None
    lib.mlxd_fused_batch.argtypes = [vp, i32, vp, i32, ctypes.POINTER(BatchDesc)]
    lib.mlxd_batch_wait.argtypes = [vp, i32, i32]
    lib.mlxd_fused_batch_on_stream.argtypes = [vp, vp, vp, i32, ctypes.POINTER(BatchDesc)]
    lib.mlxd_image_resize.argtypes = [vp, vp, i32, i32, i32, vp, i32, i32]
    lib.mlxd_image_crop.argtypes = [vp, vp, i32, i32, i32, i32, i32, i32, i32, vp]
    lib.mlxd_image_hflip.argtypes = [vp, vp, i32, i32, i32, vp]
    lib.mlxd_image_affine.argtypes = [vp, vp, i32, i32, i32, ctypes.POINTER(ctypes.c_float), i32, i32, vp]
    lib.mlxd_image_channel_reduction.argtypes = [vp, vp, i32, i32, ctypes.POINTER(ctypes.c_int32), ctypes.c_int32, vp]
    lib.mlxd_batch_pad.argtypes = [vp, ctypes.POINTER(vp), ctypes.POINTER(ctypes.c_int32),
                                   ctypes.POINTER(ctypes.c_int32), i32, i32, i32, i32, ctypes.c_double, vp]
    lib.mlxd_cast_scale_normalise.argtypes = [vp, vp, i64, i32, ctypes.c_float, vp, vp, vp]
    lib.mlxd_stats_get.argtypes = [vp, ctypes.POINTER(Stats)]
    lib.mlxd_device_alloc.argtypes = [vp, ctypes.c_size_t]
    lib.mlxd_device_alloc.restype = vp
    lib.mlxd_device_free.argtypes = [vp, vp]
    lib.mlxd_device_free.restype = None
    lib.mlxd_ctx_set_timing.argtypes = [vp, i32]
    lib.mlxd_fused_batch_noalloc.argtypes = [i32, vp, vp, i32, ctypes.POINTER(BatchDesc)]
    lib.mlxd_noalloc_status.argtypes = [i32, vp, ctypes.POINTER(ctypes.c_int32)]
    lib.mlxd_stream_status.argtypes = [vp, vp, ctypes.POINTER(ctypes.c_int32)]
    lib.mlxd_device_pci_bus_id.argtypes = [i32, ctypes.c_char_p, ctypes.c_size_t]
    _lib = lib
    return lib


def _addr(a):
    if isinstance(a, np.ndarray):
        return a.ctypes.data
    return int(a)


def make_batch_desc(dst, slot_h, slot_w, channels, out_dtype=F32, divisor=255.0, mean=None, std=None,
                    pad_value=0.0, gray=None, src_mem=MEM_HOST, dst_mem=MEM_HOST):
    """gray = (m0, m1, m2, bias) fixed-point ints, or None."""
    b = BatchDesc()
    b.dst = _addr(dst)
    b.slot_h, b.slot_w, b.channels = slot_h, slot_w, channels
    if gray is not None:
        b.gray = 1
        b.gray_m[0], b.gray_m[1], b.gray_m[2] = gray[0], gray[1], gray[2]
        b.gray_bias = gray[3]
    b.out_dtype = out_dtype
    b.divisor = divisor
    if mean is not None:
        b.normalise = 1
        for i, (m, s) in enumerate(zip(mean, std)):
            b.mean[i] = m
            b.std_[i] = s
    b.pad_value = pad_value
    b.src_mem, b.dst_mem = src_mem, dst_mem
    return b


def fused_batch_noalloc(device, stream, descs, batch):
    """mlxd_fused_batch_noalloc: device-resident sources and destination, the
    caller's CUDA stream, no context and no allocation (see include/mlxd_b200.h)."""
    lib = load()
    assert descs.dtype == SAMPLE_DTYPE and descs.flags.c_contiguous
    rc = lib.mlxd_fused_batch_noalloc(device, ctypes.c_void_p(stream), descs.ctypes.data, len(descs),
                                      ctypes.byref(batch))
    if rc != OK:
        raise MlxdError(rc, lib.mlxd_last_error().decode())


def device_pci_bus_id(device):
    """"dddd:bb:dd.f" of a CUDA device (its directory name under /sys/bus/pci/devices)."""
    buf = ctypes.create_string_buffer(32)
    rc = load().mlxd_device_pci_bus_id(device, buf, 32)
    if rc != OK:
        raise MlxdError(rc, load().mlxd_last_error().decode())
    return buf.value.decode()


def noalloc_status(device, stream):
    """mlxd_noalloc_status: the self-check word of the last allocation-free launch (0 = clean)."""
    lib = load()
    word = ctypes.c_int32(-1)
    rc = lib.mlxd_noalloc_status(device, ctypes.c_void_p(stream), ctypes.byref(word))
    if rc not in (OK, ERR_DEVICE):
        raise MlxdError(rc, lib.mlxd_last_error().decode())
    return word.value


class Context:
    """One device, ``n_lanes`` independent lanes (see include/mlxd_b200.h)."""

    def __init__(self, device=0, n_lanes=1):
        self.lib = load()
        h = ctypes.c_void_p()
        self._check(self.lib.mlxd_ctx_create(device, n_lanes, ctypes.byref(h)))
        self.handle = h
        self.n_lanes = n_lanes

    def _check(self, rc):
        if rc != OK:
            raise MlxdError(rc, self.lib.mlxd_last_error().decode())

    def close(self):
        if getattr(self, "handle", None):
            self.lib.mlxd_ctx_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def fused_batch(self, lane, descs, batch):
        assert descs.dtype == SAMPLE_DTYPE and descs.flags.c_contiguous
        self._check(self.lib.mlxd_fused_batch(self.handle, lane, descs.ctypes.data, len(descs), ctypes.byref(batch)))

    def wait(self, lane, timeout_ms=-1):
        self._check(self.lib.mlxd_batch_wait(self.handle, lane, timeout_ms))

    def fused_batch_on_stream(self, stream, descs, batch):
        assert descs.dtype == SAMPLE_DTYPE and descs.flags.c_contiguous
        self._check(self.lib.mlxd_fused_batch_on_stream(
            self.handle, ctypes.c_void_p(stream), descs.ctypes.data, len(descs), ctypes.byref(batch)))

    def stream_status(self, stream):
        """mlxd_stream_status: waits for the stream, returns the self-check word (0 = clean)."""
        word = ctypes.c_int32(-1)
        rc = self.lib.mlxd_stream_status(self.handle, ctypes.c_void_p(stream), ctypes.byref(word))
        if rc not in (OK, ERR_DEVICE):
            self._check(rc)
        return word.value

    # ---- one entry per op, host buffers, synchronous ----
    def image_resize(self, img, dw, dh):
        h, w, c = img.shape
        out = np.empty((dh, dw, c), np.uint8)
        self._check(self.lib.mlxd_image_resize(self.handle, img.ctypes.data, h, w, c, out.ctypes.data, dh, dw))
        return out

    def image_crop(self, img, x, y, cw, ch):
        h, w, c = img.shape
        out = np.empty((ch, cw, c), np.uint8)
        self._check(self.lib.mlxd_image_crop(self.handle, img.ctypes.data, h, w, c, x, y, cw, ch, out.ctypes.data))
        return out

    def image_hflip(self, img):
        h, w, c = img.shape
        out = np.empty_like(img)
        self._check(self.lib.mlxd_image_hflip(self.handle, img.ctypes.data, h, w, c, out.ctypes.data))
        return out

    def image_affine(self, img, mx, th, tw):
        h, w, c = img.shape
        out = np.empty((th, tw, c), np.uint8)
        m = (ctypes.c_float * 6)(*mx)
        self._check(self.lib.mlxd_image_affine(self.handle, img.ctypes.data, h, w, c, m, th, tw, out.ctypes.data))
        return out

    def image_channel_reduction(self, img, m_fixed, bias_fixed):
        h, w, c = img.shape
        assert c == 3
        out = np.empty((h, w, 1), np.uint8)
        m = (ctypes.c_int32 * 3)(*m_fixed)
        self._check(self.lib.mlxd_image_channel_reduction(self.handle, img.ctypes.data, h, w, m, bias_fixed, out.ctypes.data))
        return out

    def batch_pad(self, imgs, slot_h, slot_w, pad_value=0.0):
        n = len(imgs)
        c = imgs[0].shape[2]
        out = np.empty((n, slot_h, slot_w, c), np.uint8)
        ptrs = (ctypes.c_void_p * n)(*[a.ctypes.data for a in imgs])
        hs = (ctypes.c_int32 * n)(*[a.shape[0] for a in imgs])
        ws = (ctypes.c_int32 * n)(*[a.shape[1] for a in imgs])
        self._check(self.lib.mlxd_batch_pad(self.handle, ptrs, hs, ws, n, c, slot_h, slot_w, pad_value, out.ctypes.data))
        return out

    def cast_scale_normalise(self, x, divisor=255.0, mean=None, std=None):
        c = x.shape[-1]
        out = np.empty(x.shape, np.float32)
        mp = sp = None
        if mean is not None:
            mean = np.ascontiguousarray(mean, np.float32)
            std = np.ascontiguousarray(std, np.float32)
            mp, sp = mean.ctypes.data, std.ctypes.data
        self._check(self.lib.mlxd_cast_scale_normalise(
            self.handle, x.ctypes.data, x.size // c, c, divisor, mp, sp, out.ctypes.data))
        return out

    def set_timing(self, on=True):
        self._check(self.lib.mlxd_ctx_set_timing(self.handle, 1 if on else 0))

    def stats(self):
        s = Stats()
        self._check(self.lib.mlxd_stats_get(self.handle, ctypes.byref(s)))
        return {n: getattr(s, n) for n, _ in Stats._fields_}
