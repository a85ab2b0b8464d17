"""Test helper: reduce an op chain on one key to the canonical descriptor of the
C ABI (window+mirror -> one geometric op -> window+mirror -> gray), drawing the
random parameters with the oracle's generator in the reference's order.  This
is an independent restatement of what the host library's planner does, kept in
the tests so the two can be checked against each other."""
import numpy as np

import oracle as O


class Unfusable(Exception):
    pass


def gray_fixed(preset):
    """16.16 fixed-point multipliers and bias, truncated like
    mlx/data/core/image/ImageTransform.cpp:159-164 (float32 coefficient * 65536)."""
    bias, m = O.PRESETS[preset]
    f = [int(np.float32(np.float32(x) * np.float32(65536.0))) for x in m]
    return (f[0], f[1], f[2], int(np.float32(np.float32(bias) * np.float32(65536.0))))


class _Rect:
    def __init__(self, w, h):
        self.x, self.y, self.w, self.h, self.flip = 0, 0, w, h, 0

    def crop(self, x, y, w, h):
        if x < 0 or y < 0 or w <= 0 or h <= 0 or x + w > self.w or y + h > self.h:
            raise RuntimeError("crop out of bound")
        self.x = self.x + (self.w - x - w if self.flip else x)
        self.y += y
        self.w, self.h = w, h


def reduce_chain(shape, ops, sample=None):
    """shape = (H, W, C) of the source.  Returns a dict of descriptor fields plus
    'gray' (None or fixed-point tuple) and 'out_hw'."""
    H, W, C = shape
    pre = _Rect(W, H)
    post = None
    geom, gw, gh, mx = 0, W, H, [0.0] * 6
    gray = None

    def cur():
        return post if post is not None else pre

    for name, kw in ops:
        r = cur()
        if name == "image_center_crop":
            if kw["h"] > r.h or kw["w"] > r.w:
                raise RuntimeError("ImageCenterCrop: target image size larger than input image")
            r.crop((r.w - kw["w"]) // 2, (r.h - kw["h"]) // 2, kw["w"], kw["h"])
        elif name == "image_random_crop":
            x, y, w, h = O.draw_random_crop(r.w, r.h, kw["w"], kw["h"])
            r.crop(x, y, w, h)
        elif name == "image_random_area_crop":
            x, y, w, h = O.draw_area_crop(r.w, r.h, kw["area_range"], kw["aspect_ratio_range"], kw.get("num_trial", 10))
            if w != 0 and h != 0:
                r.crop(x, y, w, h)
        elif name == "image_random_h_flip":
            if O.draw_hflip(kw["prob"]):
                r.flip ^= 1
        elif name in ("image_resize", "image_resize_smallest_side", "image_rotate"):
            if post is not None or gray is not None:
                raise Unfusable(name)
            if name == "image_resize":
                gw, gh = kw["w"], kw["h"]
                geom = 1
            elif name == "image_resize_smallest_side":
                gh, gw = O.smallest_side_dims(r.h, r.w, kw["size"])
                geom = 1
            else:
                angle = float(sample[kw["angle_key"]]) if "angle_key" in kw else kw["angle"]
                m = O.rotate_matrix(angle)
                mx = list(m)
                import ctypes
                th, tw = ctypes.c_int64(), ctypes.c_int64()
                O.lib().oracle_affine_dims(ctypes.c_int64(r.h), ctypes.c_int64(r.w), m,
                                           ctypes.c_int(1 if kw.get("crop", False) else 0),
                                           ctypes.byref(th), ctypes.byref(tw))
                gw, gh = tw.value, th.value
                geom = 2
            post = _Rect(gw, gh)
        elif name == "image_channel_reduction":
            if C != 3:
                raise RuntimeError("image::channelReduction: expected a 3 channel uint8 array")
            if gray is not None:
                raise Unfusable(name)
            gray = gray_fixed(kw.get("preset", "default"))
        else:
            raise ValueError(name)
    if post is None:
        gw, gh = pre.w, pre.h
        post = _Rect(gw, gh)
    return dict(src_h=H, src_w=W, pre_x=pre.x, pre_y=pre.y, pre_w=pre.w, pre_h=pre.h, pre_flip=pre.flip,
                geom=geom, geom_w=gw, geom_h=gh, mx=mx,
                post_x=post.x, post_y=post.y, post_w=post.w, post_h=post.h, post_flip=post.flip,
                gray=gray, out_hw=(post.h, post.w))


def fill_descs(descs, i, fields, src_addr):
    d = descs[i]
    d["src"] = src_addr
    for k in ("src_h", "src_w", "pre_x", "pre_y", "pre_w", "pre_h", "pre_flip", "geom", "geom_w", "geom_h",
              "post_x", "post_y", "post_w", "post_h", "post_flip"):
        d[k] = fields[k]
    d["mx"] = np.asarray(fields["mx"], np.float32)


def run_fused(pkg, ctx, samples, key, ops, batch_size, cast=None, pad=0.0, out_dtype=None, lane=0):
    """Run ``ops`` on ``samples[i][key]`` through mlxd_fused_batch, one call per
    batch; returns the list of batch arrays.  ``cast`` = None (uint8 out),
    () for /255, or (mean, std)."""
    outs = []
    for b0 in range(0, len(samples), batch_size):
        chunk = samples[b0:b0 + batch_size]
        n = len(chunk)
        descs = np.zeros(n, pkg.SAMPLE_DTYPE)
        fields = []
        imgs = []
        for i, s in enumerate(chunk):
            img = np.ascontiguousarray(s[key])
            imgs.append(img)
            f = reduce_chain(img.shape, ops, s)
            fields.append(f)
            fill_descs(descs, i, f, img.ctypes.data)
        gray = fields[0]["gray"]
        c = imgs[0].shape[2]
        co = 1 if gray else c
        sh = max(f["out_hw"][0] for f in fields)
        sw = max(f["out_hw"][1] for f in fields)
        if cast is None:
            out = np.empty((n, sh, sw, co), np.uint8)
            bd = pkg.make_batch_desc(out, sh, sw, c, out_dtype=pkg._capi.U8, divisor=1.0, pad_value=pad, gray=gray)
        else:
            out = np.empty((n, sh, sw, co), np.float32)
            mean, std = (cast if len(cast) == 2 else (None, None))
            bd = pkg.make_batch_desc(out, sh, sw, c, out_dtype=pkg._capi.F32, divisor=255.0,
                                     mean=mean, std=std, pad_value=pad, gray=gray)
        ctx.fused_batch(lane, descs, bd)
        ctx.wait(lane)
        outs.append(out)
    return outs


def interpret(fields, img, affine_crop_dims=None):
    """Evaluate a canonical descriptor on the CPU with the oracle's ops - the
    meaning the C ABI gives to the descriptor fields."""
    f = fields
    cur = O.crop(img, f["pre_x"], f["pre_y"], f["pre_w"], f["pre_h"])
    if f["pre_flip"]:
        cur = O.hflip(cur)
    if f["geom"] == 1:
        cur = O.resize(cur, f["geom_w"], f["geom_h"])
    elif f["geom"] == 2:
        import ctypes
        mx = (ctypes.c_float * 6)(*f["mx"])
        out = np.empty((f["geom_h"], f["geom_w"], cur.shape[2]), np.uint8)
        i64 = ctypes.c_int64
        O.lib().oracle_affine(O._p8(cur), i64(cur.shape[0]), i64(cur.shape[1]), i64(cur.shape[2]), mx,
                              i64(f["geom_h"]), i64(f["geom_w"]), O._p8(out))
        cur = out
    cur = O.crop(cur, f["post_x"], f["post_y"], f["post_w"], f["post_h"])
    if f["post_flip"]:
        cur = O.hflip(cur)
    if f["gray"] is not None:
        g = f["gray"]
        v = (cur[..., 0].astype(np.int64) * g[0] + cur[..., 1].astype(np.int64) * g[1]
             + cur[..., 2].astype(np.int64) * g[2] + g[3])
        v = np.where(v >= 0, v // 65536, -((-v) // 65536))
        cur = np.clip(v, 0, 255).astype(np.uint8)[..., None]
    return cur
