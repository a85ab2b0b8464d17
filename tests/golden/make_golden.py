"""Generate tests/golden/golden.json from the reference compiled under oracle/_ref.

Run in the build container (needs `make -C oracle ref` first):

    python tests/golden/make_golden.py

Everything recorded here is produced by the reference's own pipeline code
(`import mlx.data` from oracle/_ref): random-draw sequences, crop rectangles,
rotate / channel-reduction / pad / batch results, and whole small pipelines.
Resize results are included too; they come from the reference's wrapper around
the resize restatement (oracle/resize_restatement.h), not from the un-vendored
stb routine, and are marked as such.
"""
import hashlib
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "oracle", "_ref"))
sys.path.insert(0, os.path.join(ROOT, "mlx-data_b200"))

import mlx.data as dx  # noqa: E402
import workloads as wl  # noqa: E402


def digest(a):
    a = np.ascontiguousarray(a)
    return {"shape": list(a.shape), "dtype": str(a.dtype), "sha256": hashlib.sha256(a.tobytes()).hexdigest()[:24],
            "sum": float(a.astype(np.float64).sum())}


def ramp():
    r = np.arange(48 * 64 * 3, dtype=np.uint32).reshape(48, 64, 3)
    return ((r * np.uint32(2654435761)) >> 24).astype(np.uint8)


def main():
    g = {}
    # random flips, seeds 0 and 1234
    for seed in (0, 1234):
        dx.core.set_state(seed)
        s = [{"image": np.arange(72, dtype=np.uint8).reshape(4, 6, 3)} for _ in range(16)]
        st = dx.buffer_from_vector(s).to_stream().image_random_h_flip("image", 0.5)
        g["flips_seed%d" % seed] = [int(x["image"][0, 0, 0] != 0) for x in st]
    # area-crop rectangles on 480x640 images, recovered from the cropped shapes and a coordinate image
    dx.core.set_state(0)
    yy, xx = np.meshgrid(np.arange(480), np.arange(640), indexing="ij")
    coord = np.stack([xx % 256, xx // 256, yy % 256], -1).astype(np.uint8)
    coord_hi = (yy // 256).astype(np.uint8)
    s = [{"image": coord, "hi": coord_hi[..., None].repeat(3, -1)} for _ in range(8)]
    st = dx.buffer_from_vector(s).to_stream().image_random_area_crop("image", (0.08, 1.0), (0.75, 4 / 3))
    rects = []
    for x in st:
        im = x["image"]
        tx = int(im[0, 0, 0]) + 256 * int(im[0, 0, 1])
        ty = int(im[0, 0, 2])  # low byte; the high part is found from the candidates below
        rects.append([tx, ty, im.shape[1], im.shape[0]])
    g["area_crop_rects_seed0_lowbyte_y"] = rects
    dx.core.set_state(0)
    st = dx.buffer_from_vector([{"image": np.zeros((480, 640, 3), np.uint8)} for _ in range(6)]).to_stream() \
        .image_random_crop("image", 224, 224)
    g["random_crop_shapes_seed0"] = [list(x["image"].shape) for x in st]
    # rotate / gray on the ramp image
    rp = ramp()
    g["ramp"] = digest(rp)
    for ang, crop in [(17.0, True), (-30.0, True), (30.0, True), (17.0, False)]:
        out = dx.buffer_from_vector([{"image": rp}]).image_rotate("image", ang, crop)[0]["image"]
        g["rotate_%g_%d" % (ang, int(crop))] = digest(out)
    for preset in ("rec709", "default", "rec2020", "green"):
        out = dx.buffer_from_vector([{"image": rp}]).image_channel_reduction("image", preset)[0]["image"]
        g["gray_" + preset] = digest(out)
    white = np.full((4, 4, 3), 255, np.uint8)
    g["gray_white_value"] = int(dx.buffer_from_vector([{"image": white}]).image_channel_reduction("image")[0]["image"].max())
    # batch + pad
    b = dx.buffer_from_vector([{"x": np.ones((2, 3), np.uint8)}, {"x": np.ones((3, 2), np.uint8)}]).batch(2, pad={"x": 7})
    g["batch_pad7"] = b[0]["x"].tolist()
    # whole small pipelines (stream, main thread, seed 0)
    for name in ("c1", "c2", "c3", "c5"):
        cfg = wl.CONFIGS[name]
        samples = wl.make_samples(name, "small", n=8)
        ops = wl.config_ops(name, "small")
        dx.core.set_state(0)
        ds = dx.buffer_from_vector(samples).to_stream()
        for op, kw in ops:
            ds = getattr(ds, op)(**kw)
        ds = ds.batch(4)
        if len(cfg["cast"]) == 0:
            ds = ds.key_transform("image", lambda x: x.astype("float32") / 255)
        else:
            mean = np.array(cfg["cast"][0], np.float32)
            std = np.array(cfg["cast"][1], np.float32)
            ds = ds.key_transform("image", lambda x: (x.astype("float32") / 255 - mean) / std)
        g["pipeline_%s_small8" % name] = {"uses_resize_restatement": True,
                                          "batches": [digest(x["image"]) for x in ds]}
    # rotate-heavy chain with one fixed angle (the reference op has no per-sample angle)
    samples = wl.make_samples("c4", "small", n=8)
    dx.core.set_state(0)
    ds = (dx.buffer_from_vector([{"image": s["image"]} for s in samples]).to_stream()
          .image_rotate("image", 21.5, crop=True).image_random_h_flip("image", 0.5)
          .image_center_crop("image", 140, 140).batch(4)
          .key_transform("image", lambda x: x.astype("float32") / 255))
    g["pipeline_c4_fixed_angle_small8"] = {"uses_resize_restatement": False,
                                           "batches": [digest(x["image"]) for x in ds]}
    with open(os.path.join(HERE, "golden.json"), "w") as f:
        json.dump(g, f, indent=1, sort_keys=True)
    print("wrote", len(g), "entries")


if __name__ == "__main__":
    main()
