"""Synthetic stand-ins for the five benchmark configurations.

The public image datasets the reference benchmarks on are not available, so
each configuration is described by its shapes and value distribution only:
uint8 RGB HWC images with uniform pixels and uniform random sizes, generated
from a seed.  ``ops`` uses the method names and keyword arguments of the
mlx-data Python API (python/src/wrap_dataset.h:83-362); ``image_rotate`` with
``angle_key`` takes a per-sample angle from the sample (the reference op has one
fixed angle per op instance, so the harness supplies the angle per sample).
"""
import numpy as np

IMAGENET_MEAN = (0.485, 0.456, 0.406)
IMAGENET_STD = (0.229, 0.224, 0.225)


def _cfg(**kw):
    return kw


# "full" follows the configuration text; "small" keeps the op chain and shrinks
# counts and sizes so a CPU check finishes in seconds.
CONFIGS = {
    "c1": _cfg(
        full=dict(n=256, h=(200, 500), w=(200, 500), batch=32),
        small=dict(n=48, h=(200, 500), w=(200, 500), batch=16),
        ops=[("image_resize_smallest_side", dict(key="image", size=256)),
             ("image_center_crop", dict(key="image", w=224, h=224))],
        cast=(), pad=0.0, seed=0),
    "c2": _cfg(
        full=dict(n=4096, h=(256, 800), w=(256, 800), batch=256),
        small=dict(n=40, h=(256, 800), w=(256, 800), batch=16),
        ops=[("image_random_area_crop", dict(key="image", area_range=(0.08, 1.0), aspect_ratio_range=(3 / 4, 4 / 3))),
             ("image_resize", dict(key="image", w=224, h=224)),
             ("image_random_h_flip", dict(key="image", prob=0.5))],
        cast=(IMAGENET_MEAN, IMAGENET_STD), pad=0.0, seed=0),
    "c3": _cfg(
        full=dict(n=2048, h=(64, 1024), w=(64, 1024), batch=64, size=320),
        small=dict(n=24, h=(64, 256), w=(64, 256), batch=8, size=80),
        ops=[("image_resize_smallest_side", dict(key="image", size=320))],
        gray_ops=[("image_resize_smallest_side", dict(key="image", size=320)),
                  ("image_channel_reduction", dict(key="image", preset="default", output_key="gray"))],
        cast=(), pad=0.0, seed=0),
    "c4": _cfg(
        full=dict(n=4096, h=(512, 512), w=(512, 512), batch=128, crop=448),
        small=dict(n=24, h=(160, 160), w=(160, 160), batch=8, crop=140),
        ops=[("image_rotate", dict(key="image", angle_key="angle", crop=True)),
             ("image_random_h_flip", dict(key="image", prob=0.5)),
             ("image_center_crop", dict(key="image", w=448, h=448))],
        cast=(), pad=0.0, seed=0),
    "c5": _cfg(
        full=dict(n=16384, h=(1080, 1080), w=(1920, 1920), batch=512),
        small=dict(n=6, h=(1080, 1080), w=(1920, 1920), batch=4),
        ops=[("image_resize_smallest_side", dict(key="image", size=512)),
             ("image_center_crop", dict(key="image", w=512, h=512)),
             ("image_random_h_flip", dict(key="image", prob=0.5))],
        cast=(IMAGENET_MEAN, IMAGENET_STD), pad=0.0, seed=0),
}


def config_ops(name, variant="full", which="ops"):
    """The op list of a configuration with the variant's sizes substituted."""
    cfg = CONFIGS[name]
    v = cfg[variant]
    out = []
    for op, kw in cfg[which]:
        kw = dict(kw)
        if name == "c3" and op == "image_resize_smallest_side":
            kw["size"] = v["size"]
        if name == "c4" and op == "image_center_crop":
            kw["w"] = kw["h"] = v["crop"]
        out.append((op, kw))
    return out


def image_sizes(name, variant="full", n=None):
    """Heights and widths: all H drawn first, then all W (one generator)."""
    cfg = CONFIGS[name]
    v = cfg[variant]
    n = v["n"] if n is None else n
    rng = np.random.default_rng(cfg["seed"])
    hs = rng.integers(v["h"][0], v["h"][1] + 1, n)
    ws = rng.integers(v["w"][0], v["w"][1] + 1, n)
    return rng, hs, ws


def make_samples(name, variant="full", n=None):
    """List of dict samples {"image": uint8 [H, W, 3]} (+ "angle" for c4)."""
    rng, hs, ws = image_sizes(name, variant, n)
    samples = []
    for h, w in zip(hs, ws):
        samples.append({"image": rng.integers(0, 256, (int(h), int(w), 3), dtype=np.uint8)})
    if name == "c4":
        angles = np.random.default_rng(1000 + CONFIGS[name]["seed"]).uniform(-30.0, 30.0, len(samples))
        for s, a in zip(samples, angles):
            s["angle"] = np.float64(a)
    return samples
