"""Test helper: run an op chain through the reference's own pipeline code.

``oracle/_ref`` holds the reference compiled from its own sources (with the
resize restatement standing in for the un-vendored stb header); when it is
importable the chain runs through its Stream API exactly as a user of the
reference would write it.  Otherwise the plain C restatement (oracle.run_chain)
is used.  Both are CPU checkers, never the product."""
import os
import sys

import numpy as np

import oracle as O

_REF = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref")


def reference_module():
    if not os.path.isdir(os.path.join(_REF, "mlx", "data")):
        return None
    if _REF not in sys.path:
        sys.path.insert(0, _REF)
    try:
        import mlx.data as dx
        return dx
    except Exception:
        return None


def _numpy_cast(cast):
    if len(cast) == 0:
        return lambda x: x.astype("float32") / 255
    mean = np.array(cast[0], dtype=np.float32)
    std = np.array(cast[1], dtype=np.float32)
    return lambda x: (x.astype("float32") / 255 - mean) / std


def build(dx, samples, ops, batch, pad, cast_keys, native_cast=False, prefetch=None, buffer_mode=False,
          product=False):
    """The same fluent chain on either module.  ``cast_keys`` = {key: () | (mean, std)}."""
    ds = dx.buffer_from_vector(samples)
    if not buffer_mode:
        ds = ds.to_stream()
    for name, kw in ops:
        kw = dict(kw)
        if "angle_key" in kw and not (product or native_cast):
            raise NotImplementedError("the reference has no per-sample angle")
        if "angle_key" in kw:
            kw.setdefault("angle", 0.0)
        ds = getattr(ds, name)(**kw)
    ds = ds.batch(batch, pad=pad)
    for key, cast in cast_keys.items():
        if native_cast:
            if len(cast) == 0:
                ds = ds.key_cast(key)
            else:
                ds = ds.key_cast(key, mean=list(cast[0]), std=list(cast[1]))
        else:
            ds = ds.key_transform(key, _numpy_cast(cast))
    if prefetch:
        ds = ds.prefetch(*prefetch) if not buffer_mode else ds.ordered_prefetch(*prefetch)
    return ds


def run_reference(samples, ops, batch, pad, cast_keys, seed=0):
    """List of batch dicts from the reference (or, without oracle/_ref, from the C restatement)."""
    dx = reference_module()
    per_sample_angle = any("angle_key" in kw for _, kw in ops)
    if dx is not None and not per_sample_angle:
        dx.core.set_state(seed)
        return [dict(b) for b in build(dx, samples, ops, batch, pad, cast_keys)]
    O.set_state(seed)
    cast = {k: (None if len(c) == 0 else (np.array(c[0], np.float32), np.array(c[1], np.float32)))
            for k, c in cast_keys.items()}
    return O.run_chain(samples, ops, batch, pad, cast)
