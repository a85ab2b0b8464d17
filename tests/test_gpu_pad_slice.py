"""Explicit pad / slice ops on image keys under a batch node.

They join the fused run (a slice of rows and columns is a crop; padding at the
end of rows or columns enlarges the image's claim on its batch slot), so a
chain with them still costs one launch per batch.  The results must equal the
reference pipeline's, which runs every op on the host - also for the cases
that cannot be fused (padding in front, a slice of the channels, a pad value
that differs from the batch's), which fall back to the host op.
"""
import numpy as np
import pytest

import refpipe

pytestmark = pytest.mark.gpu


def _images(seed, n, lo=40, hi=90):
    rng = np.random.default_rng(seed)
    return [{"image": rng.integers(0, 256, (int(rng.integers(lo, hi)), int(rng.integers(lo, hi)), 3), dtype=np.uint8),
             "id": np.int64(i)} for i in range(n)]


def _run(dx, samples, ops, batch, pad, seed):
    dx.core.set_state(seed)
    ds = dx.buffer_from_vector(samples).to_stream()
    for name, kw in ops:
        ds = getattr(ds, name)(**kw)
    return [dict(b) for b in ds.batch(batch, pad=pad)]


def _assert_same(got, want, resized):
    assert len(got) == len(want)
    for g, w in zip(got, want):
        assert sorted(g) == sorted(w)
        for k in w:
            a, b = np.asarray(g[k]), np.asarray(w[k])
            assert a.shape == b.shape and a.dtype == b.dtype, (k, a.shape, b.shape)
            if resized and k == "image":
                d = np.abs(a.astype(np.int32) - b.astype(np.int32))
                assert d.max() <= 1 and (d > 0).mean() <= 1e-3
            else:
                assert np.array_equal(a, b), k


# (ops, batch pad, does the chain resize, launches expected per batch: 1 = fully fused)
CHAINS = [
    ([("slice", dict(ikey="image", dims=[0, 1], starts=[3, 5], ends=[33, 37]))], {}, False, 1),
    ([("random_slice", dict(ikey="image", dims=[0, 1], sizes=[32, 24])),
      ("image_random_h_flip", dict(key="image", prob=0.5))], {}, False, 1),
    ([("random_slice", dict(ikey="image", dims=1, sizes=30)),
      ("image_resize_smallest_side", dict(key="image", size=48)),
      ("pad_to_multiple", dict(key="image", dim=0, pad_multiple=16, pad_value=0)),
      ("pad_to_multiple", dict(key="image", dim=1, pad_multiple=16, pad_value=0))], {}, True, 1),
    ([("image_center_crop", dict(key="image", w=36, h=30)),
      ("pad_to_size", dict(key="image", dim=1, size=40, pad_value=7)),
      ("pad", dict(key="image", dim=0, lpad=0, rpad=5, pad_value=7))], {"image": 7}, False, 1),
    # pad value differs from the batch's (0): every image is computed on its own, then batched
    ([("pad_to_size", dict(key="image", dim=0, size=96, pad_value=9))], {}, False, None),
    # padding in front and a slice of the channels run on the host
    ([("pad", dict(key="image", dim=1, lpad=2, rpad=1, pad_value=3))], {}, False, None),
    ([("slice", dict(ikey="image", dims=[2], starts=[1], ends=[3]))], {}, False, None),
    # an op after a pad needs the padded pixels
    ([("pad_to_multiple", dict(key="image", dim=1, pad_multiple=32, pad_value=5)),
      ("image_random_crop", dict(key="image", w=30, h=30)),
      ("image_random_h_flip", dict(key="image", prob=0.5))], {}, False, None),
    # slices that clip at the border
    ([("slice", dict(ikey="image", dims=[0], starts=[10], ends=[1000]))], {}, False, 1),
]


@pytest.mark.parametrize("case", range(len(CHAINS)))
def test_pad_and_slice_under_batch_match_reference(pkg, case):
    ref = refpipe.reference_module()
    if ref is None:
        pytest.skip("needs the reference compiled under oracle/_ref")
    ops, pad, resized, launches = CHAINS[case]
    samples = _images(20 + case, 11)
    want = _run(ref, samples, ops, 4, pad, seed=5 + case)
    before = pkg.core.stats()["kernel_launches"]
    got = _run(pkg, samples, ops, 4, pad, seed=5 + case)
    used = pkg.core.stats()["kernel_launches"] - before
    _assert_same(got, want, resized)
    if launches is not None:
        assert used == launches * len(want), "expected one launch per batch, saw %d for %d batches" % (used, len(want))


def test_fused_padding_with_cast(pkg):
    """pad_to_multiple followed by batch and the fused cast: the explicit
    padding and the batch padding both come out as cast(pad value)."""
    samples = _images(3, 6)
    pkg.core.set_state(0)
    ds = (pkg.buffer_from_vector(samples).to_stream()
          .pad_to_multiple("image", 0, 32, 255).pad_to_multiple("image", 1, 32, 255)
          .batch(3, pad={"image": 255}).key_cast("image"))
    for b, group in zip(ds, (samples[:3], samples[3:])):
        x = np.asarray(b["image"])
        hs = [-(-s["image"].shape[0] // 32) * 32 for s in group]
        ws = [-(-s["image"].shape[1] // 32) * 32 for s in group]
        assert x.shape == (3, max(hs), max(ws), 3) and x.dtype == np.float32
        for i, s in enumerate(group):
            h, w = s["image"].shape[:2]
            assert np.array_equal(x[i, :h, :w], s["image"].astype("float32") / 255)
            assert np.all(x[i, h:] == 1.0) and np.all(x[i, :, w:] == 1.0)
