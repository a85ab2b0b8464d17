"""Seeded random op chains through the pipeline API against the reference
pipeline (compiled under oracle/_ref): image ops, slices and explicit padding
in any order under a batch node, so the recorded-program machinery (windows,
mirrors, one geometric op, extensions, materialisation when a program is full)
is exercised in combinations no hand-written case lists."""
import numpy as np
import pytest

import refpipe

pytestmark = pytest.mark.gpu


def _chain(rng):
    ops = []
    h = w = 40                       # lower bounds of the current image size
    n_ops = int(rng.integers(1, 7))
    resized = False
    for _ in range(n_ops):
        kind = int(rng.integers(0, 9))
        if kind == 0 and h >= 12 and w >= 12:
            h, w = int(rng.integers(h // 2, h + 1)), int(rng.integers(w // 2, w + 1))
            ops.append(("image_center_crop", dict(key="image", w=w, h=h)))
        elif kind == 1 and h >= 12 and w >= 12:
            h, w = int(rng.integers(h // 2, h + 1)), int(rng.integers(w // 2, w + 1))
            ops.append(("image_random_crop", dict(key="image", w=w, h=h)))
        elif kind == 2:
            ops.append(("image_random_h_flip", dict(key="image", prob=0.5)))
        elif kind == 3:
            size = int(rng.integers(16, 90))
            ops.append(("image_resize_smallest_side", dict(key="image", size=size)))
            h = w = size
            resized = True
        elif kind == 4:
            w, h = int(rng.integers(8, 100)), int(rng.integers(8, 100))
            ops.append(("image_resize", dict(key="image", w=w, h=h)))
            resized = True
        elif kind == 5 and h >= 10 and w >= 10:
            a, b = int(rng.integers(0, h // 2)), int(rng.integers(0, w // 2))
            ops.append(("slice", dict(ikey="image", dims=[0, 1], starts=[a, b], ends=[a + h // 2, b + w // 2])))
            h, w = h // 2, w // 2
        elif kind == 6 and h >= 10 and w >= 10:
            h, w = int(rng.integers(h // 2, h + 1)), int(rng.integers(w // 2, w + 1))
            ops.append(("random_slice", dict(ikey="image", dims=[0, 1], sizes=[h, w])))
        elif kind == 7:
            ops.append(("pad_to_multiple", dict(key="image", dim=int(rng.integers(0, 2)),
                                                pad_multiple=int(rng.choice([8, 16, 24])), pad_value=int(rng.choice([0, 0, 9])))))
        elif kind == 8:
            ops.append(("pad", dict(key="image", dim=int(rng.integers(0, 2)), lpad=int(rng.choice([0, 0, 2])),
                                    rpad=int(rng.integers(0, 6)), pad_value=int(rng.choice([0, 0, 5])))))
    if not ops:
        ops.append(("image_random_h_flip", dict(key="image", prob=1.0)))
    return ops, resized


def _run(dx, samples, ops, batch, pad, seed):
    dx.core.set_state(seed)
    ds = dx.buffer_from_vector(samples).to_stream()
    for name, kw in ops:
        ds = getattr(ds, name)(**kw)
    return [np.asarray(b["image"]) for b in ds.batch(batch, pad={"image": pad})]


@pytest.mark.parametrize("seed", range(30))
def test_random_pipeline(pkg, seed):
    ref = refpipe.reference_module()
    if ref is None:
        pytest.skip("needs the reference compiled under oracle/_ref")
    rng = np.random.default_rng(7000 + seed)
    ops, resized = _chain(rng)
    samples = [{"image": rng.integers(0, 256, (int(rng.integers(40, 160)), int(rng.integers(40, 160)), 3), dtype=np.uint8)}
               for _ in range(int(rng.integers(2, 9)))]
    pad = int(rng.choice([0, 0, 9]))
    want = _run(ref, samples, ops, 4, pad, seed)
    got = _run(pkg, samples, ops, 4, pad, seed)
    assert len(got) == len(want), ops
    for g, w in zip(got, want):
        assert g.shape == w.shape and g.dtype == w.dtype, (ops, g.shape, w.shape)
        if not resized:
            assert np.array_equal(g, w), ops
        else:
            d = np.abs(g.astype(np.int32) - w.astype(np.int32))
            assert d.max() <= 1 and (d > 0).mean() <= 2e-3, ops
