"""GPU parity through the pipeline API: the same fluent chain on this package
and on the reference (compiled from its own sources under oracle/_ref), same
samples, same seed.  Exact for everything but resize, which is held to +-1
uint8 LSB and to a bound on how often a difference may occur."""
import importlib

import numpy as np
import pytest

import refpipe

pytestmark = pytest.mark.gpu

RESIZE_MISMATCH_MAX = 1e-3


def _wl():
    return importlib.import_module("mlx_data_b200.workloads")


def _check(got, want, has_resize, cast_scale):
    assert len(got) == len(want)
    for g, w in zip(got, want):
        assert sorted(g.keys()) == sorted(w.keys())
        for k in w:
            a, b = np.asarray(g[k]), np.asarray(w[k])
            assert a.shape == b.shape and a.dtype == b.dtype, (k, a.shape, b.shape, a.dtype, b.dtype)
            if not has_resize or a.ndim < 4:
                assert np.array_equal(a, b), k
            else:
                tol = 1.0 if a.dtype == np.uint8 else cast_scale * 1.0001
                d = np.abs(a.astype(np.float64) - b.astype(np.float64))
                assert d.max() <= tol, (k, d.max())
                assert (a != b).mean() <= RESIZE_MISMATCH_MAX, (k, (a != b).mean())


def _cast_scale(cast):
    return 1.0 / 255 if len(cast) == 0 else 1.0 / 255 / min(cast[1])


@pytest.mark.parametrize("name", ["c1", "c2", "c3", "c4", "c5"])
@pytest.mark.parametrize("mode", ["native_cast", "lambda_cast"])
def test_config_through_stream_api(pkg, name, mode):
    wl = _wl()
    cfg = wl.CONFIGS[name]
    samples = wl.make_samples(name, "small")
    for i, s in enumerate(samples):
        s["label"] = np.int64(i)
    ops = wl.config_ops(name, "small", "gray_ops" if name == "c3" else "ops")
    keys = {"image": cfg["cast"]}
    if name == "c3":
        keys["gray"] = ()
    pad = {k: cfg["pad"] for k in keys}
    batch = cfg["small"]["batch"]
    want = refpipe.run_reference(samples, ops, batch, pad, keys, seed=0)
    pkg.core.set_state(0)
    got = [dict(b) for b in refpipe.build(pkg, samples, ops, batch, pad, keys,
                                          native_cast=(mode == "native_cast"), product=True)]
    _check(got, want, name != "c4", _cast_scale(cfg["cast"]))
    assert [int(x) for b in got for x in b["label"]] == list(range(len(samples)))


def test_buffer_api_and_ordered_prefetch(pkg):
    wl = _wl()
    cfg = wl.CONFIGS["c2"]
    samples = wl.make_samples("c2", "small", n=24)
    ops = wl.config_ops("c2", "small")
    keys = {"image": cfg["cast"]}
    want = refpipe.run_reference(samples, ops, 8, {"image": 0.0}, keys, seed=3)
    pkg.core.set_state(3)
    buf = refpipe.build(pkg, samples, ops, 8, {"image": 0.0}, keys, native_cast=True, buffer_mode=True)
    assert len(buf) == 3
    got = [dict(buf[i]) for i in range(3)]
    _check(got, want, True, _cast_scale(cfg["cast"]))
    # ordered prefetch keeps buffer order; shapes only (workers draw from their own generator copies)
    stream = buf.ordered_prefetch(2, 2)
    shapes = [b["image"].shape for b in stream]
    assert shapes == [(8, 224, 224, 3)] * 3


def test_prefetch_threads_deterministic_chain(pkg):
    """A chain without random ops gives the same batches whatever the thread count."""
    wl = _wl()
    cfg = wl.CONFIGS["c1"]
    samples = wl.make_samples("c1", "small", n=40)
    for i, s in enumerate(samples):
        s["label"] = np.int64(i)
    ops = wl.config_ops("c1", "small")
    want = refpipe.run_reference(samples, ops, 8, {"image": 0.0}, {"image": ()}, seed=0)
    by_first = {int(b["label"][0]): b for b in want}
    stream = refpipe.build(pkg, samples, ops, 8, {"image": 0.0}, {"image": ()}, native_cast=True, prefetch=(4, 4))
    got = [dict(b) for b in stream]
    assert len(got) == len(want)
    assert sorted(int(b["label"][0]) for b in got) == sorted(by_first)
    for b in got:
        _check([b], [by_first[int(b["label"][0])]], True, 1.0 / 255)


def test_thumbnails_of_large_images(pkg):
    """Shrink ratios of 100 and more, beyond what the staged resize passes hold:
    the chain still runs as one fused batch and equals the reference pipeline."""
    rng = np.random.default_rng(21)
    shapes = [(1400, 1900, 3), (1300, 1700, 3), (120, 90, 3), (1999, 1203, 3)]
    samples = [{"image": rng.integers(0, 256, s, dtype=np.uint8)} for s in shapes]
    ops = [("image_resize_smallest_side", dict(key="image", size=10)),
           ("image_center_crop", dict(key="image", w=10, h=10)),
           ("image_random_h_flip", dict(key="image", prob=0.5))]
    want = refpipe.run_reference(samples, ops, 4, {"image": 0.0}, {"image": ()}, seed=2)
    pkg.core.set_state(2)
    got = [dict(b) for b in refpipe.build(pkg, samples, ops, 4, {"image": 0.0}, {"image": ()}, native_cast=True)]
    _check(got, want, True, 1.0 / 255)


def test_unfused_ops_one_by_one(pkg):
    """Ops applied without a batch node run as single launches and still match."""
    rng = np.random.default_rng(8)
    img = rng.integers(0, 256, (90, 130, 3), dtype=np.uint8)
    dx = refpipe.reference_module()
    if dx is None:
        pytest.skip("needs oracle/_ref")
    def chain(m):
        m.core.set_state(11)
        b = m.buffer_from_vector([{"image": img}])
        b = (b.image_random_crop("image", 100, 80).image_rotate("image", 20.0, crop=False)
             .image_resize("image", 64, 48).image_rotate("image", -10.0, crop=True)
             .image_channel_reduction("image", "rec709", output_key="gray").image_random_h_flip("gray", 1.0))
        return dict(b[0])
    got, want = chain(pkg), chain(dx)
    assert got["image"].shape == want["image"].shape
    d = np.abs(got["image"].astype(int) - want["image"].astype(int))
    assert d.max() <= 1
    assert np.abs(got["gray"].astype(int) - want["gray"].astype(int)).max() <= 1


def test_error_behaviour_matches(pkg):
    img = np.zeros((10, 12, 3), np.uint8)
    b = pkg.buffer_from_vector([{"image": img}])
    with pytest.raises(RuntimeError, match="target image size larger"):
        b.image_center_crop("image", 20, 5)[0]
    with pytest.raises(RuntimeError, match="illegal target size"):
        b.image_resize_smallest_side("image", 0)[0]
    with pytest.raises(RuntimeError, match="expected a 3 channel"):
        pkg.buffer_from_vector([{"image": np.zeros((4, 4, 1), np.uint8)}]).image_channel_reduction("image")[0]
    with pytest.raises(RuntimeError, match="unable to find preset"):
        b.image_channel_reduction("image", "nope")
    with pytest.raises(RuntimeError, match="key <missing> expected"):
        b.image_resize("missing", 4, 4)[0]
    with pytest.raises(ValueError):
        pkg.buffer_from_vector([{"image": np.zeros((4, 4, 3), np.float32)}]).image_resize("image", 2, 2)[0]
    with pytest.raises(IndexError):
        b[3]


def test_four_channel_resize_is_refused_until_accepted(pkg, oracle):
    """mlx-data weights colour by alpha when it resizes a 4-channel image; the
    kernels filter the four channels independently.  The pipeline says so
    instead of returning different pixels, and runs once the caller accepts."""
    rng = np.random.default_rng(2)
    img = rng.integers(0, 256, (40, 52, 4), dtype=np.uint8)
    b = pkg.buffer_from_vector([{"image": img}])
    with pytest.raises(RuntimeError, match="weights colour by alpha"):
        b.image_resize("image", 20, 16)[0]
    with pytest.raises(RuntimeError, match="weights colour by alpha"):
        b.image_resize_smallest_side("image", 20).batch(1)[0]
    # the other ops do not care about the channel count
    assert np.array_equal(np.asarray(b.image_center_crop("image", 8, 8)[0]["image"]), img[16:24, 22:30])
    pkg.core.set_rgba_resize_independent(True)
    try:
        got = np.asarray(b.image_resize("image", 20, 16)[0]["image"])
        want = oracle.resize(img, 20, 16)      # the restatement, not the reference: independent channels too
        assert got.shape == want.shape and np.abs(got.astype(int) - want.astype(int)).max() <= 1
    finally:
        pkg.core.set_rgba_resize_independent(False)


def test_stream_dynamic_batch_of_images(pkg):
    """The stream variant on ragged images under deterministic ops (absorbed: sized
    symbolically, fused with each batch) and under a random op (samples taken as
    the source delivers them): same batches as the reference either way."""
    ref = refpipe.reference_module()
    if ref is None:
        pytest.skip("needs the reference compiled under oracle/_ref")
    rng = np.random.default_rng(9)
    samples = []
    for i in range(37):
        h, w = int(rng.integers(20, 140)), int(rng.integers(20, 140))
        samples.append({"image": rng.integers(0, 256, (h, w, 3), dtype=np.uint8), "id": np.int64(i)})

    def chain(dx, random_op):
        ds = dx.buffer_from_vector(samples).to_stream()
        if random_op:
            ds = ds.image_random_crop("image", 20, 20)
        ds = ds.image_resize_smallest_side("image", 32).slice("image", 0, 0, 48)
        return ds.dynamic_batch(16, "image", max_data_size=5 * 32 * 64 * 3, pad={"image": 3.0})

    for random_op in (False, True):
        ref.core.set_state(4)
        want = [dict(b) for b in chain(ref, random_op)]
        pkg.core.set_state(4)
        before = pkg.core.stats()["kernel_launches"]
        got = [dict(b) for b in chain(pkg, random_op)]
        used = pkg.core.stats()["kernel_launches"] - before
        assert len(got) == len(want) and len(want) > 2
        for g, w in zip(got, want):
            assert np.array_equal(np.asarray(g["id"]), np.asarray(w["id"]))
            a, b = np.asarray(g["image"]), np.asarray(w["image"])
            assert a.shape == b.shape and a.dtype == b.dtype
            if not random_op:
                # (with the random crop the pixels depend on which worker thread of the pulling
                # pool drew the offsets - in the reference too - so only grouping and shapes compare)
                d = np.abs(a.astype(np.int32) - b.astype(np.int32))
                assert d.max() <= 1 and (d > 0).mean() <= RESIZE_MISMATCH_MAX
        if not random_op:
            # sources are ordinary host arrays: one launch per batch (two extra per batch when
            # page-locked sources are gathered by a kernel, which these are not)
            assert used == len(want)


CLIP_CHAINS = {
    "resize_crop_flip": [("image_resize_smallest_side", dict(key="image", size=48)),
                         ("image_random_crop", dict(key="image", w=40, h=36)),
                         ("image_random_h_flip", dict(key="image", prob=0.5))],
    "area_crop_resize": [("image_random_area_crop", dict(key="image", area_range=(0.3, 1.0),
                                                          aspect_ratio_range=(0.75, 4 / 3))),
                         ("image_resize", dict(key="image", w=32, h=24))],
    "rotate_gray": [("image_rotate", dict(key="image", angle=20.0, crop=True)),
                    ("image_channel_reduction", dict(key="image", preset="default"))],
    "center_crop_only": [("image_center_crop", dict(key="image", w=30, h=20))],
}


@pytest.mark.parametrize("name", sorted(CLIP_CHAINS))
def test_clips_through_stream_api(pkg, name):
    """4-D [F, H, W, C] entries: every frame gets the op, random parameters are
    drawn once per clip (mlx/data/op/ImageTransform.cpp:33-70, 160-182, 293-357)."""
    if refpipe.reference_module() is None:
        pytest.skip("needs the reference compiled under oracle/_ref")
    ops = CLIP_CHAINS[name]
    rng = np.random.default_rng(77)
    samples = []
    for i in range(6):
        f, h, w = int(rng.integers(2, 6)), int(rng.integers(50, 90)), int(rng.integers(50, 90))
        samples.append({"image": rng.integers(0, 256, (f, h, w, 3), dtype=np.uint8), "label": np.int64(i)})
    keys = {"image": ()}
    want = refpipe.run_reference(samples, ops, 2, {"image": 9.0}, keys, seed=5)
    pkg.core.set_state(5)
    got = [dict(b) for b in refpipe.build(pkg, samples, ops, 2, {"image": 9.0}, keys, native_cast=True, product=True)]
    has_resize = any(n.startswith("image_resize") for n, _ in ops)
    _check(got, want, has_resize, 1.0 / 255)


def test_pinned_sources_are_gathered(pkg):
    """Samples in page-locked memory are staged by the gather kernel: only the
    rectangle each chain reads crosses the bus, and the batches do not change."""
    rng = np.random.default_rng(31)
    ops = [("image_center_crop", dict(key="image", w=61, h=45)),
           ("image_resize", dict(key="image", w=40, h=52)),
           ("image_random_h_flip", dict(key="image", prob=0.5))]
    plain, pinned = [], []
    for i in range(10):
        h, w = int(rng.integers(70, 130)), int(rng.integers(90, 170))
        img = rng.integers(0, 256, (h, w, 3), dtype=np.uint8)
        plain.append({"image": img})
        buf = pkg.core.pinned_empty([h, w, 3], "uint8")
        np.asarray(buf)[...] = img
        pinned.append({"image": buf})
    keys = {"image": ()}
    want = refpipe.run_reference(plain, ops, 4, {"image": 0.0}, keys, seed=9)
    pkg.core.set_state(9)
    s0 = pkg.core.stats()
    got = [dict(b) for b in refpipe.build(pkg, pinned, ops, 4, {"image": 0.0}, keys, native_cast=True, product=True)]
    s1 = pkg.core.stats()
    _check(got, want, True, 1.0 / 255)
    full = sum(s["image"].shape[0] * s["image"].shape[1] * 3 for s in plain)
    moved = s1["h2d_bytes"] - s0["h2d_bytes"]
    # a 61 x 45 window (plus filter margin) of images of at least 90 x 70 pixels
    assert 0 < moved < 0.8 * full, (moved, full)


def test_dynamic_batch_of_images(pkg):
    """Size-sorted batches of ragged images (the padding blow-up of plain batching
    on mixed sizes): same batches as the reference, ops fused below the batch."""
    ref = refpipe.reference_module()
    if ref is None:
        pytest.skip("needs the reference compiled under oracle/_ref")
    rng = np.random.default_rng(8)
    samples = []
    for i in range(23):
        h, w = int(rng.integers(20, 140)), int(rng.integers(20, 140))
        samples.append({"image": rng.integers(0, 256, (h, w, 3), dtype=np.uint8), "id": np.int64(i)})

    def chain(dx):
        return (dx.buffer_from_vector(samples)
                .image_resize_smallest_side("image", 32)
                .dynamic_batch("image", max_data_size=6 * 32 * 64 * 3, pad={"image": 3.0}))

    want = [dict(b) for b in chain(ref)]
    before = pkg.core.stats()["kernel_launches"]
    got_buf = chain(pkg).key_cast("image")
    # the samples were sized from their recorded programs: no launch so far
    assert pkg.core.stats()["kernel_launches"] == before
    got = [dict(got_buf[i]) for i in range(len(got_buf))]
    assert pkg.core.stats()["kernel_launches"] == before + len(got)    # one fused launch per batch
    assert len(got) == len(want)
    for g, w in zip(got, want):
        assert np.array_equal(np.asarray(g["id"]), np.asarray(w["id"]))
        a = np.asarray(g["image"])
        b = np.asarray(w["image"]).astype("float32") / 255
        assert a.shape == b.shape and a.dtype == np.float32
        d = np.abs(a.astype(np.float64) - b.astype(np.float64))
        assert d.max() <= 1.0001 / 255
        assert (a != b).mean() <= RESIZE_MISMATCH_MAX
