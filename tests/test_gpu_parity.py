"""GPU parity: the CUDA path, called through the C ABI, against the CPU oracle on
the same seeded inputs.  Bit-exact for crop / flip / rotate / gray / pad / batch
/ cast; resize within +-1 uint8 LSB (float outputs within 1/255 * scale) with an
additional bound on how often any difference may occur."""
import numpy as np
import pytest

import chain

pytestmark = pytest.mark.gpu

RESIZE_MISMATCH_MAX = 1e-3  # fraction of values allowed to differ by one LSB


def _rand(shape, seed):
    return np.random.default_rng(seed).integers(0, 256, shape, dtype=np.uint8)


def assert_resize_close(got, want):
    d = np.abs(got.astype(np.int32) - want.astype(np.int32))
    assert got.shape == want.shape
    assert d.max() <= 1, "resize differs by %d LSB at %s" % (d.max(), np.argwhere(d == d.max())[:4].tolist())
    assert (d > 0).mean() <= RESIZE_MISMATCH_MAX, "resize mismatch fraction %g" % (d > 0).mean()


# ---------------------------------------------------------------- standalone ops
@pytest.mark.parametrize("shape", [(1, 1, 3), (1, 37, 3), (41, 1, 1), (17, 23, 4), (64, 64, 3), (131, 257, 3), (300, 500, 2)])
def test_hflip(ctx, oracle, shape):
    img = _rand(shape, 1)
    assert np.array_equal(ctx.image_hflip(img), oracle.hflip(img))


@pytest.mark.parametrize("shape,rect", [((50, 70, 3), (3, 5, 64, 40)), ((50, 70, 1), (0, 0, 70, 50)),
                                         ((9, 9, 4), (8, 8, 1, 1)), ((200, 333, 3), (101, 7, 129, 190))])
def test_crop(ctx, oracle, shape, rect):
    img = _rand(shape, 2)
    x, y, w, h = rect
    assert np.array_equal(ctx.image_crop(img, x, y, w, h), oracle.crop(img, x, y, w, h))


def test_crop_out_of_bounds_is_rejected(ctx, pkg):
    img = _rand((10, 10, 3), 3)
    with pytest.raises(pkg.MlxdError) as e:
        ctx.image_crop(img, 5, 5, 6, 6)
    assert e.value.code == pkg._capi.ERR_INVALID


@pytest.mark.parametrize("shape,angle,crop", [((48, 64, 3), 17.0, True), ((48, 64, 3), -30.0, True),
                                               ((48, 64, 3), 17.0, False), ((5, 9, 3), 30.0, False),
                                               ((5, 9, 1), 0.0, True), ((130, 90, 4), 123.4, False),
                                               ((257, 255, 3), -7.25, True)])
def test_rotate(ctx, oracle, shape, angle, crop):
    import ctypes
    img = _rand(shape, 4)
    want = oracle.rotate(img, angle, crop)
    mx = oracle.rotate_matrix(angle)
    got = ctx.image_affine(img, list(mx), want.shape[0], want.shape[1])
    assert np.array_equal(got, want)


@pytest.mark.parametrize("preset", ["default", "rec709", "rec2020", "green"])
def test_channel_reduction(ctx, oracle, preset):
    img = _rand((77, 129, 3), 5)
    m = chain.gray_fixed(preset)
    assert np.array_equal(ctx.image_channel_reduction(img, m[:3], m[3]), oracle.channel_reduction(img, preset))
    white = np.full((4, 4, 3), 255, np.uint8)
    m = chain.gray_fixed("default")
    assert ctx.image_channel_reduction(white, m[:3], m[3]).max() == 254


@pytest.mark.parametrize("shape,dst", [
    ((300, 400, 3), (256, 341)), ((500, 333, 3), (384, 256)), ((210, 205, 3), (262, 256)),
    ((64, 64, 3), (320, 320)), ((7, 5, 1), (3, 11)), ((1, 1, 3), (9, 9)), ((33, 1, 4), (5, 8)),
    ((1080, 1920, 3), (512, 910)), ((600, 800, 3), (60, 80)), ((1024, 64, 3), (320, 20)),
    ((900, 1300, 3), (40, 33)), ((100, 100, 3), (100, 37)), ((100, 100, 2), (51, 100))])
def test_resize(ctx, oracle, shape, dst):
    # The 4-channel case checks kernel against restatement only: both filter the
    # four channels independently, while the reference's resize library treats
    # 4 channels as RGBA and weights colour by alpha.  It is not a parity case.
    img = _rand(shape, 6)
    dh, dw = dst
    got = ctx.image_resize(img, dw, dh)
    assert_resize_close(got, oracle.resize(img, dw, dh))


def test_resize_identity_is_exact(ctx):
    img = _rand((37, 53, 3), 7)
    assert np.array_equal(ctx.image_resize(img, 53, 37), img)


def test_batch_pad(ctx, oracle):
    imgs = [_rand((h, w, 3), 10 + i) for i, (h, w) in enumerate([(2, 3), (3, 2), (17, 70), (65, 5), (1, 1)])]
    for pad in (0.0, 7.0, 255.0):
        want = oracle.batch_pad(imgs, pad)
        got = ctx.batch_pad(imgs, want.shape[1], want.shape[2], pad)
        assert np.array_equal(got, want)
    ones = [np.ones((2, 3, 1), np.uint8), np.ones((3, 2, 1), np.uint8)]
    got = ctx.batch_pad(ones, 3, 3, 7.0)[..., 0]
    assert got.tolist() == [[[1, 1, 1], [1, 1, 1], [7, 7, 7]], [[1, 1, 7], [1, 1, 7], [1, 1, 7]]]


@pytest.mark.parametrize("c", [1, 3, 4])
def test_cast(ctx, c):
    x = _rand((5, 41, 67, c), 11)
    got = ctx.cast_scale_normalise(x)
    assert got.dtype == np.float32
    assert np.array_equal(got, x.astype("float32") / 255)
    mean = np.array([0.485, 0.456, 0.406, 0.5][:c], np.float32)
    std = np.array([0.229, 0.224, 0.225, 0.25][:c], np.float32)
    got = ctx.cast_scale_normalise(x, 255.0, mean, std)
    assert np.array_equal(got, (x.astype("float32") / 255 - mean) / std)
    big = _rand((3 * 4096 + 5, 1, c), 12)
    assert np.array_equal(ctx.cast_scale_normalise(big), big.astype("float32") / 255)


def test_cast_with_more_parameter_sets_than_the_table_cache_holds(pkg):
    """Every distinct (divisor, mean, std) gets a device table that the context
    keeps; the cache is bounded (256 tables), emptied when full.  Results stay
    exact across the emptying, also for parameter sets seen before it."""
    own = pkg.Context(device=0, n_lanes=1)
    try:
        x = _rand((2, 9, 13, 3), 13)
        std = np.array([0.229, 0.224, 0.225], np.float32)
        for i in list(range(300)) + [0, 1, 299]:
            mean = np.array([0.1 + i / 1000.0, 0.456, 0.406], np.float32)
            got = own.cast_scale_normalise(x, 255.0, mean, std)
            assert np.array_equal(got, (x.astype("float32") / 255 - mean) / std), i
    finally:
        own.close()


# ---------------------------------------------------------------- fused chains
def _oracle_batches(oracle, samples, ops, batch, cast, pad, key="image"):
    oracle.set_state(0)
    c = None
    if cast is not None:
        c = {key: None if len(cast) == 0 else (np.array(cast[0], np.float32), np.array(cast[1], np.float32))}
    return [b[key] for b in oracle.run_chain(samples, ops, batch, {key: pad}, c)]


def _fused_batches(pkg, ctx, oracle, samples, ops, batch, cast, pad):
    oracle.set_state(0)
    return chain.run_fused(pkg, ctx, samples, "image", ops, batch, cast, pad)


def _compare(got, want, has_resize, cast):
    assert len(got) == len(want)
    for g, w in zip(got, want):
        assert g.shape == w.shape and g.dtype == w.dtype
        if not has_resize:
            assert np.array_equal(g, w)
        elif cast is None:
            assert_resize_close(g, w)
        else:
            # one uint8 LSB after the cast: 1/255, divided by the smallest std
            scale = 1.0 / 255 if len(cast) == 0 else 1.0 / 255 / min(cast[1])
            d = np.abs(g.astype(np.float64) - w.astype(np.float64))
            assert d.max() <= scale * 1.0001
            assert (g != w).mean() <= RESIZE_MISMATCH_MAX


@pytest.mark.parametrize("name", ["c1", "c2", "c3", "c4", "c5"])
def test_config_small(pkg, ctx, oracle, name):
    wl = pkg_workloads(pkg)
    cfg = wl.CONFIGS[name]
    samples = wl.make_samples(name, "small")
    ops = wl.config_ops(name, "small")
    batch = cfg["small"]["batch"]
    want = _oracle_batches(oracle, samples, ops, batch, cfg["cast"], cfg["pad"])
    got = _fused_batches(pkg, ctx, oracle, samples, ops, batch, cfg["cast"], cfg["pad"])
    _compare(got, want, name != "c4", cfg["cast"])


def test_config_c3_gray_key(pkg, ctx, oracle):
    wl = pkg_workloads(pkg)
    cfg = wl.CONFIGS["c3"]
    samples = wl.make_samples("c3", "small")
    ops = wl.config_ops("c3", "small", "gray_ops")
    batch = cfg["small"]["batch"]
    oracle.set_state(0)
    want = [b["gray"] for b in oracle.run_chain(samples, ops, batch, {"gray": 0.0}, {"gray": None})]
    flat = [(n, {k: v for k, v in kw.items() if k != "output_key"}) for n, kw in ops]
    got = chain.run_fused(pkg, ctx, samples, "image", flat, batch, (), 0.0)
    _compare(got, want, True, ())


def pkg_workloads(pkg):
    import importlib
    return importlib.import_module("mlx_data_b200.workloads")


CHAINS = {
    "crop_flip_u8": ([("image_random_crop", dict(key="image", w=40, h=33)),
                      ("image_random_h_flip", dict(key="image", prob=0.5))], None, 9.0),
    "flip_then_crop_then_resize": ([("image_random_h_flip", dict(key="image", prob=1.0)),
                                    ("image_center_crop", dict(key="image", w=51, h=47)),
                                    ("image_resize", dict(key="image", w=30, h=64)),
                                    ("image_random_h_flip", dict(key="image", prob=0.5))], (), 0.0),
    "crop_rotate_crop_gray": ([("image_center_crop", dict(key="image", w=57, h=49)),
                               ("image_random_h_flip", dict(key="image", prob=0.5)),
                               ("image_rotate", dict(key="image", angle=33.0, crop=False)),
                               ("image_center_crop", dict(key="image", w=31, h=29)),
                               ("image_channel_reduction", dict(key="image", preset="rec709"))], (), 3.0),
    "upsample_ragged_pad": ([("image_resize_smallest_side", dict(key="image", size=150)),
                             ("image_random_h_flip", dict(key="image", prob=0.5))], None, 200.0),
    "area_crop_only": ([("image_random_area_crop", dict(key="image", area_range=(0.08, 1.0),
                                                        aspect_ratio_range=(0.75, 4 / 3)))], (), 1.0),
}


@pytest.mark.parametrize("name", sorted(CHAINS))
def test_mixed_chain(pkg, ctx, oracle, name):
    ops, cast, pad = CHAINS[name]
    rng = np.random.default_rng(21)
    samples = [{"image": rng.integers(0, 256, (int(rng.integers(60, 120)), int(rng.integers(60, 120)), 3), dtype=np.uint8)}
               for _ in range(11)]
    want = _oracle_batches(oracle, samples, ops, 4, cast, pad)
    got = _fused_batches(pkg, ctx, oracle, samples, ops, 4, cast, pad)
    has_resize = any(n.startswith("image_resize") for n, _ in ops)
    _compare(got, want, has_resize, cast)


def test_device_resident_on_stream(pkg, ctx, oracle):
    """Device sources and destination through mlxd_fused_batch_on_stream."""
    torch = pytest.importorskip("torch")
    wl = pkg_workloads(pkg)
    cfg = wl.CONFIGS["c2"]
    samples = wl.make_samples("c2", "small", n=8)
    ops = wl.config_ops("c2", "small")
    want = _oracle_batches(oracle, samples, ops, 8, cfg["cast"], 0.0)[0]
    dev = [torch.from_numpy(s["image"]).cuda() for s in samples]
    oracle.set_state(0)
    descs = np.zeros(8, pkg.SAMPLE_DTYPE)
    for i, s in enumerate(samples):
        chain.fill_descs(descs, i, chain.reduce_chain(s["image"].shape, ops, s), dev[i].data_ptr())
    out = torch.empty((8, 224, 224, 3), dtype=torch.float32, device="cuda")
    bd = pkg.make_batch_desc(out.data_ptr(), 224, 224, 3, mean=cfg["cast"][0], std=cfg["cast"][1],
                             src_mem=pkg._capi.MEM_DEVICE, dst_mem=pkg._capi.MEM_DEVICE)
    ctx.fused_batch_on_stream(torch.cuda.current_stream().cuda_stream, descs, bd)
    torch.cuda.synchronize()
    _compare([out.cpu().numpy()], [want], True, cfg["cast"])


def test_errors(pkg, ctx):
    img = _rand((10, 10, 3), 30)
    with pytest.raises(pkg.MlxdError) as e:
        ctx.image_resize(img, 0, 5)
    assert e.value.code == pkg._capi.ERR_INVALID
    with pytest.raises(pkg.MlxdError):
        ctx.wait(99)
    # an empty batch is a no-op
    descs = np.zeros(0, pkg.SAMPLE_DTYPE)
    out = np.zeros((1, 4, 4, 3), np.float32)
    ctx.fused_batch(0, descs, pkg.make_batch_desc(out, 4, 4, 3))
    ctx.wait(0)
    s = ctx.stats()
    assert s["kernel_launches"] > 0 and s["h2d_bytes"] > 0


# ---------------------------------------------------------------- float32 kernel, resize corner cases
FAST_RESIZE_CASES = [
    # (source H, W), channels, ops: pitches that are / are not multiples of 8 bytes, up- and down-scaling,
    # ratios that force smaller passes, windows at odd offsets, mirrored outputs, tiny images
    ((96, 128), 3, [("image_resize", dict(key="image", w=61, h=47))]),
    ((96, 128), 1, [("image_resize", dict(key="image", w=61, h=47))]),
    ((96, 128), 4, [("image_resize", dict(key="image", w=61, h=47))]),
    ((97, 131), 3, [("image_resize", dict(key="image", w=200, h=150))]),
    ((97, 131), 1, [("image_resize", dict(key="image", w=33, h=29)), ("image_random_h_flip", dict(key="image", prob=1.0))]),
    ((97, 131), 4, [("image_resize", dict(key="image", w=131, h=40))]),
    ((513, 777), 3, [("image_center_crop", dict(key="image", w=701, h=451)),
                     ("image_resize", dict(key="image", w=90, h=70)),
                     ("image_center_crop", dict(key="image", w=77, h=63))]),
    ((700, 1100), 3, [("image_resize", dict(key="image", w=37, h=25))]),
    ((600, 40), 3, [("image_resize", dict(key="image", w=40, h=19))]),
    ((5, 3), 3, [("image_resize", dict(key="image", w=67, h=130))]),
    ((1, 1), 4, [("image_resize", dict(key="image", w=17, h=3))]),
    ((240, 320), 3, [("image_resize_smallest_side", dict(key="image", size=96)),
                     ("image_random_h_flip", dict(key="image", prob=1.0)),
                     ("image_center_crop", dict(key="image", w=80, h=80))]),
    # mirrored sources: the flip comes before the resize
    ((97, 131), 3, [("image_random_h_flip", dict(key="image", prob=1.0)),
                    ("image_resize", dict(key="image", w=33, h=29))]),
    ((96, 128), 1, [("image_random_h_flip", dict(key="image", prob=1.0)),
                    ("image_center_crop", dict(key="image", w=101, h=77)),
                    ("image_resize", dict(key="image", w=160, h=120))]),
    ((513, 777), 3, [("image_random_h_flip", dict(key="image", prob=1.0)),
                     ("image_random_crop", dict(key="image", w=701, h=451)),
                     ("image_resize", dict(key="image", w=90, h=70)),
                     ("image_random_h_flip", dict(key="image", prob=1.0)),
                     ("image_center_crop", dict(key="image", w=77, h=63))]),
    ((5, 3), 3, [("image_random_h_flip", dict(key="image", prob=1.0)),
                 ("image_resize", dict(key="image", w=67, h=130))]),
    ((700, 1100), 4, [("image_random_h_flip", dict(key="image", prob=1.0)),
                      ("image_resize", dict(key="image", w=37, h=25))]),
    ((300, 410), 3, [("image_random_h_flip", dict(key="image", prob=0.5)),
                     ("image_resize_smallest_side", dict(key="image", size=128))]),
]


@pytest.mark.parametrize("case", range(len(FAST_RESIZE_CASES)))
@pytest.mark.parametrize("cast", [(), "norm"])
def test_float32_resize_cases(pkg, ctx, oracle, case, cast):
    (h, w), c, ops = FAST_RESIZE_CASES[case]
    rng = np.random.default_rng(100 + case)
    # three samples per batch, the later ones one row / column smaller: ragged slots and padding
    samples = [{"image": rng.integers(0, 256, (max(1, h - i), max(1, w - 2 * i), c), dtype=np.uint8)} for i in range(3)]
    if cast == "norm":
        cast = ([0.485, 0.456, 0.406, 0.5][:c], [0.229, 0.224, 0.225, 0.25][:c])
    want = _oracle_batches(oracle, samples, ops, 3, cast, 5.0)
    got = _fused_batches(pkg, ctx, oracle, samples, ops, 3, cast, 5.0)
    _compare(got, want, True, cast)


# ---------------------------------------------------------------- shrink ratios beyond the on-chip passes
DIRECT_RESIZE_CASES = [
    # one output row of these takes more source rows (2 * ratio + 1) than a pass can stage (192): every
    # pixel is filtered from global memory by the kernel for such samples
    ((1500, 1500), 3, [("image_resize", dict(key="image", w=12, h=12))]),
    ((2100, 64), 1, [("image_resize", dict(key="image", w=32, h=10))]),
    ((1300, 900), 4, [("image_random_h_flip", dict(key="image", prob=1.0)),
                      ("image_resize", dict(key="image", w=9, h=7)),
                      ("image_center_crop", dict(key="image", w=5, h=5))]),
    ((1200, 301), 3, [("image_resize", dict(key="image", w=11, h=4)),
                      ("image_random_h_flip", dict(key="image", prob=1.0))]),
    ((1000, 40), 2, [("image_resize", dict(key="image", w=40, h=5))]),
]


@pytest.mark.parametrize("case", range(len(DIRECT_RESIZE_CASES)))
@pytest.mark.parametrize("cast", [None, (), "norm"])
def test_resize_beyond_the_on_chip_footprint(pkg, ctx, oracle, case, cast):
    """A batch of two such samples and one small image that takes the staged
    passes, same chain: uint8, float32 and normalised float32 out."""
    (h, w), c, ops = DIRECT_RESIZE_CASES[case]
    rng = np.random.default_rng(500 + case)
    shapes = [(h, w), (h - 7, w - 3), (57, 64)]
    samples = [{"image": rng.integers(0, 256, (a, b, c), dtype=np.uint8)} for a, b in shapes]
    if cast == "norm":
        cast = ([0.485, 0.456, 0.406, 0.5][:c], [0.229, 0.224, 0.225, 0.25][:c])
    want = _oracle_batches(oracle, samples, ops, 3, cast, 3.0)
    got = _fused_batches(pkg, ctx, oracle, samples, ops, 3, cast, 3.0)
    _compare(got, want, True, cast)


def test_resize_beyond_the_on_chip_footprint_gray(pkg, ctx, oracle):
    ops = [("image_resize", dict(key="image", w=14, h=9)),
           ("image_channel_reduction", dict(key="image", preset="default"))]
    rng = np.random.default_rng(77)
    samples = [{"image": rng.integers(0, 256, s, dtype=np.uint8)} for s in [(1100, 1400, 3), (90, 70, 3)]]
    for cast in (None, ()):
        want = _oracle_batches(oracle, samples, ops, 2, cast, 0.0)
        got = _fused_batches(pkg, ctx, oracle, samples, ops, 2, cast, 0.0)
        assert got[0].shape[-1] == 1
        _compare(got, want, True, cast)


# ---------------------------------------------------------------- float32 kernel, channel reduction
GRAY_CASES = [
    [("image_resize", dict(key="image", w=61, h=47)),
     ("image_channel_reduction", dict(key="image", preset="default"))],
    [("image_random_h_flip", dict(key="image", prob=1.0)),
     ("image_resize_smallest_side", dict(key="image", size=150)),
     ("image_center_crop", dict(key="image", w=100, h=90)),
     ("image_channel_reduction", dict(key="image", preset="rec601"))],
    [("image_random_crop", dict(key="image", w=70, h=50)),
     ("image_random_h_flip", dict(key="image", prob=0.5)),
     ("image_channel_reduction", dict(key="image", preset="rec709"))],
    [("image_rotate", dict(key="image", angle=-17.0, crop=True)),
     ("image_channel_reduction", dict(key="image", preset="rec2020"))],
    [("image_channel_reduction", dict(key="image", preset="green"))],
]


@pytest.mark.parametrize("case", range(len(GRAY_CASES)))
@pytest.mark.parametrize("cast", [(), "norm"])
def test_float32_gray_cases(pkg, ctx, oracle, case, cast):
    """Chains that end in the channel reduction, float32 out: the quantised
    pixel goes through the fixed-point mix, then the one-channel cast."""
    ops = GRAY_CASES[case]
    rng = np.random.default_rng(300 + case)
    samples = [{"image": rng.integers(0, 256, (97 - 3 * i, 131 - 5 * i, 3), dtype=np.uint8)} for i in range(4)]
    if cast == "norm":
        cast = ([0.45], [0.225])
    has_resize = any(n.startswith("image_resize") for n, _ in ops)
    want = _oracle_batches(oracle, samples, ops, 4, cast, 2.0)
    got = _fused_batches(pkg, ctx, oracle, samples, ops, 4, cast, 2.0)
    assert got[0].shape[-1] == 1
    _compare(got, want, has_resize, cast)
