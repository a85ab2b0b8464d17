"""GPU parity at the launch geometry the benchmark runs: the five configurations
at their configured image sizes, with enough samples per launch that the kernel
takes the same band and pass structure as a full batch, compared with the CPU
oracle on every slot.  Crop / flip / rotate / pad / cast are held bit-exact;
resize to +-1 uint8 LSB with a bound on how often a value may differ.  The
resize arithmetic of the reference lives in an un-vendored header (stb), so the
resize oracle is a restatement of its published behaviour, not the reference's
own code."""
import importlib

import numpy as np
import pytest

import chain

pytestmark = pytest.mark.gpu

RESIZE_MISMATCH_MAX = 1e-3
MEAN = (0.485, 0.456, 0.406)
STD = (0.229, 0.224, 0.225)


def _wl():
    return importlib.import_module("mlx_data_b200.workloads")


def _lut(cast):
    """float32 value of every uint8 after the cast, per channel: [3, 256]."""
    x = np.arange(256, dtype=np.uint8).reshape(256, 1).repeat(3, 1)
    if len(cast) == 0:
        return (x.astype("float32") / 255).T.copy()
    mean, std = np.array(cast[0], np.float32), np.array(cast[1], np.float32)
    return ((x.astype("float32") / 255 - mean) / std).T.copy()


def _cast(u8, lut):
    out = np.empty(u8.shape, np.float32)
    for c in range(u8.shape[-1]):
        out[..., c] = lut[c][u8[..., c]]
    return out


def _check_slot(got, want_u8, lut, has_resize, where):
    want = _cast(want_u8, lut)
    if not has_resize:
        assert np.array_equal(got, want), where
        return 0
    step = np.abs(np.diff(lut, axis=1)).max()        # one uint8 LSB after the cast
    d = np.abs(got.astype(np.float64) - want.astype(np.float64))
    assert d.max() <= step * 1.0001, (where, d.max())
    return int((got != want).sum())


def _descs_for(pkg, oracle, samples, ops, addrs, seed):
    oracle.set_state(seed)
    descs = np.zeros(len(samples), pkg.SAMPLE_DTYPE)
    fields = []
    for i, s in enumerate(samples):
        f = chain.reduce_chain(s["image"].shape, ops, s)
        fields.append(f)
        chain.fill_descs(descs, i, f, addrs[i])
    return descs, fields


def _run_device(pkg, ctx, torch, descs, n, sh, sw, cast, pad):
    capi = pkg._capi
    out = torch.full((n, sh, sw, 3), -5.0, dtype=torch.float32, device="cuda")
    mean, std = (cast if len(cast) == 2 else (None, None))
    bd = pkg.make_batch_desc(out.data_ptr(), sh, sw, 3, mean=mean, std=std, pad_value=pad,
                             src_mem=capi.MEM_DEVICE, dst_mem=capi.MEM_DEVICE)
    stream = torch.cuda.current_stream().cuda_stream
    ctx.fused_batch_on_stream(stream, descs, bd)
    assert ctx.stream_status(stream) == 0
    return out.cpu().numpy()


def _run_host(pkg, ctx, descs, n, sh, sw, cast, pad):
    out = np.full((n, sh, sw, 3), -5.0, np.float32)
    mean, std = (cast if len(cast) == 2 else (None, None))
    bd = pkg.make_batch_desc(out, sh, sw, 3, mean=mean, std=std, pad_value=pad)
    ctx.fused_batch(0, descs, bd)
    ctx.wait(0)
    return out


def _compare_batch(got, fields, expected_u8, lut, pad, has_resize):
    """expected_u8[i]: the post-window image of sample i (uint8); the rest of the slot is pad."""
    n, sh, sw, _ = got.shape
    padv = np.array([lut[c][int(pad)] for c in range(3)], np.float32)
    differing = 0
    total = 0
    for i in range(n):
        e = expected_u8[i]
        h, w = e.shape[:2]
        differing += _check_slot(got[i, :h, :w], e, lut, has_resize, "sample %d" % i)
        total += e.size
        assert np.array_equal(got[i, h:, :, :], np.broadcast_to(padv, (sh - h, sw, 3))), "pad rows of %d" % i
        assert np.array_equal(got[i, :h, w:, :], np.broadcast_to(padv, (h, sw - w, 3))), "pad columns of %d" % i
    assert differing <= RESIZE_MISMATCH_MAX * total, (differing, total)


@pytest.mark.parametrize("feed", ["device", "host"])
def test_c5_full_size_launch(pkg, ctx, oracle, feed):
    """1080 x 1920 -> smallest side 512 -> centre crop 512 x 512 -> random flip -> normalise, 128 slots
    from 8 distinct sources: the bands, passes and tables of a full 512-image launch."""
    torch = pytest.importorskip("torch")
    wl = _wl()
    ops = wl.config_ops("c5", "full")
    rng = np.random.default_rng(50)
    sources = [rng.integers(0, 256, (1080, 1920, 3), dtype=np.uint8) for _ in range(8)]
    base = []
    for s in sources:
        r = oracle.resize_smallest_side(s, 512)
        base.append(oracle.center_crop(r, 512, 512))
    n = 128
    samples = [{"image": sources[i % 8]} for i in range(n)]
    cast = (MEAN, STD)
    lut = _lut(cast)
    if feed == "device":
        dev = [torch.from_numpy(s).cuda() for s in sources]
        addrs = [dev[i % 8].data_ptr() for i in range(n)]
    else:
        addrs = [sources[i % 8].ctypes.data for i in range(n)]
    descs, fields = _descs_for(pkg, oracle, samples, ops, addrs, seed=17)
    flips = [f["post_flip"] for f in fields]
    assert 0 < sum(flips) < n
    expected = [oracle.hflip(base[i % 8]) if flips[i] else base[i % 8] for i in range(n)]
    if feed == "device":
        got = _run_device(pkg, ctx, torch, descs, n, 512, 512, cast, 0.0)
    else:
        got = _run_host(pkg, ctx, descs, n, 512, 512, cast, 0.0)
    _compare_batch(got, fields, expected, lut, 0.0, True)


def test_c2_full_batch(pkg, ctx, oracle):
    """256 images of 256..800 pixels a side -> random area crop -> 224 x 224 -> random flip -> normalise."""
    torch = pytest.importorskip("torch")
    wl = _wl()
    ops = wl.config_ops("c2", "full")
    samples = wl.make_samples("c2", "full", n=256)
    cast = (MEAN, STD)
    lut = _lut(cast)
    dev = [torch.from_numpy(s["image"]).cuda() for s in samples]
    descs, fields = _descs_for(pkg, oracle, samples, ops, [d.data_ptr() for d in dev], seed=0)
    expected = [chain.interpret(f, s["image"]) for f, s in zip(fields, samples)]
    got = _run_device(pkg, ctx, torch, descs, 256, 224, 224, cast, 0.0)
    _compare_batch(got, fields, expected, lut, 0.0, True)


def test_c1_full_batches(pkg, ctx, oracle):
    """200..500 pixels a side -> smallest side 256 -> centre crop 224 x 224 -> /255, batches of 32."""
    torch = pytest.importorskip("torch")
    wl = _wl()
    ops = wl.config_ops("c1", "full")
    samples = wl.make_samples("c1", "full", n=64)
    lut = _lut(())
    for b0 in (0, 32):
        chunk = samples[b0:b0 + 32]
        dev = [torch.from_numpy(s["image"]).cuda() for s in chunk]
        descs, fields = _descs_for(pkg, oracle, chunk, ops, [d.data_ptr() for d in dev], seed=0)
        expected = [chain.interpret(f, s["image"]) for f, s in zip(fields, chunk)]
        got = _run_device(pkg, ctx, torch, descs, 32, 224, 224, (), 0.0)
        _compare_batch(got, fields, expected, lut, 0.0, True)


def test_c3_configured_geometry(pkg, ctx, oracle):
    """64..1024 pixels a side -> smallest side 320, ragged slots padded to the batch maximum; the
    batch holds a 15:1 strip (a 5000-pixel-wide slot), a 5x enlargement and a 3.2x reduction."""
    torch = pytest.importorskip("torch")
    wl = _wl()
    ops = wl.config_ops("c3", "full")
    rng = np.random.default_rng(33)
    shapes = [(64, 1000), (64, 64), (1024, 1024), (1000, 70), (333, 777), (512, 320), (65, 1024), (700, 129)]
    for b0 in (0, 4):
        chunk = [{"image": rng.integers(0, 256, (h, w, 3), dtype=np.uint8)} for h, w in shapes[b0:b0 + 4]]
        dev = [torch.from_numpy(s["image"]).cuda() for s in chunk]
        descs, fields = _descs_for(pkg, oracle, chunk, ops, [d.data_ptr() for d in dev], seed=0)
        expected = [chain.interpret(f, s["image"]) for f, s in zip(fields, chunk)]
        sh = max(e.shape[0] for e in expected)
        sw = max(e.shape[1] for e in expected)
        got = _run_device(pkg, ctx, torch, descs, len(chunk), sh, sw, (), 0.0)
        _compare_batch(got, fields, expected, _lut(()), 0.0, True)
    # the configuration's own size distribution, one batch of 8
    samples = wl.make_samples("c3", "full", n=8)
    dev = [torch.from_numpy(s["image"]).cuda() for s in samples]
    descs, fields = _descs_for(pkg, oracle, samples, ops, [d.data_ptr() for d in dev], seed=0)
    expected = [chain.interpret(f, s["image"]) for f, s in zip(fields, samples)]
    sh = max(e.shape[0] for e in expected)
    sw = max(e.shape[1] for e in expected)
    got = _run_device(pkg, ctx, torch, descs, 8, sh, sw, (), 0.0)
    _compare_batch(got, fields, expected, _lut(()), 0.0, True)


def test_c4_configured_geometry(pkg, ctx, oracle):
    """512 x 512 -> rotate by a per-sample angle in [-30, 30] (cropped to the input size) -> random
    flip -> centre crop 448 x 448 -> /255; bit-exact."""
    torch = pytest.importorskip("torch")
    wl = _wl()
    ops = wl.config_ops("c4", "full")
    samples = wl.make_samples("c4", "full", n=32)
    dev = [torch.from_numpy(s["image"]).cuda() for s in samples]
    descs, fields = _descs_for(pkg, oracle, samples, ops, [d.data_ptr() for d in dev], seed=0)
    expected = [chain.interpret(f, s["image"]) for f, s in zip(fields, samples)]
    got = _run_device(pkg, ctx, torch, descs, 32, 448, 448, (), 0.0)
    _compare_batch(got, fields, expected, _lut(()), 0.0, False)
