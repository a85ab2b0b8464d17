"""The CUDA path against the golden vectors recorded from the reference
(tests/golden/golden.json).  Exact where no resize is involved; pipelines with a
resize are compared value by value with the oracle elsewhere, here only shapes
and near-equality of the sums are checked for them."""
import hashlib
import importlib
import json
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def golden():
    with open(os.path.join(HERE, "golden", "golden.json")) as f:
        return json.load(f)


def digest(a):
    a = np.ascontiguousarray(a)
    return {"shape": list(a.shape), "dtype": str(a.dtype), "sha256": hashlib.sha256(a.tobytes()).hexdigest()[:24],
            "sum": float(a.astype(np.float64).sum())}


def ramp():
    r = np.arange(48 * 64 * 3, dtype=np.uint32).reshape(48, 64, 3)
    return ((r * np.uint32(2654435761)) >> 24).astype(np.uint8)


def test_random_draw_sequences(pkg, golden):
    for seed in (0, 1234):
        pkg.core.set_state(seed)
        s = [{"image": np.arange(72, dtype=np.uint8).reshape(4, 6, 3)} for _ in range(16)]
        st = pkg.buffer_from_vector(s).to_stream().image_random_h_flip("image", 0.5)
        assert [int(x["image"][0, 0, 0] != 0) for x in st] == golden["flips_seed%d" % seed]
    pkg.core.set_state(0)
    yy, xx = np.meshgrid(np.arange(480), np.arange(640), indexing="ij")
    coord = np.stack([xx % 256, xx // 256, yy % 256], -1).astype(np.uint8)
    st = pkg.buffer_from_vector([{"image": coord} for _ in range(8)]).to_stream() \
        .image_random_area_crop("image", (0.08, 1.0), (0.75, 4 / 3))
    rects = []
    for x in st:
        im = x["image"]
        rects.append([int(im[0, 0, 0]) + 256 * int(im[0, 0, 1]), int(im[0, 0, 2]), im.shape[1], im.shape[0]])
    assert rects == golden["area_crop_rects_seed0_lowbyte_y"]


def test_rotate_gray_pad(pkg, golden):
    rp = ramp()
    for ang, crop in [(17.0, True), (-30.0, True), (30.0, True), (17.0, False)]:
        out = pkg.buffer_from_vector([{"image": rp}]).image_rotate("image", ang, crop)[0]["image"]
        assert digest(out) == golden["rotate_%g_%d" % (ang, int(crop))]
    for preset in ("rec709", "default", "rec2020", "green"):
        out = pkg.buffer_from_vector([{"image": rp}]).image_channel_reduction("image", preset)[0]["image"]
        assert digest(out) == golden["gray_" + preset]
    b = pkg.buffer_from_vector([{"x": np.ones((2, 3), np.uint8)}, {"x": np.ones((3, 2), np.uint8)}]).batch(2, pad={"x": 7})
    assert b[0]["x"].tolist() == golden["batch_pad7"]


def test_rotate_pipeline_exact(pkg, golden):
    wl = importlib.import_module("mlx_data_b200.workloads")
    samples = [{"image": s["image"]} for s in wl.make_samples("c4", "small", n=8)]
    pkg.core.set_state(0)
    ds = (pkg.buffer_from_vector(samples).to_stream().image_rotate("image", 21.5, crop=True)
          .image_random_h_flip("image", 0.5).image_center_crop("image", 140, 140).batch(4).key_cast("image"))
    assert [digest(b["image"]) for b in ds] == golden["pipeline_c4_fixed_angle_small8"]["batches"]


@pytest.mark.parametrize("name", ["c1", "c2", "c3", "c5"])
def test_resize_pipelines_shapes_and_sums(pkg, golden, name):
    wl = importlib.import_module("mlx_data_b200.workloads")
    cfg = wl.CONFIGS[name]
    samples = wl.make_samples(name, "small", n=8)
    pkg.core.set_state(0)
    ds = pkg.buffer_from_vector(samples).to_stream()
    for op, kw in wl.config_ops(name, "small"):
        ds = getattr(ds, op)(**kw)
    ds = ds.batch(4)
    ds = ds.key_cast("image") if len(cfg["cast"]) == 0 else ds.key_cast("image", mean=list(cfg["cast"][0]),
                                                                        std=list(cfg["cast"][1]))
    want = golden["pipeline_%s_small8" % name]["batches"]
    got = [digest(b["image"]) for b in ds]
    assert len(got) == len(want)
    for g, w in zip(got, want):
        assert g["shape"] == w["shape"] and g["dtype"] == w["dtype"]
        n = float(np.prod(w["shape"]))
        scale = 1 / 255 if len(cfg["cast"]) == 0 else 1 / 255 / min(cfg["cast"][1])
        assert abs(g["sum"] - w["sum"]) <= n * scale * 1e-3
