"""The CPU oracle against the golden vectors recorded from the reference itself
(tests/golden/golden.json, made by tests/golden/make_golden.py from the build
under oracle/_ref).  This pins the restatement before it is trusted as the
checker of the CUDA path."""
import hashlib
import importlib
import json
import os

import numpy as np
import pytest

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


def test_flip_draws(oracle, golden):
    for seed in (0, 1234):
        oracle.set_state(seed)
        assert [int(oracle.draw_hflip(0.5)) for _ in range(16)] == golden["flips_seed%d" % seed]


def test_area_crop_rectangles(oracle, golden):
    oracle.set_state(0)
    got = [list(oracle.draw_area_crop(640, 480, (0.08, 1.0), (0.75, 4 / 3))) for _ in range(8)]
    assert got == golden["area_crop_rects_seed0_lowbyte_y"]


def test_rotate_and_gray(oracle, golden):
    rp = ramp()
    assert digest(rp) == golden["ramp"]
    for ang, crop in [(17.0, True), (-30.0, True), (30.0, True), (17.0, False)]:
        assert digest(oracle.rotate(rp, ang, crop)) == golden["rotate_%g_%d" % (ang, int(crop))]
    for preset in ("rec709", "default", "rec2020", "green"):
        assert digest(oracle.channel_reduction(rp, preset)) == golden["gray_" + preset]
    assert oracle.channel_reduction(np.full((4, 4, 3), 255, np.uint8)).max() == golden["gray_white_value"] == 254


def test_batch_pad(oracle, golden):
    got = oracle.batch_pad([np.ones((2, 3, 1), np.uint8), np.ones((3, 2, 1), np.uint8)], 7.0)[..., 0]
    assert got.tolist() == golden["batch_pad7"]


@pytest.mark.parametrize("name", ["c1", "c2", "c3", "c5"])
def test_small_pipelines(pkg, oracle, golden, name):
    wl = importlib.import_module("mlx_data_b200.workloads")
    cfg = wl.CONFIGS[name]
    samples = wl.make_samples(name, "small", n=8)
    ops = wl.config_ops(name, "small")
    oracle.set_state(0)
    cast = {"image": None if len(cfg["cast"]) == 0 else (np.array(cfg["cast"][0], np.float32),
                                                         np.array(cfg["cast"][1], np.float32))}
    got = [digest(b["image"]) for b in oracle.run_chain(samples, ops, 4, {"image": 0.0}, cast)]
    assert got == golden["pipeline_%s_small8" % name]["batches"]


def test_rotate_pipeline_fixed_angle(pkg, oracle, golden):
    wl = importlib.import_module("mlx_data_b200.workloads")
    samples = [{"image": s["image"]} for s in wl.make_samples("c4", "small", n=8)]
    ops = [("image_rotate", dict(key="image", angle=21.5, crop=True)),
           ("image_random_h_flip", dict(key="image", prob=0.5)),
           ("image_center_crop", dict(key="image", w=140, h=140))]
    oracle.set_state(0)
    got = [digest(b["image"]) for b in oracle.run_chain(samples, ops, 4, {"image": 0.0}, {"image": None})]
    assert got == golden["pipeline_c4_fixed_angle_small8"]["batches"]
