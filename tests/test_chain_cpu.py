"""CPU checks of the descriptor semantics: an op chain reduced to the canonical
descriptor and evaluated stage by stage must equal the chain applied op by op."""
import importlib

import numpy as np
import pytest

import chain


def _wl(pkg):
    return importlib.import_module("mlx_data_b200.workloads")


@pytest.mark.parametrize("name", ["c1", "c2", "c3", "c4"])
def test_reduced_chain_equals_op_by_op(pkg, oracle, name):
    wl = _wl(pkg)
    samples = wl.make_samples(name, "small", n=6)
    ops = wl.config_ops(name, "small")
    oracle.set_state(0)
    want = []
    for s in samples:
        for op in ops:
            s = oracle.apply_op(s, op)
        want.append(s["image"])
    oracle.set_state(0)
    for s, w in zip(samples, want):
        f = chain.reduce_chain(s["image"].shape, ops, s)
        assert np.array_equal(chain.interpret(f, s["image"]), w)


def test_flip_crop_compose(oracle):
    rng = np.random.default_rng(3)
    img = rng.integers(0, 256, (40, 50, 3), dtype=np.uint8)
    ops = [("image_random_h_flip", dict(key="image", prob=1.0)),
           ("image_center_crop", dict(key="image", w=31, h=20)),
           ("image_random_crop", dict(key="image", w=10, h=9)),
           ("image_resize", dict(key="image", w=20, h=7)),
           ("image_random_h_flip", dict(key="image", prob=1.0)),
           ("image_center_crop", dict(key="image", w=9, h=5)),
           ("image_channel_reduction", dict(key="image", preset="rec2020"))]
    oracle.set_state(5)
    s = {"image": img}
    for op in ops:
        s = oracle.apply_op(s, op)
    oracle.set_state(5)
    f = chain.reduce_chain(img.shape, ops)
    assert f["pre_flip"] == 1 and f["post_flip"] == 1 and f["gray"] is not None
    assert np.array_equal(chain.interpret(f, img), s["image"])


def test_second_geometric_op_is_not_fusable(oracle):
    ops = [("image_resize", dict(key="image", w=20, h=7)), ("image_rotate", dict(key="image", angle=3.0))]
    with pytest.raises(chain.Unfusable):
        chain.reduce_chain((30, 30, 3), ops)
