"""pad, pad_to_size, pad_to_multiple against the reference (host-side array ops)."""
import numpy as np
import pytest

import refpipe


def _samples():
    rng = np.random.default_rng(3)
    out = []
    for i in range(9):
        out.append({
            "tokens": rng.integers(0, 100, (int(rng.integers(1, 30)),), dtype=np.int64),
            "feat": rng.normal(size=(int(rng.integers(1, 9)), 5)).astype(np.float32),
            "image": rng.integers(0, 256, (int(rng.integers(3, 9)), int(rng.integers(3, 9)), 3), dtype=np.uint8),
        })
    return out


CHAINS = [
    [("pad", dict(key="tokens", dim=0, lpad=2, rpad=3, pad_value=-1))],
    [("pad", dict(key="feat", dim=1, lpad=0, rpad=4, pad_value=0.5)),
     ("pad", dict(key="feat", dim=-2, lpad=1, rpad=0, pad_value=2.0, output_key="feat2"))],
    [("pad_to_multiple", dict(key="tokens", dim=0, pad_multiple=8, pad_value=7))],
    [("pad_to_size", dict(key="tokens", dim=0, size=16, pad_value=9))],
    [("pad", dict(key="image", dim=0, lpad=1, rpad=2, pad_value=200)),
     ("pad_to_multiple", dict(key="image", dim=1, pad_multiple=4, pad_value=17))],
    [("pad_if", dict(cond=False, key="tokens", dim=0, lpad=5, rpad=5, pad_value=1)),
     ("pad_to_multiple_if", dict(cond=True, key="tokens", dim=0, pad_multiple=5, pad_value=3)),
     ("pad_to_size_if", dict(cond=True, key="feat", dim=0, size=10, pad_value=-2.0))],
]


@pytest.mark.parametrize("case", range(len(CHAINS)))
def test_pad_ops_match_reference(pkg, case):
    ref = refpipe.reference_module()
    if ref is None:
        pytest.skip("needs the reference compiled under oracle/_ref")
    samples = _samples()

    def run(dx):
        ds = dx.buffer_from_vector(samples)
        for name, kw in CHAINS[case]:
            ds = getattr(ds, name)(**kw)
        return [dict(ds[i]) for i in range(len(ds))]

    want, got = run(ref), run(pkg)
    assert len(want) == len(got)
    for w, g in zip(want, got):
        assert sorted(w) == sorted(g)
        for k in w:
            a, b = np.asarray(g[k]), np.asarray(w[k])
            assert a.shape == b.shape and a.dtype == b.dtype and np.array_equal(a, b), k


def test_pad_rejects_negative(pkg):
    with pytest.raises(RuntimeError):
        pkg.buffer_from_vector(_samples()).pad("tokens", 0, -1, 0, 0)


def test_pad_to_size_with_a_list_of_sizes(pkg):
    """The nearest listed size above the current one; arrays at or beyond every
    listed size are left as they are (mlx/data/op/Pad.cpp:45-63).  Checked
    against numpy: the compiled reference crashes on a list argument here."""
    samples = [{"tokens": np.arange(n, dtype=np.int64)} for n in (1, 8, 9, 16, 23, 24, 30)]
    buf = pkg.buffer_from_vector(samples).pad_to_size("tokens", 0, [24, 8, 16], 5)
    for i, s in enumerate(samples):
        n = len(s["tokens"])
        larger = [x for x in (8, 16, 24) if x > n]
        want = np.concatenate([s["tokens"], np.full((min(larger) - n if larger else 0,), 5, np.int64)])
        assert np.array_equal(np.asarray(buf[i]["tokens"]), want)


SLICE_CHAINS = [
    [("slice", dict(ikey="tokens", dims=0, starts=2, ends=11))],
    [("slice", dict(ikey="feat", dims=[0, 1], starts=[0, 1], ends=[3, 4]))],
    [("slice", dict(ikey="image", dims=[1, -1], starts=[1, 0], ends=[100, 2], output_key="part"))],
    [("random_slice", dict(ikey="tokens", dims=0, sizes=4))],
    [("random_slice", dict(ikey="image", dims=[0, 1], sizes=[3, 2])),
     ("random_slice", dict(ikey="feat", dims=[1], sizes=[3]))],
]


@pytest.mark.parametrize("case", range(len(SLICE_CHAINS)))
def test_slice_ops_match_reference(pkg, case):
    ref = refpipe.reference_module()
    if ref is None:
        pytest.skip("needs the reference compiled under oracle/_ref")
    samples = _samples()

    def run(dx):
        dx.core.set_state(11)
        ds = dx.buffer_from_vector(samples)
        for name, kw in SLICE_CHAINS[case]:
            ds = getattr(ds, name)(**kw)
        return [dict(ds[i]) for i in range(len(ds))]

    want, got = run(ref), run(pkg)
    for w, g in zip(want, got):
        assert sorted(w) == sorted(g)
        for k in w:
            a, b = np.asarray(g[k]), np.asarray(w[k])
            assert a.shape == b.shape and a.dtype == b.dtype and np.array_equal(a, b), k


def test_conditional_twins_of_slice_and_sample_transform(pkg):
    b = pkg.buffer_from_vector([{"a": np.arange(10, dtype=np.int64)}])
    assert np.asarray(b.slice_if(True, "a", 0, 2, 5)[0]["a"]).tolist() == [2, 3, 4]
    assert np.asarray(b.slice_if(False, "a", 0, 2, 5)[0]["a"]).shape == (10,)
    assert np.asarray(b.random_slice_if(True, "a", 0, 3)[0]["a"]).shape == (3,)
    assert np.asarray(b.random_slice_if(False, "a", 0, 3)[0]["a"]).shape == (10,)
    assert np.asarray(b.sample_transform_if(True, lambda s: {"a": s["a"] * 2})[0]["a"])[:3].tolist() == [0, 2, 4]
    assert np.asarray(b.sample_transform_if(False, lambda s: {})[0]["a"])[:3].tolist() == [0, 1, 2]
