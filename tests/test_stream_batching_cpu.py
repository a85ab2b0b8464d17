"""Stream.dynamic_batch, Stream.repeat, Buffer.shuffle and
stream_python_iterable on samples that need no GPU: against the reference
compiled under oracle/_ref where the result is deterministic, by properties
otherwise."""
import numpy as np
import pytest

import refpipe


def _samples(seed, n, lo=1, hi=60):
    rng = np.random.default_rng(seed)
    return [{"tokens": rng.integers(0, 1000, (int(rng.integers(lo, hi)),), dtype=np.int64), "id": np.int64(i)}
            for i in range(n)]


def _same_batches(got, want):
    assert len(got) == len(want)
    for i, (g, w) in enumerate(zip(got, want)):
        assert sorted(g) == sorted(w)
        for k in w:
            a, b = np.asarray(g[k]), np.asarray(w[k])
            assert a.shape == b.shape and a.dtype == b.dtype and np.array_equal(a, b), (i, k)


CASES = [
    dict(buffer_size=200, max_data_size=256),                              # one round holds everything
    dict(buffer_size=23, max_data_size=256),                               # many rounds, last one short
    dict(buffer_size=23, min_data_size=100, max_data_size=120),            # rounds leave samples out, carried over
    dict(buffer_size=16, min_data_size=100, max_data_size=120, max_skipped_samples=3),
    dict(buffer_size=16, min_data_size=100, max_data_size=120, max_skipped_samples=-1),
    dict(buffer_size=10, max_data_size=40, drop_outliers=True),
    dict(buffer_size=10, max_data_size=40),
    dict(buffer_size=12, min_data_size=30),
    dict(buffer_size=12),
    dict(buffer_size=19, max_data_size=300, dim={"tokens": 0}, pad={"tokens": 7}),
    dict(buffer_size=19, min_data_size=50, max_data_size=200, pad={"tokens": -1}),
]


@pytest.mark.parametrize("case", range(len(CASES)))
def test_stream_dynamic_batch_matches_reference(pkg, case):
    ref = refpipe.reference_module()
    if ref is None:
        pytest.skip("needs the reference compiled under oracle/_ref")
    kw = dict(CASES[case])
    size = kw.pop("buffer_size")
    samples = _samples(70 + case, 97)
    want = [dict(b) for b in ref.buffer_from_vector(samples).to_stream().dynamic_batch(size, "tokens", **kw)]
    got = [dict(b) for b in pkg.buffer_from_vector(samples).to_stream().dynamic_batch(size, "tokens", **kw)]
    assert len(want) > 0
    _same_batches(got, want)


def test_stream_dynamic_batch_after_reset_and_with_threads(pkg):
    samples = _samples(3, 64)
    ds = pkg.buffer_from_vector(samples).to_stream().dynamic_batch(16, "tokens", max_data_size=128, num_threads=4)
    first = [dict(b) for b in ds]
    assert next(iter(ds), None) is None       # stays exhausted
    ds.reset()
    again = [dict(b) for b in ds]
    # several pulling threads may reorder samples between rounds; every sample still shows up once per pass
    for run in (first, again):
        ids = np.concatenate([np.asarray(b["id"]).reshape(-1) for b in run])
        assert sorted(ids.tolist()) == list(range(64))
        for b in run:
            t = np.asarray(b["tokens"])
            assert t.size <= 128 or t.shape[0] == 1


def test_stream_dynamic_batch_shuffle_is_a_permutation_of_the_batches(pkg):
    samples = _samples(11, 80)
    plain = [dict(b) for b in pkg.buffer_from_vector(samples).to_stream().dynamic_batch(
        200, "tokens", max_data_size=256)]
    pkg.core.set_state(5)
    mixed = [dict(b) for b in pkg.buffer_from_vector(samples).to_stream().dynamic_batch(
        200, "tokens", max_data_size=256, shuffle=True)]
    key = lambda b: tuple(np.asarray(b["id"]).reshape(-1).tolist())
    assert sorted(map(key, plain)) == sorted(map(key, mixed))
    assert list(map(key, plain)) != list(map(key, mixed))


def test_stream_dynamic_batch_rejects_bad_arguments(pkg):
    s = pkg.buffer_from_vector(_samples(0, 4)).to_stream()
    with pytest.raises(RuntimeError):
        s.dynamic_batch(0, "tokens")
    with pytest.raises(Exception):
        next(s.dynamic_batch(4, "no such key", max_data_size=10))


@pytest.mark.parametrize("times", [0, 1, 3])
def test_repeat_counts_passes(pkg, times):
    ref = refpipe.reference_module()
    samples = [{"x": np.int64(i)} for i in range(5)]
    got = [int(s["x"]) for s in pkg.buffer_from_vector(samples).to_stream().repeat(times)] if times else None
    if times:
        assert got == list(range(5)) * (times + 1)
        if ref is not None:
            assert got == [int(s["x"]) for s in ref.buffer_from_vector(samples).to_stream().repeat(times)]
    else:
        # no limit: the stream never ends
        ds = pkg.buffer_from_vector(samples).to_stream().repeat(times)
        assert [int(next(ds)["x"]) for _ in range(23)] == [i % 5 for i in range(23)]


def test_repeat_reset_restores_the_passes(pkg):
    samples = [{"x": np.int64(i)} for i in range(3)]
    ds = pkg.buffer_from_vector(samples).to_stream().repeat(1)
    assert len(list(ds)) == 6
    assert len(list(ds)) == 0
    ds.reset()
    assert len(list(ds)) == 6


def test_buffer_shuffle_matches_reference_draw(pkg):
    ref = refpipe.reference_module()
    samples = [{"x": np.int64(i)} for i in range(50)]
    pkg.core.set_state(21)
    got = [int(s["x"]) for s in pkg.buffer_from_vector(samples).shuffle()]
    assert sorted(got) == list(range(50)) and got != list(range(50))
    assert [int(s["x"]) for s in pkg.buffer_from_vector(samples).shuffle_if(False)] == list(range(50))
    if ref is not None:
        ref.core.set_state(21)
        assert got == [int(s["x"]) for s in ref.buffer_from_vector(samples).shuffle()]


def test_stream_python_iterable(pkg):
    made = []

    def factory():
        made.append(1)
        return ({"x": np.array([i, i + 1], dtype=np.int32)} for i in range(4))

    ds = pkg.stream_python_iterable(factory)
    assert [np.asarray(s["x"]).tolist() for s in ds] == [[i, i + 1] for i in range(4)]
    assert next(ds, None) is None and len(made) == 1
    ds.reset()
    assert np.asarray(next(ds)["x"]).tolist() == [0, 1] and len(made) == 2
    # composes with the rest of the pipeline
    ds = pkg.stream_python_iterable(lambda: ({"x": np.full((i + 1,), i, dtype=np.int64)} for i in range(6)))
    batches = [np.asarray(b["x"]) for b in ds.batch(4, pad={"x": -1})]
    assert [b.shape for b in batches] == [(4, 4), (2, 6)]
    assert batches[0][0].tolist() == [0, -1, -1, -1]
    with pytest.raises(Exception):
        next(pkg.stream_python_iterable(lambda: iter([3])))


def test_buffer_perm(pkg):
    ref = refpipe.reference_module()
    samples = [{"x": np.int64(i)} for i in range(6)]
    order = [5, 0, 0, 3]
    got = [int(s["x"]) for s in pkg.buffer_from_vector(samples).perm(order)]
    assert got == order
    if ref is not None:
        assert got == [int(s["x"]) for s in ref.buffer_from_vector(samples).perm(order)]
    with pytest.raises(RuntimeError):
        pkg.buffer_from_vector(samples).perm([6])
