"""Buffer.dynamic_batch against the reference on samples that need no GPU
(1-D and 2-D arrays of ragged sizes): same batches, same order, same padding."""
import numpy as np
import pytest

import refpipe


def _samples(seed, n, two_d=False):
    rng = np.random.default_rng(seed)
    out = []
    for i in range(n):
        length = int(rng.integers(1, 60))
        if two_d:
            arr = rng.integers(0, 1000, (length, int(rng.integers(1, 5))), dtype=np.int64)
        else:
            arr = rng.integers(0, 1000, (length,), dtype=np.int64)
        out.append({"tokens": arr, "id": np.int64(i)})
    return out


CASES = [
    dict(max_data_size=256),
    dict(min_data_size=64, max_data_size=256),
    dict(min_data_size=100, max_data_size=120),
    dict(max_data_size=40),
    dict(max_data_size=40, drop_outliers=True),
    dict(min_data_size=30),
    dict(),
    dict(max_data_size=300, dim={"tokens": 0}, pad={"tokens": 7}),
    dict(min_data_size=50, max_data_size=200, pad={"tokens": -1}),
]


@pytest.mark.parametrize("case", range(len(CASES)))
@pytest.mark.parametrize("two_d", [False, True])
def test_dynamic_batch_matches_reference(pkg, case, two_d):
    ref = refpipe.reference_module()
    if ref is None:
        pytest.skip("needs the reference compiled under oracle/_ref")
    kw = CASES[case]
    if two_d and "dim" in kw:
        kw = dict(kw, dim={"tokens": 0})
    samples = _samples(40 + case, 57, two_d)
    want = ref.buffer_from_vector(samples).dynamic_batch("tokens", **kw)
    got = pkg.buffer_from_vector(samples).dynamic_batch("tokens", **kw)
    assert len(got) == len(want)
    for i in range(len(want)):
        w, g = dict(want[i]), dict(got[i])
        assert sorted(w) == sorted(g)
        for k in w:
            a, b = np.asarray(g[k]), np.asarray(w[k])
            assert a.shape == b.shape and a.dtype == b.dtype and np.array_equal(a, b), (i, k)


def test_dynamic_batch_with_size_buffer(pkg):
    ref = refpipe.reference_module()
    if ref is None:
        pytest.skip("needs the reference compiled under oracle/_ref")
    samples = _samples(5, 31)
    # sizes that disagree with the arrays on purpose: they alone drive the grouping
    sizes = [{"tokens": np.array([60 - len(s["tokens"])], dtype=np.int64)} for s in samples]
    want = ref.buffer_from_vector(samples).dynamic_batch(
        "tokens", size_buffer=ref.buffer_from_vector(sizes), max_data_size=128)
    got = pkg.buffer_from_vector(samples).dynamic_batch(
        "tokens", size_buffer=pkg.buffer_from_vector(sizes), max_data_size=128)
    assert len(got) == len(want)
    for i in range(len(want)):
        assert np.array_equal(np.asarray(got[i]["id"]), np.asarray(want[i]["id"]))
        assert np.array_equal(np.asarray(got[i]["tokens"]), np.asarray(want[i]["tokens"]))


def test_dynamic_batch_sizes_images_without_a_gpu(pkg):
    """Image ops under a buffer dynamic_batch are sized from their recorded
    programs: building the batches needs no pixels (and so no GPU); the number
    of batches equals the reference's, which computes every image to size it."""
    ref = refpipe.reference_module()
    if ref is None:
        pytest.skip("needs the reference compiled under oracle/_ref")
    rng = np.random.default_rng(12)
    samples = [{"image": rng.integers(0, 256, (int(rng.integers(20, 140)), int(rng.integers(20, 140)), 3), dtype=np.uint8)}
               for _ in range(41)]

    def chain(dx):
        return (dx.buffer_from_vector(samples)
                .image_resize_smallest_side("image", 32)
                .slice("image", 1, 0, 50)
                .pad_to_multiple("image", 0, 8, 0)
                .dynamic_batch("image", max_data_size=5 * 32 * 64 * 3))

    assert len(chain(pkg)) == len(chain(ref)) > 3
