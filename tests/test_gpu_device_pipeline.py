"""The pipeline API with samples and batches resident in GPU memory, launched on
the caller's CUDA stream: results against the CPU oracle, the placement a
pipeline was built with staying with it, and recycled output blocks moving
between streams."""
import importlib

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

OPS = [("image_random_crop", dict(key="image", w=64, h=48)),
       ("image_random_h_flip", dict(key="image", prob=0.5))]


def _host_samples(n, seed):
    rng = np.random.default_rng(seed)
    return [{"image": rng.integers(0, 256, (int(rng.integers(60, 120)), int(rng.integers(70, 130)), 3), dtype=np.uint8)}
            for _ in range(n)]


def _pipeline(pkg, samples, batch):
    ds = pkg.buffer_from_vector(samples)
    for name, kw in OPS:
        ds = getattr(ds, name)(**kw)
    return ds.batch(batch).key_cast("image")


def _want(oracle, host, batch, seed):
    oracle.set_state(seed)
    return [b["image"] for b in oracle.run_chain(host, OPS, batch, {"image": 0.0}, {"image": None})]


@pytest.fixture
def restore_placement(pkg):
    yield
    pkg.core.set_stream(0, False)
    pkg.core.set_device_output(False)


def test_device_resident_pipeline_on_two_streams(pkg, oracle, restore_placement):
    torch = pytest.importorskip("torch")
    host = _host_samples(16, 1)
    dev = [{"image": torch.from_numpy(s["image"]).cuda()} for s in host]
    torch.cuda.synchronize()
    want = _want(oracle, host, 8, seed=3)
    pkg.core.set_device_output(True)
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    # the same pipeline three times: stream A, stream B, stream A again.  Each
    # round drops its batches, so the next one is handed the same pooled blocks -
    # from the other stream, which it has to wait for first.
    for rnd, st in enumerate((streams[0], streams[1], streams[0])):
        pkg.core.set_stream(st.cuda_stream, True)
        pkg.core.set_state(3)
        pipe = _pipeline(pkg, dev, 8)
        got = []
        with torch.cuda.stream(st):
            for i in range(len(pipe)):
                b = pipe[i]["image"]
                assert type(b).__name__ == "DeviceArray"
                got.append(torch.as_tensor(b, device="cuda").clone())     # consumer queued on the same stream
                del b
        assert pkg.core.stream_status(st.cuda_stream) == 0
        for g, w in zip(got, want):
            assert np.array_equal(g.cpu().numpy(), w), "round %d" % rnd
        del pipe, got
    # and a host-output batch on the lanes right after, which may take a block the streams used
    pkg.core.set_stream(0, False)
    pkg.core.set_device_output(False)
    pkg.core.set_state(3)
    host_pipe = _pipeline(pkg, host, 8)
    for i, w in enumerate(want):
        assert np.array_equal(np.asarray(host_pipe[i]["image"]), w)


def test_pipeline_keeps_the_placement_it_was_built_with(pkg, oracle, restore_placement):
    torch = pytest.importorskip("torch")
    host = _host_samples(8, 2)
    want = _want(oracle, host, 4, seed=9)
    pkg.core.set_device_output(True)
    built_with_device_output = _pipeline(pkg, host, 4)         # host samples in, batches left on the GPU
    pkg.core.set_device_output(False)
    built_with_host_output = _pipeline(pkg, host, 4)
    pkg.core.set_device_output(True)                            # flipping the default changes neither
    pkg.core.set_state(9)
    a = [built_with_device_output[i]["image"] for i in range(2)]
    pkg.core.set_state(9)
    b = [built_with_host_output[i]["image"] for i in range(2)]
    assert all(type(x).__name__ == "DeviceArray" for x in a)
    assert all(isinstance(x, np.ndarray) for x in b)
    for x, y, w in zip(a, b, want):
        assert np.array_equal(torch.as_tensor(x, device="cuda").cpu().numpy(), w)
        assert np.array_equal(y, w)
