"""Failure reporting without a fault: a lane wait that runs out of time, and a
kernel whose bounded wait runs out (a test hook makes the first resize pass
expect bytes that no copy delivers).  In both cases the caller gets an error
code, nothing hangs, and the same context goes on to produce correct batches."""
import os

import numpy as np
import pytest

import chain

pytestmark = pytest.mark.gpu

OPS = [("image_resize", dict(key="image", w=48, h=40))]


def _descs(pkg, samples, ops):
    descs = np.zeros(len(samples), pkg.SAMPLE_DTYPE)
    fields = []
    for i, s in enumerate(samples):
        f = chain.reduce_chain(s["image"].shape, ops, s)
        fields.append(f)
        chain.fill_descs(descs, i, f, s["image"].ctypes.data)
    return descs, fields


def test_lane_wait_times_out_and_recovers(pkg, oracle):
    torch = pytest.importorskip("torch")
    capi = pkg._capi
    own = pkg.Context(device=0, n_lanes=1)
    try:
        rng = np.random.default_rng(0)
        # enough work that it cannot be done the moment it is queued
        samples = [{"image": rng.integers(0, 256, (1080, 1920, 3), dtype=np.uint8)} for _ in range(24)]
        ops = [("image_resize_smallest_side", dict(key="image", size=512))]
        descs, fields = _descs(pkg, samples, ops)
        h, w = fields[0]["out_hw"]
        # page-locked destination: the copy back is asynchronous, the call returns with work in flight
        out = torch.zeros((len(samples), h, w, 3), dtype=torch.float32).pin_memory().numpy()
        bd = pkg.make_batch_desc(out, h, w, 3)
        own.fused_batch(0, descs, bd)
        with pytest.raises(pkg.MlxdError) as e:
            own.wait(0, timeout_ms=0)
        assert e.value.code == capi.ERR_TIMEOUT
        own.wait(0)                                   # the work was still queued; now it is done
        want = oracle.resize(samples[0]["image"], w, h).astype("float32") / 255
        d = np.abs(out[0].astype(np.float64) - want.astype(np.float64))
        assert d.max() <= 1.0001 / 255
    finally:
        own.close()


def test_bounded_wait_runs_out_is_reported_and_cleared(pkg, oracle):
    capi = pkg._capi
    own = pkg.Context(device=0, n_lanes=1)
    rng = np.random.default_rng(1)
    samples = [{"image": rng.integers(0, 256, (60, 90, 3), dtype=np.uint8)}]     # one band, one pass
    descs, fields = _descs(pkg, samples, OPS)
    out = np.zeros((1, 40, 48, 3), np.float32)
    bd = pkg.make_batch_desc(out, 40, 48, 3)
    try:
        os.environ["MLXD_TEST_STARVE_WAIT"] = "1"
        try:
            own.fused_batch(0, descs, bd)
        finally:
            os.environ.pop("MLXD_TEST_STARVE_WAIT", None)
        with pytest.raises(pkg.MlxdError) as e:
            own.wait(0)
        assert e.value.code == capi.ERR_DEVICE and "self-check" in str(e.value)
        # reported once, then cleared: the same lane produces a correct batch
        out[...] = -1
        own.fused_batch(0, descs, bd)
        own.wait(0)
        want = oracle.resize(samples[0]["image"], 48, 40).astype("float32") / 255
        d = np.abs(out[0].astype(np.float64) - want.astype(np.float64))
        assert d.max() <= 1.0001 / 255 and (d > 0).mean() <= 1e-3
    finally:
        own.close()
