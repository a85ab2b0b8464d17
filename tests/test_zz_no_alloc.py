"""The allocation-free entry point, mlxd_fused_batch_noalloc.

It exists for callers that cannot allocate in the data path (a loader running
inside a training step that owns the GPU's memory pool, a service that bans
allocator calls once warm): its descriptor and cast tables live in a fixed
array inside the library instead of memory allocated per call.  Its output
must equal, bit for bit, what the allocating entry point
mlxd_fused_batch_on_stream writes for the same descriptors - also on a second
call, which finds the previous call's contents in the shared array.  The
calls must leave the device's free memory as they found it and the kernel's
self-check word clean.
"""
import importlib

import numpy as np
import pytest

import chain

pytestmark = pytest.mark.gpu


def _descs(pkg, oracle, samples, ops, dev_ptrs, seed):
    oracle.set_state(seed)
    descs = np.zeros(len(samples), pkg.SAMPLE_DTYPE)
    fields = []
    for i, s in enumerate(samples):
        f = chain.reduce_chain(s["image"].shape, ops, s)
        fields.append(f)
        chain.fill_descs(descs, i, f, dev_ptrs[i])
    return descs, fields


@pytest.mark.parametrize("name", ["c2", "c4"])
def test_noalloc_matches_allocating_entry_point_twice(pkg, ctx, oracle, name):
    torch = pytest.importorskip("torch")
    capi = pkg._capi
    wl = importlib.import_module("mlx_data_b200.workloads")
    cfg = wl.CONFIGS[name]
    ops = wl.config_ops(name, "small")
    stream = torch.cuda.current_stream().cuda_stream
    for call, seed in enumerate((5, 6)):          # two calls in a row, different random parameters
        samples = wl.make_samples(name, "small", n=12)[call * 2:call * 2 + 8]
        dev = [torch.from_numpy(s["image"]).cuda() for s in samples]
        descs, fields = _descs(pkg, oracle, samples, ops, [d.data_ptr() for d in dev], seed)
        sh = max(f["out_hw"][0] for f in fields)
        sw = max(f["out_hw"][1] for f in fields)
        n = len(samples)
        cast = cfg["cast"]
        mean, std = (cast if len(cast) == 2 else (None, None))
        want = torch.full((n, sh, sw, 3), -7.0, dtype=torch.float32, device="cuda")
        got = torch.full((n, sh, sw, 3), -9.0, dtype=torch.float32, device="cuda")
        bd = pkg.make_batch_desc(want.data_ptr(), sh, sw, 3, mean=mean, std=std, pad_value=3.0,
                                 src_mem=capi.MEM_DEVICE, dst_mem=capi.MEM_DEVICE)
        ctx.fused_batch_on_stream(stream, descs, bd)
        bd2 = pkg.make_batch_desc(got.data_ptr(), sh, sw, 3, mean=mean, std=std, pad_value=3.0,
                                  src_mem=capi.MEM_DEVICE, dst_mem=capi.MEM_DEVICE)
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        capi.fused_batch_noalloc(0, stream, descs, bd2)
        torch.cuda.synchronize()
        if call == 1:   # the first call may still load the kernel's code; the second finds everything in place
            assert torch.cuda.mem_get_info()[0] == free_before, "the call changed the device's free memory"
        assert capi.noalloc_status(0, stream) == 0
        assert torch.equal(got, want), "call %d differs" % call
        assert float(want.min()) > -7.0  # every element was written


def test_noalloc_uint8_output_and_limits(pkg, ctx):
    torch = pytest.importorskip("torch")
    capi = pkg._capi
    stream = torch.cuda.current_stream().cuda_stream
    img = torch.randint(0, 256, (40, 50, 3), dtype=torch.uint8, device="cuda")
    descs = np.zeros(1, pkg.SAMPLE_DTYPE)
    f = chain.reduce_chain((40, 50, 3), [("image_center_crop", dict(key="image", w=30, h=20))])
    chain.fill_descs(descs, 0, f, img.data_ptr())
    out = torch.zeros((1, 24, 32, 3), dtype=torch.uint8, device="cuda")
    bd = pkg.make_batch_desc(out.data_ptr(), 24, 32, 3, out_dtype=capi.U8, divisor=1.0, pad_value=9.0,
                             src_mem=capi.MEM_DEVICE, dst_mem=capi.MEM_DEVICE)
    capi.fused_batch_noalloc(0, stream, descs, bd)
    torch.cuda.synchronize()
    ref = torch.full((24, 32, 3), 9, dtype=torch.uint8, device="cuda")
    ref[:20, :30] = img[10:30, 10:40]
    assert torch.equal(out[0], ref)
    # more samples than the fixed array holds: refused, nothing runs
    too_many = np.zeros(capi.NOALLOC_MAX_SAMPLES + 1, pkg.SAMPLE_DTYPE)
    with pytest.raises(pkg.MlxdError) as e:
        capi.fused_batch_noalloc(0, stream, too_many, bd)
    assert e.value.code == capi.ERR_INVALID and "at most" in str(e.value)
    # host memory is refused: this entry point copies no pixels
    host = pkg.make_batch_desc(np.zeros((1, 24, 32, 3), np.uint8), 24, 32, 3, out_dtype=capi.U8, divisor=1.0)
    with pytest.raises(pkg.MlxdError):
        capi.fused_batch_noalloc(0, stream, descs, host)
