"""load_image feeding the fused path: binary PNM, PNG and JPEG files (and in-memory
copies) are read or decoded into page-locked memory, then resized, cropped, batched and cast in
one launch per batch; the result must equal the oracle's on the pixel arrays
the files were written from."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

OPS = [("image_resize_smallest_side", dict(key="image", size=40)),
       ("image_center_crop", dict(key="image", w=36, h=32)),
       ("image_random_h_flip", dict(key="image", prob=0.5))]


def _write(path, arr, fmt="pnm"):
    h, w = arr.shape[:2]
    if fmt == "jpg":
        import io
        from PIL import Image
        b = io.BytesIO()
        Image.fromarray(arr if arr.shape[2] == 3 else arr[..., 0]).save(b, format="JPEG", quality=85, subsampling=h % 3)
        path.write_bytes(b.getvalue())
        # what a libjpeg-turbo decoder makes of the file (three channels, also for a grey file)
        return np.asarray(Image.open(io.BytesIO(b.getvalue())).convert("RGB"))
    if fmt == "png":
        from test_png_cpu import write_png
        path.write_bytes(write_png(arr.astype(np.int64), 8, 2 if arr.shape[2] == 3 else 0, interlace=bool(h % 2)))
        return arr
    magic = b"P6" if arr.shape[2] == 3 else b"P5"
    path.write_bytes(magic + b"\n# c\n%d %d\n255\n" % (w, h) + arr.tobytes())
    return arr


@pytest.mark.parametrize("channels", [3, 1])
@pytest.mark.parametrize("from_memory", [False, True])
@pytest.mark.parametrize("fmt", ["pnm", "png", "jpg"])
def test_load_then_fused_chain(pkg, oracle, tmp_path, channels, from_memory, fmt):
    rng = np.random.default_rng(5 + channels)
    arrays = [rng.integers(0, 256, (int(rng.integers(50, 90)), int(rng.integers(50, 90)), channels), dtype=np.uint8)
              for _ in range(6)]
    samples = []
    for i, a in enumerate(arrays):
        name = "im%d.%s" % (i, fmt if fmt != "pnm" else ("ppm" if channels == 3 else "pgm"))
        arrays[i] = _write(tmp_path / name, a, fmt)   # the pixels the file holds
        if from_memory:
            samples.append({"image": np.frombuffer((tmp_path / name).read_bytes(), dtype=np.uint8)})
        else:
            samples.append({"image": name.encode()})
    pkg.core.set_state(11)
    ds = pkg.buffer_from_vector(samples).to_stream().load_image("image", prefix=str(tmp_path), from_memory=from_memory)
    loaded = [np.asarray(s["image"]) for s in ds]
    for got, want in zip(loaded, arrays):
        assert got.dtype == np.uint8 and got.shape == want.shape and np.array_equal(got, want)
    ds = pkg.buffer_from_vector(samples).to_stream().load_image("image", prefix=str(tmp_path), from_memory=from_memory)
    for name, kw in OPS:
        ds = getattr(ds, name)(**kw)
    before = pkg.core.stats()["kernel_launches"]
    pkg.core.set_state(11)
    got = [np.asarray(b["image"]) for b in ds.batch(3).key_cast("image")]
    launches = pkg.core.stats()["kernel_launches"] - before
    oracle.set_state(11)
    want = [b["image"] for b in oracle.run_chain([{"image": a} for a in arrays], OPS, 3, {"image": 0.0}, {"image": None})]
    assert len(got) == len(want) == 2
    for g, w in zip(got, want):
        assert g.shape == w.shape and g.dtype == np.float32
        d = np.abs(g.astype(np.float64) - w.astype(np.float64))
        assert d.max() <= 1.0001 / 255 and (d > 0).mean() <= 1e-3
    # page-locked sources: one gather launch and one fused launch per batch
    assert launches == 2 * len(want)
