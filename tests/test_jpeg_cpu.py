"""The JPEG decoder (baseline and progressive) behind load_image, on the CPU, against Pillow's
decoder - libjpeg-turbo at its defaults, which is what the reference calls
(mlx/data/core/image/ImageJPEG.cpp:99-146): accurate integer IDCT, triangle
chroma upsampling, fixed-point YCbCr -> RGB, grey copied to three channels.
Every pixel must be the same integer."""
import io

import numpy as np
import pytest

Image = pytest.importorskip("PIL.Image")
from PIL import ImageFile  # noqa: E402

ImageFile.MAXBLOCK = 1 << 22   # Pillow's encoder wants the whole progressive file in one buffer


def _enc(img, **kw):
    b = io.BytesIO()
    img.save(b, format="JPEG", **kw)
    return b.getvalue()


def _pillow(file):
    return np.asarray(Image.open(io.BytesIO(file)).convert("RGB"))


def _picture(rng, h, w, c, noise):
    """Blocks of colour with noise on top: energy in every DCT band."""
    a = rng.integers(0, 256, (h // 4 + 2, w // 4 + 2, c)).astype(np.float64)
    a = np.kron(a, np.ones((4, 4, 1)))[:h, :w] + rng.normal(0, noise, (h, w, c))
    a = np.clip(a, 0, 255).astype(np.uint8)
    return a if c == 3 else a[..., 0]


SIZES = [(1, 1), (2, 3), (7, 9), (8, 8), (16, 16), (17, 33), (33, 17), (64, 48), (101, 77), (240, 321)]


@pytest.mark.parametrize("subsampling", [0, 1, 2])
@pytest.mark.parametrize("quality", [10, 50, 90, 100])
@pytest.mark.parametrize("progressive", [False, True])
def test_colour_files(pkg, subsampling, quality, progressive):
    rng = np.random.default_rng(subsampling * 10 + quality)
    for h, w in SIZES:
        for noise in (4, 60):
            file = _enc(Image.fromarray(_picture(rng, h, w, 3, noise), "RGB"), quality=quality, subsampling=subsampling,
                        progressive=progressive, optimize=progressive and noise == 60)
            assert (b"\xff\xc2" in file) == progressive
            got = pkg.core.jpeg_decode(file)
            want = _pillow(file)
            assert got.shape == want.shape == (h, w, 3)
            assert np.array_equal(got, want), (h, w, noise, int(np.abs(got.astype(int) - want.astype(int)).max()))


def test_grey_files_come_back_with_three_channels(pkg):
    rng = np.random.default_rng(3)
    for i, (h, w) in enumerate(SIZES):
        file = _enc(Image.fromarray(_picture(rng, h, w, 1, 30), "L"), quality=80, progressive=bool(i % 2))
        got = pkg.core.jpeg_decode(file)
        assert got.shape == (h, w, 3)
        assert np.array_equal(got, _pillow(file))
        assert np.array_equal(got[..., 0], got[..., 1]) and np.array_equal(got[..., 0], got[..., 2])


def test_optimised_tables_and_restart_markers(pkg):
    rng = np.random.default_rng(4)
    a = Image.fromarray(_picture(rng, 150, 203, 3, 25), "RGB")
    for kw in (dict(optimize=True), dict(restart_marker_blocks=3), dict(restart_marker_rows=1, subsampling=0),
               dict(optimize=True, restart_marker_blocks=1, subsampling=1),
               dict(progressive=True, restart_marker_blocks=2), dict(progressive=True, restart_marker_rows=1, subsampling=1)):
        file = _enc(a, quality=70, **kw)
        assert np.array_equal(pkg.core.jpeg_decode(file), _pillow(file)), kw
    # the restart markers are really there
    assert b"\xff\xd0" in _enc(a, quality=70, restart_marker_blocks=3)


def test_four_component_files_keep_their_first_three_channels(pkg):
    """libjpeg hands such a file out as CMYK and the reference keeps channels
    0-2 of that.  Pillow shows CMYK files inverted (the Adobe convention), so
    libjpeg's own samples are 255 minus Pillow's."""
    rng = np.random.default_rng(9)
    for h, w in SIZES:
        for kw in (dict(), dict(subsampling=2, progressive=True), dict(quality=30, subsampling=1)):
            a = np.stack([_picture(rng, h, w, 1, 15) for _ in range(4)], axis=-1)
            file = _enc(Image.fromarray(a, "CMYK"), **kw)
            im = Image.open(io.BytesIO(file))
            assert im.mode == "CMYK"
            got = pkg.core.jpeg_decode(file)
            assert np.array_equal(got, 255 - np.asarray(im)[..., :3]), (h, w, kw)


def test_what_is_not_read_is_refused_by_name(pkg):
    rng = np.random.default_rng(6)
    a = Image.fromarray(_picture(rng, 40, 40, 3, 10), "RGB")
    good = _enc(a)
    with pytest.raises(RuntimeError, match="JPEG"):
        pkg.core.jpeg_decode(b"\x00" + good)
    with pytest.raises(RuntimeError, match="no image data|cut short|runs past"):
        pkg.core.jpeg_decode(good[: good.index(b"\xff\xda")])


def test_load_image_reports_jpeg_sizes(pkg, tmp_path):
    rng = np.random.default_rng(8)
    file = _enc(Image.fromarray(_picture(rng, 31, 45, 3, 10), "RGB"))
    (tmp_path / "a.jpg").write_bytes(file)
    got = pkg.buffer_from_vector([{"file": b"a.jpg"}]).load_image("file", prefix=str(tmp_path), info=True)
    assert np.asarray(got[0]["file"]).tolist() == [45, 31]
    mem = pkg.buffer_from_vector([{"file": np.frombuffer(file, dtype=np.uint8)}]).load_image(
        "file", info=True, from_memory=True)
    assert np.asarray(mem[0]["file"]).tolist() == [45, 31]
