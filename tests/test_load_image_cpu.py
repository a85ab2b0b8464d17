"""load_image: header handling that needs no GPU (image info, refusals).  The
pixel path, which lands in page-locked memory, is in the GPU suite."""
import numpy as np
import pytest


def _ppm(path, arr, comment=False):
    h, w = arr.shape[:2]
    magic = b"P6" if arr.ndim == 3 else b"P5"
    head = magic + b"\n" + (b"# made by a test\n" if comment else b"") + b"%d %d\n255\n" % (w, h)
    path.write_bytes(head + arr.tobytes())


def test_info_from_file_and_memory(pkg, tmp_path):
    rng = np.random.default_rng(0)
    colour = rng.integers(0, 256, (7, 11, 3), dtype=np.uint8)
    grey = rng.integers(0, 256, (5, 3), dtype=np.uint8)
    _ppm(tmp_path / "a.ppm", colour, comment=True)
    _ppm(tmp_path / "b.pgm", grey)
    buf = pkg.buffer_from_vector([{"file": b"a.ppm"}, {"file": b"b.pgm"}])
    got = buf.load_image("file", prefix=str(tmp_path), info=True, output_key="size")
    assert np.asarray(got[0]["size"]).tolist() == [11, 7]
    assert np.asarray(got[1]["size"]).tolist() == [3, 5]
    assert bytes(np.asarray(got[0]["file"]).tobytes()) == b"a.ppm"          # the name stays under its key
    raw = np.frombuffer((tmp_path / "a.ppm").read_bytes(), dtype=np.uint8)
    mem = pkg.buffer_from_vector([{"file": raw}]).load_image("file", info=True, from_memory=True)
    assert np.asarray(mem[0]["file"]).tolist() == [11, 7]
    # the conditional twin leaves the sample alone
    same = buf.load_image_if(False, "file", prefix=str(tmp_path), info=True)
    assert bytes(np.asarray(same[0]["file"]).tobytes()) == b"a.ppm"


def test_refusals(pkg, tmp_path):
    (tmp_path / "x.gif").write_bytes(b"GIF89a" + bytes(64))
    (tmp_path / "ascii.ppm").write_bytes(b"P3\n1 1\n255\n1 2 3\n")
    (tmp_path / "deep.ppm").write_bytes(b"P6\n1 1\n65535\n" + bytes(6))
    (tmp_path / "x.png").write_bytes(b"\x89PNG\r\n\x1a\n" + bytes(64))
    with pytest.raises(RuntimeError, match="IHDR"):
        pkg.buffer_from_vector([{"file": b"x.png"}]).load_image("file", prefix=str(tmp_path), info=True)[0]
    for name in ("x.gif", "ascii.ppm", "deep.ppm"):
        with pytest.raises(RuntimeError, match="binary PNM"):
            pkg.buffer_from_vector([{"file": name.encode()}]).load_image("file", prefix=str(tmp_path), info=True)[0]
    with pytest.raises(RuntimeError, match="unable to load image"):
        pkg.buffer_from_vector([{"file": b"missing.ppm"}]).load_image("file", prefix=str(tmp_path))[0]
    with pytest.raises(RuntimeError, match="int8"):
        pkg.buffer_from_vector([{"file": np.arange(4, dtype=np.int64)}]).load_image("file")[0]
