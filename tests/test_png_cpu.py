"""The PNG decoder behind load_image, on the CPU: files written by Pillow (its
own filter choices and palette handling) and files written here chunk by chunk
(every filter type, Adam7 interlacing, 1/2/4/16-bit samples, split IDAT
chunks), against the pixels the format defines and the channel policy of the
reference's loader: grey 1, grey+alpha 2, everything else 3 channels, alpha
dropped, 16-bit samples reduced to their high byte, low-depth grey scaled to
0..255 (mlx/data/core/image/ImageSTBI.cpp:14-58 and stb_image's documented
conversions; stb itself is not available, so the last two are unpinned)."""
import io
import struct
import zlib

import numpy as np
import pytest


# ---------------------------------------------------------------- a small PNG writer
def _chunk(kind, body):
    return struct.pack(">I", len(body)) + kind + body + struct.pack(">I", zlib.crc32(kind + body))


def _paeth(a, b, c):
    p = a + b - c
    pa, pb, pc = abs(p - a), abs(p - b), abs(p - c)
    return a if pa <= pb and pa <= pc else (b if pb <= pc else c)


def _filter_rows(rows, unit, kinds):
    """rows: list of bytes (unfiltered scanlines) -> filtered stream with filter bytes."""
    out = bytearray()
    prev = bytes(len(rows[0])) if rows else b""
    for y, cur in enumerate(rows):
        kind = kinds[y % len(kinds)]
        line = bytearray(len(cur))
        for i, v in enumerate(cur):
            left = cur[i - unit] if i >= unit else 0
            up = prev[i]
            corner = prev[i - unit] if i >= unit else 0
            pred = [0, left, up, (left + up) >> 1, _paeth(left, up, corner)][kind]
            line[i] = (v - pred) & 0xFF
        out.append(kind)
        out += line
        prev = cur
    return bytes(out)


def _pack(samples, depth):
    """samples [W * spp] of one scanline -> bytes."""
    if depth == 8:
        return bytes(int(v) for v in samples)
    if depth == 16:
        return b"".join(struct.pack(">H", int(v)) for v in samples)
    bits = 0
    n = 0
    out = bytearray()
    for v in samples:
        bits = (bits << depth) | int(v)
        n += depth
        if n == 8:
            out.append(bits)
            bits = n = 0
    if n:
        out.append(bits << (8 - n))
    return bytes(out)


ADAM7 = [(0, 0, 8, 8), (4, 0, 8, 8), (0, 4, 4, 8), (2, 0, 4, 4), (0, 2, 2, 4), (1, 0, 2, 2), (0, 1, 1, 2)]


def write_png(samples, depth, color, interlace=False, kinds=(0, 1, 2, 3, 4), palette=None, trns=None, pieces=3):
    """samples: [H, W, spp] integers in the file's own range."""
    h, w, spp = samples.shape
    unit = max(1, spp * depth // 8)
    stream = b""
    if not interlace:
        stream = _filter_rows([_pack(samples[y].reshape(-1), depth) for y in range(h)], unit, kinds)
    else:
        for x0, y0, dx, dy in ADAM7:
            sub = samples[y0::dy, x0::dx]
            if sub.shape[0] and sub.shape[1]:
                stream += _filter_rows([_pack(r.reshape(-1), depth) for r in sub], unit, kinds)
    z = zlib.compress(stream, 6)
    cut = [len(z) * i // pieces for i in range(pieces + 1)]
    body = _chunk(b"IHDR", struct.pack(">IIBBBBB", w, h, depth, color, 0, 0, 1 if interlace else 0))
    body += _chunk(b"gAMA", struct.pack(">I", 45455))          # ancillary chunks are skipped
    if palette is not None:
        body += _chunk(b"PLTE", bytes(int(v) for v in np.asarray(palette).reshape(-1)))
    if trns is not None:
        body += _chunk(b"tRNS", bytes(trns))
    for a, b in zip(cut[:-1], cut[1:]):
        body += _chunk(b"IDAT", z[a:b])
    return b"\x89PNG\r\n\x1a\n" + body + _chunk(b"IEND", b"")


def expected(samples, depth, color, palette=None):
    s = np.asarray(samples).astype(np.int64)
    if color == 3:
        return np.asarray(palette, dtype=np.uint8)[s[..., 0]]
    if depth == 16:
        s = s >> 8
    elif depth < 8:
        s = s * {1: 255, 2: 85, 4: 17}[depth]
    return s[..., :3 if color in (2, 6) else (2 if color == 4 else 1)].astype(np.uint8)


SPP = {0: 1, 2: 3, 3: 1, 4: 2, 6: 4}
CASES = [(c, d) for c, ds in {0: (1, 2, 4, 8, 16), 2: (8, 16), 3: (1, 2, 4, 8), 4: (8, 16), 6: (8, 16)}.items() for d in ds]


@pytest.mark.parametrize("color,depth", CASES)
@pytest.mark.parametrize("interlace", [False, True])
def test_every_colour_type_and_depth(pkg, color, depth, interlace):
    rng = np.random.default_rng(color * 100 + depth)
    for h, w in [(1, 1), (3, 5), (17, 23), (9, 64)]:
        samples = rng.integers(0, 1 << depth, (h, w, SPP[color]))
        palette = rng.integers(0, 256, (1 << depth, 3)) if color == 3 else None
        trns = bytes(rng.integers(0, 256, 1 << depth).tolist()) if color == 3 and depth == 4 else None
        if color == 0 and depth == 8:
            trns = struct.pack(">H", 7)                         # a colour key on grey: pixels stay as they are
        file = write_png(samples, depth, color, interlace, palette=palette, trns=trns)
        got = pkg.core.png_decode(file)
        want = expected(samples, depth, color, palette)
        assert got.shape == want.shape and got.dtype == np.uint8
        assert np.array_equal(got, want), (h, w)


@pytest.mark.parametrize("kind", range(5))
def test_each_filter_alone(pkg, kind):
    rng = np.random.default_rng(kind)
    samples = rng.integers(0, 256, (12, 19, 3))
    got = pkg.core.png_decode(write_png(samples, 8, 2, kinds=(kind,), pieces=1))
    assert np.array_equal(got, samples.astype(np.uint8))


def test_files_written_by_pillow(pkg):
    Image = pytest.importorskip("PIL.Image")
    rng = np.random.default_rng(5)

    def enc(img, **kw):
        b = io.BytesIO()
        img.save(b, format="PNG", **kw)
        return b.getvalue()

    for mode, shape in [("L", (40, 33)), ("LA", (21, 30, 2)), ("RGB", (64, 48, 3)), ("RGBA", (30, 31, 4))]:
        a = rng.integers(0, 256, shape, dtype=np.uint8)
        a[: shape[0] // 2] = a[0]                                # smooth rows: Pillow picks different filters
        got = pkg.core.png_decode(enc(Image.fromarray(a, mode), optimize=bool(shape[0] % 2)))
        want = a.reshape(shape[0], shape[1], -1)
        want = want if mode in ("L", "LA") else want[..., :3]
        assert np.array_equal(got, want), mode
    # palette images, with and without transparency: three channels either way
    rgb = Image.fromarray(rng.integers(0, 256, (25, 37, 3), dtype=np.uint8), "RGB")
    pal = rgb.quantize(colors=50)
    want = np.asarray(pal.convert("RGB"))
    assert np.array_equal(pkg.core.png_decode(enc(pal)), want)
    assert np.array_equal(pkg.core.png_decode(enc(pal, transparency=3)), want)
    # one bit per pixel and 16-bit grey
    bits = rng.integers(0, 2, (19, 21), dtype=np.uint8).astype(bool)
    assert np.array_equal(pkg.core.png_decode(enc(Image.fromarray(bits)))[..., 0], bits.astype(np.uint8) * 255)
    deep = rng.integers(0, 65536, (11, 14)).astype(np.uint16)
    assert np.array_equal(pkg.core.png_decode(enc(Image.fromarray(deep)))[..., 0], (deep >> 8).astype(np.uint8))


def test_malformed_files_are_refused(pkg):
    good = write_png(np.zeros((4, 4, 3), dtype=np.int64), 8, 2)
    for bad, why in [
        (good[:40], "no image data"),
        (good.replace(b"IDAT", b"IDAX"), "no image data"),
        (good[:8] + good[8:33].replace(b"\x08\x02", b"\x03\x02") + good[33:], "unsupported"),
        (b"\x89PNG\r\n\x1a\n" + bytes(40), "IHDR"),
    ]:
        with pytest.raises(RuntimeError, match=why):
            pkg.core.png_decode(bad)
    # compressed data that ends early: the IDAT chunk rewritten with half its bytes
    whole = write_png(np.arange(48).reshape(4, 4, 3), 8, 2, pieces=1)
    at = whole.index(b"IDAT")
    n = struct.unpack(">I", whole[at - 4:at])[0]
    cut = whole[:at - 4] + _chunk(b"IDAT", whole[at + 4:at + 4 + n // 2]) + whole[at + 8 + n:]
    with pytest.raises(RuntimeError, match="corrupt|not enough"):
        pkg.core.png_decode(cut)


def test_load_image_reports_png_sizes(pkg, tmp_path):
    file = write_png(np.zeros((6, 9, 4), dtype=np.int64), 8, 6)
    (tmp_path / "a.png").write_bytes(file)
    got = pkg.buffer_from_vector([{"file": b"a.png"}]).load_image("file", prefix=str(tmp_path), info=True)
    assert np.asarray(got[0]["file"]).tolist() == [9, 6]
    mem = pkg.buffer_from_vector([{"file": np.frombuffer(file, dtype=np.uint8)}]).load_image(
        "file", info=True, from_memory=True)
    assert np.asarray(mem[0]["file"]).tolist() == [9, 6]
