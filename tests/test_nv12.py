"""NV12 -> RGB24 oracle (CPU) pinned to the reference's own kernel source and to BT.709.

The reference holds no vectors for its colour-conversion kernel
(packages/torchcodec-xpu/src/torchcodec_xpu/ColorConversionKernel.cpp), but the file itself compiles
for the host on top of a stand-in for the SYCL names it uses (oracle/nv12_ref_wrap.cpp ->
oracle/_ref/libnv12_ref.so, built where the reference tree is present and carried along as a built
file). The restatement is compared with it bit for bit: get_tile_offset over every byte of multi-tile
surfaces, yuv2rgb over all 2^24 triples, the whole kernel over random Tile-Y frames. Beside that:
known answers of the standard (limited-range black / white / grey, the 100 % primaries) and the
structural properties of the tiled layout."""
import numpy as np
import pytest

import oracle
from oracle import build as oracle_build


def _reference(contracted=False):
    if not oracle_build.build_nv12_reference():
        pytest.skip("oracle/_ref is not built and the reference tree is not here")
    return oracle.Nv12Reference(contracted)


@pytest.mark.parametrize("stride,rows", [(256, 64), (384, 96), (128, 32), (1920 + 128, 64)])
def test_tile_y_offsets_equal_the_references_get_tile_offset(stride, rows):
    """Every (x, y) of surfaces of 1 x 1, 2 x 2, 3 x 3 and 16 x 2 tiles (ColorConversionKernel.cpp:29-80)."""
    ref = _reference()
    for y in range(rows):
        for x in range(0, stride):
            assert oracle.nv12_offset(x, y, stride, True) == ref.tile_offset(x, y, stride), (x, y)


@pytest.mark.parametrize("fullrange", [False, True])
def test_every_yuv_triple_equals_the_references_yuv2rgb(fullrange):
    """All 2^24 triples (ColorConversionKernel.cpp:82-100), and what fusing the dot products'
    multiply-adds (which a device compiler may do with sycl::dot) would change."""
    ours = oracle.nv12_all_triples(fullrange)
    ref = _reference().all_triples(fullrange)
    assert np.array_equal(ours, ref)
    fused = _reference(contracted=True).all_triples(fullrange)
    differ = np.any(fused != ref, axis=-1)
    # contraction changes the last bit of a few products; after x255 and truncation that moves a
    # channel by at most one step, for a small share of the triples
    assert np.abs(fused.astype(np.int16) - ref.astype(np.int16)).max() <= 1
    assert differ.mean() < 0.05, differ.mean()


@pytest.mark.parametrize("fullrange", [False, True])
def test_whole_frames_equal_the_references_kernel(fullrange):
    """convertNV12ToRGB (ColorConversionKernel.cpp:131-181) over a random Tile-Y surface whose width
    and height are not multiples of the tile."""
    ref = _reference()
    rng = np.random.default_rng(5)
    w, h, stride = 300, 70, 384
    yp = rng.integers(0, 256, size=(96, stride), dtype=np.uint8)      # plane heights padded to 32 rows
    uv = rng.integers(0, 256, size=(64, stride), dtype=np.uint8)
    want = ref.convert(yp, uv, w, h, stride, fullrange)
    got = oracle.nv12_to_rgb(yp, uv, w, h, stride, fullrange, tiled=True)
    assert np.array_equal(got, want)


def _golden():
    import os
    return np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "nv12_reference.npz"))


def test_committed_vectors_of_the_references_kernel():
    """tests/golden/nv12_reference.npz holds what the reference's kernel (compiled for the host, see
    tests/golden/make_nv12_golden.py) returned for two Tile-Y frames, a surface's tile offsets and
    4096 YUV triples; the restatement reproduces all of it without the reference tree."""
    g = _golden()
    for name in ("a", "b"):
        w, h, stride = (int(v) for v in g[f"{name}_shape"])
        for key, fullrange in (("limited", False), ("full", True)):
            got = oracle.nv12_to_rgb(g[f"{name}_y"], g[f"{name}_uv"], w, h, stride, fullrange, tiled=True)
            assert np.array_equal(got, g[f"{name}_rgb_{key}"]), (name, key)
    offs = g["tile_offsets_256x64"]
    for y in range(offs.shape[0]):
        for x in range(offs.shape[1]):
            assert oracle.nv12_offset(x, y, 256, True) == int(offs[y, x])
    for key, fullrange in (("limited", False), ("full", True)):
        want = g[f"triples_rgb_{key}"]
        for (yy, u, v), rgb in zip(g["triples"][:512], want[:512]):
            assert oracle.nv12_pixel(int(yy), int(u), int(v), fullrange) == tuple(int(c) for c in rgb)


@pytest.mark.parametrize("yuv,rgb", [
    ((16, 128, 128), (0, 0, 0)),          # black
    ((235, 128, 128), (255, 255, 255)),   # white
    ((126, 128, 128), (128, 128, 128)),   # mid grey: (126 - 16) / 219 * 255 = 128.08
    ((63, 102, 240), (255, 0, 0)),        # BT.709 red   (Y 62.7, Cb 102.4, Cr 240)
    ((32, 240, 118), (0, 0, 255)),        # BT.709 blue  (Y 31.8, Cb 240, Cr 117.6)
])
def test_limited_range_known_answers(yuv, rgb):
    got = oracle.nv12_pixel(*yuv)
    assert all(abs(g - w) <= 1 for g, w in zip(got, rgb)), (got, rgb)


def test_green_primary_and_clamping():
    r, g, b = oracle.nv12_pixel(173, 42, 26)      # BT.709 green (Y 172.8, Cb 41.6, Cr 26.3)
    assert r <= 1 and g == 255 and b <= 2
    assert oracle.nv12_pixel(255, 128, 128) == (255, 255, 255)   # above nominal white: clamped, not wrapped
    assert oracle.nv12_pixel(0, 128, 128) == (0, 0, 0)           # below nominal black: clamped at zero


def test_full_range_formula_as_the_reference_writes_it():
    # ColorConversionKernel.cpp:84-88: chroma is (c - 128) / 255 - 0.5, so neutral chroma 128 is NOT
    # neutral in this mode; the restatement keeps that, digit for digit
    y, u, v = 200, 128, 128
    s0, s1, s2 = np.float32(y) / np.float32(255), np.float32(-0.5), np.float32(-0.5)
    want = []
    for m in ((1.0, 0.0, 1.5748), (1.0, -0.187324, -0.468124), (1.0, 1.8556, 0.0)):
        d = np.float32(s0 * np.float32(m[0]))
        d = np.float32(d + np.float32(s1 * np.float32(m[1])))
        d = np.float32(d + np.float32(s2 * np.float32(m[2])))
        want.append(int(min(max(np.float32(d * np.float32(255)), 0), 255)))
    assert oracle.nv12_pixel(y, u, v, fullrange=True) == tuple(want)


def test_tile_y_offsets_are_a_bijection_with_contiguous_16_byte_columns():
    stride, rows = 384, 64
    seen = np.zeros(stride * rows, dtype=np.int32)
    for y in range(rows):
        for x in range(stride):
            seen[oracle.nv12_offset(x, y, stride, True)] += 1
    assert np.all(seen == 1)
    # a tile is 128 bytes x 32 rows = 4096 bytes and tiles follow each other row-major
    assert oracle.nv12_offset(128, 0, stride, True) // 4096 == 1
    assert oracle.nv12_offset(0, 32, stride, True) // 4096 == stride // 128
    # 16 aligned bytes of a row stay together; the next row of the same column is 16 bytes on
    for y in (0, 5, 31):
        for x in (0, 16, 64, 112):
            base = oracle.nv12_offset(x, y, stride, True)
            assert [oracle.nv12_offset(x + i, y, stride, True) for i in range(16)] == list(range(base, base + 16))
    assert oracle.nv12_offset(0, 1, stride, True) - oracle.nv12_offset(0, 0, stride, True) == 16
    # the two 64-byte halves trade places in every second group of 4 rows
    assert oracle.nv12_offset(0, 0, stride, True) == 0
    # (without the swap column 4 of group 0 starts at byte 256 and column 0 of group 1 at byte 512)
    assert oracle.nv12_offset(64, 0, stride, True) == 512 and oracle.nv12_offset(0, 4, stride, True) == 256
    assert oracle.nv12_offset(64, 4, stride, True) == (1 * 8 + 4) * 64
    # linear layout
    assert oracle.nv12_offset(7, 3, stride, False) == 3 * stride + 7


def test_frame_conversion_uses_one_chroma_sample_per_2x2_block():
    w, h, stride = 6, 4, 8
    yp = np.full((h, stride), 126, dtype=np.uint8)
    uv = np.full((h // 2, stride), 128, dtype=np.uint8)
    uv[1, 2:4] = (102, 240)      # chroma of the block at columns 2-3, rows 2-3: red-ish
    rgb = oracle.nv12_to_rgb(yp, uv, w, h, stride)
    assert rgb.shape == (h, w, 3)
    grey = oracle.nv12_pixel(126, 128, 128)
    red = oracle.nv12_pixel(126, 102, 240)
    for y in range(h):
        for x in range(w):
            want = red if (y >= 2 and 2 <= x <= 3) else grey
            assert tuple(int(c) for c in rgb[y, x]) == want
