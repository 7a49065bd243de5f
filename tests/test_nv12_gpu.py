"""GPU parity: b200tbe_nv12_to_rgb vs the CPU oracle, bit for bit (byte output)."""
import numpy as np
import pytest
import torch

import oracle
from torchlib_xpu_b200 import cabi, workloads

pytestmark = pytest.mark.gpu


def _surface(rng, width, height, stride, tiled):
    rows_y = (height + 31) // 32 * 32 if tiled else height
    rows_uv = ((height + 1) // 2 + 31) // 32 * 32 if tiled else (height + 1) // 2
    y = rng.integers(0, 256, size=(rows_y, stride), dtype=np.uint8)
    uv = rng.integers(0, 256, size=(rows_uv, stride), dtype=np.uint8)
    return y, uv


@pytest.mark.parametrize("width,height,stride", [
    (64, 32, 128),         # one tile
    (1920, 1080, 1920),    # full HD: 16-pixel fast path, odd number of row pairs in a tile
    (1280, 720, 1408),     # pitch wider than the frame
    (100, 50, 128),        # width not a multiple of 16: per-pixel path
    (33, 17, 128),         # odd width and height
    (16, 1, 128),          # single row: the second row of the pair is absent
])
@pytest.mark.parametrize("tiled", [False, True])
@pytest.mark.parametrize("fullrange", [False, True])
def test_matches_oracle_bit_for_bit(width, height, stride, tiled, fullrange):
    if tiled and stride % 128:
        pytest.skip("Tile-Y pitch is a multiple of 128")
    rng = workloads.rng_for(900 + width + height)
    y, uv = _surface(rng, width, height, stride, tiled)
    want = oracle.nv12_to_rgb(y, uv, width, height, stride, fullrange, tiled)
    got = cabi.nv12_to_rgb(torch.from_numpy(y).cuda(), torch.from_numpy(uv).cuda(), width, height, stride,
                           fullrange, tiled).cpu().numpy()
    assert np.array_equal(got, want)


def test_committed_vectors_of_the_references_kernel():
    """The CUDA kernel against what the reference's own kernel returned (tests/golden/nv12_reference.npz,
    made by tests/golden/make_nv12_golden.py from the reference's source compiled for the host): two
    Tile-Y frames in both ranges, and 4096 YUV triples laid out as a one-row linear surface."""
    import os
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "nv12_reference.npz"))
    for name in ("a", "b"):
        w, h, stride = (int(v) for v in g[f"{name}_shape"])
        for key, fullrange in (("limited", False), ("full", True)):
            got = cabi.nv12_to_rgb(torch.from_numpy(g[f"{name}_y"]).cuda(), torch.from_numpy(g[f"{name}_uv"]).cuda(),
                                   w, h, stride, fullrange, True).cpu().numpy()
            assert np.array_equal(got, g[f"{name}_rgb_{key}"]), (name, key)
    # triples: pixel pairs (2 i, 2 i + 1) of one row share chroma pair i, so give both the same luma
    t = g["triples"]
    n = t.shape[0]
    y = np.repeat(t[:, 0], 2)[None, :].copy()
    uv = t[:, 1:3].reshape(1, 2 * n).copy()
    for key, fullrange in (("limited", False), ("full", True)):
        got = cabi.nv12_to_rgb(torch.from_numpy(y).cuda(), torch.from_numpy(uv).cuda(), 2 * n, 1, 2 * n,
                               fullrange, False).cpu().numpy()
        assert np.array_equal(got[0, 0::2], g[f"triples_rgb_{key}"])
        assert np.array_equal(got[0, 1::2], g[f"triples_rgb_{key}"])


def test_every_yuv_triple_of_a_sweep_matches():
    """All 256 luma values against a grid of chroma pairs: the float path has no off-by-one."""
    width, height, stride = 256, 64, 256
    y = np.tile(np.arange(256, dtype=np.uint8), (height, 1))
    uv = np.zeros((height // 2, stride), dtype=np.uint8)
    for r in range(height // 2):
        uv[r, 0::2] = (r * 8 + np.arange(128)) % 256
        uv[r, 1::2] = (255 - r * 8 - 2 * np.arange(128)) % 256
    for fullrange in (False, True):
        want = oracle.nv12_to_rgb(y, uv, width, height, stride, fullrange)
        got = cabi.nv12_to_rgb(torch.from_numpy(y).cuda(), torch.from_numpy(uv).cuda(), width, height,
                               stride, fullrange).cpu().numpy()
        assert np.array_equal(got, want)


def test_unaligned_pointers_take_the_pixel_path_and_bad_arguments_are_refused():
    rng = workloads.rng_for(950)
    width, height, stride = 64, 8, 64
    y, uv = _surface(rng, width, height, stride, False)
    want = oracle.nv12_to_rgb(y, uv, width, height, stride)
    yb = torch.zeros(y.size + 1, dtype=torch.uint8, device="cuda")
    yb[1:] = torch.from_numpy(y).cuda().flatten()
    got = cabi.nv12_to_rgb(yb[1:], torch.from_numpy(uv).cuda(), width, height, stride).cpu().numpy()
    assert np.array_equal(got, want)
    with pytest.raises(cabi.B200TbeError):
        cabi.nv12_to_rgb(torch.from_numpy(y).cuda(), torch.from_numpy(uv).cuda(), width, height, 32)      # pitch < width
    with pytest.raises(cabi.B200TbeError):
        cabi.nv12_to_rgb(torch.from_numpy(y).cuda(), torch.from_numpy(uv).cuda(), width, height, 64, tiled=True)
    empty = cabi.nv12_to_rgb(torch.from_numpy(y).cuda(), torch.from_numpy(uv).cuda(), 0, 0, stride)
    assert empty.numel() == 0
