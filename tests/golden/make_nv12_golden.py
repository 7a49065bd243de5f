"""Writes tests/golden/nv12_reference.npz: outputs of the reference's own colour-conversion kernel
(packages/torchcodec-xpu/src/torchcodec_xpu/ColorConversionKernel.cpp, compiled for the host by
oracle/build.py into oracle/_ref/libnv12_ref.so) on seeded inputs. Run where the reference tree is
present:

    python tests/golden/make_nv12_golden.py

Contents: two Tile-Y frames (inputs and the kernel's RGB, limited and "full" range), the tile offsets
of a 2 x 2-tile surface, and a 4096-entry sample of the 2^24 YUV triples with the kernel's RGB."""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import oracle  # noqa: E402


def main():
    ref = oracle.Nv12Reference()
    rng = np.random.default_rng(20)
    out = {}
    for name, (w, h, stride) in {"a": (100, 38, 128), "b": (300, 70, 384)}.items():
        rows_y = (h + 31) // 32 * 32
        rows_uv = ((h + 1) // 2 + 31) // 32 * 32
        yp = rng.integers(0, 256, size=(rows_y, stride), dtype=np.uint8)
        uv = rng.integers(0, 256, size=(rows_uv, stride), dtype=np.uint8)
        out[f"{name}_shape"] = np.asarray([w, h, stride], dtype=np.int32)
        out[f"{name}_y"] = yp
        out[f"{name}_uv"] = uv
        out[f"{name}_rgb_limited"] = ref.convert(yp, uv, w, h, stride, False)
        out[f"{name}_rgb_full"] = ref.convert(yp, uv, w, h, stride, True)
    stride, rows = 256, 64
    out["tile_offsets_256x64"] = np.asarray(
        [[ref.tile_offset(x, y, stride) for x in range(stride)] for y in range(rows)], dtype=np.int32)
    triples = rng.integers(0, 256, size=(4096, 3), dtype=np.uint8)
    table = {False: ref.all_triples(False), True: ref.all_triples(True)}
    out["triples"] = triples
    out["triples_rgb_limited"] = table[False][triples[:, 0], triples[:, 1], triples[:, 2]]
    out["triples_rgb_full"] = table[True][triples[:, 0], triples[:, 1], triples[:, 2]]
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "nv12_reference.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
