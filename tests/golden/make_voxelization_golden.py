"""Generates tests/golden/voxelization_golden.npz from the reference's own CPU code
for hard voxelization (oracle/_ref, built by oracle/build_ref.py from the reference
tree).

Run where the reference tree is available:
    python oracle/build_ref.py && python tests/golden/make_voxelization_golden.py
Per case the fixture holds the seeded inputs and the four outputs the reference
code produced.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "voxelization_golden.npz")

CASES = [
    # name, points, features, voxel_size, coors_range, max_points, max_voxels, spread
    ("lidar_like", 3000, 4, (0.5, 0.5, 1.0), (0, -10, -3, 20, 10, 1), 5, 600, 1.2),
    ("dense_cap_points", 2000, 3, (2.0, 2.0, 2.0), (0, 0, 0, 8, 8, 4), 3, 64, 1.0),
    ("cap_voxels", 1500, 5, (0.25, 0.25, 0.5), (0, 0, 0, 10, 10, 2), 4, 100, 1.0),
    ("many_outside", 1000, 4, (1.0, 1.0, 1.0), (0, 0, 0, 4, 4, 2), 8, 40, 3.0),
    ("single_point", 1, 3, (1.0, 1.0, 1.0), (0, 0, 0, 4, 4, 4), 2, 3, 1.0),
]


def make_points(rng, n, f, cr, spread):
    lo = np.array(cr[:3], dtype=np.float32)
    hi = np.array(cr[3:], dtype=np.float32)
    centre, half = (lo + hi) / 2, (hi - lo) / 2 * spread
    xyz = centre + (rng.random((n, 3), dtype=np.float32) * 2 - 1) * half
    rest = rng.random((n, f - 3), dtype=np.float32)
    return np.concatenate([xyz, rest], 1).astype(np.float32)


def main():
    assert oracle.ref_lib() is not None, "build oracle/_ref first (python oracle/build_ref.py)"
    rng = np.random.default_rng(20241127)
    store = {"names": np.array([c[0] for c in CASES])}
    for name, n, f, vs, cr, mp, mv, spread in CASES:
        pts = make_points(rng, n, f, cr, spread)
        voxels, coors, npv, num = oracle.voxelization(pts, vs, cr, mp, mv, use_ref=True)
        store[name + "/points"] = pts
        store[name + "/voxel_size"] = np.array(vs, dtype=np.float32)
        store[name + "/coors_range"] = np.array(cr, dtype=np.float32)
        store[name + "/params"] = np.array([mp, mv, num], dtype=np.int64)
        store[name + "/voxels"] = voxels
        store[name + "/coors"] = coors
        store[name + "/num_points_per_voxel"] = npv
        print(name, "voxel_num", num, "max points in a voxel", int(npv.max()))
    np.savez_compressed(OUT, **store)
    print(OUT, os.path.getsize(OUT), "bytes")


if __name__ == "__main__":
    main()
