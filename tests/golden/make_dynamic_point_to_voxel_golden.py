"""Generates tests/golden/dynamic_point_to_voxel_golden.npz from the reference's own
CPU code (oracle/_ref, built by oracle/build_ref.py from the reference tree).

Run where the reference tree is available:
    python oracle/build_ref.py && python tests/golden/make_dynamic_point_to_voxel_golden.py
Per case: seeded feats and coors, and for both reductions what the reference code
produced (voxel_feats / voxel_coors / voxel_points_count cut to voxel_num rows,
point2voxel_map, voxel_num, coors after the in-place -1 fill), and for the maximum a seeded
grad_voxel_feats with the grad_feats the reference's backward code made of it.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "dynamic_point_to_voxel_golden.npz")

CASES = [
    # name, points, channels, coordinate ranges (low, high) per axis
    ("small_grid", 1500, 4, [(0, 6), (0, 9), (0, 7)]),
    ("with_negatives", 1200, 3, [(-2, 8), (-1, 12), (-1, 5)]),
    ("wide_coordinates", 900, 5, [(0, 70000), (0, 300), (0, 1 << 20)]),
    ("one_voxel", 300, 2, [(3, 4), (5, 6), (7, 8)]),
    ("all_invalid", 50, 2, [(-3, 0), (-3, 0), (-3, 0)]),
    ("single_point", 1, 3, [(2, 3), (0, 1), (9, 10)]),
]


def main():
    assert oracle.ref_lib() is not None, "build oracle/_ref first (python oracle/build_ref.py)"
    rng = np.random.default_rng(20241128)
    store = {"names": np.array([c[0] for c in CASES])}
    for name, n, c, ranges in CASES:
        coors = np.stack([rng.integers(lo, hi, n) for lo, hi in ranges], 1).astype(np.int32)
        feats = (rng.standard_normal((n, c)) * 10).astype(np.float32)
        store[name + "/feats"], store[name + "/coors"] = feats, coors
        for mode in ("max", "mean"):
            vf, vc, p2v, cnt, num, filled = oracle.dynamic_point_to_voxel_forward(feats, coors, mode, use_ref=True)
            store["%s/%s/voxel_feats" % (name, mode)] = vf[:num]
            store["%s/voxel_coors" % name] = vc[:num]
            store["%s/voxel_points_count" % name] = cnt[:num]
            store["%s/point2voxel_map" % name] = p2v
            store["%s/voxel_num" % name] = np.array([num], dtype=np.int32)
            store["%s/coors_filled" % name] = filled
        vf, vc, p2v, cnt, num, _ = oracle.dynamic_point_to_voxel_forward(feats, coors, "max", use_ref=True)
        grad = rng.standard_normal((max(num, 1), c)).astype(np.float32)
        store[name + "/grad_voxel_feats"] = grad
        store[name + "/grad_feats"] = oracle.dynamic_point_to_voxel_backward(grad, feats, vf[:max(num, 1)], p2v, num,
                                                                             use_ref=True)
        print(name, "voxel_num", num)
    np.savez_compressed(OUT, **store)
    print(OUT, os.path.getsize(OUT), "bytes")


if __name__ == "__main__":
    main()
