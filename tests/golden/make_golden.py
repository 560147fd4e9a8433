"""Generates tests/golden/sparse_conv_golden.npz from the reference's own CPU
code (oracle/_ref, built by oracle/build_ref.py from the reference tree).

Run where the reference tree is available:
    python oracle/build_ref.py && python tests/golden/make_golden.py
The fixture holds, per case, the inputs and the outputs the reference code
produced: indice_pairs, out_indices, indice_num for the rulebook and
features_out for the convolution in each of the three filter layouts.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "sparse_conv_golden.npz")


def out_space(space, pad, stride, dil, ks):
    return [(i + 2 * p - d * (k - 1) - 1) // s + 1 for i, p, s, d, k in zip(space, pad, stride, dil, ks)]


def random_indices(rng, batch, space, n):
    D, H, W = space
    lin = rng.choice(batch * D * H * W, size=n, replace=False)
    b, rem = np.divmod(lin, D * H * W)
    z, rem = np.divmod(rem, H * W)
    y, x = np.divmod(rem, W)
    return np.stack([b, z, y, x], 1).astype(np.int32)


CASES = [
    # name, batch, space, n, ks, stride, pad, dil, sub_m, ci, co
    ("subm_k3", 2, (6, 9, 8), 150, (3, 3, 3), (1, 1, 1), (1, 1, 1), (1, 1, 1), 1, 5, 7),
    ("subm_k3_repeated", 2, (6, 9, 8), 150, (3, 3, 3), (1, 1, 1), (1, 1, 1), (1, 1, 1), 1, 5, 7),
    ("down_k3_s2", 2, (7, 10, 9), 120, (3, 3, 3), (2, 2, 2), (1, 1, 1), (1, 1, 1), 0, 4, 6),
    ("dilated_k3_d2", 1, (8, 8, 8), 90, (3, 3, 3), (1, 1, 1), (2, 2, 2), (2, 2, 2), 0, 3, 3),
    ("k311_s211_p0", 2, (6, 7, 5), 100, (3, 1, 1), (2, 1, 1), (0, 0, 0), (1, 1, 1), 0, 8, 4),
    ("k2_s2_p0", 1, (8, 8, 8), 80, (2, 2, 2), (2, 2, 2), (0, 0, 0), (1, 1, 1), 0, 2, 5),
    ("subm_k133", 1, (5, 12, 12), 200, (1, 3, 3), (1, 1, 1), (0, 1, 1), (1, 1, 1), 1, 6, 6),
    ("mixed_stride", 1, (9, 9, 9), 110, (3, 3, 3), (1, 2, 1), (1, 0, 2), (2, 1, 1), 0, 3, 2),
]


def main():
    assert oracle.ref_lib() is not None, "build oracle/_ref first (python oracle/build_ref.py)"
    rng = np.random.default_rng(20241125)
    store = {}
    names = []
    for name, batch, space, n, ks, stride, pad, dil, sub_m, ci, co in CASES:
        osp = list(space) if sub_m else out_space(space, pad, stride, dil, ks)
        idx = random_indices(rng, batch, space, n)
        if name == "subm_k3_repeated":
            idx[-3:] = idx[:3]  # repeated coordinates: the last row wins
        pairs, out_idx, num, n_out = oracle.get_indice_pairs(idx, batch, pad, stride, dil, ks, osp, sub_m,
                                                             use_ref=True)
        feat = rng.standard_normal((n, ci)).astype(np.float32)
        K = int(np.prod(ks))
        w = (rng.standard_normal(tuple(ks) + (ci, co)) / np.sqrt(K * ci)).astype(np.float32)  # ARRAY
        w_ndhwc = np.ascontiguousarray(np.transpose(w, (4, 0, 1, 2, 3)))
        w_ncdhw = np.ascontiguousarray(np.transpose(w, (4, 3, 0, 1, 2)))
        n_rows = max(n_out, 1)
        outs = {}
        for layout, wl in (("ARRAY", w), ("NDHWC", w_ndhwc), ("NCDHW", w_ncdhw)):
            outs[layout] = oracle.indice_convolution_forward(feat, wl, layout, ks, pairs, num, n_rows, co,
                                                             use_ref=True)
        assert np.array_equal(outs["ARRAY"], outs["NDHWC"]) and np.array_equal(outs["ARRAY"], outs["NCDHW"])
        names.append(name)
        store[name + "/params"] = np.array([batch, *space, *ks, *stride, *pad, *dil, *osp, sub_m, ci, co, n_out],
                                           dtype=np.int64)
        store[name + "/indices"] = idx
        store[name + "/indice_pairs"] = pairs
        store[name + "/out_indices"] = out_idx
        store[name + "/indice_num"] = num
        store[name + "/features"] = feat
        store[name + "/filters_array"] = w
        store[name + "/features_out"] = outs["ARRAY"]
    store["names"] = np.array(names)
    # float -> half bit patterns of the reference's converter
    import ctypes
    xs = np.concatenate([
        rng.standard_normal(400).astype(np.float32) * np.float32(10.0) ** rng.integers(-9, 6, 400).astype(np.float32),
        np.array([0.0, -0.0, 65504.0, 65520.0, 1e6, -1e6, 6.1e-5, 5.96e-8, 2.98e-8, 1e-9, np.inf, -np.inf],
                 dtype=np.float32)]).astype(np.float32)
    r = oracle.ref_lib()
    store["half/x"] = xs
    store["half/bits"] = np.array([r.mluops_ref_float_to_half_bits(ctypes.c_float(float(v))) for v in xs],
                                  dtype=np.uint16)
    np.savez_compressed(OUT, **store)
    print(OUT, os.path.getsize(OUT), "bytes")


if __name__ == "__main__":
    main()
