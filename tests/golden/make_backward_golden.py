"""Generates tests/golden/sparse_conv_backward_golden.npz from the reference's own
CPU code for the two backward operators (oracle/_ref, built by oracle/build_ref.py
from the reference tree).

Run where the reference tree is available, after make_golden.py:
    python oracle/build_ref.py && python tests/golden/make_backward_golden.py
The rulebooks, features and filters are those of sparse_conv_golden.npz; this
fixture adds, per case, a seeded output_grad and what the reference code made of
it: input_grad (float arithmetic, and the reference's half emulation on inputs
rounded through half) and filters_grad (float, and float on half-rounded inputs).
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
import oracle  # noqa: E402
import helpers  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "sparse_conv_golden.npz")
OUT = os.path.join(HERE, "sparse_conv_backward_golden.npz")


def main():
    assert oracle.ref_lib() is not None, "build oracle/_ref first (python oracle/build_ref.py)"
    golden = np.load(SRC)
    rng = np.random.default_rng(20241126)
    store = {"names": golden["names"]}
    for name in helpers.golden_names(golden):
        c = helpers.golden_case(golden, name)
        n_rows = c["features_out"].shape[0]
        og = rng.standard_normal((n_rows, c["co"])).astype(np.float32)
        store[name + "/output_grad"] = og
        w = c["filters_array"]
        grads = {}
        for layout in ("ARRAY", "NDHWC", "NCDHW"):
            grads[layout] = oracle.indice_convolution_backward_data(
                og, helpers.permute_filter(w, layout), layout, c["ks"], c["indice_pairs"], c["indice_num"],
                c["ci"], False, use_ref=True)
        assert np.array_equal(grads["ARRAY"], grads["NDHWC"]) and np.array_equal(grads["ARRAY"], grads["NCDHW"])
        store[name + "/input_grad"] = grads["ARRAY"]
        og_h, w_h, f_h = (oracle.round_through_half(a) for a in (og, w, c["features"]))
        store[name + "/input_grad_half"] = oracle.indice_convolution_backward_data(
            og_h, w_h, "ARRAY", c["ks"], c["indice_pairs"], c["indice_num"], c["ci"], True, use_ref=True)
        if c["ks"][1] == c["ks"][2]:  # the reference reads kw with the H accessor
            store[name + "/filters_grad"] = oracle.indice_convolution_backward_filter(
                c["features"], og, c["ks"], c["indice_pairs"], c["indice_num"], use_ref=True)
            store[name + "/filters_grad_half"] = oracle.indice_convolution_backward_filter(
                f_h, og_h, c["ks"], c["indice_pairs"], c["indice_num"], use_ref=True)
    np.savez_compressed(OUT, **store)
    print(OUT, os.path.getsize(OUT), "bytes")


if __name__ == "__main__":
    main()
