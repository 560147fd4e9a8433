"""CPU-only: pins the oracle (plain-C restatement) against the reference.

Three anchors: (1) the reference's own function bodies compiled from the
reference tree (oracle/_ref; skipped where that library has not been built),
(2) golden vectors that library produced, committed under tests/golden/, and
(3) a case small enough to check by hand.
"""
import ctypes

import numpy as np
import pytest

import helpers


def test_golden_rulebooks(oracle, golden):
    for name in helpers.golden_names(golden):
        c = helpers.golden_case(golden, name)
        pairs, out_idx, num, n_out = oracle.get_indice_pairs(
            c["indices"], c["batch"], c["pad"], c["stride"], c["dil"], c["ks"], c["out_space"], c["sub_m"],
            out_rows=c["out_indices"].shape[0], sentinel_quirk=True)
        assert np.array_equal(num, c["indice_num"]), name
        assert np.array_equal(pairs, c["indice_pairs"]), name
        assert np.array_equal(out_idx, c["out_indices"]), name
        assert n_out == c["n_out"], name
        # the true count equals the reference's count whenever a slot is unused
        if helpers.has_unused_slot(num, c["indices"].shape[0]):
            assert oracle.get_indice_pairs(c["indices"], c["batch"], c["pad"], c["stride"], c["dil"], c["ks"],
                                           c["out_space"], c["sub_m"])[3] == n_out


@pytest.mark.parametrize("layout", ["ARRAY", "NDHWC", "NCDHW"])
def test_golden_convolutions(oracle, golden, layout):
    for name in helpers.golden_names(golden):
        c = helpers.golden_case(golden, name)
        w = helpers.permute_filter(c["filters_array"], layout)
        out = oracle.indice_convolution_forward(c["features"], w, layout, c["ks"], c["indice_pairs"],
                                                c["indice_num"], c["features_out"].shape[0], c["co"])
        assert np.array_equal(out, c["features_out"]), name


def test_golden_half_bits(oracle, golden):
    assert np.array_equal(oracle.float_to_half_bits(golden["half/x"]), golden["half/bits"])


def test_against_reference_code(oracle):
    if oracle.ref_lib() is None:
        pytest.skip("oracle/_ref not built (reference tree absent)")
    rng = np.random.default_rng(11)
    done = 0
    while done < 150:
        g = helpers.random_geometry(rng, sub_m=bool(rng.integers(0, 2)))
        if g is None:
            continue
        idx = helpers.random_indices(rng, g["batch"], g["space"], g["n"])
        args = (idx, g["batch"], g["pad"], g["stride"], g["dil"], g["ks"], g["out_space"], g["sub_m"])
        a = oracle.get_indice_pairs(*args, sentinel_quirk=True)
        b = oracle.get_indice_pairs(*args, use_ref=True)
        for x, y in zip(a[:3], b[:3]):
            assert np.array_equal(x, y), g
        ci, co = int(rng.integers(1, 9)), int(rng.integers(1, 9))
        feat = rng.standard_normal((g["n"], ci)).astype(np.float32)
        w = rng.standard_normal(tuple(g["ks"]) + (ci, co)).astype(np.float32)
        layout = ["ARRAY", "NDHWC", "NCDHW"][done % 3]
        wl = helpers.permute_filter(w, layout)
        n_rows = max(a[3], 1)
        o1 = oracle.indice_convolution_forward(feat, wl, layout, g["ks"], a[0], a[2], n_rows, co)
        o2 = oracle.indice_convolution_forward(feat, wl, layout, g["ks"], a[0], a[2], n_rows, co, use_ref=True)
        assert np.array_equal(o1, o2), g
        done += 1
    r = oracle.ref_lib()
    xs = (rng.standard_normal(5000) * 10.0 ** rng.integers(-9, 6, 5000)).astype(np.float32)
    ref_bits = np.array([r.mluops_ref_float_to_half_bits(ctypes.c_float(float(v))) for v in xs], dtype=np.uint16)
    assert np.array_equal(oracle.float_to_half_bits(xs), ref_bits)


def test_two_voxel_case_by_hand(oracle):
    """Two adjacent voxels in the interior of a 4x4x4 grid, 3x3x3 kernel, pad 1."""
    idx = np.array([[0, 1, 1, 1], [0, 1, 1, 2]], dtype=np.int32)
    ones, k3, sp = [1, 1, 1], [3, 3, 3], [4, 4, 4]
    pairs, out_idx, num, n_out = oracle.get_indice_pairs(idx, 1, ones, ones, ones, k3, sp, True)
    # centre offset pairs each voxel with itself; x-1 / x+1 pair them with each other
    assert num.sum() == 4 and num[13] == 2 and num[12] == 1 and num[14] == 1
    assert pairs[13, 0, :2].tolist() == [0, 1] and pairs[13, 1, :2].tolist() == [0, 1]
    # offset 14 (kw=2): output x = input x - 1 -> input 1 feeds output 0
    assert pairs[14, 0, 0] == 1 and pairs[14, 1, 0] == 0
    assert pairs[12, 0, 0] == 0 and pairs[12, 1, 0] == 1
    assert np.array_equal(out_idx, idx) and n_out == 2
    # default mode: every offset is valid for both voxels (no unused slot): 54
    # pairs onto 36 distinct cells; this is the input class on which the
    # reference's `unique.size() - 1` undercounts by one.
    pairs, out_idx, num, n_out = oracle.get_indice_pairs(idx, 1, ones, ones, ones, k3, sp, False)
    assert num.tolist() == [2] * 27 and n_out == 36
    assert not helpers.has_unused_slot(num, 2)
    quirk = oracle.get_indice_pairs(idx, 1, ones, ones, ones, k3, sp, False, sentinel_quirk=True)
    assert quirk[3] == 35
    # ascending linear order of out_indices
    lin = (out_idx[:36, 1] * 4 + out_idx[:36, 2]) * 4 + out_idx[:36, 3]
    assert np.all(np.diff(lin) > 0)


def test_pair_lists_are_ordered(oracle):
    rng = np.random.default_rng(5)
    idx = helpers.random_indices(rng, 2, [6, 8, 8], 300)
    pairs, _, num, n_out = oracle.get_indice_pairs(idx, 2, [1] * 3, [2] * 3, [1] * 3, [3] * 3, [3, 4, 4], False)
    for k in range(27):
        p = int(num[k])
        assert np.all(np.diff(pairs[k, 0, :p]) > 0)
        assert np.all(pairs[k, :, p:] == -1)
        assert np.all((pairs[k, 1, :p] >= 0) & (pairs[k, 1, :p] < n_out))


def test_diffs(oracle):
    base = np.array([1.0, -2.0, 0.0, 4.0], dtype=np.float32)
    test = np.array([1.5, -2.0, 0.25, 4.0], dtype=np.float32)
    d1, d2, d3 = oracle.diffs(test, base, False)
    assert d1 == pytest.approx(0.75 / 7.0, rel=1e-6)
    assert d2 == pytest.approx(np.sqrt((0.25 + 0.0625) / 21.0), rel=1e-6)
    assert d3 == pytest.approx(0.5, rel=1e-6)


def test_round_through_half_matches_ieee_for_normal_values(oracle):
    rng = np.random.default_rng(3)
    x = rng.standard_normal(20000).astype(np.float32)
    assert np.array_equal(oracle.round_through_half(x), x.astype(np.float16).astype(np.float32))
    assert oracle.float_to_half_bits(np.array([1e6], dtype=np.float32))[0] == 0x7BFF  # saturates
