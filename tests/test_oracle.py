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


@pytest.mark.parametrize("layout", ["ARRAY", "NDHWC", "NCDHW"])
def test_golden_input_gradients(oracle, golden, backward_golden, layout):
    """input_grad the reference's own CPU code produced, float and half emulation."""
    for name in helpers.golden_names(golden):
        c = helpers.golden_case(golden, name)
        og = backward_golden[name + "/output_grad"]
        w = helpers.permute_filter(c["filters_array"], layout)
        out = oracle.indice_convolution_backward_data(og, w, layout, c["ks"], c["indice_pairs"], c["indice_num"],
                                                      c["ci"], False)
        assert np.array_equal(out, backward_golden[name + "/input_grad"]), name
        og_h, w_h = oracle.round_through_half(og), oracle.round_through_half(w)
        out = oracle.indice_convolution_backward_data(og_h, w_h, layout, c["ks"], c["indice_pairs"],
                                                      c["indice_num"], c["ci"], True)
        assert np.array_equal(out, backward_golden[name + "/input_grad_half"]), name


def test_golden_filter_gradients(oracle, golden, backward_golden):
    """filters_grad the reference's own CPU code produced."""
    checked = 0
    for name in helpers.golden_names(golden):
        if name + "/filters_grad" not in backward_golden:
            continue
        c = helpers.golden_case(golden, name)
        og = backward_golden[name + "/output_grad"]
        out = oracle.indice_convolution_backward_filter(c["features"], og, c["ks"], c["indice_pairs"],
                                                        c["indice_num"])
        assert np.array_equal(out, backward_golden[name + "/filters_grad"]), name
        out = oracle.indice_convolution_backward_filter(oracle.round_through_half(c["features"]),
                                                        oracle.round_through_half(og), c["ks"], c["indice_pairs"],
                                                        c["indice_num"])
        assert np.array_equal(out, backward_golden[name + "/filters_grad_half"]), name
        checked += 1
    assert checked >= 6


def test_backward_against_reference_code(oracle):
    if oracle.ref_lib() is None:
        pytest.skip("oracle/_ref not built (reference tree absent)")
    rng = np.random.default_rng(12)
    done = 0
    while done < 60:
        g = helpers.random_geometry(rng, sub_m=bool(rng.integers(0, 2)))
        if g is None:
            continue
        idx = helpers.random_indices(rng, g["batch"], g["space"], g["n"])
        pairs, _, num, n_out = oracle.get_indice_pairs(idx, g["batch"], g["pad"], g["stride"], g["dil"], g["ks"],
                                                       g["out_space"], g["sub_m"])
        ci, co = int(rng.integers(1, 9)), int(rng.integers(1, 9))
        is_half = bool(done % 2)
        feat = rng.standard_normal((g["n"], ci)).astype(np.float32)
        og = rng.standard_normal((max(n_out, 1), co)).astype(np.float32)
        w = rng.standard_normal(tuple(g["ks"]) + (ci, co)).astype(np.float32)
        if is_half:
            feat, og, w = (oracle.round_through_half(a) for a in (feat, og, w))
        layout = ["ARRAY", "NDHWC", "NCDHW"][done % 3]
        wl = helpers.permute_filter(w, layout)
        a = oracle.indice_convolution_backward_data(og, wl, layout, g["ks"], pairs, num, ci, is_half)
        b = oracle.indice_convolution_backward_data(og, wl, layout, g["ks"], pairs, num, ci, is_half, use_ref=True)
        assert np.array_equal(a, b), g
        if g["ks"][1] == g["ks"][2]:
            a = oracle.indice_convolution_backward_filter(feat, og, g["ks"], pairs, num)
            b = oracle.indice_convolution_backward_filter(feat, og, g["ks"], pairs, num, use_ref=True)
            assert np.array_equal(a, b), g
        done += 1


def test_backward_is_the_adjoint_of_forward(oracle):
    """<conv(x), dy> == <x, backward_data(dy)> == <W, backward_filter(x, dy)> in float64 terms."""
    rng = np.random.default_rng(13)
    g = None
    while g is None:
        g = helpers.random_geometry(rng, sub_m=False)
    idx = helpers.random_indices(rng, g["batch"], g["space"], g["n"])
    pairs, _, num, n_out = oracle.get_indice_pairs(idx, g["batch"], g["pad"], g["stride"], g["dil"], g["ks"],
                                                   g["out_space"], 0)
    ci, co = 5, 3
    x = rng.standard_normal((g["n"], ci)).astype(np.float32)
    dy = rng.standard_normal((n_out, co)).astype(np.float32)
    w = rng.standard_normal(tuple(g["ks"]) + (ci, co)).astype(np.float32)
    y = oracle.indice_convolution_forward(x, w, "ARRAY", g["ks"], pairs, num, n_out, co)
    dx = oracle.indice_convolution_backward_data(dy, w, "ARRAY", g["ks"], pairs, num, ci, False)
    dw = oracle.indice_convolution_backward_filter(x, dy, g["ks"], pairs, num)
    lhs = float(np.sum(y.astype(np.float64) * dy))
    assert abs(lhs - float(np.sum(x.astype(np.float64) * dx))) <= 1e-4 * (1 + abs(lhs))
    assert abs(lhs - float(np.sum(w.reshape(dw.shape).astype(np.float64) * dw))) <= 1e-4 * (1 + abs(lhs))


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
