"""Status-code conformance of the C ABI, following the reference's API tests
(test/mlu_op_gtest/api_gtest/src/gtest/get_indice_pairs/*.cpp and
.../indice_convolution_forward/*.cpp).  Every case fails (or succeeds) in the
argument checks, before any launch, so the suite runs without a GPU on a
host-only handle; the buffers handed in are dummy non-NULL addresses.
"""
import ctypes

import pytest

VP = ctypes.c_void_p


@pytest.fixture(scope="module")
def handle(ops):
    h = ops.Handle(0)
    yield h
    h.destroy()


def tdesc(ops, layout, dtype, dims):
    return ops.TensorDesc(layout, dtype, dims)


# ----------------------------------------------------------------- get_indice_pairs

def conv_params(dimNb=5, batch=1, pad=(1, 1, 1), stride=(1, 1, 1), dilation=(1, 1, 1), input_space=(1, 1, 1),
                filter_space=(3, 3, 3), output_space=(3, 3, 3), sub_m=0, transpose=0, inverse=0):
    return dict(dimNb=dimNb, batch=batch, pad=pad, stride=stride, dilation=dilation, input_space=input_space,
                filter_space=filter_space, output_space=output_space, sub_m=sub_m, transpose=transpose,
                inverse=inverse)


def run_get_indice_pairs(ops, handle, params, indices, pairs, out_indices, num):
    """Mirrors get_indice_pairs_general::compute(): Set -> WorkspaceSize -> GetIndicePairs;
    returns the first non-success status, or the status of the final call."""
    lib = ops.lib()
    desc = VP()
    assert lib.mluOpCreateSparseConvolutionDescriptor(ctypes.byref(desc)) == ops.STATUS_SUCCESS
    ia = ops.int_array
    st = lib.mluOpSetSparseConvolutionDescriptor(
        desc, params["dimNb"], params["batch"], ia(params["pad"]), ia(params["stride"]), ia(params["dilation"]),
        ia(params["input_space"]), ia(params["filter_space"]), ia(params["output_space"]), params["sub_m"],
        params["transpose"], params["inverse"])
    try:
        if st != ops.STATUS_SUCCESS:
            return st
        descs = [tdesc(ops, ops.LAYOUT_ARRAY, dt, dims) for dt, dims in (indices, pairs, out_indices, num)]
        size = ctypes.c_size_t(64)
        st = lib.mluOpGetIndicePairsWorkspaceSize(handle.ptr, desc, descs[0].ptr, descs[1].ptr, descs[2].ptr,
                                                  descs[3].ptr, ctypes.byref(size))
        if st != ops.STATUS_SUCCESS:
            return st
        dummy = (ctypes.c_char * 4096)()
        p = VP((ctypes.addressof(dummy) + 15) // 16 * 16)
        return lib.mluOpGetIndicePairs(handle.ptr, desc, descs[0].ptr, p, p, size.value, descs[1].ptr, p,
                                       descs[2].ptr, p, descs[3].ptr, p)
    finally:
        lib.mluOpDestroySparseConvolutionDescriptor(desc)


I32, I16, F32, F16, I64 = 6, 4, 2, 1, 9
GOOD = dict(indices=(I32, (1, 4)), pairs=(I32, (27, 2, 1)), out_indices=(I32, (27, 4)), num=(I32, (27,)))


def gip(ops, handle, params=None, **over):
    t = dict(GOOD)
    t.update(over)
    return run_get_indice_pairs(ops, handle, params or conv_params(), t["indices"], t["pairs"], t["out_indices"],
                                t["num"])


def test_gip_zero_elements_succeed(ops, handle):
    # get_indice_pairs_general.cpp:279-313
    p = conv_params(output_space=(1, 1, 1))
    assert gip(ops, handle, p, indices=(I32, (0, 4)), pairs=(I32, (27, 2, 0)), out_indices=(I32, (1, 4))) == 0
    assert gip(ops, handle, conv_params(), out_indices=(I32, (0, 4))) == 0


def test_gip_bad_dtype(ops, handle):
    # :315-331
    assert gip(ops, handle, indices=(I16, (1, 4)), pairs=(I16, (27, 2, 1)), out_indices=(I16, (27, 4)),
               num=(I16, (27,))) == ops.STATUS_BAD_PARAM


@pytest.mark.parametrize("indices", [(F32, (1, 4)), (I32, (2, 4)), (I32, (1, 5)), (I32, (4,)), (I32, (1, 4, 1))])
def test_gip_bad_indices(ops, handle, indices):
    # :333-355
    assert gip(ops, handle, indices=indices) == ops.STATUS_BAD_PARAM


@pytest.mark.parametrize("pairs", [(I16, (27, 2, 1)), (I32, (28, 2, 1)), (I32, (27, 1, 1)), (I32, (27, 2, 2)),
                                   (I32, (27, 2)), (I32, (27, 2, 1, 1))])
def test_gip_bad_indice_pairs(ops, handle, pairs):
    # :357-381
    assert gip(ops, handle, pairs=pairs) == ops.STATUS_BAD_PARAM


@pytest.mark.parametrize("out_indices", [(F32, (27, 4)), (I32, (28, 4)), (I32, (27, 3)), (I32, (27,)),
                                         (I32, (27, 4, 1))])
def test_gip_bad_out_indices(ops, handle, out_indices):
    # :383-405
    assert gip(ops, handle, out_indices=out_indices) == ops.STATUS_BAD_PARAM


@pytest.mark.parametrize("num", [(I16, (27,)), (I32, (28,)), (I32, (27, 1))])
def test_gip_bad_indice_num(ops, handle, num):
    # :407-433
    assert gip(ops, handle, num=num) == ops.STATUS_BAD_PARAM


@pytest.mark.parametrize("params", [
    conv_params(dimNb=4), conv_params(batch=0), conv_params(batch=-1), conv_params(pad=(-1, 1, 1)),
    conv_params(stride=(1, 0, -1)), conv_params(dilation=(1, 0, -1)), conv_params(transpose=1),
    conv_params(inverse=1)])
def test_gip_bad_descriptor_params(ops, handle, params):
    # :435-488 -- rejected by mluOpSetSparseConvolutionDescriptor
    assert gip(ops, handle, params, out_indices=(I32, (1, 4))) == ops.STATUS_BAD_PARAM


def test_gip_more_inputs_than_cells(ops, handle):
    # :490-506
    p = conv_params(filter_space=(1, 1, 1))
    assert gip(ops, handle, p, indices=(I32, (2, 4)), pairs=(I32, (1, 2, 2)), num=(I32, (1,))) == ops.STATUS_BAD_PARAM


def test_gip_kernel_volume_mismatch(ops, handle):
    # :508-524
    p = conv_params(filter_space=(1, 1, 1))
    assert gip(ops, handle, p, pairs=(I32, (2, 2, 1)), num=(I32, (2,))) == ops.STATUS_BAD_PARAM


@pytest.mark.parametrize("params", [conv_params(stride=(2, 1, 1), output_space=(1, 1, 1), sub_m=1),
                                    conv_params(dilation=(1, 1, 2), output_space=(1, 1, 1), sub_m=1)])
def test_gip_subm_needs_unit_stride_and_dilation(ops, handle, params):
    # :526-549
    assert gip(ops, handle, params, out_indices=(I32, (1, 4))) == ops.STATUS_BAD_PARAM


@pytest.mark.parametrize("axis", [0, 1, 2])
def test_gip_stride_and_dilation_both_set(ops, handle, axis):
    # :551-579
    v = [1, 1, 1]
    v[axis] = 2
    assert gip(ops, handle, conv_params(stride=tuple(v), dilation=tuple(v))) == ops.STATUS_BAD_PARAM


def test_gip_subm_space_mismatch(ops, handle):
    # :581-597
    p = conv_params(filter_space=(1, 1, 1), sub_m=1)
    assert gip(ops, handle, p, pairs=(I32, (1, 2, 1)), num=(I32, (1,))) == ops.STATUS_BAD_PARAM


def test_gip_null_sweep(ops, handle):
    # get_indice_pairs.cpp:212-311 and get_indice_pairs_workspace.cpp:144-211
    lib = ops.lib()
    conv = ops.SparseConvDesc(1, (1, 1, 1), (1, 1, 1), (1, 1, 1), (3, 3, 3), (3, 3, 3), (3, 3, 3), 0)
    d = [tdesc(ops, ops.LAYOUT_ARRAY, I32, dims) for dims in ((1, 4), (27, 2, 1), (27, 4), (27,))]
    dummy = (ctypes.c_char * 4096)()
    p = VP(ctypes.addressof(dummy))
    size = ctypes.c_size_t(0)
    ws_args = [handle.ptr, conv.ptr, d[0].ptr, d[1].ptr, d[2].ptr, d[3].ptr, ctypes.byref(size)]
    assert lib.mluOpGetIndicePairsWorkspaceSize(*ws_args) == 0 and size.value > 0
    for i in range(len(ws_args)):
        a = list(ws_args)
        a[i] = None
        assert lib.mluOpGetIndicePairsWorkspaceSize(*a) == ops.STATUS_BAD_PARAM, i
    args = [handle.ptr, conv.ptr, d[0].ptr, p, p, 64, d[1].ptr, p, d[2].ptr, p, d[3].ptr, p]
    for i in (0, 1, 2, 3, 4, 6, 7, 8, 9, 10, 11):
        a = list(args)
        a[i] = None
        assert lib.mluOpGetIndicePairs(*a) == ops.STATUS_BAD_PARAM, i


def test_gip_coordinate_rows_must_be_16_byte_aligned(ops, handle):
    """indices and out_indices rows are moved as single 16-byte words: a pointer that is only
    4-byte aligned is refused in the argument checks instead of faulting on the device."""
    lib = ops.lib()
    p = conv_params()
    desc = VP()
    assert lib.mluOpCreateSparseConvolutionDescriptor(ctypes.byref(desc)) == 0
    ia = ops.int_array
    assert lib.mluOpSetSparseConvolutionDescriptor(desc, 5, 1, ia(p["pad"]), ia(p["stride"]), ia(p["dilation"]),
                                                   ia(p["input_space"]), ia(p["filter_space"]), ia(p["output_space"]),
                                                   0, 0, 0) == 0
    descs = [tdesc(ops, ops.LAYOUT_ARRAY, dt, dims) for dt, dims in
             (GOOD["indices"], GOOD["pairs"], GOOD["out_indices"], GOOD["num"])]
    size = ctypes.c_size_t(0)
    assert lib.mluOpGetIndicePairsWorkspaceSize(handle.ptr, desc, descs[0].ptr, descs[1].ptr, descs[2].ptr,
                                                descs[3].ptr, ctypes.byref(size)) == 0
    dummy = (ctypes.c_char * 4096)()
    good = (ctypes.addressof(dummy) + 15) // 16 * 16
    for which in (3, 9):  # indices, out_indices
        args = [handle.ptr, desc, descs[0].ptr, VP(good), VP(good), max(size.value, 1 << 20), descs[1].ptr, VP(good),
                descs[2].ptr, VP(good), descs[3].ptr, VP(good)]
        args[which] = VP(good + 4)
        assert lib.mluOpGetIndicePairs(*args) == ops.STATUS_BAD_PARAM, which
    lib.mluOpDestroySparseConvolutionDescriptor(desc)


def test_gip_strided_descriptor_not_supported(ops, handle):
    lib = ops.lib()
    conv = ops.SparseConvDesc(1, (1, 1, 1), (1, 1, 1), (1, 1, 1), (3, 3, 3), (3, 3, 3), (3, 3, 3), 0)
    d = [tdesc(ops, ops.LAYOUT_ARRAY, I32, dims) for dims in ((2, 4), (27, 2, 2), (27, 4), (27,))]
    st = lib.mluOpSetTensorDescriptorEx(d[0].ptr, ops.LAYOUT_ARRAY, I32, 2, ops.int_array((2, 4)),
                                        ops.int_array((8, 1)))
    assert st == 0
    size = ctypes.c_size_t(0)
    assert lib.mluOpGetIndicePairsWorkspaceSize(handle.ptr, conv.ptr, d[0].ptr, d[1].ptr, d[2].ptr, d[3].ptr,
                                                ctypes.byref(size)) == ops.STATUS_NOT_SUPPORTED


def test_gip_limits(ops, handle):
    lib = ops.lib()
    size = ctypes.c_size_t(0)
    # more than a million input voxels is accepted (the reference stops at 1,000,000)
    conv = ops.SparseConvDesc(16, (1, 1, 1), (1, 1, 1), (1, 1, 1), (41, 1600, 1408), (3, 3, 3), (41, 1600, 1408), 1)
    L = 2400000
    d = [tdesc(ops, ops.LAYOUT_ARRAY, I32, dims) for dims in ((L, 4), (27, 2, L), (L, 4), (27,))]
    assert lib.mluOpGetIndicePairsWorkspaceSize(handle.ptr, conv.ptr, d[0].ptr, d[1].ptr, d[2].ptr, d[3].ptr,
                                                ctypes.byref(size)) == 0
    cells = 16 * 41 * 1600 * 1408
    # the stated bound: an occupancy table of 8 bytes per 32 cells, 4 bytes per voxel, scan descriptors
    assert 8 * L <= size.value <= cells // 4 + 16 * L + (1 << 20)
    # 2^31 elements in indice_pairs -> NOT_SUPPORTED
    L = 39768216
    d = [tdesc(ops, ops.LAYOUT_ARRAY, I32, dims) for dims in ((L, 4), (27, 2, L), (L, 4), (27,))]
    assert lib.mluOpGetIndicePairsWorkspaceSize(handle.ptr, conv.ptr, d[0].ptr, d[1].ptr, d[2].ptr, d[3].ptr,
                                                ctypes.byref(size)) == ops.STATUS_NOT_SUPPORTED
    # grid with 2^31 cells -> NOT_SUPPORTED
    conv = ops.SparseConvDesc(32, (1, 1, 1), (1, 1, 1), (1, 1, 1), (41, 1600, 1408), (3, 3, 3), (41, 1600, 1408), 1)
    d = [tdesc(ops, ops.LAYOUT_ARRAY, I32, dims) for dims in ((10, 4), (27, 2, 10), (10, 4), (27,))]
    assert lib.mluOpGetIndicePairsWorkspaceSize(handle.ptr, conv.ptr, d[0].ptr, d[1].ptr, d[2].ptr, d[3].ptr,
                                                ctypes.byref(size)) == ops.STATUS_NOT_SUPPORTED


def test_sparse_conv_descriptor_status_codes(ops):
    lib = ops.lib()
    # get_indice_pairs_structs.cpp:31-134
    assert lib.mluOpCreateSparseConvolutionDescriptor(None) == ops.STATUS_NOT_INITIALIZED
    assert lib.mluOpDestroySparseConvolutionDescriptor(None) == ops.STATUS_EXECUTION_FAILED
    n = ctypes.c_int(0)
    assert lib.mluOpGetSparseConvolutionNumActOut(None, ctypes.byref(n)) == ops.STATUS_NOT_INITIALIZED
    conv = ops.SparseConvDesc(1, (0, 0, 0), (1, 1, 1), (1, 1, 1), (3, 3, 3), (3, 3, 3), (1, 1, 1), 0)
    assert lib.mluOpGetSparseConvolutionNumActOut(conv.ptr, None) == ops.STATUS_NOT_INITIALIZED
    assert conv.num_act_out() == 0
    ia = ops.int_array
    assert lib.mluOpSetSparseConvolutionDescriptor(conv.ptr, 5, 1, None, ia((1, 1, 1)), ia((1, 1, 1)),
                                                   ia((1, 1, 1)), ia((1, 1, 1)), ia((1, 1, 1)), 0, 0,
                                                   0) == ops.STATUS_BAD_PARAM
    assert lib.mluOpSetSparseConvolutionDescriptor(conv.ptr, 5, 1, ia((0, 0, 0)), ia((1, 1, 1)), ia((1, 1, 1)),
                                                   ia((0, 1, 1)), ia((1, 1, 1)), ia((1, 1, 1)), 0, 0,
                                                   0) == ops.STATUS_BAD_PARAM


# ----------------------------------------------------- indice_convolution_forward

def run_conv(ops, handle, features, filters, pairs, out, indice_num, num_act_out, inverse=0, sub_m=0,
             filter_layout=3, null_size=False):
    """Mirrors indice_convolution_forward_general::compute(): WorkspaceSize, then the
    convolution; returns the first non-success status."""
    lib = ops.lib()
    d_f = tdesc(ops, ops.LAYOUT_ARRAY, *features)
    d_w = tdesc(ops, filter_layout, *filters)
    d_p = tdesc(ops, ops.LAYOUT_ARRAY, *pairs)
    d_o = tdesc(ops, ops.LAYOUT_ARRAY, *out)
    num = ops.i64_array(indice_num)
    size = ctypes.c_size_t(64)
    st = lib.mluOpGetIndiceConvolutionForwardWorkspaceSize(handle.ptr, d_f.ptr, d_w.ptr, d_p.ptr, d_o.ptr, num,
                                                           num_act_out, inverse, sub_m,
                                                           None if null_size else ctypes.byref(size))
    if st != ops.STATUS_SUCCESS:
        return st
    dummy = (ctypes.c_char * 4096)()
    p = VP(ctypes.addressof(dummy))
    return lib.mluOpIndiceConvolutionForward(handle.ptr, d_f.ptr, p, d_w.ptr, p, d_p.ptr, p, num, num_act_out,
                                             inverse, sub_m, p, size.value, d_o.ptr, p)


CONV_GOOD = dict(features=(F32, (2, 3)), filters=(F32, (5, 1, 2, 2, 3)), pairs=(I32, (4, 2, 2)),
                 out=(F32, (9, 5)), indice_num=[1, 1, 1, 1], num_act_out=9)


def conv(ops, handle, **over):
    a = dict(CONV_GOOD)
    a.update(over)
    return run_conv(ops, handle, **a)


def test_conv_zero_elements_succeed(ops, handle):
    # indice_convolution_forward_general.cpp:246-276
    assert conv(ops, handle, features=(F32, (0, 3)), pairs=(I32, (4, 2, 0)), indice_num=[0, 0, 0, 0]) == 0
    assert conv(ops, handle, out=(F32, (0, 5)), num_act_out=0) == 0
    # the size pointer is only checked after the zero-element return (reference :600-609)
    assert conv(ops, handle, out=(F32, (0, 5)), num_act_out=0, null_size=True) == 0
    assert conv(ops, handle, null_size=True) == ops.STATUS_BAD_PARAM


@pytest.mark.parametrize("features", [(F16, (2, 3)), (F32, (3, 2, 1)), (F32, (2, 4)), (F32, (3, 3))])
def test_conv_bad_features(ops, handle, features):
    # :278-297
    assert conv(ops, handle, features=features) == ops.STATUS_BAD_PARAM


def test_conv_bad_filters_dtype(ops, handle):
    # :299-314
    assert conv(ops, handle, filters=(F16, (5, 1, 2, 2, 3))) == ops.STATUS_BAD_PARAM


def test_conv_bad_filters_rank_or_layout(ops, handle):
    # :316-332
    assert conv(ops, handle, filters=(F32, (5, 1, 2, 2))) == ops.STATUS_NOT_SUPPORTED
    assert conv(ops, handle, filter_layout=ops.LAYOUT_NHWC) == ops.STATUS_NOT_SUPPORTED


@pytest.mark.parametrize("pairs", [(I64, (4, 2, 2)), (I32, (4, 2)), (I32, (5, 2, 2)), (I32, (4, 3, 2)),
                                   (I32, (4, 2, 3))])
def test_conv_bad_indice_pairs(ops, handle, pairs):
    # :334-356
    assert conv(ops, handle, pairs=pairs) == ops.STATUS_BAD_PARAM


@pytest.mark.parametrize("out", [(F16, (9, 5)), (F32, (9, 5, 5)), (F32, (10, 5)), (F32, (9, 6))])
def test_conv_bad_features_out(ops, handle, out):
    # :358-378
    assert conv(ops, handle, out=out) == ops.STATUS_BAD_PARAM


@pytest.mark.parametrize("over", [dict(indice_num=[-1, 1, 1, 1]), dict(indice_num=[1, 1, 4, 1]),
                                  dict(num_act_out=19), dict(inverse=2), dict(sub_m=2)])
def test_conv_bad_params(ops, handle, over):
    # :380-403
    assert conv(ops, handle, **over) == ops.STATUS_BAD_PARAM


def test_conv_inverse_not_supported(ops, handle):
    # :405-419
    assert conv(ops, handle, inverse=1) == ops.STATUS_NOT_SUPPORTED


def test_conv_large_tensors_not_supported(ops, handle):
    # :421-490
    assert conv(ops, handle, features=(F32, (21474837, 100)), filters=(F32, (5, 1, 2, 2, 100)),
                pairs=(I32, (4, 2, 21474837))) == ops.STATUS_NOT_SUPPORTED
    assert conv(ops, handle, features=(F32, (2, 3000)), filters=(F32, (89479, 2, 2, 2, 3000)),
                out=(F32, (9, 89479)), indice_num=[1] * 8) == ops.STATUS_NOT_SUPPORTED
    assert conv(ops, handle, features=(F32, (89478486, 2)), filters=(F32, (5, 3, 2, 2, 2)),
                pairs=(I32, (12, 2, 89478486)), indice_num=[1] * 12) == ops.STATUS_NOT_SUPPORTED
    assert conv(ops, handle, filters=(F32, (500, 1, 2, 2, 3)), out=(F32, (4294968, 500)),
                num_act_out=4294968) == ops.STATUS_NOT_SUPPORTED


def test_conv_null_sweep(ops, handle):
    # indice_convolution_forward.cpp:232-339, indice_convolution_forward_workspace.cpp:145-212
    lib = ops.lib()
    d_f = tdesc(ops, ops.LAYOUT_ARRAY, F32, (2, 3))
    d_w = tdesc(ops, ops.LAYOUT_NDHWC, F32, (5, 1, 2, 2, 3))
    d_p = tdesc(ops, ops.LAYOUT_ARRAY, I32, (4, 2, 2))
    d_o = tdesc(ops, ops.LAYOUT_ARRAY, F32, (9, 5))
    num = ops.i64_array([1, 1, 1, 1])
    size = ctypes.c_size_t(0)
    ws = [handle.ptr, d_f.ptr, d_w.ptr, d_p.ptr, d_o.ptr, num, 9, 0, 0, ctypes.byref(size)]
    assert lib.mluOpGetIndiceConvolutionForwardWorkspaceSize(*ws) == 0 and size.value > 0
    for i in (0, 1, 2, 3, 4, 5, 9):
        a = list(ws)
        a[i] = None
        assert lib.mluOpGetIndiceConvolutionForwardWorkspaceSize(*a) == ops.STATUS_BAD_PARAM, i
    dummy = (ctypes.c_char * 4096)()
    p = VP(ctypes.addressof(dummy))
    args = [handle.ptr, d_f.ptr, p, d_w.ptr, p, d_p.ptr, p, num, 9, 0, 0, p, 64, d_o.ptr, p]
    for i in (0, 1, 2, 3, 4, 5, 6, 7, 11, 13, 14):
        a = list(args)
        a[i] = None
        assert lib.mluOpIndiceConvolutionForward(*a) == ops.STATUS_BAD_PARAM, i


def test_conv_accepts_more_than_a_million_rows(ops, handle):
    L = 1600000
    d_f = tdesc(ops, ops.LAYOUT_ARRAY, F16, (L, 128))
    d_w = tdesc(ops, ops.LAYOUT_ARRAY, F16, (3, 3, 3, 128, 128))
    d_p = tdesc(ops, ops.LAYOUT_ARRAY, I32, (27, 2, L))
    d_o = tdesc(ops, ops.LAYOUT_ARRAY, F16, (L, 128))
    size = ctypes.c_size_t(0)
    st = ops.lib().mluOpGetIndiceConvolutionForwardWorkspaceSize(
        handle.ptr, d_f.ptr, d_w.ptr, d_p.ptr, d_o.ptr, ops.i64_array([L] * 27), L, 0, 1, ctypes.byref(size))
    assert st == 0 and size.value >= 27 * L * 4


# --------------------------------------------------------------- core entry points

def test_handle_and_queue(ops):
    lib = ops.lib()
    assert lib.mluOpCreate(None) == ops.STATUS_BAD_PARAM
    assert lib.mluOpDestroy(None) == ops.STATUS_BAD_PARAM
    h = ops.Handle(0)
    q = VP(123)
    assert lib.mluOpGetQueue(h.ptr, ctypes.byref(q)) == 0 and not q.value
    assert lib.mluOpSetQueue(None, None) == ops.STATUS_BAD_PARAM
    assert lib.mluOpGetQueue(h.ptr, None) == ops.STATUS_BAD_PARAM
    mode = ctypes.c_int(0)
    assert lib.mluOpGetAtomicsMode(h.ptr, ctypes.byref(mode)) == 0 and mode.value == 1
    assert lib.mluOpSetAtomicsMode(h.ptr, 2) == 0
    assert lib.mluOpSetAtomicsMode(h.ptr, 7) == ops.STATUS_BAD_PARAM
    major, minor, patch = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    lib.mluOpGetLibVersion(ctypes.byref(major), ctypes.byref(minor), ctypes.byref(patch))
    assert (major.value, minor.value, patch.value) == (1, 11, 1)
    h.destroy()


def test_tensor_descriptor_round_trip(ops):
    lib = ops.lib()
    assert lib.mluOpCreateTensorDescriptor(None) == ops.STATUS_BAD_PARAM
    assert lib.mluOpDestroyTensorDescriptor(None) == ops.STATUS_BAD_PARAM
    d = ops.TensorDesc(ops.LAYOUT_NDHWC, F16, (5, 1, 2, 2, 3))
    assert lib.mluOpGetTensorElementNum(d.ptr) == 60
    layout, dtype, n = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    dims, strides = (ctypes.c_int * 8)(), (ctypes.c_int * 8)()
    assert lib.mluOpGetTensorDescriptorEx(d.ptr, ctypes.byref(layout), ctypes.byref(dtype), ctypes.byref(n), dims,
                                          strides) == 0
    assert (layout.value, dtype.value, n.value) == (ops.LAYOUT_NDHWC, F16, 5)
    assert list(dims)[:5] == [5, 1, 2, 2, 3] and list(strides)[:5] == [12, 12, 6, 3, 1]
    # more than MLUOP_DIM_MAX dims go to the heap
    assert lib.mluOpSetTensorDescriptor(d.ptr, ops.LAYOUT_ARRAY, F32, 10, ops.int_array([2] * 10)) == 0
    assert lib.mluOpGetTensorElementNum(d.ptr) == 1024
    assert lib.mluOpSetTensorDescriptor(d.ptr, ops.LAYOUT_ARRAY, F32, 2, None) == ops.STATUS_BAD_PARAM
    assert lib.mluOpSetTensorDescriptor(d.ptr, -1, F32, 2, ops.int_array([1, 2])) == ops.STATUS_BAD_PARAM
    assert lib.mluOpResetTensorDescriptor(d.ptr) == 0 and lib.mluOpGetTensorElementNum(d.ptr) == 0
    size = ctypes.c_size_t(0)
    assert lib.mluOpGetSizeOfDataType(F16, ctypes.byref(size)) == 0 and size.value == 2
    assert lib.mluOpGetSizeOfDataType(0, ctypes.byref(size)) == ops.STATUS_BAD_PARAM
    assert lib.mluOpGetErrorString(7) == b"MLUOP_STATUS_NOT_SUPPORTED"


def test_descriptor_pool_recycles(ops):
    lib = ops.lib()
    seen = set()
    for _ in range(500):
        p = VP()
        assert lib.mluOpCreateTensorDescriptor(ctypes.byref(p)) == 0
        seen.add(p.value)
        assert lib.mluOpDestroyTensorDescriptor(p) == 0
    assert len(seen) < 10


# ------------------------------------------------- neighbour-table fast path (extension)

def test_table_entry_points_argument_checks(ops, handle):
    lib = ops.lib()
    d_p = tdesc(ops, ops.LAYOUT_ARRAY, I32, (4, 2, 2))
    size = ctypes.c_size_t(0)
    assert lib.mluOpGetIndiceNeighbourTableSize(handle.ptr, d_p.ptr, 9, ctypes.byref(size)) == 0
    assert size.value == 4 * 512 * 4  # K rows padded to 512 output rows
    for a in ([None, d_p.ptr, 9, ctypes.byref(size)], [handle.ptr, None, 9, ctypes.byref(size)],
              [handle.ptr, d_p.ptr, 9, None], [handle.ptr, d_p.ptr, -1, ctypes.byref(size)]):
        assert lib.mluOpGetIndiceNeighbourTableSize(*a) == ops.STATUS_BAD_PARAM
    bad = tdesc(ops, ops.LAYOUT_ARRAY, I32, (4, 3, 2))
    assert lib.mluOpGetIndiceNeighbourTableSize(handle.ptr, bad.ptr, 9, ctypes.byref(size)) == ops.STATUS_BAD_PARAM
    dummy = (ctypes.c_char * 16384)()
    p = VP((ctypes.addressof(dummy) + 15) // 16 * 16)
    num = ops.i64_array([1, 1, 1, 1])
    args = [handle.ptr, d_p.ptr, p, num, 9, p, 8192]
    assert lib.mluOpBuildIndiceNeighbourTable(*args) == ops.STATUS_EXECUTION_FAILED  # checks pass; host-only handle
    for i in (0, 1, 2, 3, 5):
        a = list(args)
        a[i] = None
        assert lib.mluOpBuildIndiceNeighbourTable(*a) == ops.STATUS_BAD_PARAM, i
    assert lib.mluOpBuildIndiceNeighbourTable(handle.ptr, d_p.ptr, p, num, 9, p, 100) == ops.STATUS_BAD_PARAM
    assert lib.mluOpBuildIndiceNeighbourTable(handle.ptr, d_p.ptr, p, ops.i64_array([3, 1, 1, 1]), 9, p,
                                              8192) == ops.STATUS_BAD_PARAM
    big = tdesc(ops, ops.LAYOUT_ARRAY, I32, (129, 2, 2))
    assert lib.mluOpBuildIndiceNeighbourTable(handle.ptr, big.ptr, p, ops.i64_array([1] * 129), 9, p,
                                              1 << 20) == ops.STATUS_NOT_SUPPORTED
    # the convolution from a table: the forward entry point's checks, plus the table size
    d_f = tdesc(ops, ops.LAYOUT_ARRAY, F32, (2, 3))
    d_w = tdesc(ops, ops.LAYOUT_NDHWC, F32, (5, 1, 2, 2, 3))
    d_o = tdesc(ops, ops.LAYOUT_ARRAY, F32, (9, 5))
    ws = ctypes.c_size_t(0)
    assert lib.mluOpGetIndiceConvolutionForwardFromTableWorkspaceSize(handle.ptr, d_f.ptr, d_w.ptr, d_p.ptr, d_o.ptr,
                                                                      num, 9, 0, 0, ctypes.byref(ws)) == 0
    full = ctypes.c_size_t(0)
    assert lib.mluOpGetIndiceConvolutionForwardWorkspaceSize(handle.ptr, d_f.ptr, d_w.ptr, d_p.ptr, d_o.ptr, num, 9,
                                                             0, 0, ctypes.byref(full)) == 0
    assert 0 < ws.value < full.value  # the table no longer lives in the workspace
    conv = [handle.ptr, d_f.ptr, p, d_w.ptr, p, d_p.ptr, p, 8192, num, 9, 0, 0, p, 8192, d_o.ptr, p]
    assert lib.mluOpIndiceConvolutionForwardFromTable(*conv) == ops.STATUS_EXECUTION_FAILED
    for i in (0, 1, 2, 3, 4, 5, 6, 8, 12, 14, 15):
        a = list(conv)
        a[i] = None
        assert lib.mluOpIndiceConvolutionForwardFromTable(*a) == ops.STATUS_BAD_PARAM, i
    odd = list(conv)
    odd[6] = VP(p.value + 4)  # the table is read 16 bytes at a time
    assert lib.mluOpIndiceConvolutionForwardFromTable(*odd) == ops.STATUS_BAD_PARAM
    small = list(conv)
    small[7] = 100
    assert lib.mluOpIndiceConvolutionForwardFromTable(*small) == ops.STATUS_BAD_PARAM
    inv = list(conv)
    inv[10] = 1
    assert lib.mluOpIndiceConvolutionForwardFromTable(*inv) == ops.STATUS_NOT_SUPPORTED
