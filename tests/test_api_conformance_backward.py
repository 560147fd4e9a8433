"""Status-code conformance of the two backward operators, following the
reference's API tests (test/mlu_op_gtest/api_gtest/src/gtest/
indice_convolution_backward_data/*.cpp and .../indice_convolution_backward_filter/*.cpp).
Every case is decided by the argument checks, before any launch, so the suite
runs without a GPU on a host-only handle; buffers are dummy non-NULL addresses.
"""
import ctypes

import pytest

VP = ctypes.c_void_p
F16, F32, I16, I32, I64, CF32 = 1, 2, 4, 6, 9, 16
NCHW, NHWC, HWCN, NDHWC, ARRAY, NCDHW, TNC, NTC, NC, NLC = 0, 1, 2, 3, 4, 5, 6, 7, 8, 9


@pytest.fixture(scope="module")
def handle(ops):
    h = ops.Handle(0)
    yield h
    h.destroy()


def dummy():
    buf = (ctypes.c_char * 4096)()
    return buf, VP(ctypes.addressof(buf))


# --------------------------------------------------- indice_convolution_backward_data

BD_GOOD = dict(output_grad=(ARRAY, F32, (10, 10)), filters=(HWCN, F32, (3, 3, 21, 10)),
               pairs=(ARRAY, I32, (9, 2, 10)), input_grad=(ARRAY, F32, (10, 21)), indice_num=[10] * 9, inverse=0,
               sub_m=0)


def run_bd(ops, handle, output_grad, filters, pairs, input_grad, indice_num, inverse, sub_m):
    """Mirrors indice_convolution_backward_data_general::compute(): the workspace query, then the operator."""
    lib = ops.lib()
    descs = [ops.TensorDesc(*t) for t in (output_grad, filters, pairs, input_grad)]
    d_g, d_w, d_p, d_i = (d.ptr for d in descs)
    num = ops.i64_array(indice_num)
    size = ctypes.c_size_t(64)
    st = lib.mluOpGetIndiceConvolutionBackwardDataWorkspaceSize(handle.ptr, d_g, d_w, d_p, d_i, num, inverse,
                                                                ctypes.byref(size))
    if st == ops.STATUS_SUCCESS:
        keep, p = dummy()
        st = lib.mluOpIndiceConvolutionBackwardData(handle.ptr, d_g, p, d_w, p, d_p, p, num, inverse, sub_m, p,
                                                    max(size.value, 64), d_i, p)
    for d in descs:
        d.destroy()
    return st


def bd(ops, handle, **over):
    a = dict(BD_GOOD)
    a.update(over)
    return run_bd(ops, handle, **a)


def test_bd_zero_elements_succeed(ops, handle):
    # indice_convolution_backward_data_general.cpp: zero_element_Y_0 ... zero_element_L_0
    zeros = [0] * 9
    assert bd(ops, handle, output_grad=(ARRAY, F32, (0, 10)), indice_num=zeros) == 0
    assert bd(ops, handle, output_grad=(ARRAY, F32, (10, 0)), filters=(HWCN, F32, (3, 3, 21, 0))) == 0
    assert bd(ops, handle, filters=(HWCN, F32, (3, 3, 0, 10)), input_grad=(ARRAY, F32, (10, 0))) == 0
    assert bd(ops, handle, filters=(HWCN, F32, (0, 3, 21, 10)), pairs=(ARRAY, I32, (0, 2, 10))) == 0
    assert bd(ops, handle, pairs=(ARRAY, I32, (9, 2, 0)), input_grad=(ARRAY, F32, (0, 21)), indice_num=zeros) == 0


def test_bd_bad_dtype(ops, handle):
    assert bd(ops, handle, output_grad=(ARRAY, I32, (10, 10)), filters=(HWCN, I32, (3, 3, 21, 10)),
              input_grad=(ARRAY, I32, (10, 21))) == ops.STATUS_BAD_PARAM


@pytest.mark.parametrize("t", [(ARRAY, F16, (10, 10)), (ARRAY, I32, (10, 10)), (ARRAY, F32, (10, 9)),
                               (ARRAY, F32, (10,)), (ARRAY, F32, (10, 10, 10))])
def test_bd_bad_output_grad(ops, handle, t):
    assert bd(ops, handle, output_grad=t) == ops.STATUS_BAD_PARAM


@pytest.mark.parametrize("t", [(HWCN, F16, (3, 3, 21, 10)), (HWCN, I32, (3, 3, 21, 10)), (HWCN, F32, (2, 3, 21, 10)),
                               (HWCN, F32, (3, 2, 21, 10)), (HWCN, F32, (3, 3, 20, 10)), (HWCN, F32, (3, 3, 21, 9)),
                               (HWCN, F32, (3, 21, 10)), (HWCN, F32, (3, 3, 3, 3, 21, 10)),
                               (TNC, F32, (3, 3, 21, 10)), (NTC, F32, (3, 3, 21, 10)), (NC, F32, (3, 3, 21, 10)),
                               (NLC, F32, (3, 3, 21, 10))])
def test_bd_bad_filters(ops, handle, t):
    assert bd(ops, handle, filters=t) == ops.STATUS_BAD_PARAM


@pytest.mark.parametrize("t", [(ARRAY, F32, (9, 2, 10)), (ARRAY, I16, (9, 2, 10)), (ARRAY, I32, (8, 2, 10)),
                               (ARRAY, I32, (9, 1, 10)), (ARRAY, I32, (9, 2, 9)), (ARRAY, I32, (9, 2)),
                               (ARRAY, I32, (9, 2, 10, 1))])
def test_bd_bad_indice_pairs(ops, handle, t):
    assert bd(ops, handle, pairs=t) == ops.STATUS_BAD_PARAM


@pytest.mark.parametrize("t", [(ARRAY, F16, (10, 21)), (ARRAY, I32, (10, 21)), (ARRAY, F32, (9, 21)),
                               (ARRAY, F32, (10, 20)), (ARRAY, F32, (10,)), (ARRAY, F32, (10, 21, 1))])
def test_bd_bad_input_grad(ops, handle, t):
    assert bd(ops, handle, input_grad=t) == ops.STATUS_BAD_PARAM


@pytest.mark.parametrize("over", [dict(indice_num=[-1] + [10] * 8), dict(indice_num=[20] + [10] * 8),
                                  dict(inverse=-1), dict(sub_m=-1), dict(sub_m=2)])
def test_bd_bad_params(ops, handle, over):
    assert bd(ops, handle, **over) == ops.STATUS_BAD_PARAM


def test_bd_inverse_not_supported(ops, handle):
    assert bd(ops, handle, inverse=1) == ops.STATUS_NOT_SUPPORTED


def test_bd_subm_rules(ops, handle):
    # bad_L_Y: sub_m needs as many output_grad rows as input_grad rows
    assert bd(ops, handle, output_grad=(ARRAY, F32, (9, 10)), indice_num=[1] * 9, sub_m=1) == ops.STATUS_BAD_PARAM
    # the centre offset must hold the largest count; kernel extents must be odd
    assert bd(ops, handle, indice_num=[5, 5, 5, 5, 4, 5, 5, 5, 5], sub_m=1) == ops.STATUS_BAD_PARAM
    assert bd(ops, handle, filters=(HWCN, F32, (2, 2, 21, 10)), pairs=(ARRAY, I32, (4, 2, 10)),
              indice_num=[1, 1, 10, 1], sub_m=1) == ops.STATUS_BAD_PARAM


def test_bd_accepts_every_filter_layout(ops, handle):
    """All six layouts of the reference pass the checks (a host-only handle then refuses to launch)."""
    for t in [(HWCN, F32, (3, 3, 21, 10)), (NHWC, F32, (10, 3, 3, 21)), (NCHW, F32, (10, 21, 3, 3)),
              (ARRAY, F32, (3, 3, 21, 10))]:
        assert bd(ops, handle, filters=t) == ops.STATUS_EXECUTION_FAILED, t
    for t in [(NDHWC, F32, (10, 1, 3, 3, 21)), (NCDHW, F32, (10, 21, 1, 3, 3)), (ARRAY, F32, (1, 3, 3, 21, 10))]:
        assert bd(ops, handle, filters=t) == ops.STATUS_EXECUTION_FAILED, t


def test_bd_null_sweep(ops, handle):
    # indice_convolution_backward_data.cpp (api test) :192-296 and the workspace test
    lib = ops.lib()
    descs = [ops.TensorDesc(*BD_GOOD[k]) for k in ("output_grad", "filters", "pairs", "input_grad")]
    d_g, d_w, d_p, d_i = (d.ptr for d in descs)
    num = ops.i64_array([10] + [0] * 8)
    size = ctypes.c_size_t(0)
    ws = [handle.ptr, d_g, d_w, d_p, d_i, num, 0, ctypes.byref(size)]
    assert lib.mluOpGetIndiceConvolutionBackwardDataWorkspaceSize(*ws) == 0 and size.value > 0
    for i in (0, 1, 2, 3, 4, 5, 7):
        a = list(ws)
        a[i] = None
        assert lib.mluOpGetIndiceConvolutionBackwardDataWorkspaceSize(*a) == ops.STATUS_BAD_PARAM, i
    keep, p = dummy()
    args = [handle.ptr, d_g, p, d_w, p, d_p, p, num, 0, 0, p, 64, d_i, p]
    for i in (0, 1, 2, 3, 4, 5, 6, 7, 10, 12, 13):
        a = list(args)
        a[i] = None
        assert lib.mluOpIndiceConvolutionBackwardData(*a) == ops.STATUS_BAD_PARAM, i
    for d in descs:
        d.destroy()


# ------------------------------------------------- indice_convolution_backward_filter

BF_GOOD = dict(features=(ARRAY, F32, (3, 5)), output_grad=(ARRAY, F32, (3, 3)), pairs=(ARRAY, I32, (9, 2, 3)),
               filters_grad=(ARRAY, F32, (3, 3, 5, 3)), indice_num=[1, 2, 3, 3, 3, 3, 2, 1, 0], inverse=0, sub_m=0)


def run_bf(ops, handle, features, output_grad, pairs, filters_grad, indice_num, inverse, sub_m):
    lib = ops.lib()
    descs = [ops.TensorDesc(*t) for t in (features, output_grad, pairs, filters_grad)]
    d_f, d_g, d_p, d_w = (d.ptr for d in descs)
    num = ops.i64_array(indice_num)
    size = ctypes.c_size_t(1)
    st = lib.mluOpGetIndiceConvolutionBackwardFilterWorkspaceSize(handle.ptr, d_f, d_g, d_p, d_w, num, inverse,
                                                                  sub_m, ctypes.byref(size))
    if st == ops.STATUS_SUCCESS:
        keep, p = dummy()
        st = lib.mluOpIndiceConvolutionBackwardFilter(handle.ptr, d_f, p, d_g, p, d_p, p, num, inverse, sub_m, p,
                                                      max(size.value, 1), d_w, p)
    for d in descs:
        d.destroy()
    return st


def bf(ops, handle, **over):
    a = dict(BF_GOOD)
    a.update(over)
    return run_bf(ops, handle, **a)


def test_bf_zero_elements_succeed(ops, handle):
    # the reference's cases pass counts 1..9 with three rows: a zero-element tensor returns before they matter
    num = list(range(1, 10))
    assert bf(ops, handle, features=(ARRAY, F32, (0, 5)), pairs=(ARRAY, I32, (9, 2, 0)), indice_num=num) == 0
    assert bf(ops, handle, output_grad=(ARRAY, F32, (0, 3)), indice_num=num) == 0
    assert bf(ops, handle, pairs=(ARRAY, I32, (0, 2, 3)), filters_grad=(ARRAY, F32, (3, 0, 5, 3)),
              indice_num=num) == 0


def test_bf_bad_dtype(ops, handle):
    assert bf(ops, handle, features=(ARRAY, CF32, (3, 5)), output_grad=(ARRAY, CF32, (3, 3)),
              filters_grad=(ARRAY, CF32, (3, 3, 5, 3))) == ops.STATUS_BAD_PARAM


@pytest.mark.parametrize("t", [(ARRAY, F16, (3, 5)), (ARRAY, F32, (3, 5, 1)), (ARRAY, F32, (3, 15)),
                               (ARRAY, F32, (13, 3))])
def test_bf_bad_features(ops, handle, t):
    assert bf(ops, handle, features=t) == ops.STATUS_BAD_PARAM


@pytest.mark.parametrize("t", [(ARRAY, I64, (9, 2, 3)), (ARRAY, I32, (11, 2, 3)), (ARRAY, I32, (9, 1, 3)),
                               (ARRAY, I32, (9, 2, 3, 4))])
def test_bf_bad_indice_pairs(ops, handle, t):
    assert bf(ops, handle, pairs=t) == ops.STATUS_BAD_PARAM


@pytest.mark.parametrize("t", [(ARRAY, F16, (3, 3)), (ARRAY, F32, (3, 3, 3)), (ARRAY, F32, (3, 4))])
def test_bf_bad_output_grad(ops, handle, t):
    assert bf(ops, handle, output_grad=t) == ops.STATUS_BAD_PARAM


@pytest.mark.parametrize("t", [(ARRAY, F16, (3, 3, 5, 3)), (ARRAY, F32, (3, 3, 5)), (ARRAY, F32, (3, 3, 15, 3)),
                               (ARRAY, F32, (3, 3, 5, 13))])
def test_bf_bad_filters_grad(ops, handle, t):
    assert bf(ops, handle, filters_grad=t) == ops.STATUS_BAD_PARAM


def test_bf_bad_inverse_and_counts(ops, handle):
    assert bf(ops, handle, inverse=1) == ops.STATUS_BAD_PARAM
    assert bf(ops, handle, indice_num=[4] + [0] * 8) == ops.STATUS_BAD_PARAM
    assert bf(ops, handle, indice_num=[-1] + [0] * 8) == ops.STATUS_BAD_PARAM


def test_bf_large_tensors_not_supported(ops, handle):
    assert bf(ops, handle, features=(ARRAY, F32, (1147483648, 5))) == ops.STATUS_NOT_SUPPORTED
    assert bf(ops, handle, output_grad=(ARRAY, F32, (715827883, 3))) == ops.STATUS_NOT_SUPPORTED
    assert bf(ops, handle, pairs=(ARRAY, I32, (715827883, 2, 3))) == ops.STATUS_NOT_SUPPORTED
    assert bf(ops, handle, filters_grad=(ARRAY, F32, (47721859, 3, 5, 3))) == ops.STATUS_NOT_SUPPORTED


def test_bf_passes_checks_then_needs_a_device(ops, handle):
    assert bf(ops, handle) == ops.STATUS_EXECUTION_FAILED
    assert bf(ops, handle, filters_grad=(ARRAY, F32, (1, 3, 3, 5, 3))) == ops.STATUS_EXECUTION_FAILED


def test_bf_null_sweep(ops, handle):
    # indice_convolution_backward_filter.cpp (api test) :228-340
    lib = ops.lib()
    descs = [ops.TensorDesc(*BF_GOOD[k]) for k in ("features", "output_grad", "pairs", "filters_grad")]
    d_f, d_g, d_p, d_w = (d.ptr for d in descs)
    num = ops.i64_array(BF_GOOD["indice_num"])
    size = ctypes.c_size_t(0)
    ws = [handle.ptr, d_f, d_g, d_p, d_w, num, 0, 0, ctypes.byref(size)]
    assert lib.mluOpGetIndiceConvolutionBackwardFilterWorkspaceSize(*ws) == 0 and size.value > 0
    for i in (0, 1, 2, 3, 4, 5, 8):
        a = list(ws)
        a[i] = None
        assert lib.mluOpGetIndiceConvolutionBackwardFilterWorkspaceSize(*a) == ops.STATUS_BAD_PARAM, i
    keep, p = dummy()
    args = [handle.ptr, d_f, p, d_g, p, d_p, p, num, 0, 0, p, 64, d_w, p]
    for i in (0, 1, 2, 3, 4, 5, 6, 7, 10, 12, 13):
        a = list(args)
        a[i] = None
        assert lib.mluOpIndiceConvolutionBackwardFilter(*a) == ops.STATUS_BAD_PARAM, i
    for d in descs:
        d.destroy()


# ------------------------------------------------- neighbour-table fast path of the gradients (extensions)

def test_gradient_table_entry_points_argument_checks(ops, handle):
    lib = ops.lib()
    keep = (ctypes.c_char * 65536)()
    p = VP((ctypes.addressof(keep) + 15) // 16 * 16)
    # the input table: [K][L padded to 512] int32
    d_p = ops.TensorDesc(ARRAY, I32, (9, 2, 10))
    size = ctypes.c_size_t(0)
    assert lib.mluOpGetIndiceInputNeighbourTableSize(handle.ptr, d_p.ptr, ctypes.byref(size)) == 0
    assert size.value == 9 * 512 * 4
    for a in ([None, d_p.ptr, ctypes.byref(size)], [handle.ptr, None, ctypes.byref(size)], [handle.ptr, d_p.ptr, None]):
        assert lib.mluOpGetIndiceInputNeighbourTableSize(*a) == ops.STATUS_BAD_PARAM
    num = ops.i64_array([10] * 9)
    build = [handle.ptr, d_p.ptr, p, num, 10, p, size.value]
    assert lib.mluOpBuildIndiceInputNeighbourTable(*build) == ops.STATUS_EXECUTION_FAILED  # checks pass; host-only handle
    for i in (0, 1, 2, 3, 5):
        a = list(build)
        a[i] = None
        assert lib.mluOpBuildIndiceInputNeighbourTable(*a) == ops.STATUS_BAD_PARAM, i
    assert lib.mluOpBuildIndiceInputNeighbourTable(handle.ptr, d_p.ptr, p, num, 10, p, 100) == ops.STATUS_BAD_PARAM
    assert lib.mluOpBuildIndiceInputNeighbourTable(handle.ptr, d_p.ptr, p, num, 10, VP(p.value + 4),
                                                   size.value) == ops.STATUS_BAD_PARAM
    assert lib.mluOpBuildIndiceInputNeighbourTable(handle.ptr, d_p.ptr, p, ops.i64_array([11] + [10] * 8), 10, p,
                                                   size.value) == ops.STATUS_BAD_PARAM
    # the input gradient from it: the reference-shaped entry point's checks, plus table and workspace sizes
    descs = [ops.TensorDesc(*BD_GOOD[k]) for k in ("output_grad", "filters", "pairs", "input_grad")]
    d_g, d_w, d_pp, d_i = (d.ptr for d in descs)
    ws = ctypes.c_size_t(0)
    assert lib.mluOpGetIndiceConvolutionBackwardDataFromTableWorkspaceSize(handle.ptr, d_g, d_w, d_pp, d_i, num, 0,
                                                                           ctypes.byref(ws)) == 0
    full = ctypes.c_size_t(0)
    assert lib.mluOpGetIndiceConvolutionBackwardDataWorkspaceSize(handle.ptr, d_g, d_w, d_pp, d_i, num, 0,
                                                                  ctypes.byref(full)) == 0
    assert 0 < ws.value < full.value  # the table no longer lives in the workspace
    args = [handle.ptr, d_g, p, d_w, p, d_pp, p, size.value, num, 0, 0, p, ws.value, d_i, p]
    assert lib.mluOpIndiceConvolutionBackwardDataFromTable(*args) == ops.STATUS_EXECUTION_FAILED
    for i in (0, 1, 2, 3, 4, 5, 6, 8, 11, 13, 14):
        a = list(args)
        a[i] = None
        assert lib.mluOpIndiceConvolutionBackwardDataFromTable(*a) == ops.STATUS_BAD_PARAM, i
    odd = list(args)
    odd[6] = VP(p.value + 4)  # the table is read 16 bytes at a time
    assert lib.mluOpIndiceConvolutionBackwardDataFromTable(*odd) == ops.STATUS_BAD_PARAM
    small = list(args)
    small[7] = 100
    assert lib.mluOpIndiceConvolutionBackwardDataFromTable(*small) == ops.STATUS_BAD_PARAM
    inv = list(args)
    inv[9] = 1
    assert lib.mluOpIndiceConvolutionBackwardDataFromTable(*inv) == ops.STATUS_NOT_SUPPORTED
    # the input gradient of a centred submanifold layer from its FORWARD table, offsets mirrored
    assert lib.mluOpIndiceConvolutionBackwardDataFromForwardTable(*args) == ops.STATUS_BAD_PARAM  # sub_m must be 1
    sub = list(args)
    sub[10] = 1
    # float tensors are not the tensor-memory kernel's: an answer, the caller uses the input table
    assert lib.mluOpIndiceConvolutionBackwardDataFromForwardTable(*sub) == ops.STATUS_NOT_SUPPORTED
    for i in (0, 1, 2, 3, 4, 5, 6, 8, 11, 13, 14):
        a = list(sub)
        a[i] = None
        assert lib.mluOpIndiceConvolutionBackwardDataFromForwardTable(*a) == ops.STATUS_BAD_PARAM, i
    hd = [ops.TensorDesc(ARRAY, F16, (10, 16)), ops.TensorDesc(HWCN, F16, (3, 3, 24, 16)),
          ops.TensorDesc(ARRAY, I32, (9, 2, 10)), ops.TensorDesc(ARRAY, F16, (10, 24))]
    hws = ctypes.c_size_t(0)
    assert lib.mluOpGetIndiceConvolutionBackwardDataFromTableWorkspaceSize(handle.ptr, hd[0].ptr, hd[1].ptr, hd[2].ptr,
                                                                           hd[3].ptr, num, 0, ctypes.byref(hws)) == 0
    hbuf = (ctypes.c_char * (hws.value + 64))()
    hwp = VP((ctypes.addressof(hbuf) + 15) // 16 * 16)
    half = [handle.ptr, hd[0].ptr, p, hd[1].ptr, p, hd[2].ptr, p, size.value, num, 0, 1, hwp, hws.value, hd[3].ptr, p]
    assert lib.mluOpIndiceConvolutionBackwardDataFromForwardTable(*half) == ops.STATUS_EXECUTION_FAILED  # host-only
    rows = list(half)
    bad_rows = ops.TensorDesc(ARRAY, F16, (11, 16))  # a submanifold layer has as many output as input rows
    rows[1] = bad_rows.ptr
    assert lib.mluOpIndiceConvolutionBackwardDataFromForwardTable(*rows) == ops.STATUS_BAD_PARAM
    for d in hd + [bad_rows]:
        d.destroy()
    # the filter gradient from the forward table: float tensors are not the kernel's, half 64 -> 64 are
    fdescs = [ops.TensorDesc(*BF_GOOD[k]) for k in ("features", "output_grad", "pairs", "filters_grad")]
    d_f, d_og, d_fp, d_fw = (d.ptr for d in fdescs)
    fnum = ops.i64_array(BF_GOOD["indice_num"])
    fargs = [handle.ptr, d_f, p, d_og, p, d_fp, p, 9 * 512 * 4, fnum, 0, 0, p, 1 << 16, d_fw, p]
    assert lib.mluOpIndiceConvolutionBackwardFilterFromTable(*fargs) == ops.STATUS_NOT_SUPPORTED
    for i in (0, 1, 2, 3, 4, 5, 6, 8, 11, 13, 14):
        a = list(fargs)
        a[i] = None
        assert lib.mluOpIndiceConvolutionBackwardFilterFromTable(*a) == ops.STATUS_BAD_PARAM, i
    hdescs = [ops.TensorDesc(ARRAY, F16, (3, 64)), ops.TensorDesc(ARRAY, F16, (3, 64)),
              ops.TensorDesc(ARRAY, I32, (9, 2, 3)), ops.TensorDesc(ARRAY, F16, (3, 3, 64, 64))]
    hsize = ctypes.c_size_t(0)
    assert lib.mluOpGetIndiceConvolutionBackwardFilterWorkspaceSize(handle.ptr, hdescs[0].ptr, hdescs[1].ptr,
                                                                    hdescs[2].ptr, hdescs[3].ptr, fnum, 0, 0,
                                                                    ctypes.byref(hsize)) == 0
    big = (ctypes.c_char * (hsize.value + 64))()
    wp = VP((ctypes.addressof(big) + 15) // 16 * 16)
    hargs = [handle.ptr, hdescs[0].ptr, p, hdescs[1].ptr, p, hdescs[2].ptr, p, 9 * 512 * 4, fnum, 0, 0, wp,
             hsize.value, hdescs[3].ptr, p]
    assert lib.mluOpIndiceConvolutionBackwardFilterFromTable(*hargs) == ops.STATUS_EXECUTION_FAILED  # host-only handle
    hsmall = list(hargs)
    hsmall[7] = 100
    assert lib.mluOpIndiceConvolutionBackwardFilterFromTable(*hsmall) == ops.STATUS_BAD_PARAM
    hodd = list(hargs)
    hodd[6] = VP(p.value + 4)
    assert lib.mluOpIndiceConvolutionBackwardFilterFromTable(*hodd) == ops.STATUS_BAD_PARAM
    for d in [d_p] + descs + fdescs + hdescs:
        d.destroy()
