"""GPU parity of mluOpIndiceConvolutionBackwardData and mluOpIndiceConvolutionBackwardFilter
against the CPU oracle, through the C ABI.  Acceptance: diff1 and diff2 <= 3e-3 for half
(the thresholds the reference generates its test cases with,
indice_convolution_backward_data.cpp:331 and indice_convolution_backward_filter.cpp:97),
<= 1e-5 for float."""
import numpy as np
import pytest
import torch

import helpers

# guard_bands: outputs and workspaces of every call sit between poisoned bands, checked after the test
pytestmark = [pytest.mark.gpu, pytest.mark.usefixtures("guard_bands")]


def assert_close(oracle, got, ref, is_half):
    d1, d2, _ = oracle.diffs(got, ref, is_half)
    tol = helpers.TOL_HALF if is_half else helpers.TOL_FLOAT
    assert d1 <= tol and d2 <= tol, (d1, d2)


def gpu_backward_data(ops, handle, og, w_array, layout, pairs, num, sub_m):
    w = helpers.permute_filter(w_array, layout)
    out = ops.indice_convolution_backward_data(handle, torch.from_numpy(og).cuda(), torch.from_numpy(w).cuda(), layout,
                                               torch.from_numpy(pairs).cuda(), [int(v) for v in num], sub_m)
    torch.cuda.synchronize()
    return out.float().cpu().numpy()


def gpu_backward_filter(ops, handle, feat, og, ks, pairs, num, sub_m):
    out = ops.indice_convolution_backward_filter(handle, torch.from_numpy(feat).cuda(), torch.from_numpy(og).cuda(),
                                                 ks, torch.from_numpy(pairs).cuda(), [int(v) for v in num], sub_m)
    torch.cuda.synchronize()
    return out.float().cpu().numpy()


@pytest.mark.parametrize("layout", ["ARRAY", "NDHWC", "NCDHW"])
def test_golden_input_gradients(ops, oracle, gpu_handle, golden, backward_golden, layout):
    """input_grad the reference's own CPU code produced (float, and its half emulation)."""
    for name in helpers.golden_names(golden):
        c = helpers.golden_case(golden, name)
        og = backward_golden[name + "/output_grad"]
        got = gpu_backward_data(ops, gpu_handle, og, c["filters_array"], layout, c["indice_pairs"], c["indice_num"],
                                c["sub_m"])
        assert_close(oracle, got, backward_golden[name + "/input_grad"], False)
        got = gpu_backward_data(ops, gpu_handle, og.astype(np.float16), c["filters_array"].astype(np.float16), layout,
                                c["indice_pairs"], c["indice_num"], c["sub_m"])
        assert_close(oracle, got, oracle.round_through_half(backward_golden[name + "/input_grad_half"]), True)


def test_golden_filter_gradients(ops, oracle, gpu_handle, golden, backward_golden):
    """filters_grad the reference's own CPU code produced."""
    for name in helpers.golden_names(golden):
        if name + "/filters_grad" not in backward_golden:
            continue
        c = helpers.golden_case(golden, name)
        og = backward_golden[name + "/output_grad"]
        got = gpu_backward_filter(ops, gpu_handle, c["features"], og, c["ks"], c["indice_pairs"], c["indice_num"],
                                  c["sub_m"])
        assert_close(oracle, got.reshape(-1, c["ci"], c["co"]), backward_golden[name + "/filters_grad"], False)
        got = gpu_backward_filter(ops, gpu_handle, c["features"].astype(np.float16), og.astype(np.float16), c["ks"],
                                  c["indice_pairs"], c["indice_num"], c["sub_m"])
        ref = oracle.round_through_half(backward_golden[name + "/filters_grad_half"])
        assert_close(oracle, got.reshape(-1, c["ci"], c["co"]), ref, True)


def make_case(oracle, rng, batch, space, n, ks, stride, pad, sub_m, ci, co, dtype):
    osp = list(space) if sub_m else helpers.out_space(space, pad, stride, [1] * 3, ks)
    idx = helpers.random_indices(rng, batch, space, n)
    pairs, _, num, n_out = oracle.get_indice_pairs(idx, batch, pad, stride, [1] * 3, ks, osp, sub_m)
    feat = rng.standard_normal((n, ci)).astype(np.float32).astype(dtype)
    og = rng.standard_normal((n_out, co)).astype(np.float32).astype(dtype)
    K = int(np.prod(ks))
    w = (rng.standard_normal(tuple(ks) + (ci, co)) / np.sqrt(K * co)).astype(np.float32).astype(dtype)
    return pairs, num, n_out, feat, og, w


CHANNELS = [(4, 16), (16, 16), (16, 32), (32, 32), (32, 64), (64, 64), (64, 128), (128, 128), (3, 5), (20, 48),
            (128, 16), (130, 140)]


@pytest.mark.parametrize("ci,co", CHANNELS)
@pytest.mark.parametrize("dtype", [np.float16, np.float32])
def test_channel_sweep(ops, oracle, gpu_handle, ci, co, dtype):
    """Every kernel variant of both operators: tensor-core tiles for half with
    power-of-two channels, FMA otherwise; submanifold and strided rulebooks."""
    rng = np.random.default_rng(ci * 1000 + co + 7)
    is_half = dtype == np.float16
    for sub_m, stride in ((1, [1] * 3), (0, [2] * 3)):
        pairs, num, n_out, feat, og, w = make_case(oracle, rng, 2, [8, 14, 12], 700, [3] * 3, stride, [1] * 3, sub_m,
                                                   ci, co, dtype)
        ref = oracle.indice_convolution_backward_data(og.astype(np.float32), w.astype(np.float32), "ARRAY", [3] * 3,
                                                      pairs, num, ci, is_half)
        if is_half:
            ref = oracle.round_through_half(ref)
        got = gpu_backward_data(ops, gpu_handle, og, w, "ARRAY", pairs, num, sub_m)
        assert_close(oracle, got, ref, is_half)
        ref = oracle.indice_convolution_backward_filter(feat.astype(np.float32), og.astype(np.float32), [3] * 3, pairs,
                                                        num)
        if is_half:
            ref = oracle.round_through_half(ref)
        got = gpu_backward_filter(ops, gpu_handle, feat, og, [3] * 3, pairs, num, sub_m)
        assert_close(oracle, got.reshape(ref.shape), ref, is_half)


def test_four_dimensional_filters(ops, oracle, gpu_handle):
    """HWCN / NHWC / NCHW filters (a 1 x 3 x 3 kernel described without its depth axis)."""
    rng = np.random.default_rng(21)
    ks = [1, 3, 3]
    pairs, num, n_out, feat, og, w = make_case(oracle, rng, 1, [5, 12, 12], 300, ks, [1] * 3, [0, 1, 1], 1, 16, 32,
                                               np.float32)
    ref = oracle.indice_convolution_backward_data(og, w, "ARRAY", ks, pairs, num, 16, False)
    w4 = w[0]  # [kh,kw,Ci,Co]
    d_og, d_pairs = torch.from_numpy(og).cuda(), torch.from_numpy(pairs).cuda()
    nums = [int(v) for v in num]
    for layout, wl in (("HWCN", w4), ("NHWC", np.transpose(w4, (3, 0, 1, 2))), ("NCHW", np.transpose(w4, (3, 2, 0, 1)))):
        got = ops.indice_convolution_backward_data(gpu_handle, d_og, torch.from_numpy(np.ascontiguousarray(wl)).cuda(),
                                                   layout, d_pairs, nums, 1)
        assert_close(oracle, got.cpu().numpy(), ref, False)
    got = ops.indice_convolution_backward_filter(gpu_handle, torch.from_numpy(feat).cuda(), d_og, [3, 3], d_pairs, nums,
                                                 1)
    ref = oracle.indice_convolution_backward_filter(feat, og, ks, pairs, num)
    assert_close(oracle, got.cpu().numpy().reshape(ref.shape), ref, False)


def test_rows_and_offsets_without_pairs_are_zero(ops, oracle, gpu_handle):
    rng = np.random.default_rng(22)
    pairs, num, n_out, feat, og, w = make_case(oracle, rng, 1, [6, 6, 6], 50, [3] * 3, [1] * 3, [1] * 3, 1, 16, 16,
                                               np.float16)
    zero_num = np.zeros_like(num)
    assert np.all(gpu_backward_data(ops, gpu_handle, og, w, "ARRAY", pairs, zero_num, 1) == 0)
    assert np.all(gpu_backward_filter(ops, gpu_handle, feat, og, [3] * 3, pairs, zero_num, 1) == 0)
    some = num.copy()
    some[::2] = 0
    got = gpu_backward_filter(ops, gpu_handle, feat, og, [3] * 3, pairs, some, 1).reshape(27, 16, 16)
    assert np.all(got[::2] == 0) and np.any(got[13] != 0)


def test_adjoint_identities_at_full_size(ops, oracle, workloads, gpu_handle):
    """Size-independent properties on one 200k-voxel 128-channel sample (where the CPU
    oracle would take minutes): <conv(x), dy> == <x, backward_data(dy)> == <W, backward_filter(x, dy)>,
    and two runs of each operator are bit-identical."""
    idx, feat, layers, weights = workloads.make_inputs("c3", batch=2)
    ly = layers[0]
    grid = list(workloads.CONFIGS["c3"]["grid"])
    conv = ops.SparseConvDesc(2, ly.pad, ly.stride, ly.dilation, grid, ly.filter_space, grid, 1)
    pairs, _, num, n_out = ops.get_indice_pairs(gpu_handle, conv, torch.from_numpy(idx).cuda())
    num_h = num.cpu().tolist()
    x = torch.from_numpy(feat).cuda()
    w = torch.from_numpy(weights[0]).cuda()
    gen = torch.Generator(device="cuda").manual_seed(5)
    dy = torch.randn((n_out, ly.co), generator=gen, device="cuda").half()
    y = ops.indice_convolution_forward(gpu_handle, x, w, "ARRAY", ly.filter_space, pairs, num_h, n_out, 1)
    dx = ops.indice_convolution_backward_data(gpu_handle, dy, w, "ARRAY", pairs, num_h, 1)
    dw = ops.indice_convolution_backward_filter(gpu_handle, x, dy, ly.filter_space, pairs, num_h, 1)
    lhs = float((y.double() * dy.double()).sum())
    scale = float((y.double().abs() * dy.double().abs()).sum())
    assert abs(lhs - float((x.double() * dx.double()).sum())) <= 2e-3 * scale
    assert abs(lhs - float((w.double() * dw.double()).sum())) <= 2e-3 * scale
    assert torch.equal(dx, ops.indice_convolution_backward_data(gpu_handle, dy, w, "ARRAY", pairs, num_h, 1))
    assert torch.equal(dw, ops.indice_convolution_backward_filter(gpu_handle, x, dy, ly.filter_space, pairs, num_h, 1))
    conv.destroy()


@pytest.mark.parametrize("ks", [[1, 1, 1], [5, 5, 5], [7, 7, 7], [3, 1, 5]])
@pytest.mark.parametrize("dtype", [np.float16, np.float32])
def test_kernel_volumes_outside_the_tensor_core_range(ops, oracle, gpu_handle, ks, dtype):
    """Kernel volumes 1, 125, 343 and 15: above 32 offsets the forward and the input gradient
    leave the tensor-core kernels, above 128 the pair counts travel through device memory."""
    rng = np.random.default_rng(sum(ks) + (dtype == np.float16))
    is_half = dtype == np.float16
    pad = [(k - 1) // 2 for k in ks]
    pairs, num, n_out, feat, og, w = make_case(oracle, rng, 2, [7, 9, 8], 300, ks, [1] * 3, pad, 1, 16, 32, dtype)
    f32 = lambda a: a.astype(np.float32)  # noqa: E731
    r = (lambda a: oracle.round_through_half(a)) if is_half else (lambda a: a)
    fwd = torch.from_numpy(feat).cuda()
    got = ops.indice_convolution_forward(gpu_handle, fwd, torch.from_numpy(w).cuda(), "ARRAY", ks,
                                         torch.from_numpy(pairs).cuda(), [int(v) for v in num], n_out, 1)
    ref = r(oracle.indice_convolution_forward(f32(feat), f32(w), "ARRAY", ks, pairs, num, n_out, 32))
    assert_close(oracle, got.float().cpu().numpy(), ref, is_half)
    ref = r(oracle.indice_convolution_backward_data(f32(og), f32(w), "ARRAY", ks, pairs, num, 16, is_half))
    assert_close(oracle, gpu_backward_data(ops, gpu_handle, og, w, "ARRAY", pairs, num, 1), ref, is_half)
    ref = r(oracle.indice_convolution_backward_filter(f32(feat), f32(og), ks, pairs, num))
    got = gpu_backward_filter(ops, gpu_handle, feat, og, ks, pairs, num, 1)
    assert_close(oracle, got.reshape(ref.shape), ref, is_half)


@pytest.mark.parametrize("ci,co", [(64, 64), (64, 128), (32, 32), (32, 64)])
@pytest.mark.parametrize("ks,n,space", [([3, 3, 3], 30000, [20, 40, 40]), ([1, 1, 1], 5000, [10, 30, 30]),
                                        ([5, 5, 5], 3000, [8, 16, 16]), ([3, 1, 2], 1000, [9, 10, 10]),
                                        ([4, 4, 8], 600, [8, 8, 16])])  # 128 offsets: the largest volume it takes
def test_filter_gradient_in_tensor_memory(ops, oracle, gpu_handle, trace_kernels, monkeypatch, ci, co, ks, n, space):
    """Half with 32 or 64 input channels runs filterGradTcgen05Kernel (sums of all offsets of a
    group kept in tensor memory, tiles of output rows streamed past them): several tiles
    per block, a ragged last tile, kernel volumes that leave a bundle of offsets part empty and more
    groups than one.  Checked against the oracle, against the pair-list kernel
    (MLUOP_B200_FILTER_GRAD_KERNEL=mma) and for bit-identical repeats."""
    rng = np.random.default_rng(ci * 7 + co + sum(ks) + n)
    pad = [(k - 1) // 2 for k in ks]
    for sub_m, stride in ((1, [1] * 3), (0, [2] * 3)):
        pairs, num, n_out, feat, og, w = make_case(oracle, rng, 2, space, n, ks, stride, pad, sub_m, ci, co, np.float16)
        ref = oracle.round_through_half(oracle.indice_convolution_backward_filter(
            feat.astype(np.float32), og.astype(np.float32), ks, pairs, num))
        if ci == 32:  # 32 input channels take this kernel on request only
            monkeypatch.setenv("MLUOP_B200_FILTER_GRAD_KERNEL", "tcgen05")
        with trace_kernels() as names:
            got = gpu_backward_filter(ops, gpu_handle, feat, og, ks, pairs, num, sub_m)
        assert any(nm.startswith("filterGradTcgen05Kernel") for nm in names), names
        assert_close(oracle, got.reshape(ref.shape), ref, True)
        again = gpu_backward_filter(ops, gpu_handle, feat, og, ks, pairs, num, sub_m)
        assert np.array_equal(got, again)
        monkeypatch.setenv("MLUOP_B200_FILTER_GRAD_KERNEL", "mma")
        with trace_kernels() as names:
            other = gpu_backward_filter(ops, gpu_handle, feat, og, ks, pairs, num, sub_m)
        monkeypatch.delenv("MLUOP_B200_FILTER_GRAD_KERNEL")
        assert not any(nm.startswith("filterGradTcgen05Kernel") for nm in names), names
        assert_close(oracle, got, other, True)


@pytest.mark.parametrize("dtype", [np.float16, np.float32])
def test_rows_that_start_one_element_off_an_aligned_address(ops, oracle, gpu_handle, dtype):
    """The tensor-core kernels move rows as 16-byte vectors and are chosen only for 16-byte
    aligned row arrays; a view that starts one element into a buffer (a caller's slice)
    must take the scalar kernels and give the same results, not fault."""
    rng = np.random.default_rng(31)
    is_half = dtype == np.float16
    ks = [3] * 3
    pairs, num, n_out, feat, og, w = make_case(oracle, rng, 2, [8, 12, 12], 900, ks, [1] * 3, [1] * 3, 1, 64, 64, dtype)
    f32 = lambda a: a.astype(np.float32)  # noqa: E731
    r = (lambda a: oracle.round_through_half(a)) if is_half else (lambda a: a)

    def off_by_one(a):
        buf = torch.empty((a.size + 1,), dtype=torch.from_numpy(a).dtype, device="cuda")
        view = buf[1:].view(a.shape)
        view.copy_(torch.from_numpy(a))
        assert view.data_ptr() % 16 != 0
        return view

    d_pairs, nums = torch.from_numpy(pairs).cuda(), [int(v) for v in num]
    d_w = torch.from_numpy(w).cuda()
    got = ops.indice_convolution_forward(gpu_handle, off_by_one(feat), d_w, "ARRAY", ks, d_pairs, nums, n_out, 1)
    ref = r(oracle.indice_convolution_forward(f32(feat), f32(w), "ARRAY", ks, pairs, num, n_out, 64))
    assert_close(oracle, got.float().cpu().numpy(), ref, is_half)
    got = ops.indice_convolution_backward_data(gpu_handle, off_by_one(og), d_w, "ARRAY", d_pairs, nums, 1)
    ref = r(oracle.indice_convolution_backward_data(f32(og), f32(w), "ARRAY", ks, pairs, num, 64, is_half))
    assert_close(oracle, got.float().cpu().numpy(), ref, is_half)
    got = ops.indice_convolution_backward_filter(gpu_handle, off_by_one(feat), off_by_one(og), ks, d_pairs, nums, 1)
    ref = r(oracle.indice_convolution_backward_filter(f32(feat), f32(og), ks, pairs, num))
    assert_close(oracle, got.float().cpu().numpy().reshape(ref.shape), ref, is_half)


def test_a_filter_gradient_wait_that_runs_out_is_reported_and_the_context_survives(ops, oracle, gpu_handle, monkeypatch):
    """Failure detection on the device without a fault, for the tensor-memory filter gradient: the test
    hook gives its waits a limit of about a millisecond and withholds one stage release per block, so
    the producers' wait for that stage runs out.  The kernel must record the error, leave through its
    common exit (copies drained, MMAs seen out, tensor memory freed) and return: the call reports
    MLUOP_STATUS_EXECUTION_FAILED, and the same call without the hook then gives the right answer on
    the same context."""
    rng = np.random.default_rng(13)
    space = [6, 10, 10]
    n = 2 * 6 * 10 * 10  # fully occupied: every tile is live at every offset, more items than ring stages
    pairs, num, n_out, feat, og, w = make_case(oracle, rng, 2, space, n, [3] * 3, [1] * 3, [1] * 3, 1, 64, 64,
                                               np.float16)
    monkeypatch.setenv("MLUOP_B200_TEST_FILTER_GRAD_WAIT", "2000000")
    with pytest.raises(ops.MluOpError) as err:
        gpu_backward_filter(ops, gpu_handle, feat, og, [3] * 3, pairs, num, 1)
    assert err.value.status == ops.STATUS_EXECUTION_FAILED
    monkeypatch.delenv("MLUOP_B200_TEST_FILTER_GRAD_WAIT")
    ref = oracle.round_through_half(oracle.indice_convolution_backward_filter(
        feat.astype(np.float32), og.astype(np.float32), [3] * 3, pairs, num))
    for _ in range(2):  # tensor memory was freed: later launches get their columns and compute correctly
        got = gpu_backward_filter(ops, gpu_handle, feat, og, [3] * 3, pairs, num, 1)
        assert_close(oracle, got.reshape(ref.shape), ref, True)
