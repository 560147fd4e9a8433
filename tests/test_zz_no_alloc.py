"""mluOpIndiceConvolutionForwardBuiltinWorkspace: the convolution entry point for
callers that cannot allocate device scratch (allocation-free inference loops,
plugins whose host process owns all device memory).  Its scratch is a fixed array
inside the library, so the test passes no workspace at all, calls it twice in a
row (the second call meets the first call's leftovers in the shared array) and
expects exactly the bytes the ordinary entry point produces.  The file name keeps
it last in collection order."""
import ctypes

import numpy as np
import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu
VP = ctypes.c_void_p


def builtin_conv(ops, handle, feat, w, pairs, num_host, n_out, sub_m, fill=None, out=None):
    L, ci = feat.shape
    co = w.shape[4]
    K = pairs.shape[0]
    dt = ops.DTYPE_HALF if feat.dtype == torch.float16 else ops.DTYPE_FLOAT
    if out is None:
        out = torch.empty((n_out, co), dtype=feat.dtype, device=feat.device)
    if fill is not None:
        out.fill_(fill)
    d_f = ops.TensorDesc(ops.LAYOUT_ARRAY, dt, (L, ci))
    d_w = ops.TensorDesc(ops.LAYOUT_ARRAY, dt, tuple(w.shape))
    d_p = ops.TensorDesc(ops.LAYOUT_ARRAY, ops.DTYPE_INT32, (K, 2, L))
    d_o = ops.TensorDesc(ops.LAYOUT_ARRAY, dt, (n_out, co))
    st = ops.lib().mluOpIndiceConvolutionForwardBuiltinWorkspace(
        handle.ptr, d_f.ptr, VP(feat.data_ptr()), d_w.ptr, VP(w.data_ptr()), d_p.ptr, VP(pairs.data_ptr()),
        ops.i64_array(num_host), n_out, 0, sub_m, d_o.ptr, VP(out.data_ptr()))
    return st, out


@pytest.mark.parametrize("dtype,ci,co", [(np.float16, 32, 64), (np.float32, 16, 16)])
def test_builtin_workspace_matches_ordinary_entry_point(ops, oracle, gpu_handle, dtype, ci, co):
    rng = np.random.default_rng(31)
    results = []
    for round_, (sub_m, stride) in enumerate(((1, [1] * 3), (0, [2] * 3))):
        space = [8, 20, 18]
        idx = helpers.random_indices(rng, 2, space, 2500)
        osp = space if sub_m else helpers.out_space(space, [1] * 3, stride, [1] * 3, [3] * 3)
        conv = ops.SparseConvDesc(2, [1] * 3, stride, [1] * 3, space, [3] * 3, osp, sub_m)
        pairs, _, num, n_out = ops.get_indice_pairs(gpu_handle, conv, torch.from_numpy(idx).cuda())
        num_host = num.cpu().tolist()
        feat = torch.from_numpy(rng.standard_normal((idx.shape[0], ci)).astype(np.float32).astype(dtype)).cuda()
        w = torch.from_numpy((rng.standard_normal((3, 3, 3, ci, co)) / np.sqrt(27 * ci)).astype(np.float32)
                             .astype(dtype)).cuda()
        expected = ops.indice_convolution_forward(gpu_handle, feat, w, "ARRAY", [3] * 3, pairs, num_host, n_out,
                                                  sub_m)
        # The outputs exist before the calls, and one call has already run (it loads the
        # kernels and looks the array's address up), so that the free device memory the driver
        # reports must be the same before and after the two calls under test: the entry point
        # allocates nothing, on the device or through torch.
        out1, out2 = torch.empty_like(expected), torch.empty_like(expected)
        builtin_conv(ops, gpu_handle, feat, w, pairs, num_host, n_out, sub_m, fill=1.0, out=torch.empty_like(expected))
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        reserved_before = torch.cuda.memory_reserved()
        # two calls in a row on the shared built-in scratch, different problems each round
        st1, got1 = builtin_conv(ops, gpu_handle, feat, w, pairs, num_host, n_out, sub_m, fill=7.0, out=out1)
        st2, got2 = builtin_conv(ops, gpu_handle, feat, w, pairs, num_host, n_out, sub_m, fill=-3.0, out=out2)
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        assert st1 == ops.STATUS_SUCCESS and st2 == ops.STATUS_SUCCESS
        assert free_after == free_before and torch.cuda.memory_reserved() == reserved_before
        assert torch.equal(got1, expected) and torch.equal(got2, expected)
        results.append(got2)
        conv.destroy()
    assert results[0].shape != results[1].shape or not torch.equal(results[0], results[1])


def test_builtin_workspace_refuses_what_does_not_fit(ops, gpu_handle):
    # 27 offsets x 400,000 output rows x 4 bytes of neighbour table alone exceed the built-in 32 MiB
    L = 400000
    feat = torch.zeros((L, 16), dtype=torch.float16, device="cuda")
    w = torch.zeros((3, 3, 3, 16, 16), dtype=torch.float16, device="cuda")
    pairs = torch.full((27, 2, L), -1, dtype=torch.int32, device="cuda")
    st, _ = builtin_conv(ops, gpu_handle, feat, w, pairs, [0] * 27, L, 1)
    assert st == ops.STATUS_NOT_SUPPORTED
    # argument errors are those of the ordinary entry point
    st = ops.lib().mluOpIndiceConvolutionForwardBuiltinWorkspace(None, None, None, None, None, None, None, None, 0, 0,
                                                                 0, None, None)
    assert st == ops.STATUS_BAD_PARAM
