"""Kernel tracing (include/mlu_op_trace.h): every launch of the library is
bracketed by CUDA events while tracing is on, and nothing is recorded while it is off."""
import ctypes

import numpy as np
import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu


def report(ops):
    buf = ctypes.create_string_buffer(1 << 16)
    need = ctypes.c_size_t(0)
    assert ops.lib().mluOpTraceKernelReport(buf, len(buf), ctypes.byref(need)) == 0
    lines = buf.value.decode().splitlines()
    assert lines[0] == "name,launches,total_ms,algorithmic_bytes,flops"
    assert need.value == len(buf.value) + 1
    rows = {}
    for line in lines[1:]:
        name, launches, ms, nbytes, flops = line.rsplit(",", 4)
        rows[name] = (int(launches), float(ms), float(nbytes), float(flops))
    return rows


def run_layer(ops, handle, rng):
    space = [8, 16, 16]
    idx = helpers.random_indices(rng, 2, space, 1500)
    conv = ops.SparseConvDesc(2, [1] * 3, [1] * 3, [1] * 3, space, [3] * 3, space, 1)
    pairs, _, num, n_out = ops.get_indice_pairs(handle, conv, torch.from_numpy(idx).cuda())
    feat = torch.randn((1500, 32), device="cuda").half()
    w = torch.randn((3, 3, 3, 32, 32), device="cuda").half()
    ops.indice_convolution_forward(handle, feat, w, "ARRAY", [3] * 3, pairs, num.cpu().tolist(), n_out, 1)
    torch.cuda.synchronize()
    conv.destroy()
    return int(num.sum())


def test_trace_records_only_while_enabled(ops, gpu_handle):
    lib = ops.lib()
    rng = np.random.default_rng(1)
    lib.mluOpTraceKernelEnable(0)
    lib.mluOpTraceKernelReset()
    run_layer(ops, gpu_handle, rng)
    assert report(ops) == {}
    lib.mluOpTraceKernelEnable(1)
    pairs = run_layer(ops, gpu_handle, rng)
    run_layer(ops, gpu_handle, rng)
    lib.mluOpTraceKernelEnable(0)
    rows = report(ops)
    kernels = {k: v for k, v in rows.items() if not k.startswith(("memset:", "memcpy:"))}
    lists = [k for k in kernels if k.startswith("pairListsKernel")]
    assert len(lists) == 1 and kernels[lists[0]][0] == 2 and kernels["finishPairsKernel"][0] == 2
    conv = [k for k in kernels if k.startswith("conv")]
    assert len(conv) == 1 and kernels[conv[0]][0] == 2
    assert all(v[1] > 0 for v in kernels.values())
    # the convolution states 2*P*Ci*Co flops for its launch
    assert kernels[conv[0]][3] >= 2.0 * pairs * 32 * 32
    assert report(ops) == {}  # a report clears the records
    assert lib.mluOpTraceKernelReport(None, 16, None) == ops.STATUS_BAD_PARAM


def test_size_query_then_fetch_keeps_the_records(ops, gpu_handle):
    """A report whose buffer is too small (a size query) must not drop the records."""
    lib = ops.lib()
    lib.mluOpTraceKernelReset()
    lib.mluOpTraceKernelEnable(1)
    run_layer(ops, gpu_handle, np.random.default_rng(2))
    lib.mluOpTraceKernelEnable(0)
    need = ctypes.c_size_t(0)
    assert lib.mluOpTraceKernelReport(None, 0, ctypes.byref(need)) == ops.STATUS_SUCCESS
    assert need.value > 64
    small = ctypes.create_string_buffer(32)
    assert lib.mluOpTraceKernelReport(small, len(small), None) == ops.STATUS_SUCCESS  # truncated, kept
    buf = ctypes.create_string_buffer(need.value)
    assert lib.mluOpTraceKernelReport(buf, len(buf), None) == ops.STATUS_SUCCESS
    lines = buf.value.decode().splitlines()
    assert lines[0].startswith("name,launches") and len(lines) > 3 and buf.value.decode().startswith(small.value.decode())
    assert report(ops) == {}
