import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

# Argument-check tests need a handle even on a machine without a GPU; the
# library then hands out a handle that can validate but not launch.
os.environ.setdefault("MLUOP_B200_HOST_ONLY_HANDLE", "1")
os.environ.setdefault("MLUOP_MIN_LOG_LEVEL", "3")
# Convolution calls wait for the stream and report a kernel whose bounded waits gave up.
os.environ.setdefault("MLUOP_B200_CHECK_STATUS", "1")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def pkg():
    import __graft_entry__ as entry
    entry.build()
    return entry.load_package()


@pytest.fixture(scope="session")
def ops(pkg):
    return pkg[0]


@pytest.fixture(scope="session")
def workloads(pkg):
    return pkg[1]


@pytest.fixture(scope="session")
def backbone(pkg):
    return pkg[2]


@pytest.fixture(scope="session")
def oracle():
    import __graft_entry__ as entry
    o = entry.load_oracle()
    o.build()
    return o


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    path = os.path.join(ROOT, "tests", "golden", "sparse_conv_golden.npz")
    return np.load(path)


@pytest.fixture(scope="session")
def backward_golden():
    import numpy as np
    path = os.path.join(ROOT, "tests", "golden", "sparse_conv_backward_golden.npz")
    return np.load(path)


@pytest.fixture(scope="session")
def gpu_handle(ops):
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    torch.cuda.set_device(0)
    h = ops.Handle(torch.cuda.current_stream().cuda_stream)
    yield h
    h.destroy()


@pytest.fixture
def guard_bands(ops):
    """Every buffer the harness allocates during the test (outputs, workspace) is bracketed by
    poisoned bands that are checked when the test ends (ops.Guards)."""
    with ops.guarded() as guards:
        yield guards


@pytest.fixture
def trace_kernels(ops):
    """trace_kernels() is a context manager that yields a list filled, on exit, with the names
    of the library kernels launched inside it (include/mlu_op_trace.h)."""
    import contextlib
    import ctypes

    @contextlib.contextmanager
    def tracing():
        lib = ops.lib()
        names = []
        lib.mluOpTraceKernelReset()
        lib.mluOpTraceKernelEnable(1)
        try:
            yield names
        finally:
            lib.mluOpTraceKernelEnable(0)
            buf = ctypes.create_string_buffer(1 << 16)
            assert lib.mluOpTraceKernelReport(buf, len(buf), None) == 0
            names.extend(line.rsplit(",", 4)[0] for line in buf.value.decode().splitlines()[1:])

    return tracing
