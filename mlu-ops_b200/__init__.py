"""Python harness over the C ABI of libmluops_b200.so.

The product is the shared library (include/mlu_op.h); this package only loads
it with ctypes and wraps the calls so that tests, the benchmark and the
backbone driver can pass torch CUDA tensors.  Function and argument names
follow the reference's C API.  There is no CPU fallback: if the library has not
been built, loading raises.
"""
import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "lib", "libmluops_b200.so")

# mluOpStatus_t
STATUS_SUCCESS = 0
STATUS_NOT_INITIALIZED = 1
STATUS_ALLOC_FAILED = 2
STATUS_BAD_PARAM = 3
STATUS_INTERNAL_ERROR = 4
STATUS_ARCH_MISMATCH = 5
STATUS_EXECUTION_FAILED = 6
STATUS_NOT_SUPPORTED = 7
STATUS_NUMERICAL_OVERFLOW = 8

# mluOpTensorLayout_t
LAYOUT_NCHW, LAYOUT_NHWC, LAYOUT_HWCN, LAYOUT_NDHWC, LAYOUT_ARRAY, LAYOUT_NCDHW = 0, 1, 2, 3, 4, 5
# mluOpDataType_t
DTYPE_INVALID, DTYPE_HALF, DTYPE_FLOAT, DTYPE_INT16, DTYPE_INT32, DTYPE_INT64 = 0, 1, 2, 4, 6, 9

_vp = ctypes.c_void_p
_int = ctypes.c_int
_i64 = ctypes.c_int64
_szt = ctypes.c_size_t
_intp = ctypes.POINTER(ctypes.c_int)
_i64p = ctypes.POINTER(ctypes.c_int64)

# name -> (restype, argtypes); exactly the entry points include/mlu_op.h and include/mlu_op_trace.h declare
SIGNATURES = {
    "mluOpCreate": (_int, [ctypes.POINTER(_vp)]),
    "mluOpDestroy": (_int, [_vp]),
    "mluOpSetQueue": (_int, [_vp, _vp]),
    "mluOpGetQueue": (_int, [_vp, ctypes.POINTER(_vp)]),
    "mluOpGetDevice": (_int, [_vp, _intp]),
    "mluOpGetErrorString": (ctypes.c_char_p, [_int]),
    "mluOpGetSizeOfDataType": (_int, [_int, ctypes.POINTER(_szt)]),
    "mluOpGetLibVersion": (None, [_intp, _intp, _intp]),
    "mluOpSetAtomicsMode": (_int, [_vp, _int]),
    "mluOpGetAtomicsMode": (_int, [_vp, _intp]),
    "mluOpCreateTensorDescriptor": (_int, [ctypes.POINTER(_vp)]),
    "mluOpSetTensorDescriptor": (_int, [_vp, _int, _int, _int, _intp]),
    "mluOpSetTensorDescriptor_v2": (_int, [_vp, _int, _int, _int, _i64p]),
    "mluOpSetTensorDescriptorEx": (_int, [_vp, _int, _int, _int, _intp, _intp]),
    "mluOpSetTensorDescriptorEx_v2": (_int, [_vp, _int, _int, _int, _i64p, _i64p]),
    "mluOpResetTensorDescriptor": (_int, [_vp]),
    "mluOpGetTensorDescriptor": (_int, [_vp, _intp, _intp, _intp, _intp]),
    "mluOpGetTensorDescriptor_v2": (_int, [_vp, _intp, _intp, _intp, _i64p]),
    "mluOpGetTensorDescriptorEx": (_int, [_vp, _intp, _intp, _intp, _intp, _intp]),
    "mluOpGetTensorElementNum": (ctypes.c_uint64, [_vp]),
    "mluOpDestroyTensorDescriptor": (_int, [_vp]),
    "mluOpCreateSparseConvolutionDescriptor": (_int, [ctypes.POINTER(_vp)]),
    "mluOpDestroySparseConvolutionDescriptor": (_int, [_vp]),
    "mluOpSetSparseConvolutionDescriptor": (_int, [_vp, _int, _int, _intp, _intp, _intp, _intp, _intp, _intp,
                                                  _int, _int, _int]),
    "mluOpGetSparseConvolutionNumActOut": (_int, [_vp, _intp]),
    "mluOpGetIndicePairsWorkspaceSize": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, ctypes.POINTER(_szt)]),
    "mluOpGetIndicePairs": (_int, [_vp, _vp, _vp, _vp, _vp, _szt, _vp, _vp, _vp, _vp, _vp, _vp]),
    "mluOpGetIndicePairsWithNeighbourTable": (_int, [_vp, _vp, _vp, _vp, _vp, _szt, _vp, _vp, _vp, _vp, _vp, _vp,
                                                    _vp, _szt]),
    "mluOpGetIndiceConvolutionForwardWorkspaceSize": (_int, [_vp, _vp, _vp, _vp, _vp, _i64p, _i64, _i64, _i64,
                                                            ctypes.POINTER(_szt)]),
    "mluOpIndiceConvolutionForward": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64p, _i64, _i64, _i64, _vp,
                                            _szt, _vp, _vp]),
    "mluOpIndiceConvolutionForwardBuiltinWorkspace": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64p, _i64, _i64,
                                                            _i64, _vp, _vp]),
    "mluOpGetIndiceConvolutionBackwardDataWorkspaceSize": (_int, [_vp, _vp, _vp, _vp, _vp, _i64p, _i64,
                                                                 ctypes.POINTER(_szt)]),
    "mluOpIndiceConvolutionBackwardData": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64p, _i64, _i64, _vp, _szt,
                                                 _vp, _vp]),
    "mluOpGetIndiceConvolutionBackwardFilterWorkspaceSize": (_int, [_vp, _vp, _vp, _vp, _vp, _i64p, _i64, _i64,
                                                                   ctypes.POINTER(_szt)]),
    "mluOpIndiceConvolutionBackwardFilter": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64p, _i64, _i64, _vp,
                                                   _szt, _vp, _vp]),
    "mluOpGetIndiceNeighbourTableSize": (_int, [_vp, _vp, _i64, ctypes.POINTER(_szt)]),
    "mluOpBuildIndiceNeighbourTable": (_int, [_vp, _vp, _vp, _i64p, _i64, _vp, _szt]),
    "mluOpGetIndiceConvolutionForwardFromTableWorkspaceSize": (_int, [_vp, _vp, _vp, _vp, _vp, _i64p, _i64, _i64,
                                                                     _i64, ctypes.POINTER(_szt)]),
    "mluOpIndiceConvolutionForwardFromTable": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _szt, _i64p, _i64, _i64,
                                                     _i64, _vp, _szt, _vp, _vp]),
    "mluOpGetIndiceInputNeighbourTableSize": (_int, [_vp, _vp, ctypes.POINTER(_szt)]),
    "mluOpBuildIndiceInputNeighbourTable": (_int, [_vp, _vp, _vp, _i64p, _i64, _vp, _szt]),
    "mluOpGetIndiceConvolutionBackwardDataFromTableWorkspaceSize": (_int, [_vp, _vp, _vp, _vp, _vp, _i64p, _i64,
                                                                          ctypes.POINTER(_szt)]),
    "mluOpIndiceConvolutionBackwardDataFromTable": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _szt, _i64p, _i64,
                                                          _i64, _vp, _szt, _vp, _vp]),
    "mluOpIndiceConvolutionBackwardDataFromForwardTable": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _szt, _i64p,
                                                                 _i64, _i64, _vp, _szt, _vp, _vp]),
    "mluOpIndiceConvolutionBackwardFilterFromTable": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _szt, _i64p, _i64,
                                                            _i64, _vp, _szt, _vp, _vp]),
    "mluOpGetVoxelizationWorkspaceSize": (_int, [_vp, _vp, _vp, _vp, ctypes.c_int32, ctypes.c_int32,
                                                ctypes.c_int32, ctypes.c_bool, _vp, _vp, _vp, _vp,
                                                ctypes.POINTER(_szt)]),
    "mluOpVoxelization": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32,
                                ctypes.c_bool, _vp, _szt, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "mluOpGetDynamicPointToVoxelForwardWorkspaceSize": (_int, [_vp, _vp, _vp, ctypes.POINTER(_szt)]),
    "mluOpDynamicPointToVoxelForward": (_int, [_vp, _int, _vp, _vp, _vp, _vp, _vp, _szt, _vp, _vp, _vp, _vp, _vp, _vp,
                                              _vp, _vp, _vp, _vp]),
    "mluOpGetDynamicPointToVoxelBackwardWorkspaceSize": (_int, [_vp, _int, _vp, _vp, _vp, _vp, _vp, _vp,
                                                               ctypes.POINTER(_szt)]),
    "mluOpDynamicPointToVoxelBackward": (_int, [_vp, _int, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp,
                                               _vp, _szt, _vp, _vp]),
    # include/mlu_op_trace.h
    "mluOpTraceKernelEnable": (_int, [_int]),
    "mluOpTraceKernelReset": (_int, []),
    "mluOpTraceKernelReport": (_int, [ctypes.c_char_p, _szt, ctypes.POINTER(_szt)]),
}

_lib = None


def lib():
    """The loaded C-ABI library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.isfile(LIB_PATH):
            raise RuntimeError(
                "libmluops_b200.so is missing (%s); build it with `python mlu-ops_b200/build.py`. "
                "There is no fallback path." % LIB_PATH)
        _lib = ctypes.CDLL(LIB_PATH)
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(_lib, name)
            fn.restype = restype
            fn.argtypes = argtypes
    return _lib


class MluOpError(RuntimeError):
    def __init__(self, call, status):
        self.status = status
        name = lib().mluOpGetErrorString(status).decode()
        super().__init__("%s returned %s (%d)" % (call, name, status))


def check(call, status):
    if status != STATUS_SUCCESS:
        raise MluOpError(call, status)


def int_array(values):
    return (ctypes.c_int * len(values))(*[int(v) for v in values])


def i64_array(values):
    return (ctypes.c_int64 * len(values))(*[int(v) for v in values])


class Handle:
    """mluOpHandle_t bound to a CUDA stream (raw cudaStream_t integer, 0 = default)."""

    def __init__(self, stream=0):
        self.ptr = _vp()
        check("mluOpCreate", lib().mluOpCreate(ctypes.byref(self.ptr)))
        self.set_queue(stream)

    def set_queue(self, stream):
        check("mluOpSetQueue", lib().mluOpSetQueue(self.ptr, _vp(stream)))

    def destroy(self):
        if self.ptr:
            check("mluOpDestroy", lib().mluOpDestroy(self.ptr))
            self.ptr = _vp()

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass


class TensorDesc:
    """mluOpTensorDescriptor_t with contiguous strides."""

    def __init__(self, layout, dtype, dims):
        self.ptr = _vp()
        check("mluOpCreateTensorDescriptor", lib().mluOpCreateTensorDescriptor(ctypes.byref(self.ptr)))
        check("mluOpSetTensorDescriptor_v2",
              lib().mluOpSetTensorDescriptor_v2(self.ptr, layout, dtype, len(dims), i64_array(dims)))
        self.dims = tuple(int(d) for d in dims)

    def destroy(self):
        if self.ptr:
            lib().mluOpDestroyTensorDescriptor(self.ptr)
            self.ptr = _vp()

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass


class SparseConvDesc:
    """mluOpSparseConvolutionDescriptor_t; the three-element lists are (D, H, W)."""

    def __init__(self, batch, pad, stride, dilation, input_space, filter_space, output_space, sub_m):
        self.ptr = _vp()
        check("mluOpCreateSparseConvolutionDescriptor",
              lib().mluOpCreateSparseConvolutionDescriptor(ctypes.byref(self.ptr)))
        check("mluOpSetSparseConvolutionDescriptor",
              lib().mluOpSetSparseConvolutionDescriptor(
                  self.ptr, 5, int(batch), int_array(pad), int_array(stride), int_array(dilation),
                  int_array(input_space), int_array(filter_space), int_array(output_space), int(bool(sub_m)),
                  0, 0))
        self.batch = int(batch)
        self.pad, self.stride, self.dilation = list(pad), list(stride), list(dilation)
        self.input_space, self.filter_space = list(input_space), list(filter_space)
        self.output_space, self.sub_m = list(output_space), int(bool(sub_m))

    @property
    def kernel_volume(self):
        return self.filter_space[0] * self.filter_space[1] * self.filter_space[2]

    def num_act_out(self):
        n = ctypes.c_int(0)
        check("mluOpGetSparseConvolutionNumActOut",
              lib().mluOpGetSparseConvolutionNumActOut(self.ptr, ctypes.byref(n)))
        return n.value

    def destroy(self):
        if self.ptr:
            lib().mluOpDestroySparseConvolutionDescriptor(self.ptr)
            self.ptr = _vp()

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass


def output_space(input_space, pad, stride, dilation, filter_space):
    """o = (i + 2p - d(k-1) - 1)/s + 1 per dim: the size callers pass as output_space."""
    return [(i + 2 * p - d * (k - 1) - 1) // s + 1
            for i, p, s, d, k in zip(input_space, pad, stride, dilation, filter_space)]


def _ptr(t):
    return _vp(t.data_ptr() if t is not None else 0)


class Guards:
    """Poisoned bands around every buffer the harness allocates for a call (outputs and
    workspace), checked after the call: a kernel that writes outside the buffer it was given
    is caught even when the stray write lands in memory nobody reads.  The reference's own
    harness brackets each device buffer with a mask the same way
    (test/mlu_op_gtest/pb_gtest/src/runtime.cpp:86-145); it stands in for a memory checker.

        with ops.guarded() as guards:
            ... calls through this module ...
        # leaving the block synchronises and asserts that every band is intact
    """
    BAND = 1024  # bytes before and after; a multiple of the 256-byte alignment the library assumes

    def __init__(self):
        self.items = []

    def empty(self, shape, dtype, device):
        import torch
        shape = tuple(int(v) for v in shape)
        count = 1
        for v in shape:
            count *= v
        nbytes = count * torch.empty((), dtype=dtype).element_size()
        raw = torch.empty((2 * self.BAND + nbytes,), dtype=torch.uint8, device=device)
        gen = torch.Generator(device="cpu").manual_seed(len(self.items) + 1)
        band = torch.randint(0, 256, (2 * self.BAND,), dtype=torch.uint8, generator=gen).to(device)
        raw[:self.BAND] = band[:self.BAND]
        raw[self.BAND + nbytes:] = band[self.BAND:]
        self.items.append((raw, nbytes, band))
        return raw[self.BAND:self.BAND + nbytes].view(dtype).view(shape)

    def check(self):
        import torch
        torch.cuda.synchronize()
        for i, (raw, nbytes, band) in enumerate(self.items):
            assert torch.equal(raw[:self.BAND], band[:self.BAND]), "buffer %d: bytes before it were overwritten" % i
            assert torch.equal(raw[self.BAND + nbytes:], band[self.BAND:]), \
                "buffer %d (%d bytes): bytes after it were overwritten" % (i, nbytes)
        return len(self.items)


_guards = None


class guarded:
    """Context manager: allocations of this module get guard bands inside the block."""

    def __enter__(self):
        global _guards
        self.previous, _guards = _guards, Guards()
        return _guards

    def __exit__(self, exc_type, exc, tb):
        global _guards
        mine, _guards = _guards, self.previous
        if exc_type is None:
            mine.check()
        return False


def _alloc(shape, dtype, device):
    import torch
    if _guards is not None:
        return _guards.empty(shape, dtype, device)
    return torch.empty(tuple(shape), dtype=dtype, device=device)


def get_indice_pairs_workspace_size(handle, conv, indices_desc, pairs_desc, out_indices_desc, num_desc):
    size = _szt(0)
    check("mluOpGetIndicePairsWorkspaceSize",
          lib().mluOpGetIndicePairsWorkspaceSize(handle.ptr, conv.ptr, indices_desc.ptr, pairs_desc.ptr,
                                                 out_indices_desc.ptr, num_desc.ptr, ctypes.byref(size)))
    return size.value


def max_active_outputs(L, batch, output_space, filter_space, stride, dilation):
    """Upper bound on the active outputs of a default-mode rulebook with L inputs: an input
    reaches an output through offset k only when (i + pad - k*dilation) is a multiple of the
    stride, so per dimension at most ceil(kernel / (stride / gcd(stride, dilation))) offsets
    can be valid for one input (2 of 3 for a 3-wide kernel at stride 2).  Callers size
    out_indices by it instead of by the whole output grid."""
    import math
    per_input = 1
    for k, s, d in zip(filter_space, stride, dilation):
        period = s // math.gcd(s, d)
        per_input *= -(-k // period)
    cells = batch * output_space[0] * output_space[1] * output_space[2]
    return max(1, min(L * per_input, cells))


def get_indice_pairs(handle, conv, indices, out_rows=None, workspace=None, with_table=False):
    """Rulebook of one layer through mluOpGetIndicePairs.

    indices: int32 CUDA tensor [L,4].  Returns (indice_pairs [K,2,L], out_indices
    [out_rows,4], indice_num [K] (device), num_act_out (host int)); with_table the call
    goes through mluOpGetIndicePairsWithNeighbourTable and the table (int32 [K, rows padded
    to 512]) is appended to the result.
    """
    import torch
    L = indices.shape[0]
    K = conv.kernel_volume
    if out_rows is None:
        out_rows = L if conv.sub_m else max_active_outputs(L, conv.batch, conv.output_space, conv.filter_space,
                                                           conv.stride, conv.dilation)
    dev = indices.device
    pairs = _alloc((K, 2, L), torch.int32, dev)
    out_indices = _alloc((out_rows, 4), torch.int32, dev)
    num = _alloc((K,), torch.int32, dev)
    d_in = TensorDesc(LAYOUT_ARRAY, DTYPE_INT32, (L, 4))
    d_pairs = TensorDesc(LAYOUT_ARRAY, DTYPE_INT32, (K, 2, L))
    d_out = TensorDesc(LAYOUT_ARRAY, DTYPE_INT32, (out_rows, 4))
    d_num = TensorDesc(LAYOUT_ARRAY, DTYPE_INT32, (K,))
    ws_size = get_indice_pairs_workspace_size(handle, conv, d_in, d_pairs, d_out, d_num)
    if workspace is None or workspace.numel() < ws_size:
        workspace = _alloc((max(ws_size, 1),), torch.uint8, dev)
    args = [handle.ptr, conv.ptr, d_in.ptr, _ptr(indices), _ptr(workspace), ws_size, d_pairs.ptr, _ptr(pairs),
            d_out.ptr, _ptr(out_indices), d_num.ptr, _ptr(num)]
    table = None
    try:
        if with_table:
            size = _szt(0)
            check("mluOpGetIndiceNeighbourTableSize",
                  lib().mluOpGetIndiceNeighbourTableSize(handle.ptr, d_pairs.ptr, L, ctypes.byref(size)))
            table = _alloc((K, size.value // (4 * K)), torch.int32, dev)
            check("mluOpGetIndicePairsWithNeighbourTable",
                  lib().mluOpGetIndicePairsWithNeighbourTable(*args, _ptr(table), size.value))
        else:
            check("mluOpGetIndicePairs", lib().mluOpGetIndicePairs(*args))
    finally:
        for d in (d_in, d_pairs, d_out, d_num):
            d.destroy()
    n_out = conv.num_act_out()
    if with_table:
        return pairs, out_indices, num, n_out, table
    return pairs, out_indices, num, n_out


def build_neighbour_table(handle, indice_pairs, indice_num, num_act_out):
    """The neighbour table of a rulebook from its pair lists (mluOpBuildIndiceNeighbourTable):
    int32 [K, rows padded to 512]."""
    import torch
    K, _, L = indice_pairs.shape
    d_pairs = TensorDesc(LAYOUT_ARRAY, DTYPE_INT32, (K, 2, L))
    size = _szt(0)
    try:
        check("mluOpGetIndiceNeighbourTableSize",
              lib().mluOpGetIndiceNeighbourTableSize(handle.ptr, d_pairs.ptr, num_act_out, ctypes.byref(size)))
        table = _alloc((K, size.value // (4 * K)), torch.int32, indice_pairs.device)
        check("mluOpBuildIndiceNeighbourTable",
              lib().mluOpBuildIndiceNeighbourTable(handle.ptr, d_pairs.ptr, _ptr(indice_pairs),
                                                   i64_array([int(v) for v in indice_num]), num_act_out,
                                                   _ptr(table), size.value))
    finally:
        d_pairs.destroy()
    return table


def build_input_neighbour_table(handle, indice_pairs, indice_num, num_act_out):
    """The table the input gradient works from (mluOpBuildIndiceInputNeighbourTable): for every
    kernel offset and input row the output row it feeds, int32 [K, L padded to 512]."""
    import torch
    K, _, L = indice_pairs.shape
    d_pairs = TensorDesc(LAYOUT_ARRAY, DTYPE_INT32, (K, 2, L))
    size = _szt(0)
    try:
        check("mluOpGetIndiceInputNeighbourTableSize",
              lib().mluOpGetIndiceInputNeighbourTableSize(handle.ptr, d_pairs.ptr, ctypes.byref(size)))
        table = _alloc((K, size.value // (4 * K)), torch.int32, indice_pairs.device)
        check("mluOpBuildIndiceInputNeighbourTable",
              lib().mluOpBuildIndiceInputNeighbourTable(handle.ptr, d_pairs.ptr, _ptr(indice_pairs),
                                                        i64_array([int(v) for v in indice_num]), num_act_out,
                                                        _ptr(table), size.value))
    finally:
        d_pairs.destroy()
    return table


FILTER_LAYOUTS = {"ARRAY": LAYOUT_ARRAY, "NDHWC": LAYOUT_NDHWC, "NCDHW": LAYOUT_NCDHW,
                  "HWCN": LAYOUT_HWCN, "NHWC": LAYOUT_NHWC, "NCHW": LAYOUT_NCHW}


def filter_dims(layout, filter_space, ci, co):
    kd, kh, kw = filter_space
    if layout == "ARRAY":
        return (kd, kh, kw, ci, co)
    if layout == "NDHWC":
        return (co, kd, kh, kw, ci)
    if layout == "NCDHW":
        return (co, ci, kd, kh, kw)
    raise ValueError(layout)


def indice_convolution_forward(handle, features, filters, filter_layout, filter_space, indice_pairs,
                               indice_num_host, num_act_out, sub_m, workspace=None, out=None, table=None):
    """features_out [num_act_out, Co] through mluOpIndiceConvolutionForward.

    features [L,Ci] and filters (5-D, in `filter_layout`) are CUDA tensors of the
    same dtype (float16 or float32); indice_num_host is a sequence of K ints.  table: the
    rulebook's neighbour table (build_neighbour_table); with it the call is
    mluOpIndiceConvolutionForwardFromTable and indice_pairs only gives the shapes.
    """
    import torch
    L, ci = features.shape
    dims = tuple(filters.shape)
    co = dims[4] if filter_layout == "ARRAY" else dims[0]
    K = indice_pairs.shape[0]
    dt = DTYPE_HALF if features.dtype == torch.float16 else DTYPE_FLOAT
    dev = features.device
    if out is None:
        out = _alloc((num_act_out, co), features.dtype, dev)
    d_f = TensorDesc(LAYOUT_ARRAY, dt, (L, ci))
    d_w = TensorDesc(FILTER_LAYOUTS[filter_layout], dt, dims)
    d_p = TensorDesc(LAYOUT_ARRAY, DTYPE_INT32, (K, 2, L))
    d_o = TensorDesc(LAYOUT_ARRAY, dt, (num_act_out, co))
    num = i64_array(indice_num_host)
    size = _szt(0)
    if table is not None:
        check("mluOpGetIndiceConvolutionForwardFromTableWorkspaceSize",
              lib().mluOpGetIndiceConvolutionForwardFromTableWorkspaceSize(handle.ptr, d_f.ptr, d_w.ptr, d_p.ptr,
                                                                           d_o.ptr, num, num_act_out, 0,
                                                                           int(bool(sub_m)), ctypes.byref(size)))
        if workspace is None or workspace.numel() < size.value:
            workspace = _alloc((max(size.value, 1),), torch.uint8, dev)
        check("mluOpIndiceConvolutionForwardFromTable",
              lib().mluOpIndiceConvolutionForwardFromTable(handle.ptr, d_f.ptr, _ptr(features), d_w.ptr,
                                                           _ptr(filters), d_p.ptr, _ptr(table), table.numel() * 4,
                                                           num, num_act_out, 0, int(bool(sub_m)), _ptr(workspace),
                                                           size.value, d_o.ptr, _ptr(out)))
        for d in (d_f, d_w, d_p, d_o):
            d.destroy()
        return out
    check("mluOpGetIndiceConvolutionForwardWorkspaceSize",
          lib().mluOpGetIndiceConvolutionForwardWorkspaceSize(handle.ptr, d_f.ptr, d_w.ptr, d_p.ptr, d_o.ptr,
                                                              num, num_act_out, 0, int(bool(sub_m)),
                                                              ctypes.byref(size)))
    if workspace is None or workspace.numel() < size.value:
        workspace = _alloc((max(size.value, 1),), torch.uint8, dev)
    check("mluOpIndiceConvolutionForward",
          lib().mluOpIndiceConvolutionForward(handle.ptr, d_f.ptr, _ptr(features), d_w.ptr, _ptr(filters),
                                              d_p.ptr, _ptr(indice_pairs), num, num_act_out, 0,
                                              int(bool(sub_m)), _ptr(workspace), size.value, d_o.ptr,
                                              _ptr(out)))
    for d in (d_f, d_w, d_p, d_o):
        d.destroy()
    return out


def indice_convolution_backward_data(handle, output_grad, filters, filter_layout, indice_pairs,
                                     indice_num_host, sub_m, workspace=None, out=None, table=None,
                                     forward_table=None):
    """input_grad [L, Ci] through mluOpIndiceConvolutionBackwardData.

    output_grad [N_out,Co] and filters (4-D or 5-D, in `filter_layout`: ARRAY, HWCN,
    NDHWC, NCDHW, NHWC, NCHW) are CUDA tensors of the same dtype; L is indice_pairs'
    last dimension; indice_num_host is a sequence of K ints.  table: the rulebook's input
    neighbour table (build_input_neighbour_table); with it the call is
    mluOpIndiceConvolutionBackwardDataFromTable and indice_pairs only gives the shapes.
    forward_table: the FORWARD table of a submanifold rulebook with centred padding; tried first
    (mluOpIndiceConvolutionBackwardDataFromForwardTable), NOT_SUPPORTED falls through to the rest;
    a callable is called for `table` only then.
    """
    import torch
    n_out, co = output_grad.shape
    dims = tuple(filters.shape)
    if filter_layout in ("ARRAY", "HWCN"):
        ci = dims[-2]
    elif filter_layout in ("NDHWC", "NHWC"):
        ci = dims[-1]
    else:
        ci = dims[1]
    K, _, L = indice_pairs.shape
    dt = DTYPE_HALF if output_grad.dtype == torch.float16 else DTYPE_FLOAT
    dev = output_grad.device
    if out is None:
        out = _alloc((L, ci), output_grad.dtype, dev)
    d_g = TensorDesc(LAYOUT_ARRAY, dt, (n_out, co))
    d_w = TensorDesc(FILTER_LAYOUTS[filter_layout], dt, dims)
    d_p = TensorDesc(LAYOUT_ARRAY, DTYPE_INT32, (K, 2, L))
    d_o = TensorDesc(LAYOUT_ARRAY, dt, (L, ci))
    num = i64_array(indice_num_host)
    size = _szt(0)
    if forward_table is not None and sub_m:
        check("mluOpGetIndiceConvolutionBackwardDataFromTableWorkspaceSize",
              lib().mluOpGetIndiceConvolutionBackwardDataFromTableWorkspaceSize(handle.ptr, d_g.ptr, d_w.ptr, d_p.ptr,
                                                                                d_o.ptr, num, 0, ctypes.byref(size)))
        if workspace is None or workspace.numel() < size.value:
            workspace = _alloc((max(size.value, 1),), torch.uint8, dev)
        st = lib().mluOpIndiceConvolutionBackwardDataFromForwardTable(
            handle.ptr, d_g.ptr, _ptr(output_grad), d_w.ptr, _ptr(filters), d_p.ptr, _ptr(forward_table),
            forward_table.numel() * 4, num, 0, 1, _ptr(workspace), size.value, d_o.ptr, _ptr(out))
        if st != STATUS_NOT_SUPPORTED:
            check("mluOpIndiceConvolutionBackwardDataFromForwardTable", st)
            for d in (d_g, d_w, d_p, d_o):
                d.destroy()
            return out
    if callable(table):
        table = table()
    if table is not None:
        check("mluOpGetIndiceConvolutionBackwardDataFromTableWorkspaceSize",
              lib().mluOpGetIndiceConvolutionBackwardDataFromTableWorkspaceSize(handle.ptr, d_g.ptr, d_w.ptr, d_p.ptr,
                                                                                d_o.ptr, num, 0, ctypes.byref(size)))
        if workspace is None or workspace.numel() < size.value:
            workspace = _alloc((max(size.value, 1),), torch.uint8, dev)
        check("mluOpIndiceConvolutionBackwardDataFromTable",
              lib().mluOpIndiceConvolutionBackwardDataFromTable(handle.ptr, d_g.ptr, _ptr(output_grad), d_w.ptr,
                                                                _ptr(filters), d_p.ptr, _ptr(table),
                                                                table.numel() * 4, num, 0, int(bool(sub_m)),
                                                                _ptr(workspace), size.value, d_o.ptr, _ptr(out)))
        for d in (d_g, d_w, d_p, d_o):
            d.destroy()
        return out
    check("mluOpGetIndiceConvolutionBackwardDataWorkspaceSize",
          lib().mluOpGetIndiceConvolutionBackwardDataWorkspaceSize(handle.ptr, d_g.ptr, d_w.ptr, d_p.ptr, d_o.ptr,
                                                                   num, 0, ctypes.byref(size)))
    if workspace is None or workspace.numel() < size.value:
        workspace = _alloc((max(size.value, 1),), torch.uint8, dev)
    check("mluOpIndiceConvolutionBackwardData",
          lib().mluOpIndiceConvolutionBackwardData(handle.ptr, d_g.ptr, _ptr(output_grad), d_w.ptr, _ptr(filters),
                                                   d_p.ptr, _ptr(indice_pairs), num, 0, int(bool(sub_m)),
                                                   _ptr(workspace), size.value, d_o.ptr, _ptr(out)))
    for d in (d_g, d_w, d_p, d_o):
        d.destroy()
    return out


def indice_convolution_backward_filter(handle, features, output_grad, filter_space, indice_pairs,
                                       indice_num_host, sub_m, workspace=None, out=None, table=None,
                                     forward_table=None):
    """filters_grad [kd,kh,kw,Ci,Co] through mluOpIndiceConvolutionBackwardFilter.

    features [L,Ci] and output_grad [N_out,Co] are CUDA tensors of the same dtype;
    indice_num_host is a sequence of K = kd*kh*kw ints.  table: the rulebook's FORWARD
    neighbour table; with it the call is mluOpIndiceConvolutionBackwardFilterFromTable where the
    shapes allow it (STATUS_NOT_SUPPORTED falls back to the reference-shaped call).
    """
    import torch
    L, ci = features.shape
    n_out, co = output_grad.shape
    K = indice_pairs.shape[0]
    dt = DTYPE_HALF if features.dtype == torch.float16 else DTYPE_FLOAT
    dev = features.device
    dims = tuple(filter_space) + (ci, co)
    if out is None:
        out = _alloc(dims, features.dtype, dev)
    d_f = TensorDesc(LAYOUT_ARRAY, dt, (L, ci))
    d_g = TensorDesc(LAYOUT_ARRAY, dt, (n_out, co))
    d_p = TensorDesc(LAYOUT_ARRAY, DTYPE_INT32, (K, 2, L))
    d_w = TensorDesc(LAYOUT_ARRAY, dt, dims)
    num = i64_array(indice_num_host)
    size = _szt(0)
    check("mluOpGetIndiceConvolutionBackwardFilterWorkspaceSize",
          lib().mluOpGetIndiceConvolutionBackwardFilterWorkspaceSize(handle.ptr, d_f.ptr, d_g.ptr, d_p.ptr,
                                                                     d_w.ptr, num, 0, int(bool(sub_m)),
                                                                     ctypes.byref(size)))
    if workspace is None or workspace.numel() < size.value:
        workspace = _alloc((max(size.value, 1),), torch.uint8, dev)
    st = STATUS_NOT_SUPPORTED
    if table is not None:
        st = lib().mluOpIndiceConvolutionBackwardFilterFromTable(handle.ptr, d_f.ptr, _ptr(features), d_g.ptr,
                                                                 _ptr(output_grad), d_p.ptr, _ptr(table),
                                                                 table.numel() * 4, num, 0, int(bool(sub_m)),
                                                                 _ptr(workspace), size.value, d_w.ptr, _ptr(out))
        if st != STATUS_NOT_SUPPORTED:
            check("mluOpIndiceConvolutionBackwardFilterFromTable", st)
    if st == STATUS_NOT_SUPPORTED:
        check("mluOpIndiceConvolutionBackwardFilter",
              lib().mluOpIndiceConvolutionBackwardFilter(handle.ptr, d_f.ptr, _ptr(features), d_g.ptr,
                                                         _ptr(output_grad), d_p.ptr, _ptr(indice_pairs), num, 0,
                                                         int(bool(sub_m)), _ptr(workspace), size.value, d_w.ptr,
                                                         _ptr(out)))
    for d in (d_f, d_g, d_p, d_w):
        d.destroy()
    return out


def voxelization(handle, points, voxel_size, coors_range, max_points, max_voxels, workspace=None):
    """Deterministic hard voxelization through mluOpVoxelization.

    points [N,F] float32 (x, y, z first), voxel_size [3] and coors_range [6] float32,
    all CUDA tensors.  Returns (voxels [max_voxels,max_points,F], coors [max_voxels,3]
    int32 (z,y,x), num_points_per_voxel [max_voxels] int32, voxel_num [1] int32), all on
    the device.
    """
    import torch
    n, f = points.shape
    dev = points.device
    voxels = _alloc((max_voxels, max_points, f), torch.float32, dev)
    coors = _alloc((max_voxels, 3), torch.int32, dev)
    npv = _alloc((max_voxels,), torch.int32, dev)
    num = torch.zeros((1,), dtype=torch.int32, device=dev)
    descs = [TensorDesc(LAYOUT_ARRAY, DTYPE_FLOAT, (n, f)), TensorDesc(LAYOUT_ARRAY, DTYPE_FLOAT, (3,)),
             TensorDesc(LAYOUT_ARRAY, DTYPE_FLOAT, (6,)), TensorDesc(LAYOUT_ARRAY, DTYPE_FLOAT, tuple(voxels.shape)),
             TensorDesc(LAYOUT_ARRAY, DTYPE_INT32, (max_voxels, 3)), TensorDesc(LAYOUT_ARRAY, DTYPE_INT32, (max_voxels,)),
             TensorDesc(LAYOUT_ARRAY, DTYPE_INT32, (1,))]
    d_p, d_vs, d_cr, d_v, d_c, d_n, d_num = (d.ptr for d in descs)
    size = _szt(0)
    check("mluOpGetVoxelizationWorkspaceSize",
          lib().mluOpGetVoxelizationWorkspaceSize(handle.ptr, d_p, d_vs, d_cr, max_points, max_voxels, 3, True, d_v,
                                                  d_c, d_n, d_num, ctypes.byref(size)))
    if workspace is None or workspace.numel() < size.value:
        workspace = _alloc((max(size.value, 1),), torch.uint8, dev)
    check("mluOpVoxelization",
          lib().mluOpVoxelization(handle.ptr, d_p, _ptr(points), d_vs, _ptr(voxel_size), d_cr, _ptr(coors_range),
                                  max_points, max_voxels, 3, True, _ptr(workspace), size.value, d_v, _ptr(voxels),
                                  d_c, _ptr(coors), d_n, _ptr(npv), d_num, _ptr(num)))
    for d in descs:
        d.destroy()
    return voxels, coors, npv, num


REDUCE_MODES = {"sum": 0, "mean": 1, "max": 2}


def dynamic_point_to_voxel_forward(handle, feats, coors, reduce_type="max", workspace=None):
    """Groups points by voxel through mluOpDynamicPointToVoxelForward.

    feats [N,C] float32 and coors [N,3] int32 are CUDA tensors; coors rows with a
    negative entry are overwritten with -1 (as the reference does).  Returns
    (voxel_feats [N,C], voxel_coors [N,3], point2voxel_map [N], voxel_points_count [N],
    voxel_num [1]), all on the device; the first voxel_num rows are the voxels.
    """
    import torch
    n, c = feats.shape
    dev = feats.device
    voxel_feats = _alloc((n, c), torch.float32, dev)
    voxel_coors = _alloc((n, 3), torch.int32, dev)
    p2v = _alloc((n,), torch.int32, dev)
    counts = _alloc((n,), torch.int32, dev)
    num = torch.zeros((1,), dtype=torch.int32, device=dev)
    descs = [TensorDesc(LAYOUT_ARRAY, DTYPE_FLOAT, (n, c)), TensorDesc(LAYOUT_ARRAY, DTYPE_INT32, (n, 3)),
             TensorDesc(LAYOUT_ARRAY, DTYPE_FLOAT, (n, c)), TensorDesc(LAYOUT_ARRAY, DTYPE_INT32, (n, 3)),
             TensorDesc(LAYOUT_ARRAY, DTYPE_INT32, (n,)), TensorDesc(LAYOUT_ARRAY, DTYPE_INT32, (n,)),
             TensorDesc(LAYOUT_ARRAY, DTYPE_INT32, (1,))]
    d_f, d_c, d_vf, d_vc, d_map, d_cnt, d_num = (d.ptr for d in descs)
    size = _szt(0)
    check("mluOpGetDynamicPointToVoxelForwardWorkspaceSize",
          lib().mluOpGetDynamicPointToVoxelForwardWorkspaceSize(handle.ptr, d_f, d_c, ctypes.byref(size)))
    if workspace is None or workspace.numel() < size.value:
        workspace = _alloc((max(size.value, 1),), torch.uint8, dev)
    check("mluOpDynamicPointToVoxelForward",
          lib().mluOpDynamicPointToVoxelForward(handle.ptr, REDUCE_MODES[reduce_type], d_f, _ptr(feats), d_c,
                                                _ptr(coors), _ptr(workspace), size.value, d_vf, _ptr(voxel_feats),
                                                d_vc, _ptr(voxel_coors), d_map, _ptr(p2v), d_cnt, _ptr(counts),
                                                d_num, _ptr(num)))
    for d in descs:
        d.destroy()
    return voxel_feats, voxel_coors, p2v, counts, num


def dynamic_point_to_voxel_backward(handle, grad_voxel_feats, feats, voxel_feats, point2voxel_map,
                                    voxel_points_count, voxel_num):
    """grad_feats [N,C] of the maximum reduction through mluOpDynamicPointToVoxelBackward."""
    import torch
    n, c = feats.shape
    m = grad_voxel_feats.shape[0]
    dev = feats.device
    grad_feats = _alloc((n, c), torch.float32, dev)
    descs = [TensorDesc(LAYOUT_ARRAY, DTYPE_FLOAT, (m, c)), TensorDesc(LAYOUT_ARRAY, DTYPE_FLOAT, (n, c)),
             TensorDesc(LAYOUT_ARRAY, DTYPE_FLOAT, (m, c)), TensorDesc(LAYOUT_ARRAY, DTYPE_INT32, (n,)),
             TensorDesc(LAYOUT_ARRAY, DTYPE_INT32, (m,)), TensorDesc(LAYOUT_ARRAY, DTYPE_INT32, (1,)),
             TensorDesc(LAYOUT_ARRAY, DTYPE_FLOAT, (n, c))]
    d_g, d_f, d_vf, d_map, d_cnt, d_num, d_out = (d.ptr for d in descs)
    size = _szt(0)
    check("mluOpGetDynamicPointToVoxelBackwardWorkspaceSize",
          lib().mluOpGetDynamicPointToVoxelBackwardWorkspaceSize(handle.ptr, REDUCE_MODES["max"], d_g, d_f, d_vf,
                                                                 d_map, d_cnt, d_num, ctypes.byref(size)))
    workspace = _alloc((max(size.value, 1),), torch.uint8, dev)
    check("mluOpDynamicPointToVoxelBackward",
          lib().mluOpDynamicPointToVoxelBackward(handle.ptr, REDUCE_MODES["max"], d_g, _ptr(grad_voxel_feats), d_f,
                                                 _ptr(feats), d_vf, _ptr(voxel_feats), d_map, _ptr(point2voxel_map),
                                                 d_cnt, _ptr(voxel_points_count), d_num, _ptr(voxel_num),
                                                 _ptr(workspace), size.value, d_out, _ptr(grad_feats)))
    for d in descs:
        d.destroy()
    return grad_feats
