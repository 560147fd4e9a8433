"""ctypes access to the CPU oracle (and, when built, the reference's own CPU code).

TEST INFRASTRUCTURE ONLY: imported by tests/, the smoke check and the
CPU-baseline leg of bench.py.  The shipped library never touches this package.

  oracle.lib()      -> the plain-C restatement (oracle/sparse_conv_oracle.c,
                       oracle/sparse_conv_backward_oracle.c, oracle/voxelization_oracle.c)
  oracle.ref_lib()  -> the reference's function bodies compiled by
                       oracle/build_ref.py, or None when that library is absent
"""
import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "sparse_conv_oracle.c")
SRC_BACKWARD = os.path.join(HERE, "sparse_conv_backward_oracle.c")
SRC_VOXEL = os.path.join(HERE, "voxelization_oracle.c")
LIB = os.path.join(HERE, "_build", "libmluops_oracle.so")
LIB_THREADS = os.path.join(HERE, "_build", "libmluops_oracle_threads.so")
REF_LIB = os.path.join(HERE, "_ref", "libmluops_ref_cpu.so")

_i32p = ctypes.POINTER(ctypes.c_int32)
_i64p = ctypes.POINTER(ctypes.c_int64)
_f32p = ctypes.POINTER(ctypes.c_float)
_u16p = ctypes.POINTER(ctypes.c_uint16)
_f64p = ctypes.POINTER(ctypes.c_double)

FILTER_LAYOUT = {"ARRAY": 0, "NDHWC": 1, "NCDHW": 2}


def build(force=False):
    """Compile the C oracle with gcc (a second or two)."""
    newest = max(os.path.getmtime(SRC), os.path.getmtime(SRC_BACKWARD), os.path.getmtime(SRC_VOXEL))
    if force or not os.path.isfile(LIB) or os.path.getmtime(LIB) < newest:
        os.makedirs(os.path.dirname(LIB), exist_ok=True)
        subprocess.check_call(["gcc", "-O2", "-std=c11", "-fPIC", "-shared", "-o", LIB, SRC, SRC_BACKWARD, SRC_VOXEL, "-lm"])
    if force or not os.path.isfile(LIB_THREADS) or os.path.getmtime(LIB_THREADS) < newest:
        # the all-cores timing baseline: vectorised, OpenMP where the toolchain has it
        base = ["gcc", "-O3", "-mavx2", "-mfma", "-std=c11", "-fPIC", "-shared", "-o", LIB_THREADS, SRC, "-lm"]
        if subprocess.call(base[:1] + ["-fopenmp"] + base[1:], stderr=subprocess.DEVNULL) != 0:
            subprocess.check_call(base)
    return LIB


_threads_lib = None


def threads_lib():
    """The C restatement built for timing on all cores (-O3, AVX2, OpenMP)."""
    global _threads_lib
    if _threads_lib is None:
        build()
        _threads_lib = ctypes.CDLL(LIB_THREADS)
    return _threads_lib


_lib = None
_ref = None


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(LIB)
        _lib.mluops_oracle_float_to_half_bits.restype = ctypes.c_uint16
        _lib.mluops_oracle_float_to_half_bits.argtypes = [ctypes.c_float]
        _lib.mluops_oracle_half_bits_to_float.restype = ctypes.c_float
        _lib.mluops_oracle_half_bits_to_float.argtypes = [ctypes.c_uint16]
    return _lib


def ref_lib():
    global _ref
    if _ref is None and os.path.isfile(REF_LIB):
        _ref = ctypes.CDLL(REF_LIB)
        _ref.mluops_ref_float_to_half_bits.restype = ctypes.c_uint16
        _ref.mluops_ref_float_to_half_bits.argtypes = [ctypes.c_float]
    return _ref


def _p(a, t):
    return a.ctypes.data_as(t)


def _i32x3(v):
    a = np.ascontiguousarray(np.asarray(v, dtype=np.int32))
    assert a.shape == (3,)
    return a


def kernel_volume(filter_space):
    return int(np.prod(filter_space))


def get_indice_pairs(indices, batch, pad, stride, dilation, filter_space, out_space, sub_m,
                     out_rows=None, sentinel_quirk=False, use_ref=False):
    """Rulebook of one sparse convolution.

    Returns (indice_pairs [K,2,L], out_indices [out_rows,4], indice_num [K], num_act_out).
    With use_ref the reference's own compiled code runs (num_act_out is then
    derived from out_indices, since that code does not return it).
    """
    indices = np.ascontiguousarray(indices, dtype=np.int32)
    L = indices.shape[0]
    K = kernel_volume(filter_space)
    if out_rows is None:
        out_rows = L if sub_m else min(K * L, int(batch) * int(np.prod(out_space)))
        out_rows = max(out_rows, 1)
    pairs = np.empty((K, 2, L), dtype=np.int32)
    out_indices = np.empty((out_rows, 4), dtype=np.int32)
    num = np.empty((K,), dtype=np.int32)
    pad, stride, dilation = _i32x3(pad), _i32x3(stride), _i32x3(dilation)
    fs, osp = _i32x3(filter_space), _i32x3(out_space)
    if use_ref:
        r = ref_lib()
        assert r is not None, "oracle/_ref is not built"
        rc = r.mluops_ref_get_indice_pairs(
            _p(indices, _i32p), ctypes.c_int32(L), ctypes.c_int32(batch), _p(pad, _i32p),
            _p(stride, _i32p), _p(dilation, _i32p), _p(fs, _i32p), _p(osp, _i32p),
            ctypes.c_int32(int(sub_m)), _p(pairs, _i32p), _p(out_indices, _i32p),
            ctypes.c_int64(out_rows), _p(num, _i32p))
        assert rc == 0
        n_out = L if sub_m else int((out_indices[:, 0] >= 0).sum())
        return pairs, out_indices, num, n_out
    n_out = ctypes.c_int32(0)
    rc = lib().mluops_oracle_get_indice_pairs(
        _p(indices, _i32p), ctypes.c_int32(L), ctypes.c_int32(batch), _p(pad, _i32p),
        _p(stride, _i32p), _p(dilation, _i32p), _p(fs, _i32p), _p(osp, _i32p),
        ctypes.c_int32(int(sub_m)), _p(pairs, _i32p), _p(out_indices, _i32p),
        ctypes.c_int64(out_rows), _p(num, _i32p), ctypes.byref(n_out),
        ctypes.c_int32(int(sentinel_quirk)))
    assert rc == 0, "oracle allocation failed"
    return pairs, out_indices, num, int(n_out.value)


def indice_convolution_forward(features, filters, filter_layout, filter_space, indice_pairs,
                               indice_num, num_act_out, co, use_ref=False, fast=False, threads=False):
    """features_out [num_act_out, co] float32, accumulated in the reference order.

    features/filters are float32 arrays holding the values the device sees (for
    a half device dtype: already rounded through half).  `fast` drops the
    product-rounding barrier and `threads` also shares the pairs of an offset among
    OpenMP threads (timed baselines only; filters must be ARRAY layout).
    """
    features = np.ascontiguousarray(features, dtype=np.float32)
    filters = np.ascontiguousarray(filters, dtype=np.float32)
    pairs = np.ascontiguousarray(indice_pairs, dtype=np.int32)
    num = np.ascontiguousarray(indice_num, dtype=np.int64)
    L, ci = features.shape
    K = kernel_volume(filter_space)
    out = np.empty((num_act_out, co), dtype=np.float32)
    code = FILTER_LAYOUT[filter_layout]
    if use_ref:
        r = ref_lib()
        assert r is not None, "oracle/_ref is not built"
        kdhw = _i32x3(filter_space)
        rc = r.mluops_ref_indice_convolution_forward(
            _p(features, _f32p), _p(filters, _f32p), ctypes.c_int32(code), _p(kdhw, _i32p),
            _p(pairs, _i32p), _p(num, _i64p), ctypes.c_int64(L), ctypes.c_int64(ci),
            ctypes.c_int64(co), ctypes.c_int64(num_act_out), _p(out, _f32p))
    elif threads:
        assert code == 0
        rc = threads_lib().mluops_oracle_indice_convolution_forward_threads(
            _p(features, _f32p), _p(filters, _f32p), _p(pairs, _i32p), _p(num, _i64p),
            ctypes.c_int64(L), ctypes.c_int64(ci), ctypes.c_int64(co), ctypes.c_int64(K),
            ctypes.c_int64(num_act_out), _p(out, _f32p))
    elif fast:
        assert code == 0
        rc = lib().mluops_oracle_indice_convolution_forward_fast(
            _p(features, _f32p), _p(filters, _f32p), _p(pairs, _i32p), _p(num, _i64p),
            ctypes.c_int64(L), ctypes.c_int64(ci), ctypes.c_int64(co), ctypes.c_int64(K),
            ctypes.c_int64(num_act_out), _p(out, _f32p))
    else:
        rc = lib().mluops_oracle_indice_convolution_forward(
            _p(features, _f32p), _p(filters, _f32p), ctypes.c_int32(code), _p(pairs, _i32p),
            _p(num, _i64p), ctypes.c_int64(L), ctypes.c_int64(ci), ctypes.c_int64(co),
            ctypes.c_int64(K), ctypes.c_int64(num_act_out), _p(out, _f32p))
    assert rc == 0
    return out


def indice_convolution_backward_data(output_grad, filters, filter_layout, filter_space, indice_pairs,
                                     indice_num, ci, is_half, use_ref=False):
    """input_grad [L, ci] float32 in the reference's accumulation order.  output_grad/filters
    hold the values the device sees; is_half selects the reference's half emulation
    (products and per-pair running sums rounded through half)."""
    og = np.ascontiguousarray(output_grad, dtype=np.float32)
    filters = np.ascontiguousarray(filters, dtype=np.float32)
    pairs = np.ascontiguousarray(indice_pairs, dtype=np.int32)
    num = np.ascontiguousarray(indice_num, dtype=np.int64)
    n_out, co = og.shape
    L = pairs.shape[2]
    K = kernel_volume(filter_space)
    out = np.empty((L, ci), dtype=np.float32)
    code = FILTER_LAYOUT[filter_layout]
    if use_ref:
        r = ref_lib()
        assert r is not None, "oracle/_ref is not built"
        kdhw = _i32x3(filter_space)
        rc = r.mluops_ref_indice_convolution_backward_data(
            _p(og, _f32p), _p(filters, _f32p), ctypes.c_int32(code), _p(kdhw, _i32p), _p(pairs, _i32p),
            _p(num, _i64p), ctypes.c_int64(L), ctypes.c_int64(ci), ctypes.c_int64(co),
            ctypes.c_int64(n_out), ctypes.c_int32(int(is_half)), _p(out, _f32p))
    else:
        rc = lib().mluops_oracle_indice_convolution_backward_data(
            _p(og, _f32p), _p(filters, _f32p), ctypes.c_int32(code), _p(pairs, _i32p), _p(num, _i64p),
            ctypes.c_int64(L), ctypes.c_int64(ci), ctypes.c_int64(co), ctypes.c_int64(K),
            ctypes.c_int32(int(is_half)), _p(out, _f32p))
    assert rc == 0
    return out


def indice_convolution_backward_filter(features, output_grad, filter_space, indice_pairs, indice_num,
                                       use_ref=False):
    """filters_grad [K, ci, co] float32: one float accumulator per element over the pair list."""
    feats = np.ascontiguousarray(features, dtype=np.float32)
    og = np.ascontiguousarray(output_grad, dtype=np.float32)
    pairs = np.ascontiguousarray(indice_pairs, dtype=np.int32)
    num = np.ascontiguousarray(indice_num, dtype=np.int64)
    L, ci = feats.shape
    n_out, co = og.shape
    K = kernel_volume(filter_space)
    out = np.zeros((K, ci, co), dtype=np.float32)
    if use_ref:
        r = ref_lib()
        assert r is not None, "oracle/_ref is not built"
        kdhw = _i32x3(filter_space)
        rc = r.mluops_ref_indice_convolution_backward_filter(
            _p(feats, _f32p), _p(og, _f32p), _p(kdhw, _i32p), _p(pairs, _i32p), _p(num, _i64p),
            ctypes.c_int64(L), ctypes.c_int64(ci), ctypes.c_int64(co), ctypes.c_int64(n_out),
            _p(out, _f32p))
    else:
        rc = lib().mluops_oracle_indice_convolution_backward_filter(
            _p(feats, _f32p), _p(og, _f32p), _p(pairs, _i32p), _p(num, _i64p), ctypes.c_int64(L),
            ctypes.c_int64(ci), ctypes.c_int64(co), ctypes.c_int64(K), _p(out, _f32p))
    assert rc == 0
    return out


def voxelization(points, voxel_size, coors_range, max_points, max_voxels, use_ref=False):
    """Deterministic hard voxelization of points [N,F] float32.  Returns (voxels
    [max_voxels,max_points,F] float32, coors [max_voxels,3] int32 (z,y,x),
    num_points_per_voxel [max_voxels] int32, voxel_num int)."""
    pts = np.ascontiguousarray(points, dtype=np.float32)
    vs = np.ascontiguousarray(voxel_size, dtype=np.float32)
    cr = np.ascontiguousarray(coors_range, dtype=np.float32)
    n, f = pts.shape
    voxels = np.zeros((max_voxels, max_points, f), dtype=np.float32)
    coors = np.zeros((max_voxels, 3), dtype=np.int32)
    npv = np.zeros((max_voxels,), dtype=np.int32)
    num = ctypes.c_int32(0)
    fn = None
    if use_ref:
        r = ref_lib()
        assert r is not None, "oracle/_ref is not built"
        fn = r.mluops_ref_voxelization
    else:
        fn = lib().mluops_oracle_voxelization
    rc = fn(_p(pts, _f32p), ctypes.c_int64(n), ctypes.c_int64(f), _p(vs, _f32p), _p(cr, _f32p),
            ctypes.c_int32(max_points), ctypes.c_int32(max_voxels), _p(voxels, _f32p), _p(coors, _i32p),
            _p(npv, _i32p), ctypes.byref(num))
    assert rc == 0
    return voxels, coors, npv, int(num.value)


def dynamic_point_to_voxel_forward(feats, coors, reduce_type="max", use_ref=False):
    """Groups points by voxel.  feats [N,C] float32, coors [N,3] int32 (a copy is modified).
    Returns (voxel_feats [N,C], voxel_coors [N,3], point2voxel_map [N], voxel_points_count [N],
    voxel_num, coors after the -1 fill); only the first voxel_num rows of the voxel_* arrays and
    all of point2voxel_map are defined by the reference."""
    f = np.ascontiguousarray(feats, dtype=np.float32)
    c = np.array(coors, dtype=np.int32, order="C", copy=True)
    n, cn = f.shape
    vf = np.zeros((n, cn), dtype=np.float32)
    vc = np.zeros((n, 3), dtype=np.int32)
    p2v = np.zeros((n,), dtype=np.int32)
    cnt = np.zeros((n,), dtype=np.int32)
    num = ctypes.c_int32(0)
    if use_ref:
        r = ref_lib()
        assert r is not None, "oracle/_ref is not built"
        fn = r.mluops_ref_dynamic_point_to_voxel_forward
    else:
        fn = lib().mluops_oracle_dynamic_point_to_voxel_forward
    rc = fn(_p(f, _f32p), _p(c, _i32p), ctypes.c_int64(n), ctypes.c_int64(cn), ctypes.c_int64(n),
            ctypes.c_int32(1 if reduce_type == "max" else 0), _p(vf, _f32p), _p(vc, _i32p), _p(p2v, _i32p),
            _p(cnt, _i32p), ctypes.byref(num))
    assert rc == 0
    return vf, vc, p2v, cnt, int(num.value), c


def dynamic_point_to_voxel_backward(grad_voxel_feats, feats, voxel_feats, point2voxel_map, voxel_num,
                                    use_ref=False):
    """grad_feats [N,C] float32 of the maximum reduction."""
    g = np.ascontiguousarray(grad_voxel_feats, dtype=np.float32)
    f = np.ascontiguousarray(feats, dtype=np.float32)
    vf = np.ascontiguousarray(voxel_feats, dtype=np.float32)
    p2v = np.ascontiguousarray(point2voxel_map, dtype=np.int32)
    n, c = f.shape
    out = np.zeros((n, c), dtype=np.float32)
    if use_ref:
        r = ref_lib()
        assert r is not None, "oracle/_ref is not built"
        fn = r.mluops_ref_dynamic_point_to_voxel_backward
    else:
        fn = lib().mluops_oracle_dynamic_point_to_voxel_backward
    rc = fn(_p(g, _f32p), _p(f, _f32p), _p(vf, _f32p), _p(p2v, _i32p), ctypes.c_int32(int(voxel_num)),
            ctypes.c_int64(n), ctypes.c_int64(c), _p(out, _f32p))
    assert rc == 0
    return out


def round_through_half(x):
    """float32 -> half (reference rounding) -> float32."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty_like(x)
    lib().mluops_oracle_round_through_half(_p(x, _f32p), _p(out, _f32p), ctypes.c_int64(x.size))
    return out


def float_to_half_bits(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().mluops_oracle_float_to_half_array(_p(x, _f32p), _p(out, _u16p), ctypes.c_int64(x.size))
    return out


def half_bits_to_float(h):
    h = np.ascontiguousarray(h, dtype=np.uint16)
    out = np.empty(h.shape, dtype=np.float32)
    lib().mluops_oracle_half_to_float_array(_p(h, _u16p), _p(out, _f32p), ctypes.c_int64(h.size))
    return out


def diffs(test, base, is_half):
    """(diff1, diff2, diff3) of a device result against the CPU result."""
    test = np.ascontiguousarray(test, dtype=np.float32).ravel()
    base = np.ascontiguousarray(base, dtype=np.float32).ravel()
    assert test.size == base.size
    d1, d2, d3 = ctypes.c_double(), ctypes.c_double(), ctypes.c_double()
    lib().mluops_oracle_diffs(_p(test, _f32p), _p(base, _f32p), ctypes.c_int64(test.size),
                              ctypes.c_int32(int(is_half)), ctypes.byref(d1), ctypes.byref(d2),
                              ctypes.byref(d3))
    return d1.value, d2.value, d3.value
