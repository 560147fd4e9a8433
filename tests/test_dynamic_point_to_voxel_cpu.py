"""Dynamic point-to-voxel scatter without a GPU: the oracle against the reference's
golden vectors and compiled code, and the status codes of the C ABI following the
reference's checks (kernels/dynamic_point_to_voxel/dynamic_point_to_voxel_forward/
dynamic_point_to_voxel_forward.cpp:70-191)."""
import ctypes
import os

import numpy as np
import pytest

VP = ctypes.c_void_p
F16, F32, I32, I64 = 1, 2, 6, 9
ARRAY = 4
SUM, MEAN, MAX = 0, 1, 2


@pytest.fixture(scope="module")
def dpv_golden():
    return np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden",
                                "dynamic_point_to_voxel_golden.npz"))


@pytest.fixture(scope="module")
def handle(ops):
    h = ops.Handle(0)
    yield h
    h.destroy()


def test_oracle_matches_golden(oracle, dpv_golden):
    for name in [str(n) for n in dpv_golden["names"]]:
        for mode in ("max", "mean"):
            vf, vc, p2v, cnt, num, filled = oracle.dynamic_point_to_voxel_forward(dpv_golden[name + "/feats"],
                                                                                  dpv_golden[name + "/coors"], mode)
            assert num == int(dpv_golden[name + "/voxel_num"][0]), name
            assert np.array_equal(p2v, dpv_golden[name + "/point2voxel_map"]), name
            assert np.array_equal(vc[:num], dpv_golden[name + "/voxel_coors"]), name
            assert np.array_equal(cnt[:num], dpv_golden[name + "/voxel_points_count"]), name
            assert np.array_equal(filled, dpv_golden[name + "/coors_filled"]), name
            assert np.array_equal(vf[:num].view(np.uint32),
                                  dpv_golden["%s/%s/voxel_feats" % (name, mode)].view(np.uint32)), (name, mode)


def test_oracle_against_reference_code(oracle):
    if oracle.ref_lib() is None:
        pytest.skip("oracle/_ref not built (reference tree absent)")
    rng = np.random.default_rng(51)
    for trial in range(40):
        n, c = int(rng.integers(1, 700)), int(rng.integers(1, 6))
        hi = [4, 6, 5] if trial % 3 else [40, 300, 7]
        coors = np.stack([rng.integers(-1 if trial % 2 else 0, h, n) for h in hi], 1).astype(np.int32)
        feats = (rng.standard_normal((n, c)) * 10).astype(np.float32)
        for mode in ("max", "mean"):
            a = oracle.dynamic_point_to_voxel_forward(feats, coors, mode)
            b = oracle.dynamic_point_to_voxel_forward(feats, coors, mode, use_ref=True)
            m = a[4]
            assert m == b[4] and np.array_equal(a[2], b[2]) and np.array_equal(a[5], b[5])
            assert np.array_equal(a[1][:m], b[1][:m]) and np.array_equal(a[3][:m], b[3][:m])
            assert np.array_equal(a[0][:m].view(np.uint32), b[0][:m].view(np.uint32))


def test_backward_oracle(oracle, dpv_golden):
    for name in [str(n) for n in dpv_golden["names"]]:
        feats, coors = dpv_golden[name + "/feats"], dpv_golden[name + "/coors"]
        vf, vc, p2v, cnt, num, _ = oracle.dynamic_point_to_voxel_forward(feats, coors, "max")
        grad = dpv_golden[name + "/grad_voxel_feats"]
        got = oracle.dynamic_point_to_voxel_backward(grad, feats, vf[:max(num, 1)], p2v, num)
        assert np.array_equal(got, dpv_golden[name + "/grad_feats"]), name
        # each voxel hands every channel's gradient to exactly one of its points
        assert int((got != 0).sum()) <= num * feats.shape[1]
        if oracle.ref_lib() is not None:
            assert np.array_equal(got, oracle.dynamic_point_to_voxel_backward(grad, feats, vf[:max(num, 1)], p2v, num,
                                                                              use_ref=True))


def test_backward_status_codes(ops, handle):
    lib = ops.lib()
    shapes = dict(g=(F32, (6, 4)), f=(F32, (6, 4)), vf=(F32, (6, 4)), m=(I32, (6,)), c=(I32, (6,)), n=(I32, (1,)),
                  o=(F32, (6, 4)))

    def call(reduce=MAX, null_at=None, **over):
        a = dict(shapes)
        a.update(over)
        descs = [ops.TensorDesc(ARRAY, *a[k]) for k in ("g", "f", "vf", "m", "c", "n", "o")]
        d = [x.ptr for x in descs]
        buf = (ctypes.c_char * 8192)()
        p = VP(ctypes.addressof(buf))
        args = [handle.ptr, reduce, d[0], p, d[1], p, d[2], p, d[3], p, d[4], p, d[5], p, p, 8192, d[6], p]
        if null_at is not None:
            args[null_at] = None
        st = lib.mluOpDynamicPointToVoxelBackward(*args)
        for x in descs:
            x.destroy()
        return st

    assert call() == ops.STATUS_EXECUTION_FAILED  # checks pass; a host-only handle cannot launch
    assert call(reduce=MEAN) == ops.STATUS_BAD_PARAM
    assert call(f=(F32, (0, 4)), m=(I32, (0,)), o=(F32, (0, 4)), g=(F32, (0, 4)), vf=(F32, (0, 4)), c=(I32, (0,))) == 0
    for over in (dict(g=(F16, (6, 4))), dict(f=(F32, (6, 5))), dict(vf=(F32, (5, 4))), dict(m=(I32, (5,))),
                 dict(c=(I32, (5,))), dict(n=(I32, (2,))), dict(o=(F32, (5, 4))), dict(o=(F32, (6, 3))),
                 dict(g=(F32, (7, 4)), vf=(F32, (7, 4)), c=(I32, (7,)))):
        assert call(**over) == ops.STATUS_BAD_PARAM, over
    for i in (0, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 16, 17):
        assert call(null_at=i) == ops.STATUS_BAD_PARAM, i
    d = [ops.TensorDesc(ARRAY, *shapes[k]) for k in ("g", "f", "vf", "m", "c", "n")]
    size = ctypes.c_size_t(0)
    assert lib.mluOpGetDynamicPointToVoxelBackwardWorkspaceSize(handle.ptr, MAX, *[x.ptr for x in d],
                                                                ctypes.byref(size)) == 0
    assert size.value == 6 * 4 * 4
    assert lib.mluOpGetDynamicPointToVoxelBackwardWorkspaceSize(handle.ptr, MAX, *[x.ptr for x in d],
                                                                None) == ops.STATUS_BAD_PARAM


def test_by_hand(oracle):
    coors = np.array([[1, 0, 2], [0, 5, 5], [1, 0, 2], [-1, 3, 3], [0, 5, 4]], dtype=np.int32)
    feats = np.array([[1.0], [2.0], [5.0], [9.0], [4.0]], dtype=np.float32)
    vf, vc, p2v, cnt, num, filled = oracle.dynamic_point_to_voxel_forward(feats, coors, "mean")
    assert num == 3 and vc[:3].tolist() == [[0, 5, 4], [0, 5, 5], [1, 0, 2]]
    assert p2v.tolist() == [2, 1, 2, -1, 0] and cnt[:3].tolist() == [1, 1, 2]
    assert vf[:3, 0].tolist() == [4.0, 2.0, 3.0] and filled[3].tolist() == [-1, -1, -1]


GOOD = dict(reduce=MAX, feats=(F32, (6, 4)), coors=(I32, (6, 3)), vfeats=(F32, (6, 4)), vcoors=(I32, (6, 3)),
            p2v=(I32, (6,)), cnt=(I32, (6,)), num=(I32, (1,)))


def run(ops, handle, null_at=None, **over):
    a = dict(GOOD)
    a.update(over)
    lib = ops.lib()
    descs = [ops.TensorDesc(ARRAY, *a[k]) for k in ("feats", "coors", "vfeats", "vcoors", "p2v", "cnt", "num")]
    d_f, d_c, d_vf, d_vc, d_m, d_n, d_num = (d.ptr for d in descs)
    buf = (ctypes.c_char * 8192)()
    p = VP(ctypes.addressof(buf))
    args = [handle.ptr, a["reduce"], d_f, p, d_c, p, p, 8192, d_vf, p, d_vc, p, d_m, p, d_n, p, d_num, p]
    if null_at is not None:
        args[null_at] = None
    st = lib.mluOpDynamicPointToVoxelForward(*args)
    for d in descs:
        d.destroy()
    return st


def test_status_codes(ops, handle):
    assert run(ops, handle) == ops.STATUS_EXECUTION_FAILED  # checks pass; a host-only handle cannot launch
    assert run(ops, handle, reduce=MEAN) == ops.STATUS_EXECUTION_FAILED
    assert run(ops, handle, reduce=SUM) == ops.STATUS_BAD_PARAM
    assert run(ops, handle, feats=(F32, (0, 4)), coors=(I32, (0, 3)), p2v=(I32, (0,)), vfeats=(F32, (0, 4)),
               vcoors=(I32, (0, 3)), cnt=(I32, (0,))) == 0
    for over in (dict(feats=(F16, (6, 4))), dict(coors=(I64, (6, 3))), dict(coors=(I32, (6, 2)), vcoors=(I32, (6, 2))),
                 dict(coors=(I32, (5, 3))), dict(p2v=(I32, (5,))), dict(vfeats=(F32, (6, 5))),
                 dict(vfeats=(F32, (7, 4)), vcoors=(I32, (7, 3)), cnt=(I32, (7,))), dict(vcoors=(I32, (5, 3))),
                 dict(cnt=(I32, (5,))), dict(num=(I32, (2,))), dict(p2v=(F32, (6,))), dict(feats=(F32, (6, 4, 1))),
                 dict(p2v=(I32, (6, 1)))):
        assert run(ops, handle, **over) == ops.STATUS_BAD_PARAM, over
    for i in (0, 2, 3, 4, 5, 6, 8, 9, 10, 11, 12, 13, 14, 15, 16, 17):
        assert run(ops, handle, null_at=i) == ops.STATUS_BAD_PARAM, i


def test_workspace_query(ops, handle):
    lib = ops.lib()
    d_f, d_c = ops.TensorDesc(ARRAY, F32, (1000, 4)), ops.TensorDesc(ARRAY, I32, (1000, 3))
    size = ctypes.c_size_t(0)
    assert lib.mluOpGetDynamicPointToVoxelForwardWorkspaceSize(handle.ptr, d_f.ptr, d_c.ptr, ctypes.byref(size)) == 0
    assert size.value >= 2 * 16 * 1000
    for a in ([None, d_f.ptr, d_c.ptr, ctypes.byref(size)], [handle.ptr, None, d_c.ptr, ctypes.byref(size)],
              [handle.ptr, d_f.ptr, None, ctypes.byref(size)], [handle.ptr, d_f.ptr, d_c.ptr, None]):
        assert lib.mluOpGetDynamicPointToVoxelForwardWorkspaceSize(*a) == ops.STATUS_BAD_PARAM
