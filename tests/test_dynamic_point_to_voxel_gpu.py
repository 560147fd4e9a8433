"""GPU parity of mluOpDynamicPointToVoxelForward against the CPU oracle, through the C ABI.
The grouping is integer work and the reductions run in the reference's order, so every
output is compared bit for bit (rows up to voxel_num, which is all the reference defines)."""
import os

import numpy as np
import pytest
import torch

# guard_bands: outputs and workspaces of every call sit between poisoned bands, checked after the test
pytestmark = [pytest.mark.gpu, pytest.mark.usefixtures("guard_bands")]


@pytest.fixture(scope="module")
def dpv_golden():
    return np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden",
                                "dynamic_point_to_voxel_golden.npz"))


def run_gpu(ops, handle, feats, coors, mode):
    d_coors = torch.from_numpy(np.ascontiguousarray(coors, dtype=np.int32)).cuda()
    out = ops.dynamic_point_to_voxel_forward(handle, torch.from_numpy(np.ascontiguousarray(feats)).cuda(), d_coors,
                                             mode)
    torch.cuda.synchronize()
    vf, vc, p2v, cnt, num = (t.cpu().numpy() for t in out)
    return vf, vc, p2v, cnt, int(num[0]), d_coors.cpu().numpy()


def assert_same(got, ref, mode):
    m = ref[4]
    assert got[4] == m
    assert np.array_equal(got[2], ref[2]) and np.array_equal(got[5], ref[5])
    assert np.array_equal(got[1][:m], ref[1][:m]) and np.array_equal(got[3][:m], ref[3][:m])
    assert np.array_equal(got[0][:m].view(np.uint32), ref[0][:m].view(np.uint32))
    # rows the reference leaves undefined: zeros, and the reduction's fill value
    assert not got[1][m:].any() and not got[3][m:].any()
    assert np.all(got[0][m:] == (-np.inf if mode == "max" else 0.0))


@pytest.mark.parametrize("mode", ["max", "mean"])
def test_golden_vectors(ops, gpu_handle, dpv_golden, mode):
    """Outputs the reference's own CPU code produced."""
    for name in [str(n) for n in dpv_golden["names"]]:
        got = run_gpu(ops, gpu_handle, dpv_golden[name + "/feats"], dpv_golden[name + "/coors"], mode)
        m = int(dpv_golden[name + "/voxel_num"][0])
        assert got[4] == m, name
        assert np.array_equal(got[2], dpv_golden[name + "/point2voxel_map"]), name
        assert np.array_equal(got[1][:m], dpv_golden[name + "/voxel_coors"]), name
        assert np.array_equal(got[3][:m], dpv_golden[name + "/voxel_points_count"]), name
        assert np.array_equal(got[5], dpv_golden[name + "/coors_filled"]), name
        assert np.array_equal(got[0][:m].view(np.uint32),
                              dpv_golden["%s/%s/voxel_feats" % (name, mode)].view(np.uint32)), name


@pytest.mark.parametrize("seed", range(8))
def test_random_clouds(ops, oracle, gpu_handle, seed):
    rng = np.random.default_rng(200 + seed)
    n, c = int(rng.integers(1, 20000)), int(rng.integers(1, 9))
    hi = [[5, 7, 6], [41, 1600, 1408], [300, 70000, 3], [1 << 30, 2, 1 << 24]][seed % 4]
    coors = np.stack([rng.integers(-1 if seed % 2 else 0, h, n) for h in hi], 1).astype(np.int32)
    feats = (rng.standard_normal((n, c)) * 10).astype(np.float32)
    for mode in ("max", "mean"):
        assert_same(run_gpu(ops, gpu_handle, feats, coors, mode),
                    oracle.dynamic_point_to_voxel_forward(feats, coors, mode), mode)


def test_lidar_frame_properties(ops, gpu_handle):
    """300,000 points on a 41 x 1600 x 1408 grid: voxel_coors strictly ascending, the map
    consistent with it, counts and per-voxel maxima as a scatter of the inputs gives them."""
    rng = np.random.default_rng(10)
    n = 300000
    coors = np.stack([np.clip(rng.normal(20, 4, n), -1, 40), np.clip(rng.normal(800, 150, n), -1, 1599),
                      np.clip(rng.normal(700, 150, n), -1, 1407)], 1).astype(np.int32)
    feats = rng.standard_normal((n, 4)).astype(np.float32)
    vf, vc, p2v, cnt, num, filled = run_gpu(ops, gpu_handle, feats, coors, "max")
    valid = np.all(coors >= 0, 1)
    assert np.array_equal(p2v >= 0, valid) and np.all(filled[~valid] == -1)
    lin = (vc[:num, 0].astype(np.int64) * 1600 + vc[:num, 1]) * 1408 + vc[:num, 2]
    assert np.all(np.diff(lin) > 0)
    assert np.array_equal(vc[:num][p2v[valid]], coors[valid])
    assert np.array_equal(np.bincount(p2v[valid], minlength=num), cnt[:num])
    ref = np.full((num, 4), -np.inf, dtype=np.float32)
    np.maximum.at(ref, p2v[valid], feats[valid])
    assert np.array_equal(vf[:num], ref)


def test_backward_matches_oracle(ops, oracle, gpu_handle, dpv_golden):
    """grad_feats of the maximum reduction: golden vectors of the reference's CPU code, then random
    clouds with many tied features (the smallest point index must win a tie)."""
    def gpu_backward(feats, coors, grad_rows):
        d_feats = torch.from_numpy(np.ascontiguousarray(feats)).cuda()
        d_coors = torch.from_numpy(np.ascontiguousarray(coors, dtype=np.int32)).cuda()
        vf, vc, p2v, cnt, num = ops.dynamic_point_to_voxel_forward(gpu_handle, d_feats, d_coors, "max")
        grad = torch.zeros_like(vf)
        grad[:grad_rows.shape[0]] = torch.from_numpy(grad_rows).cuda()
        out = ops.dynamic_point_to_voxel_backward(gpu_handle, grad, d_feats, vf, p2v, cnt, num)
        torch.cuda.synchronize()
        return out.cpu().numpy()

    for name in [str(n) for n in dpv_golden["names"]]:
        got = gpu_backward(dpv_golden[name + "/feats"], dpv_golden[name + "/coors"],
                           dpv_golden[name + "/grad_voxel_feats"])
        assert np.array_equal(got.view(np.uint32), dpv_golden[name + "/grad_feats"].view(np.uint32)), name
    rng = np.random.default_rng(300)
    for trial in range(4):
        n, c = int(rng.integers(100, 20000)), int(rng.integers(1, 9))
        coors = np.stack([rng.integers(-1, h, n) for h in (5, 9, 7)], 1).astype(np.int32)
        feats = np.round(rng.standard_normal((n, c)) * 2).astype(np.float32)
        vf, vc, p2v, cnt, num, _ = oracle.dynamic_point_to_voxel_forward(feats, coors, "max")
        grad = rng.standard_normal((max(num, 1), c)).astype(np.float32)
        ref = oracle.dynamic_point_to_voxel_backward(grad, feats, vf[:max(num, 1)], p2v, num)
        assert np.array_equal(gpu_backward(feats, coors, grad), ref)
