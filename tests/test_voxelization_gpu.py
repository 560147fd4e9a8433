"""GPU parity of mluOpVoxelization against the CPU oracle, through the C ABI.
Every output is integer work or a copy of input floats: the comparison is bit-exact."""
import os

import numpy as np
import pytest
import torch

# guard_bands: outputs and workspaces of every call sit between poisoned bands, checked after the test
pytestmark = [pytest.mark.gpu, pytest.mark.usefixtures("guard_bands")]


@pytest.fixture(scope="module")
def vox_golden():
    return np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "voxelization_golden.npz"))


def run_gpu(ops, handle, pts, vs, cr, mp, mv):
    dev = "cuda"
    out = ops.voxelization(handle, torch.from_numpy(np.ascontiguousarray(pts, dtype=np.float32)).to(dev),
                           torch.tensor(vs, dtype=torch.float32, device=dev),
                           torch.tensor(cr, dtype=torch.float32, device=dev), mp, mv)
    torch.cuda.synchronize()
    voxels, coors, npv, num = (t.cpu().numpy() for t in out)
    return voxels, coors, npv, int(num[0])


def assert_same(got, ref):
    assert got[3] == ref[3]
    assert np.array_equal(got[1], ref[1]) and np.array_equal(got[2], ref[2])
    assert np.array_equal(got[0].view(np.uint32), ref[0].view(np.uint32))


def test_golden_vectors(ops, gpu_handle, vox_golden):
    """Outputs the reference's own CPU code produced."""
    for name in [str(n) for n in vox_golden["names"]]:
        mp, mv, num = (int(v) for v in vox_golden[name + "/params"])
        got = run_gpu(ops, gpu_handle, vox_golden[name + "/points"], vox_golden[name + "/voxel_size"].tolist(),
                      vox_golden[name + "/coors_range"].tolist(), mp, mv)
        assert_same(got, (vox_golden[name + "/voxels"], vox_golden[name + "/coors"],
                          vox_golden[name + "/num_points_per_voxel"], num))


@pytest.mark.parametrize("seed", range(8))
def test_random_clouds(ops, oracle, gpu_handle, seed):
    rng = np.random.default_rng(100 + seed)
    n, f = int(rng.integers(1, 6000)), int(rng.integers(3, 7))
    pts = rng.random((n, f)).astype(np.float32) * np.array([22, 24, 6] + [1] * (f - 3), dtype=np.float32) - \
        np.array([1, 12, 4] + [0] * (f - 3), dtype=np.float32)
    vs = [[0.5, 0.5, 1.0], [2.0, 3.0, 4.0], [0.1, 0.1, 0.2], [5.0, 5.0, 4.0]][seed % 4]
    cr = [0, -10, -3, 20, 10, 1]
    mp, mv = int(rng.integers(1, 12)), int(rng.integers(1, 3000))
    assert_same(run_gpu(ops, gpu_handle, pts, vs, cr, mp, mv), oracle.voxelization(pts, vs, cr, mp, mv))


def test_crowded_voxel_keeps_the_first_points(ops, oracle, gpu_handle):
    """Thousands of points in a handful of voxels: the per-voxel lists are contended."""
    rng = np.random.default_rng(7)
    pts = rng.random((20000, 4)).astype(np.float32) * np.array([2, 2, 1, 1], dtype=np.float32)
    got = run_gpu(ops, gpu_handle, pts, [1, 1, 1], [0, 0, 0, 2, 2, 1], 35, 10)
    assert_same(got, oracle.voxelization(pts, [1, 1, 1], [0, 0, 0, 2, 2, 1], 35, 10))
    assert got[3] == 4 and got[2][:4].tolist() == [35] * 4
    # two runs are bit-identical
    assert_same(run_gpu(ops, gpu_handle, pts, [1, 1, 1], [0, 0, 0, 2, 2, 1], 35, 10), got)


def test_lidar_frame_properties(ops, gpu_handle):
    """A 300,000-point frame (where the quadratic CPU oracle would take minutes): every kept
    point sits in the voxel its coordinates name, points of a voxel are in index order, voxels are
    in order of their first points, and counts add up."""
    rng = np.random.default_rng(9)
    n = 300000
    pts = np.concatenate([rng.normal(0, 18, (n, 2)), rng.normal(-1, 0.8, (n, 1)), rng.random((n, 1))], 1).astype(
        np.float32)
    pts[:, 3] = np.arange(n, dtype=np.float32)  # the index travels with the point (exact below 2^24)
    vs, cr, mp, mv = [0.05, 0.05, 0.1], [-40, -40, -3, 40, 40, 1], 5, 160000
    voxels, coors, npv, num = run_gpu(ops, gpu_handle, pts, vs, cr, mp, mv)
    assert 0 < num <= mv and not npv[num:].any() and not voxels[num:].any()
    assert npv[:num].min() >= 1 and npv[:num].max() <= mp
    firsts = voxels[:num, 0, 3]
    assert np.all(np.diff(firsts) > 0)  # voxel order = order of first points
    lo, size = np.array(cr[:3], dtype=np.float32), np.array(vs, dtype=np.float32)
    for m in range(mp):
        live = npv[:num] > m
        p = voxels[:num][live, m]
        c = np.floor((p[:, :3] - lo) / size).astype(np.int32)[:, ::-1]
        assert np.array_equal(c, coors[:num][live])
        if m:
            assert np.all(p[:, 3] > voxels[:num][live, m - 1, 3])  # index order inside a voxel
    inside = np.all((np.floor((pts[:, :3] - lo) / size) >= 0) &
                    (np.floor((pts[:, :3] - lo) / size) < np.round((np.array(cr[3:]) - lo) / size)), 1)
    assert int(npv[:num].sum()) <= int(inside.sum())
