"""GPU parity of mluOpGetIndicePairs against the CPU oracle: bit-exact
indice_pairs, out_indices, indice_num and num_act_out, through the C ABI."""
import numpy as np
import pytest
import torch

import helpers

# guard_bands: outputs and workspaces of every call sit between poisoned bands, checked after the test
pytestmark = [pytest.mark.gpu, pytest.mark.usefixtures("guard_bands")]


def run_gpu(ops, handle, idx, g, out_rows=None):
    conv = ops.SparseConvDesc(g["batch"], g["pad"], g["stride"], g["dil"], g["space"], g["ks"], g["out_space"],
                              g["sub_m"])
    d_idx = torch.from_numpy(np.ascontiguousarray(idx)).cuda()
    pairs, out_idx, num, n_out = ops.get_indice_pairs(handle, conv, d_idx, out_rows)
    torch.cuda.synchronize()
    conv.destroy()
    return pairs.cpu().numpy(), out_idx.cpu().numpy(), num.cpu().numpy(), n_out


def check_against_oracle(ops, oracle, handle, idx, g, out_rows=None):
    pairs, out_idx, num, n_out = run_gpu(ops, handle, idx, g, out_rows)
    r_pairs, r_out, r_num, r_n = oracle.get_indice_pairs(idx, g["batch"], g["pad"], g["stride"], g["dil"], g["ks"],
                                                         g["out_space"], g["sub_m"], out_rows=out_idx.shape[0])
    assert n_out == r_n
    assert np.array_equal(num, r_num)
    assert np.array_equal(out_idx, r_out)
    assert np.array_equal(pairs, r_pairs)
    return pairs, out_idx, num, n_out


def test_golden_vectors(ops, gpu_handle, golden):
    """Outputs of the reference's own CPU code, committed as fixtures."""
    for name in helpers.golden_names(golden):
        c = helpers.golden_case(golden, name)
        if not helpers.has_unused_slot(c["indice_num"], c["indices"].shape[0]):
            continue
        g = dict(batch=c["batch"], space=c["space"], ks=c["ks"], stride=c["stride"], pad=c["pad"], dil=c["dil"],
                 out_space=c["out_space"], sub_m=c["sub_m"])
        pairs, out_idx, num, n_out = run_gpu(ops, gpu_handle, c["indices"], g, c["out_indices"].shape[0])
        assert np.array_equal(num, c["indice_num"]), name
        assert np.array_equal(pairs, c["indice_pairs"]), name
        assert np.array_equal(out_idx, c["out_indices"]), name
        assert n_out == c["n_out"], name


@pytest.mark.parametrize("sub_m", [0, 1])
def test_random_small_geometries(ops, oracle, gpu_handle, sub_m):
    """All stride / pad / dilation / kernel-shape combinations on tiny grids."""
    rng = np.random.default_rng(100 + sub_m)
    done = 0
    while done < 60:
        g = helpers.random_geometry(rng, sub_m)
        if g is None:
            continue
        idx = helpers.random_indices(rng, g["batch"], g["space"], g["n"])
        check_against_oracle(ops, oracle, gpu_handle, idx, g)
        done += 1


def test_config0_full_size(ops, oracle, workloads, gpu_handle):
    idx, _, layers, _ = workloads.make_inputs("c0")
    ly = layers[0]
    grid = workloads.CONFIGS["c0"]["grid"]
    g = dict(batch=1, space=list(grid), ks=ly.filter_space, stride=ly.stride, pad=ly.pad, dil=ly.dilation,
             out_space=list(grid), sub_m=1)
    _, _, num, n_out = check_against_oracle(ops, oracle, gpu_handle, idx, g)
    assert n_out == 16000 and num[13] == 16000


def test_config1_full_size(ops, oracle, workloads, gpu_handle):
    idx, _, layers, _ = workloads.make_inputs("c1")
    ly = layers[0]
    grid = list(workloads.CONFIGS["c1"]["grid"])
    osp = helpers.out_space(grid, ly.pad, ly.stride, ly.dilation, ly.filter_space)
    assert osp == [21, 800, 704]
    g = dict(batch=2, space=grid, ks=ly.filter_space, stride=ly.stride, pad=ly.pad, dil=ly.dilation,
             out_space=osp, sub_m=0)
    pairs, out_idx, num, n_out = check_against_oracle(ops, oracle, gpu_handle, idx, g)
    assert 0 < n_out <= out_idx.shape[0]


def test_subm_scaled_config3(ops, oracle, workloads, gpu_handle):
    """Submanifold rulebook on the LiDAR-like distribution, two samples of the 200k-voxel config."""
    idx, _, layers, _ = workloads.make_inputs("c3", batch=2)
    ly = layers[0]
    grid = list(workloads.CONFIGS["c3"]["grid"])
    g = dict(batch=2, space=grid, ks=ly.filter_space, stride=ly.stride, pad=ly.pad, dil=ly.dilation,
             out_space=grid, sub_m=1)
    check_against_oracle(ops, oracle, gpu_handle, idx, g)


def test_subm_repeated_coordinates_keep_last_row(ops, oracle, gpu_handle):
    rng = np.random.default_rng(9)
    g = dict(batch=1, space=[6, 6, 6], ks=[3, 3, 3], stride=[1] * 3, pad=[1] * 3, dil=[1] * 3, out_space=[6, 6, 6],
             sub_m=1)
    idx = helpers.random_indices(rng, 1, g["space"], 100)
    idx[80:] = idx[:20]
    check_against_oracle(ops, oracle, gpu_handle, idx, g)


def test_degenerate_no_valid_pair(ops, oracle, gpu_handle):
    """Kernel 1, stride 2, pad 0: only even coordinates produce an output."""
    g = dict(batch=1, space=[5, 5, 5], ks=[1, 1, 1], stride=[2, 2, 2], pad=[0, 0, 0], dil=[1, 1, 1],
             out_space=[3, 3, 3], sub_m=0)
    idx = np.array([[0, 1, 1, 1], [0, 3, 1, 3], [0, 1, 3, 3]], dtype=np.int32)
    pairs, out_idx, num, n_out = run_gpu(ops, gpu_handle, idx, g)
    assert n_out == 0 and num.sum() == 0 and np.all(pairs == -1) and np.all(out_idx == -1)


def test_single_voxel_and_ragged_tile_sizes(ops, oracle, gpu_handle):
    rng = np.random.default_rng(21)
    for n in (1, 31, 32, 33, 255, 256, 257, 1023, 1025):
        for sub_m in (0, 1):
            g = dict(batch=2, space=[8, 16, 16], ks=[3, 3, 3], stride=[1] * 3 if sub_m else [2] * 3, pad=[1] * 3,
                     dil=[1] * 3, sub_m=sub_m)
            g["out_space"] = g["space"] if sub_m else helpers.out_space(g["space"], g["pad"], g["stride"],
                                                                        g["dil"], g["ks"])
            idx = helpers.random_indices(rng, 2, g["space"], n)
            check_against_oracle(ops, oracle, gpu_handle, idx, g)


def test_out_of_range_rows_produce_no_pairs(ops, gpu_handle):
    g = dict(batch=1, space=[4, 4, 4], ks=[3, 3, 3], stride=[1] * 3, pad=[1] * 3, dil=[1] * 3, out_space=[4, 4, 4],
             sub_m=1)
    idx = np.array([[0, 1, 1, 1], [3, 1, 1, 2], [0, 9, 1, 1], [0, 1, 1, 2]], dtype=np.int32)
    pairs, out_idx, num, n_out = run_gpu(ops, gpu_handle, idx, g)
    assert num[13] == 2 and pairs[13, 0, :2].tolist() == [0, 3]
    assert num.sum() == 4


def test_out_indices_too_small_is_reported(ops, gpu_handle):
    g = dict(batch=1, space=[8, 8, 8], ks=[3, 3, 3], stride=[2] * 3, pad=[1] * 3, dil=[1] * 3, out_space=[4, 4, 4],
             sub_m=0)
    idx = helpers.random_indices(np.random.default_rng(2), 1, g["space"], 100)
    with pytest.raises(ops.MluOpError) as e:
        run_gpu(ops, gpu_handle, idx, g, out_rows=3)
    assert e.value.status == ops.STATUS_BAD_PARAM


def test_workspace_too_small_is_rejected(ops, gpu_handle):
    conv = ops.SparseConvDesc(1, [1] * 3, [1] * 3, [1] * 3, [4, 4, 4], [3, 3, 3], [4, 4, 4], 1)
    idx = torch.zeros((4, 4), dtype=torch.int32, device="cuda")
    ws = torch.empty((16,), dtype=torch.uint8, device="cuda")
    L, K = 4, 27
    d = [ops.TensorDesc(ops.LAYOUT_ARRAY, ops.DTYPE_INT32, dims) for dims in ((L, 4), (K, 2, L), (L, 4), (K,))]
    pairs = torch.empty((K, 2, L), dtype=torch.int32, device="cuda")
    out = torch.empty((L, 4), dtype=torch.int32, device="cuda")
    num = torch.empty((K,), dtype=torch.int32, device="cuda")
    import ctypes
    st = ops.lib().mluOpGetIndicePairs(gpu_handle.ptr, conv.ptr, d[0].ptr, ctypes.c_void_p(idx.data_ptr()),
                                       ctypes.c_void_p(ws.data_ptr()), 16, d[1].ptr,
                                       ctypes.c_void_p(pairs.data_ptr()), d[2].ptr, ctypes.c_void_p(out.data_ptr()),
                                       d[3].ptr, ctypes.c_void_p(num.data_ptr()))
    assert st == ops.STATUS_BAD_PARAM


def test_large_scale_properties(ops, workloads, gpu_handle):
    """Size-independent properties on the largest single-call rulebooks
    (2.4 M voxels, batch 16): per-offset lists strictly ascending in the input
    id, tails -1, counts consistent, every output id in range, subm centre offset
    is the identity, default-mode out_indices strictly ascending in linear order
    and every pair's coordinates consistent with its kernel offset."""
    rng = np.random.default_rng(77)
    grid = list(workloads.LIDAR_GRID)
    idx = workloads.batch_indices(rng, grid, 16, 150000, "lidar")
    L = idx.shape[0]
    d_idx = torch.from_numpy(idx).cuda()
    for sub_m in (1, 0):
        stride = [1] * 3 if sub_m else [2] * 3
        osp = grid if sub_m else helpers.out_space(grid, [1] * 3, stride, [1] * 3, [3] * 3)
        conv = ops.SparseConvDesc(16, [1] * 3, stride, [1] * 3, grid, [3] * 3, osp, sub_m)
        pairs, out_idx, num, n_out = ops.get_indice_pairs(gpu_handle, conv, d_idx)
        num_h = num.cpu().numpy()
        pos = torch.arange(L, device="cuda")
        total = 0
        for k in range(27):
            p = int(num_h[k])
            total += p
            rows_in, rows_out = pairs[k, 0], pairs[k, 1]
            assert bool((rows_in[p:] == -1).all()) and bool((rows_out[p:] == -1).all())
            if p == 0:
                continue
            assert bool((rows_in[1:p] > rows_in[:p - 1]).all())
            assert int(rows_in[:p].min()) >= 0 and int(rows_in[:p].max()) < L
            assert int(rows_out[:p].min()) >= 0 and int(rows_out[:p].max()) < n_out
            # geometry of every pair: in + pad - k*dil == out*stride
            kd, kh, kw = k // 9, (k // 3) % 3, k % 3
            ci = d_idx[rows_in[:p].long()]
            co = out_idx[rows_out[:p].long()]
            assert bool((ci[:, 0] == co[:, 0]).all())
            for axis, kk in ((1, kd), (2, kh), (3, kw)):
                assert bool((ci[:, axis] + 1 - kk == co[:, axis] * stride[0]).all())
        if sub_m:
            assert n_out == L and int(num_h[13]) == L
            assert bool((pairs[13, 0] == pos).all()) and bool((pairs[13, 1] == pos).all())
            assert bool((out_idx == d_idx).all())
            # symmetry: pair (a, b) at offset k <=> pair (b, a) at offset 26 - k
            assert np.array_equal(num_h, num_h[::-1])
        else:
            o = out_idx[:n_out].long()
            lin = ((o[:, 0] * osp[0] + o[:, 1]) * osp[1] + o[:, 2]) * osp[2] + o[:, 3]
            assert bool((lin[1:] > lin[:-1]).all())
            assert bool((out_idx[n_out:] == -1).all())
            # every active output is hit by at least one pair
            hit = torch.zeros(n_out, dtype=torch.bool, device="cuda")
            for k in range(27):
                hit[pairs[k, 1, :int(num_h[k])].long()] = True
            assert bool(hit.all())
        assert total > 0
        conv.destroy()


def test_large_kernel_volume(ops, oracle, gpu_handle):
    """Kernel volumes above 32 (more offsets than the single-pass path holds)."""
    rng = np.random.default_rng(45)
    space = [9, 12, 12]
    idx = helpers.random_indices(rng, 2, space, 900)
    g = dict(batch=2, space=space, ks=[5, 3, 3], stride=[1] * 3, pad=[2, 1, 1], dil=[1] * 3, out_space=space, sub_m=1)
    check_against_oracle(ops, oracle, gpu_handle, idx, g)
    g = dict(batch=2, space=space, ks=[4, 3, 3], stride=[2, 1, 1], pad=[1, 1, 1], dil=[1] * 3, sub_m=0)
    g["out_space"] = helpers.out_space(space, g["pad"], g["stride"], g["dil"], g["ks"])
    check_against_oracle(ops, oracle, gpu_handle, idx, g)


@pytest.mark.parametrize("env", [{"MLUOP_B200_PAIRS_LOOKUP": "hash"}, {"MLUOP_B200_PAIRS_LOOKUP": "rank"},
                                 {"MLUOP_B200_PAIRS_PATH": "twopass"},
                                 {"MLUOP_B200_PAIRS_PATH": "twopass", "MLUOP_B200_PAIRS_LOOKUP": "hash"}])
def test_forced_variants(env):
    """Every lookup structure (hash / occupancy rank) and both pair-list paths (single pass by
    default / two pass on request) pass the same parity cases; the choice is per process, hence
    the child."""
    import os
    import subprocess
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    r = subprocess.run([sys.executable, "-m", "pytest", os.path.join(here, "test_get_indice_pairs_gpu.py"), "-m", "gpu",
                        "-x", "-q", "-k", "golden or random_small or config0 or scaled_config3 or repeated or ragged"],
                       env=dict(os.environ, **env), capture_output=True, text=True)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]


def test_device_errors_of_asynchronous_calls_are_sticky(ops, gpu_handle, monkeypatch):
    """A submanifold rulebook returns before its kernels have run, so a device-side error
    (here: a hash table undersized on purpose through the test hook, whose capacity-bounded
    probes record "table full") cannot be returned by the call itself.  It must surface as
    MLUOP_STATUS_EXECUTION_FAILED from the next entry point on the handle, once, and with
    MLUOP_B200_CHECK_STATUS=1 from the call itself.  Nothing waits or faults: every probe
    loop ends after `capacity` steps."""
    rng = np.random.default_rng(5)
    space = [16, 64, 64]
    idx = torch.from_numpy(helpers.random_indices(rng, 1, space, 1000)).cuda()
    conv = ops.SparseConvDesc(1, [1] * 3, [1] * 3, [1] * 3, space, [3] * 3, space, 1)
    monkeypatch.setenv("MLUOP_B200_TEST_HASH_CAPACITY", "64")
    with pytest.raises(ops.MluOpError) as err:  # the tests run with MLUOP_B200_CHECK_STATUS=1
        ops.get_indice_pairs(gpu_handle, conv, idx)
    assert err.value.status == ops.STATUS_EXECUTION_FAILED
    monkeypatch.setenv("MLUOP_B200_CHECK_STATUS", "0")
    ops.get_indice_pairs(gpu_handle, conv, idx)  # asynchronous: reports success
    torch.cuda.synchronize()
    monkeypatch.delenv("MLUOP_B200_TEST_HASH_CAPACITY")
    with pytest.raises(ops.MluOpError) as err:
        ops.get_indice_pairs(gpu_handle, conv, idx)
    assert err.value.status == ops.STATUS_EXECUTION_FAILED
    pairs, _, num, n_out = ops.get_indice_pairs(gpu_handle, conv, idx)  # reported once, then cleared
    torch.cuda.synchronize()
    assert n_out == 1000 and int(num.sum()) >= 1000
    conv.destroy()


def test_table_emitted_by_the_rulebook_equals_the_table_built_from_its_pairs(ops, gpu_handle):
    """mluOpGetIndicePairsWithNeighbourTable (submanifold, centred padding) must leave exactly the
    table mluOpBuildIndiceNeighbourTable derives from indice_pairs, padding rows included, and the
    same rulebook as mluOpGetIndicePairs; other rulebooks are refused before anything runs."""
    rng = np.random.default_rng(63)
    for ks, space, n in (([3, 3, 3], [9, 30, 31], 3000), ([3, 1, 3], [7, 9, 40], 700), ([1, 3, 5], [6, 12, 33], 517),
                         ([3, 3, 3], [41, 160, 140], 60000), ([1, 1, 1], [4, 4, 4], 20)):
        idx = torch.from_numpy(helpers.random_indices(rng, 2, space, n)).cuda()
        conv = ops.SparseConvDesc(2, [k // 2 for k in ks], [1] * 3, [1] * 3, space, ks, space, 1)
        ref = ops.get_indice_pairs(gpu_handle, conv, idx)
        pairs, out_idx, num, n_out, table = ops.get_indice_pairs(gpu_handle, conv, idx, with_table=True)
        torch.cuda.synchronize()
        assert n_out == ref[3] and torch.equal(pairs, ref[0]) and torch.equal(out_idx, ref[1]) and torch.equal(num, ref[2])
        built = ops.build_neighbour_table(gpu_handle, pairs, num.cpu().tolist(), n_out)
        torch.cuda.synchronize()
        assert table.shape == built.shape and torch.equal(table, built), ks
        conv.destroy()
    # default mode and off-centre padding: not supported, nothing launched
    space = [8, 8, 8]
    idx = torch.from_numpy(helpers.random_indices(rng, 1, space, 50)).cuda()
    for conv in (ops.SparseConvDesc(1, [1] * 3, [2] * 3, [1] * 3, space, [3] * 3, [4, 4, 4], 0),
                 ops.SparseConvDesc(1, [0, 1, 1], [1] * 3, [1] * 3, space, [3] * 3, space, 1)):
        with pytest.raises(ops.MluOpError) as err:
            ops.get_indice_pairs(gpu_handle, conv, idx, with_table=True)
        assert err.value.status == ops.STATUS_NOT_SUPPORTED
        conv.destroy()


def test_guard_bands_catch_a_stray_write(ops):
    """The guard itself: a write one element past a guarded buffer, or one before it, is reported."""
    for offset in (0, -1):
        with pytest.raises(AssertionError):
            with ops.guarded() as guards:
                t = guards.empty((10, 4), torch.int32, "cuda")
                flat = torch.as_strided(t, (1,), (1,), storage_offset=t.storage_offset() + (t.numel() if offset == 0 else -1))
                flat.fill_(7)
    with ops.guarded() as guards:
        t = guards.empty((10, 4), torch.int32, "cuda")
        t.fill_(7)
    assert guards.check() == 1
