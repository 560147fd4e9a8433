"""The benchmarked batches at their stated size against the oracle: c2 (4 x 120,000
voxels, 12-layer backbone), c3 (8 x 200,000 voxels, 128 -> 128 channels) and c4
(16 x 150,000 voxels, the backbone sharded by sample as the multi-GPU run shards it).

Rulebooks (indice_pairs, out_indices, indice_num, num_act_out) must be bit-exact and
every convolution within diff1, diff2 <= 3e-3, layer by layer and teacher-forced:
the oracle of layer n consumes the device's half output of layer n-1.  The oracle
is the reference's own CPU code (oracle/_ref) when it is built, else its C
restatement; it runs per sample in a process pool (tests/batch_oracle.py), so a
batch costs the wall time of one sample.
"""
import importlib

import numpy as np
import pytest
import torch

import batch_oracle
import helpers

pytestmark = pytest.mark.gpu


def _run_pool(tasks):
    results = {}
    with batch_oracle.make_pool(batch_oracle.default_workers(len(tasks))) as pool:
        # big tasks first so that the pool drains evenly
        order = sorted(tasks, key=lambda t: -sum(c["features_in"].size * c["co"] for c in t["convs"]))
        for r in pool.imap_unordered(batch_oracle._group_task, order):
            results[r["key"]] = r
    return results


def _forward_records(backbone, handle, grid, batch, idx, feat, layers, weights):
    net = backbone.SparseNetwork(handle, layers, [torch.from_numpy(w).cuda() for w in weights], grid, batch)
    out, out_idx, records = net.forward(torch.from_numpy(idx).cuda(), torch.from_numpy(feat).cuda(), keep=True)
    torch.cuda.synchronize()
    return net, out, out_idx, records


def test_c2_full_batch_against_the_oracle(workloads, backbone, gpu_handle):
    cfg = workloads.CONFIGS["c2"]
    idx, feat, layers, weights = workloads.make_inputs("c2")
    assert idx.shape[0] == 4 * 120000
    net, out, out_idx, records = _forward_records(backbone, gpu_handle, list(cfg["grid"]), cfg["batch"], idx, feat, layers, weights)
    tasks, meta = batch_oracle.group_tasks(records, weights, cfg["batch"])
    report = batch_oracle.check_records(_run_pool(tasks), meta, cfg["batch"], helpers.TOL_HALF)
    assert len(report) == 12
    assert out.shape == (records[-1].n_out, 128) and torch.equal(out_idx, records[-1].out_indices)
    net.close()


def test_c3_full_batch_against_the_oracle(workloads, backbone, gpu_handle):
    cfg = workloads.CONFIGS["c3"]
    idx, feat, layers, weights = workloads.make_inputs("c3")
    assert idx.shape[0] == 8 * 200000 and layers[0].ci == 128 and layers[0].co == 128
    net, out, out_idx, records = _forward_records(backbone, gpu_handle, list(cfg["grid"]), cfg["batch"], idx, feat, layers, weights)
    tasks, meta = batch_oracle.group_tasks(records, weights, cfg["batch"])
    report = batch_oracle.check_records(_run_pool(tasks), meta, cfg["batch"], helpers.TOL_HALF)
    assert len(report) == 1 and out.shape == (1600000, 128)
    net.close()


def test_c4_sharded_full_batch_against_the_oracle(workloads, backbone, gpu_handle):
    """16 samples split over 8 ranks (two samples each, batch index relabelled), every
    rank's layer records against the oracle, and the ranks' final rows concatenated in rank
    order against the unsharded run of the same 16 samples."""
    sharding = importlib.import_module("mluops_b200.sharding")
    cfg = workloads.CONFIGS["c4"]
    batch, world = cfg["batch"], 8
    idx, feat, layers, weights = workloads.make_inputs("c4")
    assert idx.shape[0] == 16 * 150000
    grid = list(cfg["grid"])
    w_dev = [torch.from_numpy(w).cuda() for w in weights]
    d_idx, d_feat = torch.from_numpy(idx).cuda(), torch.from_numpy(feat).cuda()
    tasks, metas, outs, idxs = [], [], [], []
    for rank in range(world):
        l_idx, l_feat, l_batch, b0 = sharding.shard_by_sample(d_idx, d_feat, batch, rank, world)
        net = backbone.SparseNetwork(gpu_handle, layers, w_dev, grid, l_batch)
        out, out_idx, records = net.forward(l_idx.contiguous(), l_feat.contiguous(), keep=True)
        torch.cuda.synchronize()
        t, m = batch_oracle.group_tasks(records, weights, l_batch, tag=rank)
        tasks += t
        metas.append((m, l_batch))
        o, i = sharding.gather_rows(out, out_idx, b0, 0, 1)
        outs.append(o)
        idxs.append(i)
        net.close()
        del records
    results = _run_pool(tasks)
    for rank, (m, l_batch) in enumerate(metas):
        assert len(batch_oracle.check_records(results, m, l_batch, helpers.TOL_HALF, tag=rank)) == 12
    del metas, tasks, results
    whole = backbone.SparseNetwork(gpu_handle, layers, w_dev, grid, batch)
    ref_out, ref_idx, _ = whole.forward(d_idx, d_feat)
    torch.cuda.synchronize()
    assert torch.equal(torch.cat(idxs), ref_idx)
    assert torch.equal(torch.cat(outs), ref_out)
    whole.close()
