"""The SECOND-style backbone through the layer-stack driver: per-layer parity
(teacher-forced: the oracle consumes the GPU's output of the previous layer, so
each convolution is judged on its own 3e-3 budget) and bit-exact rulebooks."""
import numpy as np
import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu


def test_backbone_scaled(ops, oracle, workloads, backbone, gpu_handle):
    scale = 0.1
    idx, feat, layers, weights = workloads.make_inputs("c2", scale=scale, batch=2)
    grid = list(workloads.CONFIGS["c2"]["grid"])
    net = backbone.SparseNetwork(gpu_handle, layers, [torch.from_numpy(w).cuda() for w in weights], grid, 2)
    out, out_idx, records = net.forward(torch.from_numpy(idx).cuda(), torch.from_numpy(feat).cuda(), keep=True)
    torch.cuda.synchronize()
    assert len(records) == 12 and sum(r.new_rulebook for r in records) == 8
    cur_idx = idx
    for rec, w in zip(records, weights):
        ly = rec.layer
        if rec.new_rulebook:
            r_pairs, r_out, r_num, r_n = oracle.get_indice_pairs(
                cur_idx, 2, ly.pad, ly.stride, ly.dilation, ly.filter_space, rec.out_space, ly.sub_m)
            assert rec.n_out == r_n
            assert np.array_equal(np.array(rec.indice_num), r_num)
            assert np.array_equal(rec.pairs.cpu().numpy(), r_pairs)
            assert np.array_equal(rec.out_indices.cpu().numpy(), r_out[:r_n])
        f_in = rec.features_in.float().cpu().numpy()
        ref = oracle.round_through_half(oracle.indice_convolution_forward(
            f_in, w.astype(np.float32), "ARRAY", ly.filter_space, r_pairs, r_num, r_n, ly.co))
        got = rec.features_out.float().cpu().numpy()
        d1, d2, _ = oracle.diffs(got, ref, True)
        assert d1 <= helpers.TOL_HALF and d2 <= helpers.TOL_HALF, (ly.rulebook, ly.ci, ly.co, d1, d2)
        if not ly.sub_m:
            cur_idx = r_out[:r_n]
    assert out.shape == (records[-1].n_out, 128) and out_idx.shape == (records[-1].n_out, 4)
    assert records[-1].out_space == [2, 200, 176]
    conv, pair_bytes = backbone.roofline_bytes_and_flops(records, 2)
    assert len(conv) == 12 and pair_bytes > 0
