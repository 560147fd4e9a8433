"""The SECOND-style backbone through the layer-stack driver: per-layer parity
(teacher-forced: the oracle consumes the GPU's output of the previous layer, so
each convolution is judged on its own 3e-3 budget) and bit-exact rulebooks."""
import numpy as np
import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("scale,batch", [(0.1, 2), (1.0, 1)])
def test_backbone_per_layer_parity(ops, oracle, workloads, backbone, gpu_handle, scale, batch):
    """scale 0.1 x 2 samples, and one full-size sample (120,000 voxels) of the benchmark workload."""
    idx, feat, layers, weights = workloads.make_inputs("c2", scale=scale, batch=batch)
    grid = list(workloads.CONFIGS["c2"]["grid"])
    net = backbone.SparseNetwork(gpu_handle, layers, [torch.from_numpy(w).cuda() for w in weights], grid, batch)
    out, out_idx, records = net.forward(torch.from_numpy(idx).cuda(), torch.from_numpy(feat).cuda(), keep=True)
    torch.cuda.synchronize()
    assert len(records) == 12 and sum(r.new_rulebook for r in records) == 8
    cur_idx = idx
    for rec, w in zip(records, weights):
        ly = rec.layer
        if rec.new_rulebook:
            r_pairs, r_out, r_num, r_n = oracle.get_indice_pairs(
                cur_idx, batch, ly.pad, ly.stride, ly.dilation, ly.filter_space, rec.out_space, ly.sub_m)
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


def test_sample_sharding_reproduces_the_unsharded_run(ops, workloads, backbone, gpu_handle):
    """The multi-GPU partition (config c4: samples split over ranks, batch index relabelled,
    rows concatenated in rank order) emulated on one GPU: three samples of 150,000 voxels run
    as one batch and as shards of 2 + 1 samples must give identical rows, bit for bit."""
    import importlib
    sharding = importlib.import_module("mluops_b200.sharding")
    batch, world = 3, 2
    idx, feat, layers, weights = workloads.make_inputs("c4", batch=batch)
    grid = list(workloads.CONFIGS["c4"]["grid"])
    w_dev = [torch.from_numpy(w).cuda() for w in weights]
    d_idx, d_feat = torch.from_numpy(idx).cuda(), torch.from_numpy(feat).cuda()
    net = backbone.SparseNetwork(gpu_handle, layers, w_dev, grid, batch)
    ref_out, ref_idx, _ = net.forward(d_idx, d_feat)
    outs, idxs = [], []
    for rank in range(world):
        l_idx, l_feat, l_batch, b0 = sharding.shard_by_sample(d_idx, d_feat, batch, rank, world)
        shard_net = backbone.SparseNetwork(gpu_handle, layers, w_dev, grid, l_batch)
        out, out_idx, _ = shard_net.forward(l_idx.contiguous(), l_feat.contiguous())
        o, i = sharding.gather_rows(out, out_idx, b0, 0, 1)
        outs.append(o)
        idxs.append(i)
        shard_net.close()
    torch.cuda.synchronize()
    assert torch.equal(torch.cat(idxs), ref_idx)
    assert torch.equal(torch.cat(outs), ref_out)
    net.close()


def test_neighbour_table_fast_path_is_bit_identical(ops, workloads, backbone, gpu_handle):
    """One table per rulebook (mluOpBuildIndiceNeighbourTable + ...ForwardFromTable) gives exactly the
    features the reference-shaped entry point gives."""
    idx, feat, layers, weights = workloads.make_inputs("c2", batch=1)
    grid = list(workloads.CONFIGS["c2"]["grid"])
    net = backbone.SparseNetwork(gpu_handle, layers, [torch.from_numpy(w).cuda() for w in weights], grid, 1)
    d_idx, d_feat = torch.from_numpy(idx).cuda(), torch.from_numpy(feat).cuda()
    a, ia, ra = net.forward(d_idx, d_feat)
    b, ib, _ = net.forward(d_idx, d_feat, reuse_tables=True)
    c, ic, rc = net.forward(d_idx, d_feat, reuse_tables=True, defer_counts=True)
    torch.cuda.synchronize()
    assert torch.equal(a, b) and torch.equal(ia, ib) and torch.equal(a, c) and torch.equal(ia, ic)
    assert any(r.indice_num is None for r in rc)
    net.resolve_counts(rc)
    assert [r.indice_num for r in rc] == [r.indice_num for r in ra]
    net.close()


def test_gradient_table_fast_path_is_bit_identical(ops, workloads, backbone, gpu_handle):
    """One input neighbour table per rulebook (mluOpBuildIndiceInputNeighbourTable +
    ...BackwardDataFromTable) and the forward table handed to the filter gradient
    (...BackwardFilterFromTable) give exactly the gradients of the reference-shaped entry points."""
    idx, feat, layers, weights = workloads.make_inputs("c2", batch=1)
    grid = list(workloads.CONFIGS["c2"]["grid"])
    net = backbone.SparseNetwork(gpu_handle, layers, [torch.from_numpy(w).cuda() for w in weights], grid, 1)
    d_idx, d_feat = torch.from_numpy(idx).cuda(), torch.from_numpy(feat).cuda()
    out, _, records = net.forward(d_idx, d_feat, keep=True, reuse_tables=True)
    gen = torch.Generator(device="cuda").manual_seed(11)
    grad = torch.randn(out.shape, generator=gen, device="cuda").half()
    dx_ref, dw_ref = net.backward(records, grad)
    lib = ops.lib()
    lib.mluOpTraceKernelReset()
    lib.mluOpTraceKernelEnable(1)
    dx, dw = net.backward(records, grad, reuse_tables=True)
    torch.cuda.synchronize()
    lib.mluOpTraceKernelEnable(0)
    import ctypes
    buf = ctypes.create_string_buffer(1 << 16)
    assert lib.mluOpTraceKernelReport(buf, len(buf), None) == 0
    launches = {line.rsplit(",", 4)[0]: int(line.rsplit(",", 4)[1]) for line in buf.value.decode().splitlines()[1:]}
    # input gradients: the strided rulebooks build an input table each, the submanifold ones read their
    # forward table mirrored - except the first, whose 4-channel layer is not the tensor-memory kernel's;
    # the 64-channel filter gradients take the forward table: no build
    strided = len({ly.rulebook for ly in layers if not ly.sub_m})
    assert launches["buildNeighbourKernel"] == strided + 1, launches
    assert torch.equal(dx, dx_ref)
    assert all(torch.equal(a, b) for a, b in zip(dw, dw_ref))
    net.close()


def test_rulebooks_on_a_second_stream_are_bit_identical(ops, workloads, backbone, gpu_handle):
    """mluOpGetIndicePairs through a second handle on a second stream, overlapping the
    convolutions of earlier layers, gives exactly the single-stream results, repeatedly."""
    idx, feat, layers, weights = workloads.make_inputs("c2", batch=1)
    grid = list(workloads.CONFIGS["c2"]["grid"])
    d_w = [torch.from_numpy(w).cuda() for w in weights]
    d_idx, d_feat = torch.from_numpy(idx).cuda(), torch.from_numpy(feat).cuda()
    plain = backbone.SparseNetwork(gpu_handle, layers, d_w, grid, 1)
    a, ia, _ = plain.forward(d_idx, d_feat)
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    second = ops.Handle(stream.cuda_stream)
    net = backbone.SparseNetwork(gpu_handle, layers, d_w, grid, 1, rulebook_handle=second, rulebook_stream=stream)
    for _ in range(3):
        b, ib, _ = net.forward(d_idx, d_feat)
        c, ic, _ = net.forward(d_idx, d_feat, reuse_tables=True, defer_counts=True)
        torch.cuda.synchronize()
        assert torch.equal(a, b) and torch.equal(ia, ib) and torch.equal(a, c) and torch.equal(ia, ic)
    net.close()
    plain.close()
    second.destroy()
