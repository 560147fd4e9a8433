"""The PyTorch modules over the C ABI: forward and autograd gradients of a small
layer stack against the CPU oracle, and a few optimiser steps."""
import importlib

import numpy as np
import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def sp(pkg):
    return importlib.import_module("mluops_b200.torch_sparse")


def make_input(rng, batch, space, n, c, dtype):
    idx = helpers.random_indices(rng, batch, space, n)
    feat = rng.standard_normal((n, c)).astype(np.float32)
    return idx, feat, torch.from_numpy(idx).cuda(), torch.from_numpy(feat).cuda().to(dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_layer_stack_matches_oracle(sp, oracle, dtype):
    rng = np.random.default_rng(31)
    is_half = dtype == torch.float16
    batch, space, n = 2, [8, 12, 10], 500
    idx, feat, d_idx, d_feat = make_input(rng, batch, space, n, 16, dtype)
    torch.manual_seed(3)
    l1 = sp.SubMConv3d(16, 32, 3, bias=False, indice_key="subm1", dtype=dtype).cuda()
    l2 = sp.SubMConv3d(32, 32, 3, bias=False, indice_key="subm1", dtype=dtype).cuda()
    l3 = sp.SparseConv3d(32, 64, 3, stride=2, padding=1, bias=False, dtype=dtype).cuda()
    d_feat.requires_grad_(True)
    x = sp.SparseConvTensor(d_feat, d_idx, space, batch)
    y1 = l1(x)
    y2 = l2(y1)
    y3 = l3(y2)
    assert len(x.indice_dict) == 1 and y2.indices is d_idx  # the second layer reused the first one's rulebook
    gen = torch.Generator(device="cuda").manual_seed(9)
    dy = torch.randn(y3.features.shape, generator=gen, device="cuda").to(dtype)
    y3.features.backward(dy)

    # the same stack on the CPU oracle
    def r(a):
        return oracle.round_through_half(a) if is_half else a
    f0 = r(feat)
    w = [r(l.weight.detach().float().cpu().numpy()) for l in (l1, l2, l3)]
    p1, _, n1, _ = oracle.get_indice_pairs(idx, batch, [1] * 3, [1] * 3, [1] * 3, [3] * 3, space, 1)
    osp = helpers.out_space(space, [1] * 3, [2] * 3, [1] * 3, [3] * 3)
    p3, oi3, n3, n_out3 = oracle.get_indice_pairs(idx, batch, [1] * 3, [2] * 3, [1] * 3, [3] * 3, osp, 0)
    a1 = r(oracle.indice_convolution_forward(f0, w[0], "ARRAY", [3] * 3, p1, n1, n, 32))
    a2 = r(oracle.indice_convolution_forward(a1, w[1], "ARRAY", [3] * 3, p1, n1, n, 32))
    a3 = r(oracle.indice_convolution_forward(a2, w[2], "ARRAY", [3] * 3, p3, n3, n_out3, 64))
    tol = helpers.TOL_HALF if is_half else helpers.TOL_FLOAT

    def close(got, ref, scale=1.0):
        d1, d2, _ = oracle.diffs(got.detach().float().cpu().numpy(), ref, is_half)
        assert d1 <= tol * scale and d2 <= tol * scale, (d1, d2)

    assert y3.features.shape == (n_out3, 64) and np.array_equal(y3.indices.cpu().numpy(), oi3[:n_out3])
    close(y3.features, a3)
    g3 = r(dy.float().cpu().numpy())
    dw3 = oracle.indice_convolution_backward_filter(a2, g3, [3] * 3, p3, n3)
    g2 = r(oracle.indice_convolution_backward_data(g3, w[2], "ARRAY", [3] * 3, p3, n3, 32, is_half))
    dw2 = oracle.indice_convolution_backward_filter(a1, g2, [3] * 3, p1, n1)
    g1 = r(oracle.indice_convolution_backward_data(g2, w[1], "ARRAY", [3] * 3, p1, n1, 32, is_half))
    dw1 = oracle.indice_convolution_backward_filter(f0, g1, [3] * 3, p1, n1)
    g0 = oracle.indice_convolution_backward_data(g1, w[0], "ARRAY", [3] * 3, p1, n1, 16, is_half)
    # gradients that passed through several half roundings get a proportionally wider band
    close(l3.weight.grad.reshape(27, 32, 64), r(dw3))
    close(l2.weight.grad.reshape(27, 32, 32), r(dw2), 2.0)
    close(l1.weight.grad.reshape(27, 16, 32), r(dw1), 3.0)
    close(d_feat.grad, r(g0), 3.0)


def test_functional_indice_conv_and_bias(sp, oracle):
    rng = np.random.default_rng(32)
    idx, feat, d_idx, d_feat = make_input(rng, 1, [6, 8, 8], 200, 8, torch.float32)
    layer = sp.SubMConv3d(8, 16, 3, bias=True).cuda()
    with torch.no_grad():
        layer.bias.copy_(torch.arange(16, dtype=torch.float32))
    y = layer(sp.SparseConvTensor(d_feat, d_idx, [6, 8, 8], 1))
    rb = layer.rulebook(sp.SparseConvTensor(d_feat, d_idx, [6, 8, 8], 1))
    y2 = sp.indice_conv(d_feat, layer.weight, rb.indice_pairs, rb.indice_num, rb.num_act_out, False, True)
    assert torch.allclose(y.features, y2 + layer.bias)
    dense = y.dense()
    assert dense.shape == (1, 16, 6, 8, 8)
    i = idx[0]
    assert torch.equal(dense[i[0], :, i[1], i[2], i[3]], y.features[0])


def test_a_few_optimiser_steps_reduce_the_loss(sp):
    rng = np.random.default_rng(33)
    idx, feat, d_idx, d_feat = make_input(rng, 2, [8, 12, 10], 600, 4, torch.float32)
    torch.manual_seed(1)
    net = [sp.SubMConv3d(4, 16, 3, indice_key="a").cuda(), sp.SubMConv3d(16, 16, 3, indice_key="a").cuda(),
           sp.SparseConv3d(16, 8, 3, stride=2, padding=1).cuda()]
    params = [p for l in net for p in l.parameters()]
    opt = torch.optim.SGD(params, lr=0.05)
    target = None
    losses = []
    for _ in range(8):
        x = sp.SparseConvTensor(d_feat, d_idx, [8, 12, 10], 2)
        for l in net:
            x = l(x)
            x.features = torch.relu(x.features) if l is not net[-1] else x.features
        if target is None:
            target = torch.ones_like(x.features)
        loss = ((x.features - target) ** 2).mean()
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    assert all(b < a for a, b in zip(losses, losses[1:])) and losses[-1] < 0.9 * losses[0], losses


def test_points_to_backbone_features(sp, oracle):
    """points -> Voxelization -> mean of the points of a voxel -> SparseConvTensor -> two layers."""
    rng = np.random.default_rng(34)
    n = 4000
    pts = np.concatenate([rng.random((n, 3)) * [8, 8, 2], rng.random((n, 1))], 1).astype(np.float32)
    vox = sp.Voxelization([0.5, 0.5, 0.5], [0, 0, 0, 8, 8, 2], 4, 3000).cuda()
    voxels, coors, npv = vox(torch.from_numpy(pts).cuda())
    ref = oracle.voxelization(pts, [0.5, 0.5, 0.5], [0, 0, 0, 8, 8, 2], 4, 3000)
    m = ref[3]
    assert voxels.shape[0] == m and np.array_equal(coors.cpu().numpy(), ref[1][:m])
    feats = voxels.sum(1) / npv.unsqueeze(1).float()
    idx = torch.cat([torch.zeros((m, 1), dtype=torch.int32, device="cuda"), coors], 1)
    x = sp.SparseConvTensor(feats, idx, [4, 16, 16], 1)
    y = sp.SparseConv3d(16, 8, 3, stride=2, padding=1).cuda()(sp.SubMConv3d(4, 16, 3).cuda()(x))
    assert y.features.shape[1] == 8 and y.spatial_shape == [2, 8, 8] and torch.isfinite(y.features).all()


def test_dynamic_scatter_autograd(sp, oracle):
    rng = np.random.default_rng(35)
    n, c = 3000, 5
    coors = np.stack([rng.integers(-1, h, n) for h in (4, 9, 8)], 1).astype(np.int32)
    feats = np.round(rng.standard_normal((n, c)) * 3).astype(np.float32)
    d_feats = torch.from_numpy(feats).cuda().requires_grad_(True)
    vf, vc, p2v = sp.dynamic_scatter(d_feats, torch.from_numpy(coors).cuda(), "max")
    ref = oracle.dynamic_point_to_voxel_forward(feats, coors, "max")
    m = ref[4]
    assert vf.shape == (m, c) and np.array_equal(vf.detach().cpu().numpy(), ref[0][:m])
    assert np.array_equal(vc.cpu().numpy(), ref[1][:m]) and np.array_equal(p2v.cpu().numpy(), ref[2])
    grad = rng.standard_normal((m, c)).astype(np.float32)
    vf.backward(torch.from_numpy(grad).cuda())
    assert np.array_equal(d_feats.grad.cpu().numpy(), oracle.dynamic_point_to_voxel_backward(grad, feats, ref[0][:m],
                                                                                            ref[2], m))
    mean, _, _ = sp.dynamic_scatter(d_feats, torch.from_numpy(coors).cuda(), "mean")
    assert np.array_equal(mean.cpu().numpy(), oracle.dynamic_point_to_voxel_forward(feats, coors, "mean")[0][:m])


def test_layers_that_share_a_rulebook_run_from_its_tables_bit_identically(sp):
    """Layers under one indice_key run from the rulebook's neighbour tables (built once, kept on
    the rulebook: forward, input gradient and, at 64 channels, filter gradient from a table);
    the same weights without a key rebuild the tables per call.  Same bits either way."""
    rng = np.random.default_rng(41)
    batch, space, n = 2, [8, 16, 16], 1500
    _, _, d_idx, d_feat = make_input(rng, batch, space, n, 64, torch.float16)
    results = []
    for key in ("k", None):
        torch.manual_seed(5)
        l1 = sp.SubMConv3d(64, 64, 3, bias=False, indice_key=key, dtype=torch.float16).cuda()
        l2 = sp.SubMConv3d(64, 64, 3, bias=False, indice_key=key, dtype=torch.float16).cuda()
        feat = d_feat.clone().requires_grad_(True)
        x = sp.SparseConvTensor(feat, d_idx, space, batch)
        y = l2(l1(x))
        gen = torch.Generator(device="cuda").manual_seed(6)
        y.features.backward(torch.randn(y.features.shape, generator=gen, device="cuda").half())
        if key is not None:
            rb = x.indice_dict[key]
            # forward table kept; the input gradients read it mirrored, so no input table was ever built
            assert rb.table is not None and getattr(rb, "input_table", None) is None
        results.append((y.features.detach(), feat.grad, l1.weight.grad, l2.weight.grad))
    for a, b in zip(*results):
        assert torch.equal(a, b)
