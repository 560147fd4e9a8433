"""PyTorch modules over the C ABI: the caller the library's sparse-convolution
operators are written for.

The reference library is called from mmcv's sparse-convolution code (reference
docs/design_docs/indice_convolution_forward/indice_convolution_forward.md:114-130
names the caller: `indice_conv(features, filters, indice_pairs, indice_pairs_num,
num_active_out, inverse, subm)` in mmcv/ops/sparse_ops.py, used by the
convolution modules of mmcv/ops/sparse_conv.py).  This module offers that
function and modules of the same shape over this library:

    x = SparseConvTensor(features, indices, spatial_shape, batch_size)
    y = SubMConv3d(16, 32, 3, indice_key="subm1")(x)
    z = SparseConv3d(32, 64, 3, stride=2, padding=1)(y)
    z.features.sum().backward()

Every tensor stays on the GPU; the forward runs mluOpGetIndicePairs (once per
indice_key) and mluOpIndiceConvolutionForward, the backward runs
mluOpIndiceConvolutionBackwardFilter and mluOpIndiceConvolutionBackwardData on
the rulebook the forward used.  Weights are [kd,kh,kw,Cin,Cout] (the ARRAY filter
layout), float16 or float32 like the features.  There is no CPU path.
"""
import math
import sys

import torch
from torch import nn

ops = sys.modules[__package__]

_handles = {}


def _handle(device):
    """One library handle per device, bound to the stream that is current at each call."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key not in _handles:
        with torch.cuda.device(key):
            _handles[key] = ops.Handle(0)
    h = _handles[key]
    h.set_queue(torch.cuda.current_stream(device).cuda_stream)
    return h


def _triple(v):
    return [int(x) for x in v] if isinstance(v, (list, tuple)) else [int(v)] * 3


class Rulebook:
    """What mluOpGetIndicePairs produced for one geometry (shared through indice_key)."""
    __slots__ = ("indice_pairs", "out_indices", "indice_num", "num_act_out", "out_space", "filter_space", "sub_m",
                 "shared", "table", "input_table")

    def forward_table(self, handle):
        """The neighbour table of a rulebook that several layers share (an indice_key), built at its
        first use and kept: those layers then run from it instead of each rebuilding it from the
        pair lists.  None for a rulebook of one layer or a kernel volume above 128."""
        if not getattr(self, "shared", False) or len(self.indice_num) > 128:
            return None
        if getattr(self, "table", None) is None:
            self.table = ops.build_neighbour_table(handle, self.indice_pairs, self.indice_num, self.num_act_out)
        return self.table

    def backward_table(self, handle):
        """The same for the input gradients (for every offset and input row the output row it feeds)."""
        if not getattr(self, "shared", False) or len(self.indice_num) > 128:
            return None
        if getattr(self, "input_table", None) is None:
            self.input_table = ops.build_input_neighbour_table(handle, self.indice_pairs, self.indice_num,
                                                               self.num_act_out)
        return self.input_table


class SparseConvTensor:
    """features [N,C] and int32 indices [N,4] = (batch, z, y, x) of the active voxels of a
    batch of grids of size spatial_shape = (D, H, W).  Rows must not repeat a coordinate."""

    def __init__(self, features, indices, spatial_shape, batch_size, indice_dict=None):
        assert features.is_cuda and indices.is_cuda, "sparse convolution tensors live on the GPU"
        assert indices.dtype == torch.int32 and indices.shape == (features.shape[0], 4)
        self.features = features
        self.indices = indices.contiguous()
        self.spatial_shape = [int(v) for v in spatial_shape]
        self.batch_size = int(batch_size)
        self.indice_dict = {} if indice_dict is None else indice_dict

    def dense(self):
        """[batch, C, D, H, W] with zeros where no voxel is active."""
        D, H, W = self.spatial_shape
        C = self.features.shape[1]
        out = torch.zeros((self.batch_size, D, H, W, C), dtype=self.features.dtype, device=self.features.device)
        i = self.indices.long()
        out[i[:, 0], i[:, 1], i[:, 2], i[:, 3]] = self.features
        return out.permute(0, 4, 1, 2, 3).contiguous()


class _IndiceConvFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, features, weight, rulebook):
        features = features.contiguous()
        h = _handle(features.device)
        out = ops.indice_convolution_forward(h, features, weight, "ARRAY", rulebook.filter_space,
                                             rulebook.indice_pairs, rulebook.indice_num, rulebook.num_act_out,
                                             rulebook.sub_m, table=rulebook.forward_table(h))
        ctx.save_for_backward(features, weight)
        ctx.rulebook = rulebook
        return out

    @staticmethod
    def backward(ctx, grad_out):
        features, weight = ctx.saved_tensors
        rb = ctx.rulebook
        grad_out = grad_out.contiguous()
        h = _handle(features.device)
        grad_features = grad_weight = None
        if ctx.needs_input_grad[1]:
            grad_weight = ops.indice_convolution_backward_filter(h, features, grad_out, rb.filter_space,
                                                                 rb.indice_pairs, rb.indice_num, rb.sub_m,
                                                                 table=rb.forward_table(h))
        if ctx.needs_input_grad[0]:
            grad_features = ops.indice_convolution_backward_data(h, grad_out, weight, "ARRAY", rb.indice_pairs,
                                                                 rb.indice_num, rb.sub_m,
                                                                 table=lambda: rb.backward_table(h),
                                                                 forward_table=rb.forward_table(h) if rb.sub_m else None)
        return grad_features, grad_weight, None


def indice_conv(features, filters, indice_pairs, indice_pairs_num, num_active_out, inverse=False, subm=False):
    """features_out [num_active_out, Cout], differentiable in features and filters.
    filters [kd,kh,kw,Cin,Cout]; indice_pairs [K,2,N] int32 on the GPU; indice_pairs_num: K
    counts (a host sequence, or a tensor that is read back once)."""
    assert not inverse, "inverse convolution is not supported (the library returns NOT_SUPPORTED)"
    rb = Rulebook()
    rb.indice_pairs = indice_pairs
    rb.indice_num = indice_pairs_num.cpu().tolist() if torch.is_tensor(indice_pairs_num) else list(indice_pairs_num)
    rb.num_act_out, rb.sub_m = int(num_active_out), int(bool(subm))
    rb.filter_space = list(filters.shape[:3])
    rb.out_indices = rb.out_space = None
    return _IndiceConvFunction.apply(features, filters, rb)


class SparseConvolution(nn.Module):
    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, bias=True,
                 subm=False, indice_key=None, dtype=torch.float32):
        super().__init__()
        self.in_channels, self.out_channels = int(in_channels), int(out_channels)
        self.kernel_size, self.stride = _triple(kernel_size), _triple(stride)
        self.padding, self.dilation = _triple(padding), _triple(dilation)
        self.subm, self.indice_key = bool(subm), indice_key
        if self.subm:
            assert self.stride == [1, 1, 1] and self.dilation == [1, 1, 1], "submanifold: unit stride and dilation"
            assert all(k % 2 == 1 for k in self.kernel_size), "submanifold: odd kernel extents"
            self.padding = [(k - 1) // 2 for k in self.kernel_size]
        self.weight = nn.Parameter(torch.empty(*self.kernel_size, self.in_channels, self.out_channels, dtype=dtype))
        self.bias = nn.Parameter(torch.zeros(self.out_channels, dtype=dtype)) if bias else None
        fan_in = self.in_channels * self.kernel_size[0] * self.kernel_size[1] * self.kernel_size[2]
        nn.init.uniform_(self.weight, -1.0 / math.sqrt(fan_in), 1.0 / math.sqrt(fan_in))

    def rulebook(self, x):
        """The layer's rulebook: from x.indice_dict when indice_key names one, else mluOpGetIndicePairs."""
        if self.indice_key is not None and self.indice_key in x.indice_dict:
            return x.indice_dict[self.indice_key]
        out_space = list(x.spatial_shape) if self.subm else ops.output_space(
            x.spatial_shape, self.padding, self.stride, self.dilation, self.kernel_size)
        conv = ops.SparseConvDesc(x.batch_size, self.padding, self.stride, self.dilation, x.spatial_shape,
                                  self.kernel_size, out_space, self.subm)
        pairs, out_indices, num, n_out = ops.get_indice_pairs(_handle(x.features.device), conv, x.indices)
        conv.destroy()
        rb = Rulebook()
        rb.indice_pairs, rb.out_indices = pairs, (x.indices if self.subm else out_indices[:n_out])
        rb.indice_num = num.cpu().tolist()  # the convolution API takes the counts as a host array
        rb.num_act_out, rb.out_space = n_out, out_space
        rb.filter_space, rb.sub_m = list(self.kernel_size), int(self.subm)
        rb.shared = self.indice_key is not None  # other layers will come for it: worth keeping its tables
        if self.indice_key is not None:
            x.indice_dict[self.indice_key] = rb
        return rb

    def forward(self, x):
        rb = self.rulebook(x)
        out = _IndiceConvFunction.apply(x.features, self.weight, rb)
        if self.bias is not None:
            out = out + self.bias
        return SparseConvTensor(out, rb.out_indices, rb.out_space, x.batch_size, x.indice_dict)


class SparseConv3d(SparseConvolution):
    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, bias=True,
                 indice_key=None, dtype=torch.float32):
        super().__init__(in_channels, out_channels, kernel_size, stride, padding, dilation, bias, False, indice_key,
                         dtype)


class SubMConv3d(SparseConvolution):
    def __init__(self, in_channels, out_channels, kernel_size, bias=True, indice_key=None, dtype=torch.float32):
        super().__init__(in_channels, out_channels, kernel_size, 1, 0, 1, bias, True, indice_key, dtype)


class Voxelization(nn.Module):
    """Hard voxelization of a point cloud (mluOpVoxelization, deterministic mode): the step
    before the sparse backbone.  forward(points [N,F] float32) returns (voxels [M,max_points,F],
    coors [M,3] int32 (z,y,x), num_points_per_voxel [M] int32) with M = the number of voxels
    found (one host read), as mmcv's Voxelization module does."""

    def __init__(self, voxel_size, point_cloud_range, max_num_points, max_voxels=20000):
        super().__init__()
        self.register_buffer("voxel_size", torch.tensor(voxel_size, dtype=torch.float32))
        self.register_buffer("point_cloud_range", torch.tensor(point_cloud_range, dtype=torch.float32))
        self.max_num_points, self.max_voxels = int(max_num_points), int(max_voxels)

    def forward(self, points):
        assert points.is_cuda and points.dtype == torch.float32
        h = _handle(points.device)
        voxels, coors, npv, num = ops.voxelization(h, points.contiguous(), self.voxel_size.to(points.device),
                                                   self.point_cloud_range.to(points.device), self.max_num_points,
                                                   self.max_voxels)
        m = int(num.item())
        return voxels[:m], coors[:m], npv[:m]


class _DynamicScatterMax(torch.autograd.Function):
    @staticmethod
    def forward(ctx, feats, coors):
        h = _handle(feats.device)
        feats = feats.contiguous()
        voxel_feats, voxel_coors, p2v, counts, num = ops.dynamic_point_to_voxel_forward(h, feats, coors.clone(), "max")
        m = int(num.item())
        ctx.save_for_backward(feats, voxel_feats, p2v, counts, num)
        ctx.mark_non_differentiable(voxel_coors, p2v)
        ctx.rows = m
        return voxel_feats[:m], voxel_coors[:m], p2v

    @staticmethod
    def backward(ctx, grad_voxel_feats, _grad_coors, _grad_map):
        feats, voxel_feats, p2v, counts, num = ctx.saved_tensors
        grad = torch.zeros_like(voxel_feats)
        grad[:ctx.rows] = grad_voxel_feats
        h = _handle(feats.device)
        return ops.dynamic_point_to_voxel_backward(h, grad, feats, voxel_feats, p2v, counts, num), None


def dynamic_scatter(feats, coors, reduce_type="max"):
    """Dynamic voxelization of point features (mluOpDynamicPointToVoxelForward): feats [N,C] float32,
    coors [N,3] int32 on the GPU.  Returns (voxel_feats [M,C], voxel_coors [M,3] ascending,
    point2voxel_map [N]).  "max" is differentiable in feats (mluOpDynamicPointToVoxelBackward);
    "mean" is forward only, as in the reference."""
    if reduce_type == "max":
        return _DynamicScatterMax.apply(feats, coors)
    h = _handle(feats.device)
    voxel_feats, voxel_coors, p2v, _, num = ops.dynamic_point_to_voxel_forward(h, feats.detach().contiguous(),
                                                                              coors.clone(), reduce_type)
    m = int(num.item())
    return voxel_feats[:m], voxel_coors[:m], p2v
