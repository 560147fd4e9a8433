"""Layer-stack driver over the C ABI: runs a list of sparse convolutions
(workloads.Layer) the way a framework plugin would call the library.

Per distinct geometry one mluOpGetIndicePairs call (layers that share a
`rulebook` name share its result), then per layer the indice_num device->host
copy the API requires (mluOpIndiceConvolutionForward takes a host array) and one
mluOpIndiceConvolutionForward call.  All work is enqueued on the handle's stream.
"""
import sys

import torch

# The package directory name is not a Python identifier, so the package is
# loaded by path under the name "mluops_b200" (see __graft_entry__.load_package);
# this module is always imported as its submodule.
ops = sys.modules[__package__]


class Workspace:
    """One device scratch buffer, grown on demand and reused by every call."""

    def __init__(self, device):
        self.device = device
        self.buf = torch.empty((1,), dtype=torch.uint8, device=device)

    def get(self, nbytes):
        if self.buf.numel() < nbytes:
            self.buf = torch.empty((int(nbytes * 1.25) + 256,), dtype=torch.uint8, device=self.device)
        return self.buf


class LayerRecord:
    """What one layer consumed and produced (kept for parity checks and roofline accounting)."""
    __slots__ = ("layer", "n_in", "n_out", "indice_num", "pairs", "out_indices", "features_in", "features_out",
                 "new_rulebook", "in_space", "out_space")


class SparseNetwork:
    def __init__(self, handle, layers, weights, grid, batch):
        """weights: per layer a CUDA tensor in ARRAY layout [kd,kh,kw,Ci,Co]."""
        self.handle, self.layers, self.weights = handle, layers, weights
        self.grid, self.batch = list(grid), int(batch)
        self.workspace = Workspace(weights[0].device)

    def forward(self, indices, features, keep=False):
        """indices [L,4] int32, features [L,Cin] on the GPU.
        Returns (features_out, out_indices, records)."""
        space = list(self.grid)
        rulebooks = {}
        records = []
        cur_idx, cur_feat = indices, features
        for ly, w in zip(self.layers, self.weights):
            new_rb = ly.rulebook not in rulebooks
            if new_rb:
                out_space = space if ly.sub_m else ops.output_space(space, ly.pad, ly.stride, ly.dilation,
                                                                     ly.filter_space)
                conv = ops.SparseConvDesc(self.batch, ly.pad, ly.stride, ly.dilation, space, ly.filter_space,
                                          out_space, ly.sub_m)
                L = cur_idx.shape[0]
                K = ly.kernel_volume
                cells = self.batch * out_space[0] * out_space[1] * out_space[2]
                out_rows = L if ly.sub_m else min(K * L, cells)
                pairs, out_idx, num_dev, n_out = self._pairs(conv, cur_idx, out_rows)
                num_host = num_dev.cpu().tolist()  # the convolution API takes a host array
                conv.destroy()
                rulebooks[ly.rulebook] = (pairs, out_idx, num_host, n_out, list(out_space))
            pairs, out_idx, num_host, n_out, out_space = rulebooks[ly.rulebook]
            out = self._conv(cur_feat, w, ly, pairs, num_host, n_out)
            if keep:
                rec = LayerRecord()
                rec.layer, rec.n_in, rec.n_out, rec.indice_num = ly, cur_feat.shape[0], n_out, num_host
                rec.pairs, rec.out_indices = pairs, out_idx[:n_out]
                rec.features_in, rec.features_out, rec.new_rulebook = cur_feat, out, new_rb
                rec.in_space, rec.out_space = list(space), list(out_space)
                records.append(rec)
            else:
                rec = LayerRecord()
                rec.layer, rec.n_in, rec.n_out, rec.indice_num, rec.new_rulebook = (
                    ly, cur_feat.shape[0], n_out, num_host, new_rb)
                records.append(rec)
            cur_feat = out
            if not ly.sub_m:
                cur_idx = out_idx[:n_out]
                space = out_space
        return cur_feat, cur_idx, records

    def _pairs(self, conv, indices, out_rows):
        L, K = indices.shape[0], conv.kernel_volume
        d_in = ops.TensorDesc(ops.LAYOUT_ARRAY, ops.DTYPE_INT32, (L, 4))
        d_pairs = ops.TensorDesc(ops.LAYOUT_ARRAY, ops.DTYPE_INT32, (K, 2, L))
        d_out = ops.TensorDesc(ops.LAYOUT_ARRAY, ops.DTYPE_INT32, (out_rows, 4))
        d_num = ops.TensorDesc(ops.LAYOUT_ARRAY, ops.DTYPE_INT32, (K,))
        size = ops.get_indice_pairs_workspace_size(self.handle, conv, d_in, d_pairs, d_out, d_num)
        for d in (d_in, d_pairs, d_out, d_num):
            d.destroy()
        return ops.get_indice_pairs(self.handle, conv, indices, out_rows, self.workspace.get(size))

    def _conv(self, features, weight, ly, pairs, num_host, n_out):
        return ops.indice_convolution_forward(self.handle, features, weight, "ARRAY", ly.filter_space, pairs,
                                              num_host, n_out, ly.sub_m, workspace=self._conv_ws(features, ly, n_out))

    def _conv_ws(self, features, ly, n_out):
        # upper bound of the library's request: repacked filter + neighbour table + slack
        elem = features.element_size()
        n_pad = (n_out + 127) // 128 * 128
        need = ly.kernel_volume * ly.ci * ly.co * elem + ly.kernel_volume * n_pad * 4 + ly.kernel_volume * 4 + 2048
        return self.workspace.get(need)


def roofline_bytes_and_flops(records, elem_size):
    """Algorithmic bytes and flops of a run, from its actual pair counts.

    Per convolution: P = sum_k indice_num[k]; flops = 2*P*Ci*Co; bytes =
    P*(Ci+Co)*elem + 8*P (gathered input rows, scattered output rows, two int32
    ids per pair).  Per rulebook: 16*L (indices) + 8*K*L (indice_pairs incl. -1
    tails) + 16*N_out (out_indices) + 4*K (indice_num).
    """
    conv = []
    pairs_bytes = 0
    for rec in records:
        ly = rec.layer
        P = int(sum(rec.indice_num))
        conv.append(dict(P=P, flops=2 * P * ly.ci * ly.co, bytes=P * (ly.ci + ly.co) * elem_size + 8 * P,
                         ci=ly.ci, co=ly.co, n_in=rec.n_in, n_out=rec.n_out, sub_m=ly.sub_m))
        if rec.new_rulebook:
            pairs_bytes += 16 * rec.n_in + 8 * ly.kernel_volume * rec.n_in + 16 * rec.n_out + 4 * ly.kernel_volume
    return conv, pairs_bytes
