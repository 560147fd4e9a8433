"""Layer stack on the CPU oracle (TEST INFRASTRUCTURE ONLY): runs the same list
of layers as the GPU driver, one oracle rulebook per distinct geometry and one
oracle convolution per layer, rounding each layer's output through half when the
storage dtype is half (what the reference harness does to a half output,
pb_gtest/src/executor.cpp:2247-2275).  Used by the multi-rank CPU tests and as
the timed CPU baseline of the benchmark."""
import numpy as np

from . import get_indice_pairs, indice_convolution_forward, round_through_half


def output_space(space, pad, stride, dilation, ks):
    return [(i + 2 * p - d * (k - 1) - 1) // s + 1 for i, p, s, d, k in zip(space, pad, stride, dilation, ks)]


def run_layers(indices, features, layers, weights, grid, batch, is_half=True, use_ref=False, fast=False,
               timings=None, threads=False):
    """Returns (features_out float32 [N,Co], out_indices int32 [N,4], per-layer pair totals)."""
    import time
    space = list(grid)
    rulebooks = {}
    idx = np.ascontiguousarray(indices, dtype=np.int32)
    feat = np.ascontiguousarray(features, dtype=np.float32)
    pair_totals = []
    for ly, w in zip(layers, weights):
        if ly.rulebook not in rulebooks:
            osp = list(space) if ly.sub_m else output_space(space, ly.pad, ly.stride, ly.dilation, ly.filter_space)
            t0 = time.perf_counter()
            pairs, out_idx, num, n_out = get_indice_pairs(idx, batch, ly.pad, ly.stride, ly.dilation,
                                                          ly.filter_space, osp, ly.sub_m, use_ref=use_ref)
            if timings is not None:
                timings["pairs"] = timings.get("pairs", 0.0) + time.perf_counter() - t0
            rulebooks[ly.rulebook] = (pairs, out_idx, num, n_out, osp)
        pairs, out_idx, num, n_out, osp = rulebooks[ly.rulebook]
        t0 = time.perf_counter()
        out = indice_convolution_forward(feat, np.asarray(w, dtype=np.float32), "ARRAY", ly.filter_space, pairs,
                                         num, n_out, ly.co, use_ref=use_ref, fast=fast, threads=threads)
        if timings is not None:
            timings["conv"] = timings.get("conv", 0.0) + time.perf_counter() - t0
        feat = round_through_half(out) if is_half else out
        pair_totals.append(int(num.sum()))
        if not ly.sub_m:
            idx = np.ascontiguousarray(out_idx[:n_out])
            space = osp
    return feat, idx, pair_totals
