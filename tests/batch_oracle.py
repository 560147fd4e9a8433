"""The CPU oracle run per batch sample in a process pool (test infrastructure).

Samples never interact: the batch index is the top digit of the linear voxel
index, so a pair never crosses samples.  The rulebook of a batch is therefore
the concatenation of the per-sample rulebooks (reference CPU path:
test/mlu_op_gtest/pb_gtest/src/zoo/get_indice_pairs/get_indice_pairs.cpp:288-406):
  * per offset k the pair list of the batch is the samples' lists in ascending
    sample order, input ids shifted by the sample's first input row, output ids
    by the sample's first output row (default mode: outputs are ranked by linear
    index with the batch index on top, so a sample's outputs follow all outputs
    of the samples before it; submanifold: outputs are the inputs);
  * indice_num[k] is the sum of the samples' counts;
  * out_indices is the samples' rows in order with the batch column restored.
The convolution of a sample only reads and writes that sample's rows
(.../zoo/indice_convolution_forward/indice_convolution_forward.cpp:148-171).

This lets the full benchmark batches (4 x 120,000, 8 x 200,000 and 16 x 150,000
voxels) meet the oracle in the time one sample takes: one task per (sample,
rulebook) runs the sample's rulebook and the convolutions of every layer that
uses it, compares the convolution outputs with the device's rows it was given
(teacher-forced: the oracle consumes the device's input rows of that layer) and
returns the compact pair lists, the coordinates and the four sums diff1 / diff2
are made of (pb_gtest/include/evaluator.h:431-519).
"""
import multiprocessing as mp
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _oracle():
    if ROOT not in sys.path:
        sys.path.insert(0, ROOT)
    import oracle
    return oracle


def sample_slices(batch_column, batch):
    """[(first, end)] row ranges of the samples 0..batch-1; rows must be grouped by ascending sample."""
    b = np.asarray(batch_column)
    assert b.size == 0 or (np.all(np.diff(b) >= 0) and b[0] >= 0 and b[-1] < batch), "rows not grouped by sample"
    counts = np.bincount(b, minlength=batch)
    ends = np.cumsum(counts)
    return [(int(e - c), int(e)) for c, e in zip(counts, ends)]


def _group_task(task):
    """One sample, one rulebook, the layers that use it.  All arrays are the sample's own rows."""
    o = _oracle()
    use_ref = task["use_ref"] and o.ref_lib() is not None
    idx = np.array(task["indices"], dtype=np.int32, copy=True)
    idx[:, 0] = 0
    g = task["geometry"]
    pairs, out_idx, num, n_out = o.get_indice_pairs(idx, 1, g["pad"], g["stride"], g["dilation"], g["filter_space"],
                                                    g["out_space"], g["sub_m"], use_ref=use_ref)
    K = pairs.shape[0]
    compact = [np.ascontiguousarray(pairs[k, :, :num[k]]) for k in range(K)]
    sums = []
    for conv in task["convs"]:
        f_in = conv["features_in"].astype(np.float32)
        ref = o.indice_convolution_forward(f_in, conv["weights"].astype(np.float32), "ARRAY", g["filter_space"], pairs,
                                           num, n_out, conv["co"], use_ref=use_ref)
        if conv["is_half"]:
            ref = o.round_through_half(ref)
        got = conv["features_out"]
        if got.shape[0] != n_out:  # the device disagrees about this sample's output rows
            sums.append(None)
            continue
        sums.append(diff_sums(got.astype(np.float32), ref))
    return {"key": task["key"], "compact": compact, "num": num.astype(np.int64), "n_out": int(n_out),
            "out_indices": np.ascontiguousarray(out_idx[:n_out]), "sums": sums}


def diff_sums(test, base):
    """(sum |t-b|, sum |b|, sum (t-b)^2, sum b^2) in double: the four sums of diff1 and diff2."""
    t = np.asarray(test, dtype=np.float64).ravel()
    b = np.asarray(base, dtype=np.float64).ravel()
    e = np.abs(t - b)
    return float(e.sum()), float(np.abs(b).sum()), float((e * e).sum()), float((b * b).sum())


def diffs_from_sums(sums):
    """diff1, diff2 of a tensor from the per-sample sums (evaluator.h:431-519)."""
    eps = 1e-9
    n1 = sum(s[0] for s in sums)
    d1 = sum(s[1] for s in sums)
    n2 = sum(s[2] for s in sums)
    d2 = sum(s[3] for s in sums)
    return n1 / (d1 + eps), float(np.sqrt(n2 / (d2 + eps)))


def default_workers(n_tasks):
    return max(1, min(n_tasks, os.cpu_count() or 1, 48))


def make_pool(workers):
    # spawn: the parent may hold a CUDA context, which must not be forked
    return mp.get_context("spawn").Pool(workers)


def _np(x):
    return x if isinstance(x, np.ndarray) else x.cpu().numpy()


def group_tasks(records, weights, batch, use_ref=True, tag=None):
    """Tasks for the layer records of SparseNetwork.forward(keep=True) (device tensors are
    copied to the host here) and the layers' filters (numpy, ARRAY layout).  One task per
    (rulebook, sample)."""
    groups = []
    for rec, w in zip(records, weights):
        rec.weights = w
        if rec.new_rulebook:
            groups.append([rec])
        else:
            groups[-1].append(rec)
    tasks, meta = [], []
    for gi, recs in enumerate(groups):
        first = recs[0]
        ly = first.layer
        idx_in = _np(first.in_indices)
        in_slices = sample_slices(idx_in[:, 0], batch)
        out_idx = _np(first.out_indices)
        out_slices = in_slices if ly.sub_m else sample_slices(out_idx[:, 0], batch)
        geometry = dict(pad=ly.pad, stride=ly.stride, dilation=ly.dilation, filter_space=ly.filter_space,
                        out_space=first.out_space, sub_m=ly.sub_m)
        f_in = [_np(r.features_in) for r in recs]
        f_out = [_np(r.features_out) for r in recs]
        for s in range(batch):
            (a, e), (oa, oe) = in_slices[s], out_slices[s]
            convs = [dict(features_in=fi[a:e], features_out=fo[oa:oe], weights=r.weights, co=r.layer.co,
                          is_half=fi.dtype == np.float16) for r, fi, fo in zip(recs, f_in, f_out)]
            tasks.append(dict(key=(tag, gi, s), indices=idx_in[a:e], geometry=geometry, convs=convs, use_ref=use_ref))
        meta.append(dict(records=recs, in_slices=in_slices, out_slices=out_slices))
    return tasks, meta


def assemble_rulebook(results, in_slices, sub_m, K, L):
    """Batch rulebook from the per-sample results (in sample order): (indice_pairs [K,2,L],
    out_indices [n,4], indice_num [K], n_out)."""
    num = np.zeros((K,), dtype=np.int64)
    pairs = np.full((K, 2, L), -1, dtype=np.int32)
    out_rows, out_first = [], 0
    for s, (res, (a, _)) in enumerate(zip(results, in_slices)):
        shift_out = a if sub_m else out_first
        for k in range(K):
            c = res["compact"][k]
            n = c.shape[1]
            if n:
                p = int(num[k])
                pairs[k, 0, p:p + n] = c[0] + a
                pairs[k, 1, p:p + n] = c[1] + shift_out
            num[k] += n
        rows = res["out_indices"].copy()
        rows[:, 0] = s
        out_rows.append(rows)
        out_first += res["n_out"]
    out_indices = np.concatenate(out_rows) if out_rows else np.zeros((0, 4), np.int32)
    return pairs, out_indices, num, int(out_indices.shape[0])


def check_records(results_by_key, meta, batch, tol, tag=None):
    """Compares the device's records with the assembled oracle.  Returns a list of
    per-layer (rulebook name, ci, co, diff1, diff2); raises AssertionError on a mismatch."""
    report = []
    for gi, m in enumerate(meta):
        recs = m["records"]
        first = recs[0]
        ly = first.layer
        K, L = ly.kernel_volume, first.n_in
        res = [results_by_key[(tag, gi, s)] for s in range(batch)]
        pairs, out_idx, num, n_out = assemble_rulebook(res, m["in_slices"], ly.sub_m, K, L)
        assert first.n_out == n_out, (ly.rulebook, first.n_out, n_out)
        assert np.array_equal(np.asarray(first.indice_num, dtype=np.int64), num), ly.rulebook
        assert np.array_equal(_np(first.out_indices), out_idx), ly.rulebook
        assert np.array_equal(_np(first.pairs), pairs), ly.rulebook
        for ci, rec in enumerate(recs):
            sums = [r["sums"][ci] for r in res]
            assert all(s is not None for s in sums), rec.layer.rulebook
            d1, d2 = diffs_from_sums(sums)
            report.append((rec.layer.rulebook, rec.layer.ci, rec.layer.co, d1, d2))
            assert d1 <= tol and d2 <= tol, (rec.layer.rulebook, rec.layer.ci, rec.layer.co, d1, d2)
    return report
