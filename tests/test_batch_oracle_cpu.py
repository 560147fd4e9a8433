"""The per-sample oracle (tests/batch_oracle.py) assembled over a batch must be the
whole-batch oracle, bit for bit: this is what lets the full benchmark batches meet
the oracle sample by sample in a process pool.  Checked here on the reference's
own CPU code (when built) and on the restatement, for both rulebook modes."""
import types

import numpy as np
import pytest

import batch_oracle
import helpers


def _records_from_oracle(oracle, workloads, config, batch, scale, use_ref):
    """Layer records as SparseNetwork.forward(keep=True) leaves them, produced by the
    whole-batch oracle instead of the device."""
    from oracle import backbone_cpu
    idx, feat, layers, weights = workloads.make_inputs(config, scale=scale, batch=batch)
    space = list(workloads.CONFIGS[config]["grid"])
    records, rulebooks = [], {}
    cur_idx, cur = idx, feat
    for ly, w in zip(layers, weights):
        rec = types.SimpleNamespace(layer=ly, new_rulebook=ly.rulebook not in rulebooks)
        if rec.new_rulebook:
            osp = list(space) if ly.sub_m else backbone_cpu.output_space(space, ly.pad, ly.stride, ly.dilation,
                                                                         ly.filter_space)
            rulebooks[ly.rulebook] = oracle.get_indice_pairs(cur_idx, batch, ly.pad, ly.stride, ly.dilation,
                                                             ly.filter_space, osp, ly.sub_m, use_ref=use_ref) + (osp,)
        pairs, out_idx, num, n_out, osp = rulebooks[ly.rulebook]
        out = oracle.round_through_half(oracle.indice_convolution_forward(
            cur.astype(np.float32), w.astype(np.float32), "ARRAY", ly.filter_space, pairs, num, n_out, ly.co,
            use_ref=use_ref)).astype(np.float16)
        rec.n_in, rec.n_out, rec.indice_num = cur_idx.shape[0], n_out, num.tolist()
        rec.pairs, rec.in_indices, rec.out_indices = pairs, cur_idx, out_idx[:n_out]
        rec.features_in, rec.features_out, rec.out_space = cur, out, osp
        records.append(rec)
        cur = out
        if not ly.sub_m:
            cur_idx, space = np.ascontiguousarray(out_idx[:n_out]), osp
    return records, weights


@pytest.mark.parametrize("use_ref", [False, True])
def test_per_sample_oracle_assembles_to_the_batch_oracle(oracle, workloads, use_ref):
    if use_ref and oracle.ref_lib() is None:
        pytest.skip("the reference's CPU code is not built here")
    batch = 2
    records, weights = _records_from_oracle(oracle, workloads, "c2", batch, 0.01, use_ref)
    assert sum(r.new_rulebook for r in records) == 8
    tasks, meta = batch_oracle.group_tasks(records, weights, batch, use_ref=use_ref)
    assert len(tasks) == 8 * batch
    with batch_oracle.make_pool(2) as pool:
        results = {r["key"]: r for r in pool.imap_unordered(batch_oracle._group_task, tasks)}
    report = batch_oracle.check_records(results, meta, batch, 0.0)
    assert len(report) == 12 and all(d1 == 0.0 and d2 == 0.0 for *_, d1, d2 in report)


def test_a_wrong_pair_or_row_is_caught(oracle, workloads):
    batch = 2
    records, weights = _records_from_oracle(oracle, workloads, "c1", batch, 0.02, False)
    records[0].pairs = records[0].pairs.copy()
    k = int(np.argmax(records[0].indice_num))
    records[0].pairs[k, 1, 0] += 1
    tasks, meta = batch_oracle.group_tasks(records, weights, batch, use_ref=False)
    results = {r["key"]: r for r in map(batch_oracle._group_task, tasks)}
    with pytest.raises(AssertionError):
        batch_oracle.check_records(results, meta, batch, helpers.TOL_HALF)
    records, weights = _records_from_oracle(oracle, workloads, "c3", batch, 0.005, False)
    records[0].features_out = records[0].features_out.copy()
    records[0].features_out[::7] *= np.float16(1.05)
    tasks, meta = batch_oracle.group_tasks(records, weights, batch, use_ref=False)
    results = {r["key"]: r for r in map(batch_oracle._group_task, tasks)}
    with pytest.raises(AssertionError):
        batch_oracle.check_records(results, meta, batch, helpers.TOL_HALF)
