"""The multi-rank path on CPU: two gloo ranks shard a batch by sample, each runs
the layer stack (the CPU oracle stands in for the GPU library), rank 0 gathers the
final rows; the result must be row-for-row the single-process run."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _rank_main(rank, world, port, queue):
    sys.path.insert(0, ROOT)
    import __graft_entry__ as entry
    import importlib
    _, workloads, _ = entry.load_package()
    sharding = importlib.import_module("mluops_b200.sharding")
    from oracle import backbone_cpu
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    batch = 3  # odd on purpose: ranks get 2 and 1 samples
    idx, feat, layers, weights = workloads.make_inputs("c2", scale=0.02, batch=batch)
    grid = workloads.CONFIGS["c2"]["grid"]
    l_idx, l_feat, l_batch, b0 = sharding.shard_by_sample(torch.from_numpy(idx), torch.from_numpy(feat), batch, rank,
                                                          world)
    out, out_idx, _ = backbone_cpu.run_layers(l_idx.numpy(), l_feat.numpy(), layers, weights, grid, l_batch)
    feats, idxs = sharding.gather_rows(torch.from_numpy(out), torch.from_numpy(out_idx), b0, rank, world)
    # the two-phase form the benchmark uses: coordinates first, features later, twice in a row on one object
    same_again = True
    # the ranks' row counts through the tensors' own group, then through a separate host group
    for host_group in (None, dist.new_group(backend="gloo")):
        two_phase = sharding.RowGather(b0, rank, world, host_group=host_group)
        for _ in range(2):
            two_phase.begin(torch.from_numpy(out_idx))
            f2, i2 = two_phase.finish(torch.from_numpy(out), wait=False)
            two_phase.wait()
            same_again = same_again and torch.equal(f2, feats) and torch.equal(i2, idxs)
    if rank == 0:
        ref_out, ref_idx, _ = backbone_cpu.run_layers(idx, feat, layers, weights, grid, batch)
        queue.put((bool(np.array_equal(feats.numpy(), ref_out)) and same_again,
                   bool(np.array_equal(idxs.numpy(), ref_idx)), int(feats.shape[0])))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_reproduce_single_process():
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, queue)) for r in range(2)]
    for p in procs:
        p.start()
    same_feat, same_idx, rows = queue.get(timeout=300)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert same_feat and same_idx and rows > 0


def test_sample_ranges_cover_the_batch(pkg):
    import importlib
    sharding = importlib.import_module("mluops_b200.sharding")
    for batch in (1, 4, 7, 16):
        for world in (1, 2, 3, 8):
            spans = [sharding.sample_range(batch, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == batch
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))


def test_rank_that_never_joins_times_out():
    """Failure detection on the host: a rank that never joins makes the rendezvous
    of the others fail within the process-group timeout instead of hanging."""
    import datetime
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(31500 + os.getpid() % 2000)
    with pytest.raises(Exception):
        dist.init_process_group("gloo", rank=0, world_size=2, timeout=datetime.timedelta(seconds=3))
    if dist.is_initialized():
        dist.destroy_process_group()
