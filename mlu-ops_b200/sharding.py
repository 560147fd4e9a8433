"""Batch-sample sharding of the sparse-convolution path over ranks.

Samples never interact: the batch index is the most significant digit of the
linear voxel index and a pair never crosses samples.  A rank therefore takes a
contiguous range of samples, relabels their batch index to start at zero, runs
the whole layer stack with batch = its sample count, and the final rows of all
ranks, concatenated in rank order with the batch index shifted back, are
row-for-row the single-process result (default-mode outputs are sorted by linear
index with the batch index on top; submanifold outputs keep input order and the
inputs are grouped by ascending batch index).

Only torch.distributed point-to-point and all_gather calls are used, so the same
code runs on NCCL (GPU tensors) and gloo (CPU tensors).
"""
import torch
import torch.distributed as dist


def sample_range(batch, rank, world):
    """Samples [b0, b1) owned by `rank` when `batch` samples are split over `world` ranks."""
    base, extra = divmod(batch, world)
    b0 = rank * base + min(rank, extra)
    return b0, b0 + base + (1 if rank < extra else 0)


def shard_by_sample(indices, features, batch, rank, world):
    """Rows of the rank's samples with the batch index relabelled to start at 0.
    indices [L,4] (b,z,y,x) must be grouped by ascending b.  Returns
    (local_indices, local_features, local_batch, first_sample)."""
    b0, b1 = sample_range(batch, rank, world)
    b = indices[:, 0]
    keep = (b >= b0) & (b < b1)
    local_idx = indices[keep].clone()
    local_idx[:, 0] -= b0
    return local_idx, features[keep], b1 - b0, b0


def gather_rows(features_out, out_indices, first_sample, rank, world, dst=0):
    """Final rows of every rank -> rank `dst`, in rank order, batch index shifted back
    by each rank's first sample.  Returns (features, indices) on dst, the local
    (shifted) rows elsewhere."""
    shifted = out_indices.clone()
    shifted[:, 0] += first_sample
    if world == 1:
        return features_out, shifted
    rows = torch.tensor([features_out.shape[0]], dtype=torch.int64, device=features_out.device)
    all_rows = [torch.zeros_like(rows) for _ in range(world)]
    dist.all_gather(all_rows, rows)
    counts = [int(r.item()) for r in all_rows]
    if rank == dst:
        feats = torch.empty((sum(counts), features_out.shape[1]), dtype=features_out.dtype,
                            device=features_out.device)
        idxs = torch.empty((sum(counts), 4), dtype=out_indices.dtype, device=out_indices.device)
        ops, off = [], 0
        for r in range(world):
            if r == dst:
                feats[off:off + counts[r]] = features_out
                idxs[off:off + counts[r]] = shifted
            elif counts[r] > 0:
                ops.append(dist.P2POp(dist.irecv, feats[off:off + counts[r]], r))
                ops.append(dist.P2POp(dist.irecv, idxs[off:off + counts[r]], r))
            off += counts[r]
        if ops:
            for w in dist.batch_isend_irecv(ops):
                w.wait()
        return feats, idxs
    if features_out.shape[0] > 0:
        ops = [dist.P2POp(dist.isend, features_out.contiguous(), dst), dist.P2POp(dist.isend, shifted, dst)]
        for w in dist.batch_isend_irecv(ops):
            w.wait()
    return features_out, shifted
