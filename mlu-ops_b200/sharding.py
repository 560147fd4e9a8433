"""Batch-sample sharding of the sparse-convolution path over ranks.

Samples never interact: the batch index is the most significant digit of the
linear voxel index and a pair never crosses samples.  A rank therefore takes a
contiguous range of samples, relabels their batch index to start at zero, runs
the whole layer stack with batch = its sample count, and the final rows of all
ranks, concatenated in rank order with the batch index shifted back, are
row-for-row the single-process result (default-mode outputs are sorted by linear
index with the batch index on top; submanifold outputs keep input order and the
inputs are grouped by ascending batch index).

Only torch.distributed all_gather and all_to_all calls are used, so the same code
runs on NCCL (GPU tensors) and gloo (CPU tensors).
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
    all_rows = torch.empty((world,), dtype=torch.int64, device=features_out.device)
    dist.all_gather_into_tensor(all_rows, rows)
    counts = all_rows.tolist()  # one host read for all ranks' row counts
    # One variable-size exchange per tensor: rank dst receives counts[r] rows from
    # every rank r, the other ranks receive nothing (NCCL runs it as one group of
    # sends and receives; far less host work than one send/recv pair per peer).
    co = features_out.shape[1]
    if rank == dst:
        feats = torch.empty((sum(counts), co), dtype=features_out.dtype, device=features_out.device)
        idxs = torch.empty((sum(counts), 4), dtype=out_indices.dtype, device=out_indices.device)
        recv_rows = counts
    else:
        feats = torch.empty((0, co), dtype=features_out.dtype, device=features_out.device)
        idxs = torch.empty((0, 4), dtype=out_indices.dtype, device=out_indices.device)
        recv_rows = [0] * world
    send_rows = [0] * world
    send_rows[dst] = features_out.shape[0]
    dist.all_to_all_single(feats, features_out.contiguous(), recv_rows, send_rows)
    dist.all_to_all_single(idxs, shifted, recv_rows, send_rows)
    if rank == dst:
        return feats, idxs
    return features_out, shifted
