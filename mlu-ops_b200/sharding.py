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


class RowGather:
    """Final rows of every rank -> rank `dst`, in rank order, in two phases.

    The coordinates of the final rows are known as soon as the last rulebook
    exists, which is before the last convolutions have run.  begin() therefore
    exchanges the row counts and the coordinate rows on a second stream while
    those convolutions execute; finish() is left with one variable-size exchange
    of the feature rows.  On CPU tensors (gloo) both phases run in line.

    Every rank must call begin() and finish() once per step, in that order.
    finish(wait=False) leaves the exchange running on the second stream, so that
    the next step's kernels overlap it; wait() orders the launching stream after
    it (call it before reading the gathered rows, and once at the end).
    """

    def __init__(self, first_sample, rank, world, dst=0, device=None, host_group=None):
        """host_group: a process group on CPU tensors (gloo).  With it the ranks' row counts -
        numbers every rank already has on the host - are exchanged over that group; without it
        they travel through the device and the host has to wait for the stream to read them,
        which costs a rank whatever lead its host had over its GPU."""
        self.first_sample, self.rank, self.world, self.dst = int(first_sample), rank, world, dst
        self.host_group = host_group
        self.cuda = device is not None and torch.device(device).type == "cuda"
        self.comm = torch.cuda.Stream(device) if self.cuda and world > 1 else None
        self.counts = None
        self.idxs = None
        self.shifted = None

    def _on_comm(self):
        return torch.cuda.stream(self.comm) if self.comm is not None else _NullContext()

    def begin(self, out_indices, ready=None):
        """out_indices [n,4]: this rank's final coordinate rows.  `ready` (a CUDA event,
        optional) marks the point of the launching stream after which they are valid;
        without it the second stream waits for everything enqueued so far."""
        if self.comm is not None:
            if ready is not None:
                self.comm.wait_event(ready)
            else:
                self.comm.wait_stream(torch.cuda.current_stream())
        with self._on_comm():
            shifted = out_indices.clone()
            shifted[:, 0] += self.first_sample
            self.shifted = shifted
            if self.world == 1:
                return
            n = out_indices.shape[0]
            if self.host_group is not None:
                mine = torch.tensor([n], dtype=torch.int64)
                every = [torch.empty((1,), dtype=torch.int64) for _ in range(self.world)]
                dist.all_gather(every, mine, group=self.host_group)  # host to host: no stream is waited for
                self.counts = [int(t.item()) for t in every]
            else:
                rows = torch.tensor([n], dtype=torch.int64, device=out_indices.device)
                all_rows = torch.empty((self.world,), dtype=torch.int64, device=out_indices.device)
                dist.all_gather_into_tensor(all_rows, rows)
                self.counts = all_rows.tolist()  # one host read for all ranks' row counts
            total = sum(self.counts) if self.rank == self.dst else 0
            self.idxs = torch.empty((total, 4), dtype=out_indices.dtype, device=out_indices.device)
            dist.all_to_all_single(self.idxs, shifted, self._recv_rows(), self._send_rows(n))
            if self.comm is not None:
                out_indices.record_stream(self.comm)

    def _recv_rows(self):
        return list(self.counts) if self.rank == self.dst else [0] * self.world

    def _send_rows(self, n):
        send = [0] * self.world
        send[self.dst] = n
        return send

    def wait(self):
        """Orders the launching stream after everything enqueued on the second stream."""
        if self.comm is not None:
            torch.cuda.current_stream().wait_stream(self.comm)

    def finish(self, features_out, wait=True, ready=None):
        """features_out [n,Co]: this rank's final feature rows (n as given to begin()).
        Returns (features, indices): all ranks' rows on dst, the local rows (batch index
        shifted) elsewhere.  With wait=True the launching stream is ordered after the
        exchange on return; with wait=False the caller calls wait() before it reads them.
        `ready` as in begin(): the point of the launching stream after which features_out is
        valid (default: everything enqueued so far)."""
        if self.world == 1:
            return features_out, self.shifted
        if self.comm is not None:
            if ready is not None:
                self.comm.wait_event(ready)
            else:
                self.comm.wait_stream(torch.cuda.current_stream())
        with self._on_comm():
            total = sum(self.counts) if self.rank == self.dst else 0
            feats = torch.empty((total, features_out.shape[1]), dtype=features_out.dtype,
                                device=features_out.device)
            # One variable-size exchange: rank dst receives counts[r] rows from every rank r,
            # the other ranks receive nothing (NCCL runs it as one group of sends and
            # receives; far less host work than one send/recv pair per peer).
            dist.all_to_all_single(feats, features_out.contiguous(), self._recv_rows(),
                                   self._send_rows(features_out.shape[0]))
        if self.comm is not None:
            cur = torch.cuda.current_stream()
            if wait:
                cur.wait_stream(self.comm)
            for t in (feats, self.idxs, self.shifted):
                t.record_stream(cur)
            features_out.record_stream(self.comm)
        if self.rank == self.dst:
            return feats, self.idxs
        return features_out, self.shifted


class _NullContext:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


def gather_rows(features_out, out_indices, first_sample, rank, world, dst=0):
    """Both phases of RowGather back to back: final rows of every rank -> rank `dst`,
    in rank order, batch index shifted back by each rank's first sample.  Returns
    (features, indices) on dst, the local (shifted) rows elsewhere."""
    g = RowGather(first_sample, rank, world, dst, device=features_out.device)
    g.begin(out_indices)
    return g.finish(features_out)
