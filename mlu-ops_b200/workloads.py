"""Seeded synthetic workloads for the sparse-convolution path.

No public dataset is involved: these generators are the workload.  They follow
the five configurations of the benchmark definition:

  c0  submanifold 3x3x3, batch 1, grid 40x400x352, 16,000 voxels drawn uniformly
      without replacement, fp32, Cin = Cout = 16
  c1  strided 3x3x3 s2 p1, batch 2, grid 41x1600x1408, 60,000 voxels per sample
      with a LiDAR-like distribution, fp16, 32 -> 64 channels
  c2  SECOND-style backbone, batch 4, ~120,000 voxels per sample, fp16
  c3  submanifold 3x3x3, batch 8, 200,000 voxels per sample, fp16, 128 -> 128
  c4  the c2 backbone at batch 16 x 150,000 voxels per sample, sharded by sample

LiDAR-like distribution, per sample: 70% of the voxels on a ground band
(z in [0,4), y and x uniform), 30% in 200 Gaussian blobs (centres uniform in the
grid, sigma 6 voxels per axis, rounded, clipped to the grid); duplicates are
rejected and redrawn; rows keep sampling order; samples are concatenated in
ascending batch index.
"""
import numpy as np

LIDAR_GRID = (41, 1600, 1408)


def uniform_voxels(rng, grid, n):
    """n distinct cells of `grid` = (D,H,W), uniform, in sampling order -> [n,3] (z,y,x)."""
    D, H, W = grid
    lin = rng.choice(D * H * W, size=n, replace=False)
    z, rem = np.divmod(lin, H * W)
    y, x = np.divmod(rem, W)
    return np.stack([z, y, x], axis=1).astype(np.int32)


def _take_new(cand_lin, seen, want):
    """First-occurrence-ordered entries of cand_lin not in `seen`, at most `want`."""
    _, first = np.unique(cand_lin, return_index=True)
    cand = cand_lin[np.sort(first)]
    cand = cand[~np.isin(cand, seen, assume_unique=False)]
    return cand[:want]


def lidar_like_voxels(rng, grid, n, n_blobs=200, sigma=6.0, ground_frac=0.7, band=4):
    """n distinct cells with the LiDAR-like distribution -> [n,3] (z,y,x), sampling order."""
    D, H, W = grid
    n_ground = int(round(ground_frac * n))
    chosen = np.empty((0,), dtype=np.int64)
    while chosen.size < n_ground:
        m = int((n_ground - chosen.size) * 1.1) + 16
        z = rng.integers(0, min(band, D), m)
        y = rng.integers(0, H, m)
        x = rng.integers(0, W, m)
        lin = (z.astype(np.int64) * H + y) * W + x
        chosen = np.concatenate([chosen, _take_new(lin, chosen, n_ground - chosen.size)])
    centres = np.stack([rng.uniform(0, D, n_blobs), rng.uniform(0, H, n_blobs), rng.uniform(0, W, n_blobs)], 1)
    while chosen.size < n:
        m = int((n - chosen.size) * 1.3) + 16
        which = rng.integers(0, n_blobs, m)
        pts = np.rint(centres[which] + rng.normal(0.0, sigma, (m, 3))).astype(np.int64)
        pts[:, 0] = np.clip(pts[:, 0], 0, D - 1)
        pts[:, 1] = np.clip(pts[:, 1], 0, H - 1)
        pts[:, 2] = np.clip(pts[:, 2], 0, W - 1)
        lin = (pts[:, 0] * H + pts[:, 1]) * W + pts[:, 2]
        chosen = np.concatenate([chosen, _take_new(lin, chosen, n - chosen.size)])
    z, rem = np.divmod(chosen, H * W)
    y, x = np.divmod(rem, W)
    return np.stack([z, y, x], axis=1).astype(np.int32)


def batch_indices(rng, grid, batch, per_sample, distribution="lidar", first_batch_index=0):
    """[batch*per_sample, 4] int32 rows (b, z, y, x), samples in ascending b."""
    rows = []
    for b in range(batch):
        zyx = (lidar_like_voxels(rng, grid, per_sample) if distribution == "lidar"
               else uniform_voxels(rng, grid, per_sample))
        bcol = np.full((zyx.shape[0], 1), b + first_batch_index, dtype=np.int32)
        rows.append(np.concatenate([bcol, zyx], axis=1))
    return np.ascontiguousarray(np.concatenate(rows, axis=0))


def normal(rng, shape, std, dtype):
    return (rng.standard_normal(shape) * std).astype(np.float32).astype(dtype)


class Layer:
    """One convolution of a network: geometry + channel counts; `rulebook` names
    the geometry so that layers with the same name share one rulebook."""

    def __init__(self, rulebook, sub_m, ci, co, filter_space, stride, pad, dilation=(1, 1, 1)):
        self.rulebook, self.sub_m, self.ci, self.co = rulebook, int(sub_m), ci, co
        self.filter_space, self.stride, self.pad, self.dilation = list(filter_space), list(stride), list(pad), list(dilation)

    @property
    def kernel_volume(self):
        return int(np.prod(self.filter_space))


def second_backbone_layers(c_in=4):
    """SECOND-style sparse backbone: subm c_in->16, subm 16->16; three stages of
    [3x3x3 s2 p1 conv to 32/64/64, then two subm convs]; (3,1,1) s(2,1,1) p0 conv 64->128."""
    k3, s1, s2, p1 = (3, 3, 3), (1, 1, 1), (2, 2, 2), (1, 1, 1)
    layers = [Layer("subm0", 1, c_in, 16, k3, s1, p1), Layer("subm0", 1, 16, 16, k3, s1, p1)]
    prev = 16
    for stage, width in enumerate((32, 64, 64), start=1):
        layers.append(Layer("down%d" % stage, 0, prev, width, k3, s2, p1))
        layers.append(Layer("subm%d" % stage, 1, width, width, k3, s1, p1))
        layers.append(Layer("subm%d" % stage, 1, width, width, k3, s1, p1))
        prev = width
    layers.append(Layer("down_final", 0, prev, 128, (3, 1, 1), (2, 1, 1), (0, 0, 0)))
    return layers


def layer_weights(rng, layers, dtype):
    """Per layer an ARRAY-layout filter [kd,kh,kw,Ci,Co] drawn from N(0, 1/fan_in), fan_in = K*Ci."""
    out = []
    for ly in layers:
        std = 1.0 / np.sqrt(ly.kernel_volume * ly.ci)
        out.append(normal(rng, tuple(ly.filter_space) + (ly.ci, ly.co), std, dtype))
    return out


CONFIGS = {
    "c0": dict(batch=1, grid=(40, 400, 352), per_sample=16000, distribution="uniform", dtype="float32",
               seed=0xC0),
    "c1": dict(batch=2, grid=LIDAR_GRID, per_sample=60000, distribution="lidar", dtype="float16", seed=0xC1),
    "c2": dict(batch=4, grid=LIDAR_GRID, per_sample=120000, distribution="lidar", dtype="float16", seed=0xC2),
    "c3": dict(batch=8, grid=LIDAR_GRID, per_sample=200000, distribution="lidar", dtype="float16", seed=0xC3),
    "c4": dict(batch=16, grid=LIDAR_GRID, per_sample=150000, distribution="lidar", dtype="float16", seed=0xC4),
}


def single_layer(config):
    """The one convolution of c0 / c1 / c3."""
    if config == "c0":
        return Layer("subm", 1, 16, 16, (3, 3, 3), (1, 1, 1), (1, 1, 1))
    if config == "c1":
        return Layer("down", 0, 32, 64, (3, 3, 3), (2, 2, 2), (1, 1, 1))
    if config == "c3":
        return Layer("subm", 1, 128, 128, (3, 3, 3), (1, 1, 1), (1, 1, 1))
    raise ValueError(config)


def make_inputs(config, scale=1.0, batch=None, first_batch_index=0, seed=None, first_sample=0):
    """(indices [L,4] int32, features [L,Cin], layers, weights) of a configuration.

    scale < 1 shrinks the voxel count per sample (for parity cases the CPU oracle
    finishes quickly); batch overrides the number of samples (multi-GPU shards).

    c4 is one fixed job of 16 samples that is split over ranks, so each of its
    samples has a random stream of its own: `first_sample` and `batch` select
    samples [first_sample, first_sample + batch) of that job (batch index
    relabelled to start at first_batch_index), and the rows a rank draws are
    exactly the rows of those samples in the unsharded job.
    """
    cfg = CONFIGS[config]
    base_seed = cfg["seed"] if seed is None else seed
    b = cfg["batch"] if batch is None else batch
    per = max(1, int(round(cfg["per_sample"] * scale)))
    dtype = np.float16 if cfg["dtype"] == "float16" else np.float32
    layers = second_backbone_layers() if config in ("c2", "c4") else [single_layer(config)]
    if config == "c4":
        idx_rows, feat_rows = [], []
        for i in range(b):
            rng = np.random.default_rng([base_seed, first_sample + i])
            idx_rows.append(batch_indices(rng, cfg["grid"], 1, per, cfg["distribution"], first_batch_index + i))
            feat_rows.append(normal(rng, (idx_rows[-1].shape[0], layers[0].ci), 1.0, dtype))
        indices = np.ascontiguousarray(np.concatenate(idx_rows))
        features = np.ascontiguousarray(np.concatenate(feat_rows))
    else:
        assert first_sample == 0
        rng = np.random.default_rng(base_seed)
        indices = batch_indices(rng, cfg["grid"], b, per, cfg["distribution"], first_batch_index)
        features = normal(rng, (indices.shape[0], layers[0].ci), 1.0, dtype)
    # weights come from their own stream so that every shard of a workload sees the same filters
    weights = layer_weights(np.random.default_rng([cfg["seed"], 0x5EED]), layers, dtype)
    return indices, features, layers, weights
