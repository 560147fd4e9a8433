"""Shared helpers of the tests: golden-case decoding, random geometry, parity checks."""
import numpy as np

PARAM_FIELDS = ["batch", "space", "ks", "stride", "pad", "dil", "out_space", "sub_m", "ci", "co", "n_out"]


def golden_case(golden, name):
    p = golden[name + "/params"].tolist()
    case = dict(batch=p[0], space=p[1:4], ks=p[4:7], stride=p[7:10], pad=p[10:13], dil=p[13:16],
                out_space=p[16:19], sub_m=p[19], ci=p[20], co=p[21], n_out=p[22])
    for key in ("indices", "indice_pairs", "out_indices", "indice_num", "features", "filters_array",
                "features_out"):
        case[key] = golden[name + "/" + key]
    return case


def golden_names(golden):
    return [str(n) for n in golden["names"]]


def out_space(space, pad, stride, dil, ks):
    return [(i + 2 * p - d * (k - 1) - 1) // s + 1 for i, p, s, d, k in zip(space, pad, stride, dil, ks)]


def random_indices(rng, batch, space, n):
    D, H, W = space
    lin = rng.choice(batch * D * H * W, size=n, replace=False)
    b, rem = np.divmod(lin, D * H * W)
    z, rem = np.divmod(rem, H * W)
    y, x = np.divmod(rem, W)
    return np.stack([b, z, y, x], 1).astype(np.int32)


def random_geometry(rng, sub_m):
    """A random legal convolution geometry on a small grid."""
    batch = int(rng.integers(1, 4))
    space = [int(v) for v in rng.integers(2, 11, 3)]
    ks = [int(v) for v in rng.integers(1, 4, 3)]
    if sub_m:
        ks = [k if k % 2 else k + 1 for k in ks]
        stride, dil = [1, 1, 1], [1, 1, 1]
        pad = [(k - 1) // 2 for k in ks]
        osp = list(space)
    else:
        stride = [int(v) for v in rng.integers(1, 4, 3)]
        dil = [int(rng.integers(1, 3)) if s == 1 else 1 for s in stride]
        pad = [int(v) for v in rng.integers(0, 3, 3)]
        osp = out_space(space, pad, stride, dil, ks)
        if min(osp) < 1:
            return None
    n = int(rng.integers(1, min(batch * space[0] * space[1] * space[2], 400) + 1))
    return dict(batch=batch, space=space, ks=ks, stride=stride, pad=pad, dil=dil, out_space=osp, sub_m=sub_m, n=n)


def has_unused_slot(indice_num, L):
    """True when at least one (k, j) slot of the rulebook is unused, the
    condition under which the reference's `unique.size() - 1` is the true count."""
    return int(np.sum(indice_num)) < len(indice_num) * L


def permute_filter(w_array, layout):
    """ARRAY [kd,kh,kw,Ci,Co] -> the requested layout."""
    if layout == "ARRAY":
        return np.ascontiguousarray(w_array)
    if layout == "NDHWC":
        return np.ascontiguousarray(np.transpose(w_array, (4, 0, 1, 2, 3)))
    if layout == "NCDHW":
        return np.ascontiguousarray(np.transpose(w_array, (4, 3, 0, 1, 2)))
    raise ValueError(layout)


# Acceptance thresholds of the convolution (diff1 and diff2): 3e-3 for half
# (reference indice_convolution_forward.cpp:674), 1e-5 for float (reference
# docs/design_docs/indice_convolution_forward/indice_convolution_forward.md:106-107).
TOL_HALF = 3e-3
TOL_FLOAT = 1e-5
