"""Device-side HXQ encoder: dense weight -> codebook, uint8 indices, sidecar and
optional per-group affine, as torch tensors ready for HelixLinear.

Follows the reference writer's algorithm (helix_substrate/hxq_writer_v3.py:162-232,
422-467; k-means helix_substrate/hxq_encoder.py:107-207; outliers
helix_substrate/generate_sidecars_v3.py:18-40) but runs on the GPU with plain
torch ops, because CPU k-means takes about a minute per 16 M-element tensor and
a 7B model has 196 of them.  It is the caller feeding the forward path, not part
of the timed path.

Nearest-centroid assignment uses the sorted codebook's midpoints
(``bucketize``): for a strictly increasing codebook this gives the same index as
the reference's ``argmin |w - c|`` except at exact ties (measure zero for float
data), where the reference takes the lower index and so does ``right=False``.
"""

from __future__ import annotations

from typing import Optional

import torch

_KMEANS_MAX_SAMPLES = 500_000


_subsample_cache: dict = {}


def _subsample_positions(n: int) -> torch.Tensor:
    """The reference writer's subsample: RandomState(42).choice(n, 500 000, replace=False)
    (helix_substrate/hxq_writer_v3.py:422-437).  It depends on n alone, so it is drawn once
    per tensor size (a full permutation of n on the host) and kept."""
    pos = _subsample_cache.get(n)
    if pos is None:
        import numpy as np
        pos = torch.from_numpy(np.random.RandomState(42).choice(n, _KMEANS_MAX_SAMPLES, replace=False).astype("int64"))
        if len(_subsample_cache) < 16:
            _subsample_cache[n] = pos
    return pos


def kmeans_codebook(flat: torch.Tensor, n_clusters: int = 256, max_iters: int = 10,
                    rtol: float = 1e-3) -> torch.Tensor:
    """1-D Lloyd on the reference's RandomState(42) subsample with percentile
    initialisation and the reference's relative-movement stop.  Same samples and the same
    iteration as the reference's CPU k-means; centroids can differ from it in the last bits
    (fp32 sums in another order), so a codebook made here is not bit-identical to one the
    reference writer makes - indices are always the nearest entry of whichever codebook is given."""
    n = flat.numel()
    if n > _KMEANS_MAX_SAMPLES:
        sample = flat[_subsample_positions(n).to(flat.device)]
    else:
        sample = flat
    sample = sample.float().sort().values
    q = torch.linspace(0, 1, n_clusters, device=flat.device, dtype=torch.float64)
    pos = q * (sample.numel() - 1)
    lo = pos.floor().long()
    hi = (lo + 1).clamp(max=sample.numel() - 1)
    frac = (pos - lo).float()
    cents = sample[lo] * (1 - frac) + sample[hi] * frac
    rng = float(cents[-1] - cents[0]) or 1.0
    for _ in range(max_iters):
        assign = assign_indices(sample, cents).long()
        sums = torch.zeros(n_clusters, device=flat.device).index_add_(0, assign, sample)
        cnts = torch.zeros(n_clusters, device=flat.device).index_add_(0, assign, torch.ones_like(sample))
        new = torch.where(cnts > 0, sums / cnts.clamp(min=1), cents)
        moved = float((new - cents).abs().max())
        if moved < rtol * rng:
            break
        cents = new
    return cents.sort().values.contiguous()


def assign_indices(flat: torch.Tensor, codebook: torch.Tensor) -> torch.Tensor:
    """Nearest entry of a sorted codebook, uint8."""
    cb = codebook.double()
    mids = ((cb[1:] + cb[:-1]) * 0.5).contiguous()     # exact in fp64: a rounded fp32 midpoint misplaces values next to it
    out = torch.empty(flat.numel(), dtype=torch.uint8, device=flat.device)
    step = 1 << 24                                      # bounded fp64 temporaries
    src = flat.reshape(-1)
    for a in range(0, src.numel(), step):
        out[a:a + step] = torch.bucketize(src[a:a + step].double(), mids, right=False).to(torch.uint8)
    return out.view(flat.shape)


def find_outliers_percentile(weight: torch.Tensor, percentile: float):
    """Two-sided percentile outliers: positions ascending, fp32 values."""
    flat = weight.reshape(-1).float()
    n = flat.numel()
    # numpy's linear-interpolated percentile lies between two order statistics;
    # "beyond it" is therefore decided by the order statistic on its inner side.
    import math
    pos_hi = (n - 1) * (percentile / 100.0)
    pos_lo = (n - 1) * ((100.0 - percentile) / 100.0)
    hi = torch.kthvalue(flat, min(n, int(math.floor(pos_hi)) + 1)).values
    lo = torch.kthvalue(flat, min(n, int(math.ceil(pos_lo)) + 1)).values
    pos = torch.nonzero((flat < lo) | (flat > hi)).reshape(-1)
    return pos, flat[pos]


def fit_group_affine(weight: torch.Tensor, codebook: torch.Tensor, indices: torch.Tensor,
                     group_size: int, exclude: Optional[torch.Tensor] = None):
    """Least-squares (s, t) per (row, group) of w on codebook[index], sidecar
    positions left out of the fit.  fp64 sums, fp32 result."""
    n_out, n_in = weight.shape
    ng = n_in // group_size
    w = weight.double().view(n_out, ng, group_size)
    c = codebook.double()[indices.long()].view(n_out, ng, group_size)
    m = torch.ones(n_out * n_in, dtype=torch.float64, device=weight.device)
    if exclude is not None and exclude.numel():
        m[exclude] = 0
    m = m.view(n_out, ng, group_size)
    n = m.sum(-1)
    sc, sw = (m * c).sum(-1), (m * w).sum(-1)
    scc, scw = (m * c * c).sum(-1), (m * c * w).sum(-1)
    den = n * scc - sc * sc
    ok = den.abs() > 1e-30
    s = torch.where(ok, (n * scw - sc * sw) / torch.where(ok, den, torch.ones_like(den)), torch.ones_like(den))
    t = torch.where(n > 0, (sw - s * sc) / n.clamp(min=1), torch.zeros_like(den))
    return s.float().contiguous(), t.float().contiguous()


@torch.no_grad()
def compress_weight(weight: torch.Tensor, n_clusters: int = 256, percentile: float = 99.95,
                    max_corrections: int = 0, group_size: int = 0, sidecar: bool = True,
                    st_dtype: torch.dtype = torch.float32) -> dict:
    """Encode one [out, in] matrix on its device.  Returns the constructor
    arguments of HelixLinear: codebook, indices, sidecar_positions,
    sidecar_values (fp16-rounded like the on-disk format) and, when
    ``group_size`` > 0, group_scales / group_offsets."""
    assert weight.ndim == 2 and n_clusters <= 256
    w = weight.float()
    flat = w.reshape(-1)
    cb = kmeans_codebook(flat, n_clusters)
    if cb.numel() < 256:
        cb = torch.cat([cb, cb[-1:].expand(256 - cb.numel())]).contiguous()
    idx = assign_indices(flat, cb[:n_clusters]).view_as(w)
    out = {"codebook": cb, "indices": idx}
    pos = None
    if sidecar:
        pos, vals = find_outliers_percentile(w, percentile)
        if max_corrections > 0 and pos.numel() > max_corrections:
            keep = torch.topk(vals.abs(), max_corrections).indices
            pos = pos[keep].sort().values
            vals = flat[pos]
        out["sidecar_positions"] = pos
        out["sidecar_values"] = vals.half().float()
    if group_size > 0:
        assert w.shape[1] % group_size == 0
        s, t = fit_group_affine(w, cb, idx, group_size, pos)
        out["group_scales"], out["group_offsets"] = s.to(st_dtype), t.to(st_dtype)
        out["group_size"] = group_size
    return out


def student_t_weight(shape, seed: int, device, std: float = 0.02, df: float = 5.0) -> torch.Tensor:
    """i.i.d. Student-t(df) rescaled to ``std`` - the synthetic weight
    distribution of the benchmark configurations."""
    g = torch.Generator(device=device).manual_seed(seed)
    z = torch.randn(shape, device=device, generator=g)
    chi = torch.zeros(shape, device=device)
    for _ in range(int(df)):
        chi += torch.randn(shape, device=device, generator=g) ** 2
    w = z / (chi / df).sqrt()
    return (w * (std / w.std())).contiguous()
