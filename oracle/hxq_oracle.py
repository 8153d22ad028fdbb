"""CPU restatement of the HXQ compressed-linear forward path of helix-substrate.

TEST INFRASTRUCTURE, NOT PRODUCT.  Only the test-suite, the smoke check and the
benchmark's CPU-baseline / reference legs may import this module; the shipped
path is the CUDA library and never routes through here.

Every function restates, in plain numpy, one piece of the reference's Python /
torch implementation and cites the reference file:line it follows.  Parity of
this restatement with the reference is pinned by the golden vectors under
``tests/golden/`` (made by ``tests/golden/make_golden.py``, which imports the
reference itself and records its outputs on seeded inputs).

Superset weight definition used by the CUDA kernels::

    W^[o, i] = cb[idx[o, i]] * s[o, (col0 + i) // G] + t[o, (col0 + i) // G]

``s == 1, t == 0`` is HelixLinear (helix_linear.py:81-97); ``cb[k] == k`` is
fused_affine_group_matmul (triton_affine_group_matmul.py:10-14).  The reference
pins only those two corners; the interior (k-means codebook AND group affine)
is checked "by composition" against this restatement.
"""

from __future__ import annotations

import numpy as np

F32 = np.float32


# ---------------------------------------------------------------------------
# Dequantisation (bit-exact target)
# ---------------------------------------------------------------------------

def _group_ids(n_cols: int, group_size: int, col0: int = 0) -> np.ndarray:
    return (col0 + np.arange(n_cols, dtype=np.int64)) // group_size


def gather_affine(codebook, indices, scales=None, offsets=None, group_size=0, col0=0):
    """``cb[idx]`` and, when group scale/offset are given, ``w*s + t`` per group.

    The gather follows hxq_reader_v3.py:116-127 (``codebook[indices]``).  The
    affine follows affine_group_matmul_reference
    (triton_affine_group_matmul.py:375-379): scale and offset are widened to
    fp32, the product is rounded to fp32 and then the sum is rounded to fp32
    (two roundings, no fused multiply-add).
    """
    cb = np.asarray(codebook, dtype=F32)
    idx = np.asarray(indices)
    w = cb[idx.astype(np.int64)]
    if scales is not None:
        g = _group_ids(idx.shape[1], int(group_size), int(col0))
        s = np.asarray(scales).astype(F32)[:, g]
        t = np.asarray(offsets).astype(F32)[:, g]
        w = (w * s).astype(F32) + t
        w = w.astype(F32)
    return w


def reconstruct(codebook, indices, positions=None, values=None,
                scales=None, offsets=None, group_size=0, col0=0):
    """Full dequantised weight, sidecar values OVERWRITING the codebook value.

    CDNAv3Reader.reconstruct (hxq_reader_v3.py:102-140): gather, then
    ``flat[positions] = values``.
    """
    w = gather_affine(codebook, indices, scales, offsets, group_size, col0)
    if positions is not None and len(positions):
        flat = w.ravel().copy()
        flat[np.asarray(positions, dtype=np.int64)] = np.asarray(values, dtype=F32)
        w = flat.reshape(w.shape)
    return w


def reconstruct_block(codebook, indices, start_row, end_row, positions=None, values=None,
                      scales=None, offsets=None, group_size=0, col0=0):
    """Rows ``[start_row, end_row)`` only (hxq_reader_v3.py:142-187)."""
    idx = np.asarray(indices)[start_row:end_row]
    sc = None if scales is None else np.asarray(scales)[start_row:end_row]
    of = None if offsets is None else np.asarray(offsets)[start_row:end_row]
    block = gather_affine(codebook, idx, sc, of, group_size, col0)
    if positions is not None and len(positions):
        cols = np.asarray(indices).shape[1]
        positions = np.asarray(positions, dtype=np.int64)
        lo, hi = start_row * cols, end_row * cols
        mask = (positions >= lo) & (positions < hi)
        if mask.any():
            flat = block.ravel().copy()
            flat[positions[mask] - lo] = np.asarray(values, dtype=F32)[mask]
            block = flat.reshape(block.shape)
    return block


# ---------------------------------------------------------------------------
# Sidecar derivation
# ---------------------------------------------------------------------------

def derive_sidecar(codebook, indices, positions, values,
                   scales=None, offsets=None, group_size=0, col0=0):
    """rows, cols, deltas as HelixLinear derives them (helix_linear.py:196-203,
    960-997): ``rows = pos // IN``, ``cols = pos % IN``,
    ``delta = value - cb[idx_flat[pos]]`` in fp32.  With a group affine the
    value subtracted is the affine-applied weight at that position."""
    idx = np.asarray(indices)
    n_in = idx.shape[1]
    positions = np.asarray(positions, dtype=np.int64)
    rows = positions // n_in
    cols = positions % n_in
    w_at = np.asarray(codebook, dtype=F32)[idx[rows, cols].astype(np.int64)]
    if scales is not None:
        g = (col0 + cols) // int(group_size)
        s = np.asarray(scales).astype(F32)[rows, g]
        t = np.asarray(offsets).astype(F32)[rows, g]
        w_at = ((w_at * s).astype(F32) + t).astype(F32)
    deltas = (np.asarray(values, dtype=F32) - w_at).astype(F32)
    return rows, cols, deltas


def csr_from_rows(rows, n_rows):
    """Row pointer of a row-sorted COO list (positions are ascending in the
    file, hxq_writer_v3.py:215-222, so rows are already sorted)."""
    rows = np.asarray(rows, dtype=np.int64)
    return np.searchsorted(rows, np.arange(n_rows + 1, dtype=np.int64), side="left").astype(np.int32)


# ---------------------------------------------------------------------------
# Forward
# ---------------------------------------------------------------------------

def dequant_tile(codebook, indices, start_row, end_row, rows=None, cols=None, deltas=None,
                 scales=None, offsets=None, group_size=0, col0=0):
    """HelixLinear._dequant_tile (helix_linear.py:735-781): gather then
    ``tile[r, c] += delta`` for sidecar entries inside the tile."""
    idx = np.asarray(indices)[start_row:end_row]
    sc = None if scales is None else np.asarray(scales)[start_row:end_row]
    of = None if offsets is None else np.asarray(offsets)[start_row:end_row]
    tile = gather_affine(codebook, idx, sc, of, group_size, col0)
    if rows is not None and len(rows):
        rows = np.asarray(rows, dtype=np.int64)
        mask = (rows >= start_row) & (rows < end_row)
        if mask.any():
            tile = tile.copy()
            # fancy-index "+=" as torch does it (positions are unique)
            tile[rows[mask] - start_row, np.asarray(cols, dtype=np.int64)[mask]] += \
                np.asarray(deltas, dtype=F32)[mask]
    return tile


def forward_naive(x, codebook, indices, rows=None, cols=None, deltas=None, bias=None,
                  scales=None, offsets=None, group_size=0, col0=0, chunk=256):
    """HelixLinear._forward_naive (helix_linear.py:783-822): 256-row tiles,
    ``x_f32 @ W_tile.T`` in fp32, bias added last; returns fp32 [N, OUT]."""
    idx = np.asarray(indices)
    n_out, n_in = idx.shape
    x2 = np.asarray(x, dtype=F32).reshape(-1, n_in)
    out = np.zeros((x2.shape[0], n_out), dtype=F32)
    for r0 in range(0, n_out, chunk):
        r1 = min(r0 + chunk, n_out)
        tile = dequant_tile(codebook, idx, r0, r1, rows, cols, deltas,
                            scales, offsets, group_size, col0)
        out[:, r0:r1] = x2 @ tile.T
    if bias is not None:
        out += np.asarray(bias, dtype=F32)[None, :]
    return out


def forward_f64(x, codebook, indices, rows=None, cols=None, deltas=None, bias=None,
                scales=None, offsets=None, group_size=0, col0=0):
    """Same operator with the contraction in fp64 - the yardstick the rel-L2
    tolerances are measured against (weights are the fp32 dequantised values)."""
    idx = np.asarray(indices)
    n_out, n_in = idx.shape
    w = dequant_tile(codebook, idx, 0, n_out, rows, cols, deltas,
                     scales, offsets, group_size, col0).astype(np.float64)
    x2 = np.asarray(x, dtype=np.float64).reshape(-1, n_in)
    out = x2 @ w.T
    if bias is not None:
        out += np.asarray(bias, dtype=np.float64)[None, :]
    return out


def naive_vq_matmul(x, codebook, indices, positions=None, values=None, bias=None):
    """The dense restatement the reference's kernel tests compare against
    (tests/test_triton_vq_matmul.py:56-74): gather, OVERWRITE sidecar values,
    matmul, bias."""
    w = reconstruct(codebook, indices, positions, values)
    out = np.asarray(x, dtype=F32) @ w.T
    if bias is not None:
        out = out + np.asarray(bias, dtype=F32)[None, :]
    return out.astype(F32)


def affine_group_matmul(x, indices, scales, offsets, group_size=128, bias=None):
    """affine_group_matmul_reference (triton_affine_group_matmul.py:366-383):
    ``W = idx * s + t`` per (row, group) in fp32, ``Y = x @ W.T`` (+ bias)."""
    idx = np.asarray(indices)
    n_out, n_in = idx.shape
    ng = n_in // group_size
    w = (idx.reshape(n_out, ng, group_size).astype(F32)
         * np.asarray(scales).astype(F32)[:, :, None]
         + np.asarray(offsets).astype(F32)[:, :, None]).astype(F32).reshape(n_out, n_in)
    y = np.asarray(x, dtype=F32) @ w.T
    if bias is not None:
        y = y + np.asarray(bias, dtype=F32)[None, :]
    return y.astype(F32)


def block_affine_weight(indices, scales, biases_ab, block_size=256):
    """HelixAffineLinear.decode_weight (helix_affine_linear.py:103-114):
    ``((u8 - 128) / 127) * scale[blk] + bias_ab[blk]``, blocks of ``block_size``
    along the input dimension, scale/bias stored fp16 and widened to fp32."""
    idx = np.asarray(indices)
    n_out, n_in = idx.shape
    bpr = n_in // block_size
    q = idx.reshape(n_out, bpr, block_size).astype(np.int16) - 128
    s = np.asarray(scales).astype(F32).reshape(n_out, bpr, 1)
    b = np.asarray(biases_ab).astype(F32).reshape(n_out, bpr, 1)
    return (((q.astype(F32) / F32(127.0)) * s).astype(F32) + b).astype(F32).reshape(n_out, n_in)


def block_affine_forward(x, indices, scales, biases_ab, block_size=256, bias=None):
    """HelixAffineLinear.forward on CPU tensors (helix_affine_linear.py:68-101)."""
    w = block_affine_weight(indices, scales, biases_ab, block_size)
    y = np.asarray(x, dtype=F32).reshape(-1, w.shape[1]) @ w.T
    if bias is not None:
        y = y + np.asarray(bias, dtype=F32)[None, :]
    return y.astype(F32)


# ---------------------------------------------------------------------------
# Encoder side (the callers feeding the path; not timed)
# ---------------------------------------------------------------------------

def find_outliers_percentile(tensor, percentile=99.9):
    """Two-sided percentile outliers (generate_sidecars_v3.py:18-40)."""
    flat = np.asarray(tensor).astype(F32).ravel()
    lo = np.percentile(flat, 100.0 - percentile)
    hi = np.percentile(flat, percentile)
    mask = (flat < lo) | (flat > hi)
    positions = np.where(mask)[0].astype(np.int64)
    return positions, flat[positions].astype(F32)


def sidecar_fp16_roundtrip(values):
    """Sidecar values are stored fp16 on disk and widened on read
    (generate_sidecars_v3.py:152-156,174-178)."""
    return np.asarray(values, dtype=F32).astype(np.float16).astype(F32)


def simple_kmeans(data, n_clusters=256, max_iters=10, rtol=0.001):
    """1-D Lloyd iterations with percentile initialisation and a relative
    movement stop (hxq_encoder.py:107-177, CPU branch)."""
    data = np.asarray(data, dtype=F32)
    n_clusters = min(n_clusters, len(np.unique(data)))
    centroids = np.percentile(data, np.linspace(0, 100, n_clusters)).astype(F32)
    cb_range = float(centroids[-1] - centroids[0])
    if cb_range < 1e-30:
        cb_range = 1.0
    abs_tol = rtol * cb_range
    assignments = None
    for _ in range(max_iters):
        assignments = chunked_assign(data, centroids)
        new_c = np.zeros_like(centroids)
        for i in range(n_clusters):
            m = assignments == i
            new_c[i] = np.mean(data[m]) if np.any(m) else centroids[i]
        if float(np.max(np.abs(new_c - centroids))) < abs_tol:
            break
        centroids = new_c
    return centroids, assignments


def chunked_assign(flat, codebook, chunk=1 << 18):
    """Nearest centroid by |w - c| with first-minimum tie break
    (hxq_writer_v3.py:446-467)."""
    flat = np.asarray(flat, dtype=F32)
    cb = np.asarray(codebook, dtype=F32)
    out = np.empty(len(flat), dtype=np.uint8)
    for a in range(0, len(flat), chunk):
        d = np.abs(flat[a:a + chunk, None] - cb[None, :])
        out[a:a + chunk] = np.argmin(d, axis=1).astype(np.uint8)
    return out


def assign_sorted(flat, codebook):
    """chunked_assign for a strictly increasing codebook in one pass: the nearest entry
    is found by bisecting the midpoints between neighbours (ties go to the lower index,
    as argmin's first minimum does).  Used where the 256-way distance table of
    chunked_assign is too slow (16 M-element tensors); the tests check both agree."""
    flat = np.asarray(flat, dtype=F32)
    cb = np.asarray(codebook, dtype=F32)
    mids = ((cb[1:].astype(np.float64) + cb[:-1].astype(np.float64)) * 0.5)
    return np.searchsorted(mids, flat.astype(np.float64), side="left").astype(np.uint8)


def kmeans_codebook(flat, n_clusters=256, max_samples=500_000):
    """Codebook fitted on a RandomState(42) subsample of at most 500 k values
    (hxq_writer_v3.py:422-437)."""
    flat = np.asarray(flat, dtype=F32)
    if len(flat) > max_samples:
        rng = np.random.RandomState(42)
        sample = flat[rng.choice(len(flat), max_samples, replace=False)]
    else:
        sample = flat
    cb, _ = simple_kmeans(sample, n_clusters, max_iters=10)
    return cb.astype(F32)


def fit_group_affine(weight, codebook, indices, group_size=128, exclude_positions=None):
    """Closed-form least squares of w on cb[idx] per (row, group):
    minimise sum (w - (s*c + t))^2.  The reference has no encoder for the
    codebook-with-group-affine form; this is the definition the package's
    writer follows.  Sidecar positions are left out of the fit."""
    w = np.asarray(weight, dtype=np.float64)
    n_out, n_in = w.shape
    assert n_in % group_size == 0
    ng = n_in // group_size
    c = np.asarray(codebook, dtype=np.float64)[np.asarray(indices).astype(np.int64)]
    m = np.ones_like(w)
    if exclude_positions is not None and len(exclude_positions):
        m.ravel()[np.asarray(exclude_positions, dtype=np.int64)] = 0.0
    w3, c3, m3 = (a.reshape(n_out, ng, group_size) for a in (w, c, m))
    n = m3.sum(-1)
    sc = (m3 * c3).sum(-1)
    sw = (m3 * w3).sum(-1)
    scc = (m3 * c3 * c3).sum(-1)
    scw = (m3 * c3 * w3).sum(-1)
    den = n * scc - sc * sc
    ok = np.abs(den) > 1e-30
    s = np.where(ok, (n * scw - sc * sw) / np.where(ok, den, 1.0), 1.0)
    t = np.where(n > 0, (sw - s * sc) / np.maximum(n, 1.0), 0.0)
    return s.astype(F32), t.astype(F32)


# ---------------------------------------------------------------------------
# Tensor-parallel shard descriptors (host logic mirrored by the package)
# ---------------------------------------------------------------------------

def shard_rows(n_out, rank, world):
    """Column-parallel: contiguous slice of output rows."""
    per = (n_out + world - 1) // world
    return min(rank * per, n_out), min((rank + 1) * per, n_out)


def shard_cols(n_in, rank, world):
    """Row-parallel: contiguous slice of input columns."""
    per = (n_in + world - 1) // world
    return min(rank * per, n_in), min((rank + 1) * per, n_in)


# ---------------------------------------------------------------------------
# Timed CPU baseline: the same operator with the reference's own torch ops
# ---------------------------------------------------------------------------

def forward_naive_torch(x, codebook, indices, rows=None, cols=None, deltas=None, bias=None,
                        scales=None, offsets=None, group_size=0, chunk=256):
    """HelixLinear._forward_naive with the torch calls the reference makes
    (helix_linear.py:735-822: ``codebook[idx.long()]`` gather per 256-row tile,
    in-place sidecar add, ``x @ W_tile.t()`` in fp32), plus the group affine of
    affine_group_matmul_reference (triton_affine_group_matmul.py:375-379) for the
    grouped configurations.  Used only as the timed CPU baseline: it runs on all
    the threads torch is given."""
    import torch
    cb = torch.as_tensor(codebook)
    idx = torch.as_tensor(indices)
    n_out, n_in = idx.shape
    x2 = torch.as_tensor(x).reshape(-1, n_in).float()
    out = torch.zeros(x2.shape[0], n_out, dtype=torch.float32)
    if rows is not None:
        rows_t, cols_t, deltas_t = (torch.as_tensor(a) for a in (rows, cols, deltas))
    if scales is not None:
        s_t, t_t = torch.as_tensor(scales).float(), torch.as_tensor(offsets).float()
    for r0 in range(0, n_out, chunk):
        r1 = min(r0 + chunk, n_out)
        tile = cb[idx[r0:r1].long()]
        if scales is not None:
            ng = n_in // group_size
            tile = (tile.reshape(r1 - r0, ng, group_size) * s_t[r0:r1, :, None]
                    + t_t[r0:r1, :, None]).reshape(r1 - r0, n_in)
        if rows is not None:
            mask = (rows_t >= r0) & (rows_t < r1)
            if mask.any():
                tile = tile.clone()
                tile[rows_t[mask] - r0, cols_t[mask]] += deltas_t[mask]
        out[:, r0:r1] = x2 @ tile.t()
    if bias is not None:
        out += torch.as_tensor(bias).unsqueeze(0)
    return out.numpy()
