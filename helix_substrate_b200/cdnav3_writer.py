"""CDNAv3Writer: writes the per-tensor directory the reader and HelixLinear load
(layout of helix_substrate/hxq_writer_v3.py:1-11,162-336):

    {safe_name}.cdnav3/ meta.json codebook.npy indices.bin [sidecar.npz] stats.json
                        [group_scales.npy group_offsets.npy]   <- this package's extension

Encoding runs on the GPU (hxq_writer_gpu) when ``device`` is a CUDA device, or
on the host with the reference's exact numpy algorithm (subsample-500k Lloyd
with percentile initialisation, nearest-centroid assignment, two-sided
percentile sidecar), which reproduces the reference's files bit for bit.
Writing is the caller feeding the forward path; it is never timed.
"""

from __future__ import annotations

import hashlib
import json
from datetime import datetime, timezone
from pathlib import Path
from typing import Optional

import numpy as np

from .generate_sidecars_v3 import find_outliers_percentile, write_sidecar_npz
from .tensor_policy import TensorPolicy, classify_tensor, get_default_policy

_KMEANS_MAX_SAMPLES = 500_000
_ASSIGN_CHUNK = 1 << 18


def _safe_name(tensor_name: str) -> str:
    return tensor_name.replace("/", "_").replace(".", "_")


def _cosine(a: np.ndarray, b: np.ndarray) -> float:
    na, nb = np.linalg.norm(a), np.linalg.norm(b)
    return 0.0 if na == 0 or nb == 0 else float(np.dot(a, b) / (na * nb))


def _assign(flat: np.ndarray, codebook: np.ndarray) -> np.ndarray:
    out = np.empty(len(flat), dtype=np.uint8)
    for a in range(0, len(flat), _ASSIGN_CHUNK):
        out[a:a + _ASSIGN_CHUNK] = np.argmin(np.abs(flat[a:a + _ASSIGN_CHUNK, None] - codebook[None, :]), axis=1)
    return out


def _kmeans_1d(data: np.ndarray, n_clusters: int, max_iters: int = 10, rtol: float = 1e-3) -> np.ndarray:
    n_clusters = min(n_clusters, len(np.unique(data)))
    cents = np.percentile(data, np.linspace(0, 100, n_clusters)).astype(np.float32)
    span = float(cents[-1] - cents[0])
    tol = rtol * (span if span >= 1e-30 else 1.0)
    for _ in range(max_iters):
        assign = _assign(data, cents)
        new = cents.copy()
        for i in range(n_clusters):
            m = assign == i
            if m.any():
                new[i] = np.mean(data[m])
        if float(np.max(np.abs(new - cents))) < tol:
            break
        cents = new
    return cents.astype(np.float32)


def _fit_group_affine(weight: np.ndarray, codebook: np.ndarray, indices: np.ndarray, group_size: int,
                      exclude: Optional[np.ndarray] = None):
    """Per (row, group) least squares of w on codebook[index]: minimise
    sum (w - (s c + t))^2 over the group, sidecar positions left out."""
    n_out, n_in = weight.shape
    if n_in % group_size:
        raise ValueError(f"in_features {n_in} is not a multiple of group_size {group_size}")
    ng = n_in // group_size
    w = weight.astype(np.float64).reshape(n_out, ng, group_size)
    c = codebook.astype(np.float64)[indices.astype(np.int64)].reshape(n_out, ng, group_size)
    m = np.ones(n_out * n_in)
    if exclude is not None and len(exclude):
        m[exclude] = 0.0
    m = m.reshape(n_out, ng, group_size)
    n, sc, sw = m.sum(-1), (m * c).sum(-1), (m * w).sum(-1)
    scc, scw = (m * c * c).sum(-1), (m * c * w).sum(-1)
    den = n * scc - sc * sc
    ok = np.abs(den) > 1e-30
    s = np.where(ok, (n * scw - sc * sw) / np.where(ok, den, 1.0), 1.0)
    t = np.where(n > 0, (sw - s * sc) / np.maximum(n, 1.0), 0.0)
    return s.astype(np.float32), t.astype(np.float32)


class CDNAv3Writer:
    def __init__(self, base_dir: Path, device: Optional[str] = None):
        self.base_dir = Path(base_dir)
        self.base_dir.mkdir(parents=True, exist_ok=True)
        self.device = device  # None / "cpu": host numpy encoder; "cuda[:i]": GPU encoder

    def write_tensor(self, tensor, tensor_name: str, policy: Optional[TensorPolicy] = None,
                     source_artifact: str = "") -> dict:
        tensor = np.asarray(tensor)
        if policy is None:
            policy = get_default_policy(classify_tensor(tensor_name, shape=tensor.shape))
        if policy.storage_mode == "morpho" or getattr(policy, "vector_dim", 1) != 1 or policy.n_clusters > 256:
            raise NotImplementedError("only the scalar k<=256 codebook(+sidecar) modes are on this path")
        if tensor.ndim == 1 or policy.storage_mode == "exact":
            return self._write_exact(tensor.astype(np.float16), tensor_name)
        tensor = tensor.astype(np.float32)
        if tensor.ndim > 2:
            tensor = tensor.reshape(-1, tensor.shape[-1])
        return self._write_quantized(tensor, tensor_name, policy, source_artifact)

    def _write_exact(self, tensor: np.ndarray, tensor_name: str) -> dict:
        safe = _safe_name(tensor_name)
        path = self.base_dir / f"{safe}.npy"
        np.save(path, tensor)
        (self.base_dir / f"{safe}.npy.meta.json").write_text(json.dumps(
            {"tensor_name": tensor_name, "shape": list(tensor.shape), "storage_mode": "exact"}))
        return {"tensor_name": tensor_name, "storage_mode": "exact", "shape": list(tensor.shape),
                "original_bytes": tensor.nbytes, "compressed_bytes": path.stat().st_size}

    # -- encoders -------------------------------------------------------------
    def _encode_host(self, tensor: np.ndarray, policy: TensorPolicy):
        flat = tensor.ravel()
        if policy.use_kmeans:
            sample = flat
            if len(flat) > _KMEANS_MAX_SAMPLES:
                sample = flat[np.random.RandomState(42).choice(len(flat), _KMEANS_MAX_SAMPLES, replace=False)]
            cb = _kmeans_1d(sample, policy.n_clusters)
        else:
            cb = np.linspace(float(flat.min()), float(flat.max()), policy.n_clusters).astype(np.float32)
        idx = _assign(flat, cb)
        pos = vals = None
        if policy.sidecar_enabled:
            pos, vals = find_outliers_percentile(tensor, policy.percentile)
            if policy.max_corrections > 0 and len(pos) > policy.max_corrections:
                top = np.argsort(np.abs(vals))[::-1][:policy.max_corrections]
                pos = np.sort(pos[top])
                vals = flat[pos]
        return cb, idx.reshape(tensor.shape), pos, vals

    def _encode_device(self, tensor: np.ndarray, policy: TensorPolicy):
        import torch
        from . import hxq_writer_gpu as G
        w = torch.from_numpy(tensor).to(self.device)
        enc = G.compress_weight(w, policy.n_clusters, policy.percentile, policy.max_corrections, 0,
                                policy.sidecar_enabled)
        pos = vals = None
        if policy.sidecar_enabled:
            pos = enc["sidecar_positions"].cpu().numpy()
            vals = tensor.ravel()[pos]
        return enc["codebook"][:policy.n_clusters].cpu().numpy(), enc["indices"].cpu().numpy(), pos, vals

    def _write_quantized(self, tensor: np.ndarray, tensor_name: str, policy: TensorPolicy,
                         source_artifact: str) -> dict:
        out_dir = self.base_dir / f"{_safe_name(tensor_name)}.cdnav3"
        out_dir.mkdir(parents=True, exist_ok=True)
        rows, cols = tensor.shape
        flat = tensor.ravel()
        on_gpu = self.device is not None and str(self.device).startswith("cuda")
        cb, idx, pos, vals = (self._encode_device if on_gpu else self._encode_host)(tensor, policy)

        recon = cb[idx.ravel()]
        cos0 = _cosine(flat, recon)
        max_abs = float(np.max(np.abs(flat - recon)))
        n_out, sc_bytes, cos1 = 0, 0, cos0
        G = int(getattr(policy, "group_size", 0))
        scales = offsets = None
        if G > 0:
            scales, offsets = _fit_group_affine(tensor, cb, idx, G, pos)
            np.save(out_dir / "group_scales.npy", scales)
            np.save(out_dir / "group_offsets.npy", offsets)
            g = np.arange(cols) // G
            recon = (recon.reshape(rows, cols) * scales[:, g] + offsets[:, g]).astype(np.float32).ravel()
            cos0 = _cosine(flat, recon)
            max_abs = float(np.max(np.abs(flat - recon)))
            cos1 = cos0
        if pos is not None and len(pos):
            rec = write_sidecar_npz(pos, vals, out_dir / "sidecar.npz")
            n_out, sc_bytes = rec["num_corrections"], rec["size_bytes"]
            patched = recon.copy()
            patched[pos] = vals
            cos1 = _cosine(flat, patched)
        np.save(out_dir / "codebook.npy", cb)
        sha = hashlib.sha256(cb.tobytes()).hexdigest()
        idx.astype(np.uint8).tofile(out_dir / "indices.bin")
        meta = {
            "format_version": "cdna_v3", "tensor_name": tensor_name, "shape": [rows, cols], "dtype": "float32",
            "index_dtype": "uint8", "storage_mode": policy.storage_mode,
            "tensor_class": policy.tensor_class.value, "n_clusters": policy.n_clusters,
            "percentile": policy.percentile, "use_kmeans": policy.use_kmeans,
            "sidecar_enabled": policy.sidecar_enabled, "block_rows": policy.block_rows, "vector_dim": 1,
            "codebook_sha256": sha, "svd_residual_rank": 0, "source_artifact": source_artifact,
            "created_utc": datetime.now(timezone.utc).isoformat(),
        }
        if scales is not None:
            meta["group_size"] = G
        (out_dir / "meta.json").write_text(json.dumps(meta, indent=2))
        comp = (out_dir / "indices.bin").stat().st_size + (out_dir / "codebook.npy").stat().st_size + sc_bytes
        mu = float(flat.mean())
        var = float(((flat - mu) ** 2).mean())
        kurt = float(((flat - mu) ** 4).mean() / max(var ** 2, 1e-30) - 3.0) if var > 1e-30 else 0.0
        stats = {
            "tensor_name": tensor_name, "shape": [rows, cols], "original_bytes": tensor.nbytes,
            "compressed_bytes": comp, "compression_ratio": round(tensor.nbytes / max(1, comp), 2),
            "cosine_no_sidecar": round(cos0, 6), "cosine_with_sidecar": round(cos1, 6),
            "cosine_with_svd": round(cos1, 6), "max_abs_diff": round(max_abs, 6), "num_outliers": n_out,
            "sidecar_bytes": sc_bytes, "svd_residual_rank": 0, "svd_bytes": 0,
            "weight_mean": round(mu, 8), "weight_std": round(var ** 0.5, 8),
            "weight_min": round(float(flat.min()), 8), "weight_max": round(float(flat.max()), 8),
            "weight_kurtosis": round(kurt, 4), "tensor_class": policy.tensor_class.value,
            "n_clusters": policy.n_clusters, "vector_dim": 1, "codec_decision": policy.storage_mode,
        }
        (out_dir / "stats.json").write_text(json.dumps(stats, indent=2))
        return stats
