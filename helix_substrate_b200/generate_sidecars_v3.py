"""Outlier sidecar of the CDNA-v3 layout: two-sided percentile selection and the
``sidecar.npz`` file (int64 positions ascending, fp16 values) - the format of
helix_substrate/generate_sidecars_v3.py:18-40,135-185."""

from __future__ import annotations

from pathlib import Path

import numpy as np


def find_outliers_percentile(tensor: np.ndarray, percentile: float = 99.9):
    """Positions (flat, ascending) and values beyond either tail percentile."""
    flat = np.asarray(tensor).astype(np.float32).ravel()
    lo, hi = np.percentile(flat, 100.0 - percentile), np.percentile(flat, percentile)
    positions = np.flatnonzero((flat < lo) | (flat > hi)).astype(np.int64)
    return positions, flat[positions].astype(np.float32)


def write_sidecar_npz(positions: np.ndarray, values: np.ndarray, output_path: Path) -> dict:
    output_path = Path(output_path)
    output_path.parent.mkdir(parents=True, exist_ok=True)
    np.savez_compressed(output_path, positions=np.asarray(positions, dtype=np.int64),
                        values=np.asarray(values).astype(np.float16))
    return {"format": "npz", "num_corrections": int(len(positions)), "size_bytes": output_path.stat().st_size}


def read_sidecar_v3(path: Path):
    path = Path(path)
    if path.suffix != ".npz":
        raise ValueError(f"Unknown sidecar format: {path.suffix}")
    with np.load(path) as z:
        return z["positions"].astype(np.int64), z["values"].astype(np.float32)
