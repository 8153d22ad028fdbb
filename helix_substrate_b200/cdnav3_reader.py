"""CDNAv3Reader: reads a ``{name}.cdnav3/`` tensor directory (meta.json,
codebook.npy, indices.bin, sidecar.npz, optional svd_*.npy and, as this
package's extension, group_scales.npy / group_offsets.npy) - interface of
helix_substrate/hxq_reader_v3.py:22-214.

reconstruct() / reconstruct_block() dequantise ON THE GPU through hxq_dequant
(bit-exact with the reference's numpy gather + overwrite) and return numpy
arrays; there is no CPU dequantisation in this package."""

from __future__ import annotations

import hashlib
import json
from pathlib import Path
from typing import Optional

import numpy as np

from .generate_sidecars_v3 import read_sidecar_v3


class CDNAv3Reader:
    def __init__(self, tensor_dir: Path, device: str = "cuda"):
        self.tensor_dir = Path(tensor_dir)
        if not self.tensor_dir.exists():
            raise FileNotFoundError(f"Tensor directory not found: {tensor_dir}")
        meta = self.tensor_dir / "meta.json"
        if not meta.exists():
            raise FileNotFoundError(f"meta.json not found in {tensor_dir}")
        self._meta = json.loads(meta.read_text())
        self._device = device
        self._module = None

    meta = property(lambda self: self._meta)
    shape = property(lambda self: tuple(self._meta["shape"]))
    tensor_name = property(lambda self: self._meta["tensor_name"])
    vector_dim = property(lambda self: self._meta.get("vector_dim", 1))
    group_size = property(lambda self: int(self._meta.get("group_size", 0)))
    has_sidecar = property(lambda self: (self.tensor_dir / "sidecar.npz").exists())
    has_svd_residual = property(lambda self: (self.tensor_dir / "svd_U.npy").exists())
    is_morpho = property(lambda self: self._meta.get("storage_mode") == "morpho")

    def _load_codebook(self) -> np.ndarray:
        return np.load(self.tensor_dir / "codebook.npy")

    def _load_indices(self) -> np.ndarray:
        if self.vector_dim != 1 or self._meta.get("index_dtype", "uint8") != "uint8":
            raise NotImplementedError("only scalar uint8 codebooks are on this path")
        return np.fromfile(self.tensor_dir / "indices.bin", dtype=np.uint8).reshape(self.shape)

    def _load_sidecar(self):
        p = self.tensor_dir / "sidecar.npz"
        return read_sidecar_v3(p) if p.exists() else None

    def _load_svd_factors(self):
        return tuple(np.load(self.tensor_dir / f"svd_{n}.npy") for n in ("U", "s", "Vt"))

    def _helix(self):
        if self.is_morpho:
            raise NotImplementedError("the morpho codec is outside the compressed-linear path")
        if self._module is None:
            from .helix_linear import load_helix_linear_from_cdnav3
            self._module = load_helix_linear_from_cdnav3(self.tensor_dir).to(self._device)
        return self._module

    def reconstruct(self) -> np.ndarray:
        """Full fp32 tensor: codebook gather (+ group affine), sidecar values
        overwrite, SVD residual added."""
        return self.reconstruct_block(0, self.shape[0])

    def reconstruct_block(self, start_row: int, end_row: int) -> np.ndarray:
        return self._helix()._dequant_tile(start_row, end_row).cpu().numpy()

    def get_stats(self) -> dict:
        p = self.tensor_dir / "stats.json"
        return json.loads(p.read_text()) if p.exists() else {}

    def verify_codebook(self) -> bool:
        actual = hashlib.sha256(self._load_codebook().tobytes()).hexdigest()
        return actual == self._meta.get("codebook_sha256", "")
