"""HelixLinear: nn.Linear drop-in over HXQ-compressed weights, B200 kernels only.

Same constructor, buffer names, state-dict keys and helper functions as the
reference module (helix_substrate/helix_linear.py:53-1499), so model code and
checkpoints written for it keep working.  What differs is underneath: every
forward mode runs the one CUDA path (hxq_gemv for a few tokens, hxq_gemm above),
a CPU input raises instead of falling back, and an optional per-group affine
(``group_scales`` / ``group_offsets`` / ``group_size``) is part of the weight:

    W^[o, i] = codebook[indices[o, i]] * group_scales[o, i // G] + group_offsets[o, i // G]
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Dict, Optional

import numpy as np
import torch
import torch.nn as nn

from .packed import HxqWeight, csr_from_positions, uses_gemv


@dataclass(frozen=True)
class HelixLinearStats:
    """Compression statistics for one layer (helix_linear.py:39-50)."""
    tensor_name: str
    in_features: int
    out_features: int
    rank: int
    n_outliers: int
    compression_ratio: float
    cosine_fidelity: float
    storage_bytes: int
    dense_bytes: int


_PRIMARY_OPTIONAL = ("sidecar_positions", "sidecar_values", "svd_U", "svd_s", "svd_Vt",
                     "bias", "channel_scales", "group_scales", "group_offsets")
_DERIVED = ("codebook_f16", "_sidecar_vq_vals", "_sidecar_rows", "_sidecar_cols", "_sidecar_deltas",
            "_csr_rowptr", "_csr_cols")
_SIDECAR_MODES = ("default", "always_on", "always_off", "threshold")


class HelixLinear(nn.Module):
    """y = x @ W^T + bias with W held as codebook + uint8 indices + sidecar
    (+ optional group affine, SVD residual and AWQ channel scales)."""

    _shared_buffer = None      # bf16 / fp16 scratch of the buffered mode, one per process, sized to the largest layer seen
    _shared_buffer_size = 0

    def __init__(self, in_features: int, out_features: int, codebook: torch.Tensor, indices: torch.Tensor,
                 sidecar_positions: Optional[torch.Tensor] = None, sidecar_values: Optional[torch.Tensor] = None,
                 svd_U: Optional[torch.Tensor] = None, svd_s: Optional[torch.Tensor] = None,
                 svd_Vt: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
                 tensor_name: str = "", compute_dtype: torch.dtype = torch.float32,
                 channel_scales: Optional[torch.Tensor] = None, vector_dim: int = 1,
                 group_scales: Optional[torch.Tensor] = None, group_offsets: Optional[torch.Tensor] = None,
                 group_size: int = 128):
        super().__init__()
        if vector_dim != 1:
            raise NotImplementedError("vector_dim > 1 (2-D / 4-D VQ) is outside the k=256 scalar path")
        if codebook.numel() > 256:
            raise NotImplementedError("codebooks above 256 entries (int16 indices) are outside this path")
        self._init_attrs(in_features, out_features, tensor_name, compute_dtype, vector_dim)
        self.group_size = int(group_size) if group_scales is not None else 0
        self.register_buffer("codebook", self._pad_codebook(codebook.to(torch.float32)))
        if indices.dtype != torch.uint8:
            indices = indices.to(torch.uint8)
        self.register_buffer("indices", indices.contiguous())
        opt = dict(sidecar_positions=sidecar_positions, sidecar_values=sidecar_values, svd_U=svd_U, svd_s=svd_s,
                   svd_Vt=svd_Vt, bias=bias, channel_scales=channel_scales, group_scales=group_scales,
                   group_offsets=group_offsets)
        if (sidecar_positions is None) != (sidecar_values is None):
            opt["sidecar_positions"] = opt["sidecar_values"] = None
        for name, t in opt.items():
            self.register_buffer(name, None if t is None else t.contiguous())
        for name in _DERIVED:
            self.register_buffer(name, None, persistent=False)
        self._derive()

    # ------------------------------------------------------------------ set-up
    def _init_attrs(self, in_features, out_features, tensor_name, compute_dtype, vector_dim):
        self.in_features, self.out_features = in_features, out_features
        self.tensor_name, self.compute_dtype, self.vector_dim = tensor_name, compute_dtype, vector_dim
        self._last_dispatch_path = "unknown"
        self._last_dispatch = None
        self._fused_available = False
        self._cell_skip_svd = False
        self._kurtosis_gate = None
        self._sidecar_phase = None
        self._sidecar_mode, self._sidecar_threshold = "default", 0.0
        self._sidecar_apply_count = self._sidecar_skip_count = 0
        self._sidecar_norms = []
        self._cuda_graph_mode = False
        # "fused" (default) and "naive": the fused sm_100a kernels.  "buffered": the reference's default mode
        # (helix_linear.py:556-634) - the whole weight dequantised into a shared 16-bit buffer by hxq_dequant,
        # then one dense library GEMM; worth choosing for prefill beyond ~1000 tokens.
        self._forward_mode = "fused"
        self._weight_buffer = None
        self._wave_enabled = False
        self.index_packing = None
        self._idx_rows, self._idx_cols = out_features, in_features
        self.has_svd = self.has_channel_scales = False
        self.rank = 0
        self.group_size = 0
        self.col0 = 0   # global column of local column 0 (row-parallel shards); group ids stay global
        self._packed = None
        self._packed_nosc = None
        self.weight = nn.Parameter(torch.empty(0, dtype=compute_dtype), requires_grad=False)

    @staticmethod
    def _pad_codebook(cb: torch.Tensor) -> torch.Tensor:
        """The kernels index a full 256-entry table; shorter codebooks (k-means
        on few distinct values) are padded with their last entry."""
        cb = cb.reshape(-1).contiguous()
        if cb.numel() < 256 and cb.numel() > 0:
            cb = torch.cat([cb, cb[-1:].expand(256 - cb.numel())]).contiguous()
        return cb

    def _derive(self) -> None:
        """Sidecar rows / cols / deltas and the CSR the kernels walk
        (reference derivation: helix_linear.py:184-210, 960-997)."""
        self._packed = self._packed_nosc = None
        n_in = self.in_features
        if self.sidecar_positions is not None and self.sidecar_values is not None:
            pos = self.sidecar_positions.long()
            rows, cols = pos // n_in, pos % n_in
            # gather the nnz index bytes first, widen only those (never the whole matrix)
            vq = self.codebook[self.indices.reshape(-1)[pos].long()]
            if self.group_scales is not None:
                g = (self.col0 + cols) // self.group_size - self.col0 // self.group_size
                vq = (vq * self.group_scales.float()[rows, g]) + self.group_offsets.float()[rows, g]
            vals = self.sidecar_values.float()
            rowptr, ccols = csr_from_positions(pos, self.out_features, n_in)
            derived = dict(_sidecar_vq_vals=vq.contiguous(), _sidecar_rows=rows, _sidecar_cols=cols,
                           _sidecar_deltas=(vals - vq).contiguous(),
                           _csr_rowptr=rowptr.to(pos.device), _csr_cols=ccols.to(pos.device))
        else:
            derived = dict.fromkeys(_DERIVED[1:], None)
        for name, t in derived.items():
            self.register_buffer(name, t, persistent=False)
        cb16 = self.codebook.half().contiguous() if self.compute_dtype == torch.float16 else None
        self.register_buffer("codebook_f16", cb16, persistent=False)
        self.has_svd = self.svd_U is not None
        self.rank = self.svd_U.shape[1] if self.has_svd else 0
        self.has_channel_scales = self.channel_scales is not None
        self._fused_available = self._check_fused_available()

    def _recompute_derived(self) -> None:
        """After a checkpoint filled the primary buffers: normalise empty
        optional buffers to None and rebuild everything derived
        (helix_linear.py:920-1018)."""
        if self.codebook is not None and self.codebook.ndim == 2:
            raise NotImplementedError("vector codebooks are outside the k=256 scalar path")
        for name in _PRIMARY_OPTIONAL:
            buf = getattr(self, name, None)
            if buf is not None and buf.numel() == 0:
                self.register_buffer(name, None)
        if self.codebook.numel() != 256:
            self.register_buffer("codebook", self._pad_codebook(self.codebook.float()))
        if self.group_scales is None:
            self.group_size = 0
        elif self.group_size == 0:
            self.group_size = self.in_features // self.group_scales.shape[1]
        self._derive()

    @classmethod
    def from_quantized_config(cls, in_features: int, out_features: int, tensor_name: str = "",
                              compute_dtype: torch.dtype = torch.float32, n_clusters: int = 256,
                              vector_dim: int = 1, index_packing: Optional[str] = None,
                              group_size: int = 0) -> "HelixLinear":
        """Empty shell whose buffers a checkpoint loader fills; call
        ``_recompute_derived()`` afterwards (helix_linear.py:1020-1119)."""
        if vector_dim != 1 or n_clusters > 256 or index_packing is not None:
            raise NotImplementedError("only k<=256 scalar uint8 indices are on this path")
        self = cls.__new__(cls)
        nn.Module.__init__(self)
        self._init_attrs(in_features, out_features, tensor_name, compute_dtype, vector_dim)
        self.group_size = int(group_size)
        self.register_buffer("codebook", torch.zeros(n_clusters, dtype=torch.float32))
        self.register_buffer("indices", torch.zeros(out_features, in_features, dtype=torch.uint8))
        self.register_buffer("sidecar_positions", torch.zeros(0, dtype=torch.int64))
        for name in _PRIMARY_OPTIONAL[1:]:
            self.register_buffer(name, torch.zeros(0, dtype=torch.float32))
        for name in _DERIVED:
            self.register_buffer(name, None, persistent=False)
        return self

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys,
                              unexpected_keys, error_msgs):
        """Buffers may change size while loading (empty placeholders become real
        data), so matching keys replace the buffer outright (helix_linear.py:241-274)."""
        for name in ("codebook", "indices", "weight") + _PRIMARY_OPTIONAL + _DERIVED:
            key = prefix + name
            if key in state_dict:
                t = state_dict.pop(key)
                if name == "weight":
                    self.weight = t
                elif name in _DERIVED:
                    continue  # rebuilt from the primaries
                else:
                    self.register_buffer(name, t)
        before = set(missing_keys)
        super()._load_from_state_dict(state_dict, prefix, local_metadata, strict, missing_keys,
                                      unexpected_keys, error_msgs)
        mine = {prefix + n for n in ("codebook", "indices", "weight") + _PRIMARY_OPTIONAL}
        missing_keys[:] = [k for k in missing_keys if k in before or k not in mine]
        self._packed = self._packed_nosc = None

    _KEEP_DTYPE = ("codebook", "sidecar_values", "group_scales", "group_offsets", "bias",
                   "_sidecar_deltas", "_sidecar_vq_vals")

    def _apply(self, fn, recurse=True):
        # .to(bf16) / .half() on the model must not round the codebook, the affine
        # tables or the sidecar: those buffers keep their dtype and only move.
        saved = {n: getattr(self, n) for n in self._KEEP_DTYPE if getattr(self, n, None) is not None}
        result = super()._apply(fn, recurse)
        for n, old in saved.items():
            new = getattr(self, n)
            if new is not None and new.dtype != old.dtype:
                self._buffers[n] = old.to(new.device)
        self._packed = self._packed_nosc = None
        self._fused_available = self._check_fused_available()
        return result

    def __setattr__(self, name, value):
        # tie_weights() assigns arbitrary tensors to .weight: keep it a frozen Parameter
        if name == "weight" and "_parameters" in self.__dict__ and "weight" in self._parameters:
            if isinstance(value, nn.Parameter):
                self._parameters["weight"] = value
            elif isinstance(value, torch.Tensor):
                self._parameters["weight"] = nn.Parameter(value, requires_grad=False)
            else:
                self._parameters["weight"] = nn.Parameter(torch.empty(0), requires_grad=False)
            return
        super().__setattr__(name, value)

    def set_compute_dtype(self, dtype: torch.dtype) -> None:
        self.compute_dtype = dtype
        cb16 = self.codebook.half().contiguous() if dtype == torch.float16 else None
        self.register_buffer("codebook_f16", cb16, persistent=False)

    def _check_fused_available(self) -> bool:
        return bool(self.codebook is not None and self.codebook.is_cuda)

    @property
    def _use_fused(self) -> bool:
        return self._fused_available

    def _refresh_dispatch_cache(self) -> None:
        self._fused_available = self._check_fused_available()

    # ------------------------------------------------------------------ kernels
    def packed(self, with_sidecar: bool = True) -> HxqWeight:
        """The descriptor over this module's CUDA buffers (built on first use,
        dropped whenever buffers move or reload)."""
        if not self.indices.is_cuda:
            raise RuntimeError(
                "HelixLinear runs on CUDA only: move the module and its input to a B200 "
                "(.cuda()); there is no CPU forward path. No silent fallback.")
        cached = self._packed if with_sidecar else self._packed_nosc
        if cached is not None:
            return cached
        if self.indices.dtype != torch.uint8 or self.indices.ndim != 2:
            raise NotImplementedError("only uint8 [out, in] indices are on this path")
        kw = {}
        if with_sidecar and self._csr_rowptr is not None:
            kw = dict(rowptr=self._csr_rowptr, cols=self._csr_cols, deltas=self._sidecar_deltas,
                      values=self.sidecar_values.float().contiguous())
        if self.group_scales is not None:
            kw.update(scales=self.group_scales, offsets=self.group_offsets, group_size=self.group_size)
        w = HxqWeight(self.codebook, self.indices, bias=self.bias, col0=self.col0, **kw)
        if with_sidecar:
            self._packed = w
        else:
            self._packed_nosc = w
        return w

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """x[..., in] -> y[..., out] in x's dtype (helix_linear.py:318-361).
        ``_forward_mode`` "buffered" selects the two-pass path (see ``_forward_buffered``); every
        other value runs the fused kernels."""
        if not x.is_cuda:
            raise RuntimeError(
                "HelixLinear.forward got a CPU tensor: this build has CUDA kernels only "
                "(sm_100a). No silent fallback.")
        if self._kurtosis_gate is not None and self.has_svd:
            with torch.no_grad():
                self._cell_skip_svd = not self._kurtosis_gate.step(x, cuda_graph_safe=self._cuda_graph_mode)
        if getattr(self, "_forward_mode", "fused") == "buffered":
            self._last_dispatch_path = "buffered"
            return self._forward_buffered(x)
        self._last_dispatch_path = "fused"
        return self._run(x, x.dtype if x.dtype in (torch.float16, torch.bfloat16, torch.float32) else torch.float32)

    def _run(self, x: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        shape = x.shape
        x2 = x.reshape(-1, self.in_features)
        if x2.dtype not in (torch.float32, torch.float16, torch.bfloat16):
            x2 = x2.float()
        if self.has_channel_scales:  # AWQ: weights live in scaled space (helix_linear.py:478-480)
            x2 = x2 / self.channel_scales.to(x2.dtype).unsqueeze(0)
        apply_sc = self._policy_decide(x2) if self._csr_rowptr is not None else False
        w = self.packed(with_sidecar=apply_sc)
        svd = self.has_svd and not self._cell_skip_svd
        y = w.matmul(x2, out_dtype=torch.float32 if svd else out_dtype)
        self._last_dispatch = {
            "dispatch_selected": "hxq_gemv_sm100a" if uses_gemv(x2.shape[0], x2.dtype) else "hxq_gemm_sm100a",
            "tokens": int(x2.shape[0]), "vq_dim": 1,
        }
        if svd:  # rank-r residual as two small dense products (triton_vq_matmul.py:715-721)
            xf = x2.float()
            y += ((xf @ self.svd_Vt.t()) * self.svd_s.unsqueeze(0)) @ self.svd_U.t()
            y = y.to(out_dtype)
        return y.reshape(*shape[:-1], self.out_features)

    # the reference's per-path entry points all land on the same kernels
    def _forward_fused(self, x: torch.Tensor) -> torch.Tensor:
        """fp32 result, as the reference's fused operator returns (triton_vq_matmul.py:592)."""
        return self._run(x, torch.float32)

    _forward_naive = _forward_fused
    _forward_wave = _forward_fused

    def _forward_buffered(self, x: torch.Tensor) -> torch.Tensor:
        """The reference's buffered mode (helix_linear.py:556-634): materialise the whole weight in a
        16-bit buffer shared by all modules, then one dense matmul.  The materialisation is
        ``hxq_dequant`` (codebook, group affine and sidecar in one pass over the indices: 3 bytes of
        traffic per weight where the reference's gather chain moves ~17); the matmul is the
        framework's dense GEMM, as in the reference.  Result in x's dtype (bf16 compute for fp32 x)."""
        if not x.is_cuda:
            raise RuntimeError("HelixLinear._forward_buffered got a CPU tensor. No silent fallback.")
        shape = x.shape
        x2 = x.reshape(-1, self.in_features)
        if self.has_channel_scales:
            x2 = x2 / self.channel_scales.to(x2.dtype).unsqueeze(0)
        compute_dt = x.dtype if x.dtype in (torch.float16, torch.bfloat16) else torch.bfloat16
        needed = self.out_features * self.in_features
        buf = HelixLinear._shared_buffer
        if buf is None or buf.device != x.device or buf.dtype != compute_dt or HelixLinear._shared_buffer_size < needed:
            buf = torch.empty(needed, dtype=compute_dt, device=x.device)
            HelixLinear._shared_buffer, HelixLinear._shared_buffer_size = buf, needed
        w = buf[:needed].view(self.out_features, self.in_features)
        apply_sc = self._policy_decide(x2) if self._csr_rowptr is not None else False
        self.packed(with_sidecar=apply_sc).dequant(dtype=compute_dt, out=w)
        if self.has_svd and not self._cell_skip_svd:
            w += ((self.svd_U * self.svd_s.unsqueeze(0)) @ self.svd_Vt).to(compute_dt)
        bias = None if self.bias is None else self.bias.to(compute_dt)
        y = torch.nn.functional.linear(x2.to(compute_dt), w, bias)
        self._last_dispatch = {"dispatch_selected": "hxq_dequant_sm100a+dense_gemm", "tokens": int(x2.shape[0]), "vq_dim": 1}
        return y.to(x.dtype if x.dtype in (torch.float16, torch.bfloat16, torch.float32) else torch.float32).reshape(*shape[:-1], self.out_features)

    def _dequant_tile(self, start_row: int, end_row: int) -> torch.Tensor:
        """Rows [start_row, end_row) as dense fp32 on the GPU.  Sidecar entries
        carry the stored value itself, i.e. CDNAv3Reader.reconstruct() semantics
        (hxq_reader_v3.py:128-133), bit for bit."""
        apply_sc = self._csr_rowptr is not None and getattr(self, "_apply_sidecar_this_call", True)
        tile = self.packed(with_sidecar=apply_sc).dequant(start_row, end_row, torch.float32)
        if self.has_svd and not self._cell_skip_svd:
            tile = tile + (self.svd_U[start_row:end_row] * self.svd_s.unsqueeze(0)) @ self.svd_Vt
        return tile

    def decode_weight(self) -> torch.Tensor:
        with torch.no_grad():
            return self._dequant_tile(0, self.out_features)

    # ------------------------------------------------------------------ sidecar policy
    def set_sidecar_policy(self, mode: str, threshold: float = 0.0) -> None:
        if mode not in _SIDECAR_MODES:
            raise ValueError(f"unknown sidecar mode: {mode!r}")
        self._sidecar_mode, self._sidecar_threshold = mode, float(threshold)

    def reset_sidecar_policy_stats(self) -> None:
        self._sidecar_apply_count = self._sidecar_skip_count = 0
        self._sidecar_norms = []

    def get_sidecar_policy_stats(self) -> dict:
        stats = {"n": 0}
        if self._sidecar_norms:
            a = np.asarray(self._sidecar_norms, dtype=np.float64)
            stats = {"n": int(a.size), "mean": float(a.mean()), "p50": float(np.percentile(a, 50)),
                     "p95": float(np.percentile(a, 95)), "min": float(a.min()), "max": float(a.max())}
        return {"mode": self._sidecar_mode, "threshold": self._sidecar_threshold,
                "apply_count": self._sidecar_apply_count, "skip_count": self._sidecar_skip_count,
                "norm_stats": stats}

    def _policy_decide(self, x_2d: torch.Tensor) -> bool:
        """Apply the sidecar this call? (helix_linear.py:701-733).  "threshold"
        synchronises with the device and is not graph-capturable."""
        mode = self._sidecar_mode
        if mode == "default":
            return True
        if mode == "always_on":
            self._sidecar_apply_count += 1
            return True
        if mode == "always_off":
            self._sidecar_skip_count += 1
            return False
        contrib = x_2d.index_select(1, self._sidecar_cols).float() * self._sidecar_deltas.unsqueeze(0)
        norm = float(contrib.norm().item())
        self._sidecar_norms.append(norm)
        if norm > self._sidecar_threshold:
            self._sidecar_apply_count += 1
            return True
        self._sidecar_skip_count += 1
        return False

    # ------------------------------------------------------------------ gates / graph mode
    def attach_kurtosis_gate(self, threshold: float, hysteresis_n: int = 2, ema_decay: float = 0.5) -> None:
        raise NotImplementedError("runtime SVD gating is outside the compressed-linear forward path")

    def detach_kurtosis_gate(self) -> None:
        self._kurtosis_gate = None
        self._cell_skip_svd = False

    def set_cuda_graph_mode(self, enabled: bool) -> None:
        """The kernels never synchronise, so forward() is capturable either way
        (unless the sidecar policy is "threshold"); the flag is kept for callers."""
        self._cuda_graph_mode = enabled

    def pre_step_kurtosis(self, x: torch.Tensor) -> Optional[bool]:
        return None

    # ------------------------------------------------------------------ reporting
    def dispatch_metadata(self) -> dict:
        return {
            "dispatch_path": self._last_dispatch_path,
            "device": str(self.codebook.device),
            "is_cuda": self.codebook.is_cuda,
            "triton_available": False,
            "compute_dtype": str(self.compute_dtype),
            "kernel_metadata": self._last_dispatch,
            "cell_skip_svd": self._cell_skip_svd,
            "svd_active": self.has_svd and not self._cell_skip_svd,
            "kurtosis_gate": None,
            "cuda_graph_mode": self._cuda_graph_mode,
            "wave_tiles": False,
        }

    def memory_savings(self) -> dict:
        """Bytes held vs an fp32 nn.Linear, counted as the reference counts them
        (helix_linear.py:890-918) plus the affine tables."""
        dense = self.out_features * self.in_features * 4
        comp = self.codebook.numel() * 4 + self.indices.numel() * self.indices.element_size()
        if self.codebook_f16 is not None:
            comp += self.codebook_f16.numel() * 2
        if self.sidecar_positions is not None:
            comp += self.sidecar_positions.numel() * 8 + self.sidecar_values.numel() * 4
        if self._sidecar_rows is not None:
            comp += self._sidecar_rows.numel() * 16 + self._sidecar_deltas.numel() * 4
        if self.has_svd:
            comp += (self.svd_U.numel() + self.svd_s.numel() + self.svd_Vt.numel()) * 4
        if self.has_channel_scales:
            comp += self.channel_scales.numel() * 4
        if self.group_scales is not None:
            comp += 2 * self.group_scales.numel() * self.group_scales.element_size()
        return {"dense_bytes": dense, "compressed_bytes": comp, "ratio": round(dense / max(1, comp), 2),
                "savings_pct": round(100 * (1 - comp / dense), 1)}

    def extra_repr(self) -> str:
        parts = [f"in_features={self.in_features}", f"out_features={self.out_features}"]
        if self.has_svd:
            parts.append(f"svd_rank={self.rank}")
        if self.sidecar_positions is not None:
            parts.append(f"n_outliers={self.sidecar_positions.numel()}")
        if self.group_scales is not None:
            parts.append(f"group_size={self.group_size}")
        if self.bias is not None:
            parts.append("bias=True")
        parts.append(f"compression={self.memory_savings()['ratio']}x")
        return ", ".join(parts)


# ---------------------------------------------------------------------------
# Loading from .cdnav3 directories and model surgery
# ---------------------------------------------------------------------------

def _npy(path: Path, dtype) -> torch.Tensor:
    return torch.from_numpy(np.load(path).astype(dtype, copy=True))


def load_helix_linear_from_cdnav3(tensor_dir: Path, bias: Optional[torch.Tensor] = None,
                                  compute_dtype: torch.dtype = torch.float32) -> HelixLinear:
    """One ``{name}.cdnav3/`` directory -> HelixLinear on the CPU, ready for
    ``.cuda()`` (file set: helix_linear.py:1141-1222; ``group_scales.npy`` /
    ``group_offsets.npy`` + ``meta["group_size"]`` are this package's extension)."""
    tensor_dir = Path(tensor_dir)
    meta = json.loads((tensor_dir / "meta.json").read_text())
    rows, cols = meta["shape"]
    if meta.get("vector_dim", 1) != 1 or meta.get("index_dtype", "uint8") != "uint8":
        raise NotImplementedError(f"{tensor_dir}: only scalar uint8 codebooks are on this path")
    kw = {}
    sc = tensor_dir / "sidecar.npz"
    if sc.exists():
        with np.load(sc) as z:
            kw["sidecar_positions"] = torch.from_numpy(z["positions"].astype(np.int64))
            kw["sidecar_values"] = torch.from_numpy(z["values"].astype(np.float32))
    if (tensor_dir / "svd_U.npy").exists():
        for n in ("svd_U", "svd_s", "svd_Vt"):
            kw[n] = _npy(tensor_dir / f"{n}.npy", np.float32)
    if (tensor_dir / "channel_scales.npy").exists():
        kw["channel_scales"] = _npy(tensor_dir / "channel_scales.npy", np.float32)
    if (tensor_dir / "group_scales.npy").exists():
        kw["group_scales"] = torch.from_numpy(np.load(tensor_dir / "group_scales.npy"))
        kw["group_offsets"] = torch.from_numpy(np.load(tensor_dir / "group_offsets.npy"))
        kw["group_size"] = int(meta.get("group_size", 128))
    idx = np.fromfile(tensor_dir / "indices.bin", dtype=np.uint8).reshape(rows, cols)
    return HelixLinear(cols, rows, _npy(tensor_dir / "codebook.npy", np.float32), torch.from_numpy(idx),
                       bias=bias, tensor_name=meta.get("tensor_name", ""), compute_dtype=compute_dtype, **kw)


def load_cdna_factors(cdna_dir: Path, model: Optional[nn.Module] = None,
                      compute_dtype: torch.dtype = torch.float32) -> Dict[str, HelixLinear]:
    """Every ``*.cdnav3`` directory under ``cdna_dir`` keyed by module path
    (helix_linear.py:1225-1290).  Biases come from ``*.npy.meta.json`` side
    files, overridden by the live model's nn.Linear biases when given."""
    cdna_dir = Path(cdna_dir)
    biases: Dict[str, torch.Tensor] = {}
    for mp in sorted(cdna_dir.glob("*.npy.meta.json")):
        name = json.loads(mp.read_text()).get("tensor_name", "")
        npy = mp.with_name(mp.name[: -len(".meta.json")])
        if name.endswith(".bias") and npy.exists():
            biases[name[:-5]] = torch.from_numpy(np.load(npy))
    if model is not None:
        for name, mod in model.named_modules():
            if isinstance(mod, nn.Linear) and mod.bias is not None:
                biases[name] = mod.bias.data.clone()
    out: Dict[str, HelixLinear] = {}
    for td in sorted(cdna_dir.glob("*.cdnav3")):
        if not td.is_dir() or not (td / "meta.json").exists():
            continue
        meta = json.loads((td / "meta.json").read_text())
        if meta.get("storage_mode") == "exact":
            continue
        path = _tensor_name_to_module_path(meta["tensor_name"])
        out[path] = load_helix_linear_from_cdnav3(td, bias=biases.get(path), compute_dtype=compute_dtype)
    return out


def swap_to_helix(model: nn.Module, helix_modules: Dict[str, HelixLinear],
                  compute_dtype: torch.dtype = torch.float32) -> nn.Module:
    """Replace each nn.Linear whose path is a key of ``helix_modules``
    (helix_linear.py:1293-1346); shapes must agree."""
    for name, mod in list(model.named_modules()):
        new = helix_modules.get(name)
        if new is None or not isinstance(mod, nn.Linear):
            continue
        if compute_dtype != torch.float32:
            new.set_compute_dtype(compute_dtype)
        assert new.in_features == mod.in_features, \
            f"{name}: in_features mismatch ({new.in_features} vs {mod.in_features})"
        assert new.out_features == mod.out_features, \
            f"{name}: out_features mismatch ({new.out_features} vs {mod.out_features})"
        parent = model
        *head, leaf = name.split(".")
        for part in head:
            parent = getattr(parent, part)
        setattr(parent, leaf, new)
    return model


def set_cuda_graph_mode(model: nn.Module, enabled: bool) -> int:
    n = 0
    for mod in model.modules():
        if isinstance(mod, HelixLinear):
            mod.set_cuda_graph_mode(enabled)
            n += 1
    return n


def pre_step_kurtosis_all(model: nn.Module, inputs: Optional[Dict[str, torch.Tensor]] = None) -> int:
    """No module carries a kurtosis gate in this build, so nothing is evaluated."""
    return 0


def freeze_sidecar_phase(model: nn.Module, phase: Optional[str]) -> int:
    """Kept for callers; the sidecar is always fused into the product kernel."""
    n = 0
    for mod in model.modules():
        if isinstance(mod, HelixLinear):
            mod._sidecar_phase = phase
            n += 1
    return n


def swap_summary(model: nn.Module) -> dict:
    """How much of the model is compressed (helix_linear.py:1418-1442)."""
    n_h = n_l = b_h = b_d = 0
    for mod in model.modules():
        if isinstance(mod, HelixLinear):
            ms = mod.memory_savings()
            n_h, b_h, b_d = n_h + 1, b_h + ms["compressed_bytes"], b_d + ms["dense_bytes"]
        elif isinstance(mod, nn.Linear):
            n_l, b_d = n_l + 1, b_d + mod.weight.numel() * 4
    return {"helix_modules": n_h, "linear_modules": n_l, "total_linear": n_h + n_l,
            "compressed_bytes": b_h, "dense_equivalent_bytes": b_d,
            "overall_ratio": round(b_d / max(1, b_h), 2)}


_GGUF_TO_HF = {
    "attn_q": "self_attn.q_proj", "attn_k": "self_attn.k_proj", "attn_v": "self_attn.v_proj",
    "attn_output": "self_attn.o_proj", "ffn_gate": "mlp.gate_proj", "ffn_up": "mlp.up_proj",
    "ffn_down": "mlp.down_proj",
}


def _tensor_name_to_module_path(tensor_name: str) -> str:
    """meta.json tensor name -> module path, HF and GGUF spellings
    (helix_linear.py:1464-1499)."""
    if tensor_name.startswith("blk."):
        parts = tensor_name.split(".")
        key = parts[2] if len(parts) <= 3 or parts[3] == "weight" else f"{parts[2]}_{parts[3]}"
        return f"model.layers.{int(parts[1])}.{_GGUF_TO_HF.get(key, key)}"
    if tensor_name in ("token_embd.weight", "model.embed_tokens.weight"):
        return "model.embed_tokens"
    if tensor_name in ("output.weight", "lm_head.weight"):
        return "lm_head"
    return tensor_name[:-7] if tensor_name.endswith(".weight") else tensor_name
