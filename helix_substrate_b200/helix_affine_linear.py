"""HelixAffineLinear: int8 block-affine linear with the reference's interface
(helix_substrate/helix_affine_linear.py:30-277) on the HXQ kernels:
W = ((u8 - 128) / 127) * scale[blk] + bias_ab[blk] is the superset weight with
codebook[k] = (k - 128) / 127 and a group affine of ``block_size``."""

from __future__ import annotations

from typing import Optional, Set

import torch
import torch.nn as nn

from .packed import HxqWeight


def _int8_codebook(device=None) -> torch.Tensor:
    # IEEE fp32 division on the host, the rounding of the reference's CPU
    # ``int8_vals.float() / 127.0`` (a device-side division by a scalar is a
    # multiplication by the reciprocal and differs in the last bit)
    import numpy as np
    cb = (np.arange(256, dtype=np.float32) - np.float32(128.0)) / np.float32(127.0)
    return torch.from_numpy(cb).to(device) if device is not None else torch.from_numpy(cb)


class HelixAffineLinear(nn.Module):
    def __init__(self, in_features: int, out_features: int, indices: torch.Tensor, scales: torch.Tensor,
                 biases_ab: torch.Tensor, block_size: int = 256, bias: Optional[torch.Tensor] = None,
                 tensor_name: str = ""):
        super().__init__()
        assert indices.dtype == torch.uint8
        assert in_features % block_size == 0
        self.in_features, self.out_features = in_features, out_features
        self.block_size, self.blocks_per_row = block_size, in_features // block_size
        self.tensor_name = tensor_name
        self.register_buffer("indices", indices.contiguous())
        self.register_buffer("scales", scales.contiguous())
        self.register_buffer("biases_ab", biases_ab.contiguous())
        self.register_buffer("bias", None if bias is None else bias.contiguous())
        self.register_buffer("_codebook", _int8_codebook(), persistent=False)
        self._packed = None

    def _apply(self, fn, recurse=True):
        out = super()._apply(fn, recurse)
        self._buffers["_codebook"] = _int8_codebook(self.indices.device)
        self._packed = None
        return out

    def packed(self) -> HxqWeight:
        if not self.indices.is_cuda:
            raise RuntimeError("HelixAffineLinear runs on CUDA only; there is no CPU path. No silent fallback.")
        if self._packed is None:
            sc = self.scales.reshape(self.out_features, self.blocks_per_row)
            of = self.biases_ab.reshape(self.out_features, self.blocks_per_row)
            if sc.dtype not in (torch.float16, torch.float32):
                sc, of = sc.float(), of.float()
            self._packed = HxqWeight(self._codebook, self.indices, bias=self.bias, scales=sc.contiguous(),
                                     offsets=of.to(sc.dtype).contiguous(), group_size=self.block_size)
        return self._packed

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """fp32 result like the reference (helix_affine_linear.py:68-101)."""
        if not x.is_cuda:
            raise RuntimeError("HelixAffineLinear.forward got a CPU tensor; CUDA only. No silent fallback.")
        x2 = x.reshape(-1, self.in_features)
        if x2.dtype not in (torch.float32, torch.float16, torch.bfloat16):
            x2 = x2.float()
        y = self.packed().matmul(x2, out_dtype=torch.float32)
        return y.reshape(*x.shape[:-1], self.out_features)

    def decode_weight(self) -> torch.Tensor:
        with torch.no_grad():
            return self.packed().dequant()

    def memory_savings(self) -> dict:
        dense = self.out_features * self.in_features * 4
        comp = self.indices.numel() + self.scales.numel() * 2 + self.biases_ab.numel() * 2
        return {"dense_bytes": dense, "compressed_bytes": comp, "ratio": round(dense / max(1, comp), 2),
                "savings_pct": round(100 * (1 - comp / dense), 1)}

    def extra_repr(self) -> str:
        parts = [f"in_features={self.in_features}", f"out_features={self.out_features}",
                 f"block_size={self.block_size}", f"compression={self.memory_savings()['ratio']}x"]
        if self.bias is not None:
            parts.append("bias=True")
        return ", ".join(parts)


@torch.no_grad()
def quantize_linear_to_affine(weight: torch.Tensor, block_size: int = 256) -> tuple:
    """Per-block mean / max-abs-residual int8 encoder
    (helix_affine_linear.py:146-200); runs on whatever device ``weight`` is on."""
    rows, cols = weight.shape
    assert cols % block_size == 0, f"cols {cols} not divisible by block_size {block_size}"
    bpr = cols // block_size
    w = weight.float().reshape(rows, bpr, block_size)
    mean = w.mean(dim=2)
    resid = w - mean.unsqueeze(2)
    scale = resid.abs().amax(dim=2).clamp(min=1e-6)
    q = (resid * 127.0 / scale.unsqueeze(2)).round().clamp(-128, 127)
    indices = (q.to(torch.int16) + 128).to(torch.uint8).reshape(rows, cols)
    recon = ((q / 127.0) * scale.unsqueeze(2) + mean.unsqueeze(2)).reshape(rows, cols)
    err = (recon - weight.float()).abs()
    stats = {
        "n_blocks": rows * bpr, "block_size": block_size,
        "max_abs_error": err.max().item(), "mean_abs_error": err.mean().item(),
        "cosine": float(torch.nn.functional.cosine_similarity(
            weight.float().reshape(1, -1), recon.reshape(1, -1)).item()),
    }
    return indices, scale.half().reshape(-1), mean.half().reshape(-1), stats


@torch.no_grad()
def swap_to_affine(model: nn.Module, block_size: int = 256, skip_modules: Optional[Set[str]] = None) -> tuple:
    """Replace eligible nn.Linear modules by HelixAffineLinear; returns
    ``(model, n_replaced, total_stats)`` (helix_affine_linear.py:203-277)."""
    skip_modules = {"lm_head"} if skip_modules is None else skip_modules
    n = 0
    tot = {"max_abs_error": 0.0, "sum_cosine": 0.0, "n_tensors": 0, "compressed_bytes": 0, "dense_bytes": 0}
    for name, mod in list(model.named_modules()):
        if not isinstance(mod, nn.Linear) or name in skip_modules or mod.in_features % block_size != 0:
            continue
        idx, sc, bab, stats = quantize_linear_to_affine(mod.weight.data, block_size)
        new = HelixAffineLinear(mod.in_features, mod.out_features, idx, sc, bab, block_size,
                                bias=None if mod.bias is None else mod.bias.data.clone(), tensor_name=name)
        parent = model
        *head, leaf = name.split(".")
        for part in head:
            parent = getattr(parent, part)
        setattr(parent, leaf, new)
        n += 1
        ms = new.memory_savings()
        tot["max_abs_error"] = max(tot["max_abs_error"], stats["max_abs_error"])
        tot["sum_cosine"] += stats["cosine"]
        tot["n_tensors"] += 1
        tot["compressed_bytes"] += ms["compressed_bytes"]
        tot["dense_bytes"] += ms["dense_bytes"]
    if tot["n_tensors"]:
        tot["avg_cosine"] = tot["sum_cosine"] / tot["n_tensors"]
        tot["overall_ratio"] = round(tot["dense_bytes"] / max(1, tot["compressed_bytes"]), 2)
    return model, n, tot
