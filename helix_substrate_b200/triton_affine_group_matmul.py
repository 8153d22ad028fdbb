"""fused_affine_group_matmul: per-group affine product with the reference's
name and signature (helix_substrate/triton_affine_group_matmul.py:301-383),
served by the same sm_100a kernels as HelixLinear: the quantised byte is its own
codebook value (a 0..255 ramp) and scale/offset are the group affine."""

from __future__ import annotations

import torch

from .packed import HxqWeight

HAS_TRITON = False
_ramps: dict = {}


def _ramp(device: torch.device) -> torch.Tensor:
    r = _ramps.get(device)
    if r is None:
        r = torch.arange(256, dtype=torch.float32, device=device)
        _ramps[device] = r
    return r


def _weight(indices, scales, offsets, group_size, bias) -> HxqWeight:
    assert indices.is_cuda, "the affine-group product requires CUDA tensors"
    assert indices.ndim == 2 and indices.dtype == torch.uint8
    OUT, IN = indices.shape
    assert IN % group_size == 0, f"IN ({IN}) must be a multiple of group_size ({group_size})"
    n_groups = IN // group_size
    assert scales.shape == (OUT, n_groups) and offsets.shape == (OUT, n_groups)
    if scales.dtype not in (torch.float16, torch.float32):
        scales, offsets = scales.float(), offsets.float()
    offsets = offsets.to(scales.dtype)
    return HxqWeight(_ramp(indices.device), indices.contiguous(), bias=bias,
                     scales=scales.contiguous(), offsets=offsets.contiguous(), group_size=group_size)


def fused_affine_group_matmul(x: torch.Tensor, indices: torch.Tensor, scales: torch.Tensor,
                              offsets: torch.Tensor, group_size: int = 128,
                              bias: torch.Tensor | None = None) -> torch.Tensor:
    """Y[n, o] = sum_i X[n, i] * (indices[o, i] * scale[o, i//G] + offset[o, i//G]) (+ bias), fp32."""
    assert x.is_cuda and indices.is_cuda
    assert x.ndim == 2 and indices.ndim == 2 and indices.shape[1] == x.shape[1]
    return _weight(indices, scales, offsets, group_size, bias).matmul(x, out_dtype=torch.float32)


def fused_affine_group_matmul_packed6(*args, **kwargs):
    raise NotImplementedError("6-bit packed indices (k=64) are a different codec, outside this path")


def affine_group_matmul_reference(x: torch.Tensor, indices: torch.Tensor, scales: torch.Tensor,
                                  offsets: torch.Tensor, group_size: int = 128,
                                  bias: torch.Tensor | None = None) -> torch.Tensor:
    """Two-step check of the fused product on the GPU: materialise W with
    hxq_dequant (exact fp32 affine), then a dense fp32 matmul."""
    w = _weight(indices, scales, offsets, group_size, None).dequant()
    y = x.float() @ w.t()
    if bias is not None:
        y += bias.float().unsqueeze(0)
    return y
