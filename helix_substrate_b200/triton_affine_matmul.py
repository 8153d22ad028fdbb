"""fused_affine_matmul: per-tensor affine product with the reference's name and
signature (helix_substrate/triton_affine_matmul.py:110-167):

    W[o, i] = indices[o, i] * step + offset,     Y = X @ W^T (+ bias), fp32.

Served by the same sm_100a kernels as HelixLinear: the 256 values k * step +
offset ARE a codebook, so the call is a plain codebook product with no group
affine and no sidecar (the reference splits it into step * (X @ idx^T) +
offset * rowsum(X); both are the same sum up to fp32 rounding)."""

from __future__ import annotations

import torch

from .packed import HxqWeight

HAS_TRITON = False


def _codebook(step: float, offset: float, device: torch.device) -> torch.Tensor:
    k = torch.arange(256, dtype=torch.float64, device=device)
    return (k * float(step) + float(offset)).to(torch.float32).contiguous()


def fused_affine_matmul(x: torch.Tensor, indices: torch.Tensor, step: float, offset: float,
                        bias: torch.Tensor | None = None) -> torch.Tensor:
    """Y = step * (X @ indices^T) + offset * rowsum(X) [+ bias]; x [N, IN] float, indices [OUT, IN] uint8."""
    assert x.is_cuda and indices.is_cuda, "fused_affine_matmul requires CUDA tensors"
    assert x.ndim == 2 and indices.ndim == 2
    assert x.shape[1] == indices.shape[1], f"IN mismatch: {x.shape[1]} vs {indices.shape[1]}"
    assert indices.dtype == torch.uint8, "Expected uint8 indices"
    w = HxqWeight(_codebook(step, offset, indices.device), indices.contiguous(), bias=bias)
    from . import _lib
    with _lib.weights_on_stream():   # the ramp codebook is computed per call on this stream
        return w.matmul(x, out_dtype=torch.float32)


def affine_matmul_reference(x: torch.Tensor, indices: torch.Tensor, step: float, offset: float,
                            bias: torch.Tensor | None = None) -> torch.Tensor:
    """The same product in plain torch ops (any device), as the reference states it
    (helix_substrate/triton_affine_matmul.py:170-187)."""
    rowsum = x.sum(dim=-1, keepdim=True)
    y = step * (x @ indices.to(x.dtype).t()) + offset * rowsum
    if bias is not None:
        y = y + bias.unsqueeze(0)
    return y
