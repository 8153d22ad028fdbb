"""fused_vq_matmul: the operator behind HelixLinear, same name and signature as
the reference's Triton operator (helix_substrate/triton_vq_matmul.py:521-727)
so existing imports keep working - but the body is the sm_100a C-ABI library
(hxq_gemv for a few tokens, hxq_gemm above: packed.uses_gemv).  No Triton is involved."""

from __future__ import annotations

from typing import Optional

import torch

from . import _lib
from .packed import HxqWeight, uses_gemv

KERNEL_VERSION = "hxq_b200_v1"
KERNEL_IMPL = "libhxq_b200"
HAS_TRITON = False  # kept for callers that test it; nothing here uses Triton

_csr_cache: dict = {}


def get_kernel_metadata() -> dict:
    """Version / dispatch metadata for receipts (triton_vq_matmul.py:77-97)."""
    meta = {
        "kernel_impl": KERNEL_IMPL, "kernel_version": KERNEL_VERSION, "dispatch_selected": KERNEL_VERSION,
        "triton_version": None, "torch_version": torch.__version__, "cuda_version": None,
        "compute_capability": None, "library_version": None,
    }
    try:
        meta["library_version"] = _lib.lib().hxq_version()
    except RuntimeError:
        pass
    if torch.cuda.is_available():
        meta["cuda_version"] = torch.version.cuda
        p = torch.cuda.get_device_properties(0)
        meta["compute_capability"] = f"{p.major}.{p.minor}"
    return meta


def is_available() -> bool:
    """True when the CUDA library is built and a GPU is present."""
    try:
        _lib.lib()
    except (RuntimeError, OSError):
        return False
    return torch.cuda.is_available()


def _csr(rows: torch.Tensor, cols: torch.Tensor, deltas: torch.Tensor, n_out: int):
    """Row-sorted CSR (int32) of a COO sidecar, built on the device and cached
    per tensor triple so the decode loop pays for it once."""
    key = (rows.data_ptr(), cols.data_ptr(), deltas.data_ptr(), rows.numel(), rows._version, n_out)
    hit = _csr_cache.get(key)
    if hit is not None:
        return hit
    rows = rows.long()
    if rows.numel() > 1 and bool((rows[1:] < rows[:-1]).any()):
        order = torch.sort(rows, stable=True).indices
        rows, cols, deltas = rows[order], cols[order], deltas[order]
    rowptr = torch.searchsorted(rows, torch.arange(n_out + 1, device=rows.device)).to(torch.int32)
    out = (rowptr.contiguous(), cols.to(torch.int32).contiguous(), deltas.float().contiguous())
    if len(_csr_cache) > 4096:
        _csr_cache.clear()
    _csr_cache[key] = out
    return out


def fused_vq_matmul(
    x: torch.Tensor,
    codebook: torch.Tensor,
    indices: torch.Tensor,
    sidecar_positions: Optional[torch.Tensor] = None,
    sidecar_values: Optional[torch.Tensor] = None,
    codebook_values_at_sidecar: Optional[torch.Tensor] = None,
    sidecar_rows: Optional[torch.Tensor] = None,
    sidecar_cols: Optional[torch.Tensor] = None,
    sidecar_deltas: Optional[torch.Tensor] = None,
    svd_U: Optional[torch.Tensor] = None,
    svd_s: Optional[torch.Tensor] = None,
    svd_Vt: Optional[torch.Tensor] = None,
    bias: Optional[torch.Tensor] = None,
    codebook_f16: Optional[torch.Tensor] = None,
    _dispatch_log: Optional[dict] = None,
    sidecar_phase: Optional[str] = None,
    vq_dim: int = 1,
) -> torch.Tensor:
    """x[N, IN] @ (codebook[indices] + sidecar + SVD)^T + bias -> fp32 [N, OUT].

    Sidecar either as precomputed rows/cols/deltas (preferred) or as flat
    positions + values (deltas are then derived against the codebook value).
    ``codebook_f16`` and ``sidecar_phase`` are accepted and ignored: there is
    one kernel path and the sidecar is always fused into it."""
    assert x.is_cuda, "fused_vq_matmul requires CUDA tensors"
    assert x.dtype in (torch.float32, torch.float16, torch.bfloat16), \
        f"Expected float32/float16/bfloat16, got {x.dtype}"
    assert indices.dtype in (torch.uint8, torch.int16), f"Expected uint8 or int16 indices, got {indices.dtype}"
    assert vq_dim in (1, 2, 4), f"vq_dim must be 1, 2, or 4, got {vq_dim}"
    if vq_dim != 1 or indices.dtype != torch.uint8:
        raise NotImplementedError("vector codebooks / int16 indices are outside the k=256 scalar path")
    N, IN = x.shape
    OUT = indices.shape[0]
    assert indices.shape[1] == IN, f"indices shape {tuple(indices.shape)} inconsistent with IN={IN}"

    kw = {}
    if sidecar_rows is not None:
        rp, cc, dl = _csr(sidecar_rows, sidecar_cols, sidecar_deltas, OUT)
        kw = dict(rowptr=rp, cols=cc, deltas=dl)
    elif sidecar_positions is not None and sidecar_values is not None:
        rows, cols = sidecar_positions // IN, sidecar_positions % IN
        vq = codebook_values_at_sidecar
        if vq is None:
            vq = codebook.reshape(-1)[indices.reshape(-1)[sidecar_positions].long()]
        rp, cc, dl = _csr(rows, cols, (sidecar_values - vq).float(), OUT)
        kw = dict(rowptr=rp, cols=cc, deltas=dl)
    cb = codebook.reshape(-1).float()
    if cb.numel() < 256:
        cb = torch.cat([cb, cb[-1:].expand(256 - cb.numel())])
    idx = indices if indices.stride(1) == 1 else indices.contiguous()
    w = HxqWeight(cb.contiguous(), idx, bias=bias, **kw)
    try:
        with _lib.weights_on_stream():   # the CSR / deltas / padded codebook above were made on this stream
            out = w.matmul(x, out_dtype=torch.float32)
    except _lib.HxqError as e:
        raise RuntimeError(f"hxq kernel launch failed: {e}. N={N}, IN={IN}, OUT={OUT}. No silent fallback.") from e
    if _dispatch_log is not None:
        gemv = uses_gemv(N, x.dtype)
        _dispatch_log["dispatch_selected"] = "hxq_gemv_sm100a" if gemv else "hxq_gemm_sm100a"
        _dispatch_log["block_config"] = "unit8x512" if gemv else "umma128"
        _dispatch_log["vq_dim"] = vq_dim
    if svd_U is not None:
        xf = x.float()
        out += ((xf @ svd_Vt.t()) * svd_s.unsqueeze(0)) @ svd_U.t()
    return out
