"""HxqWeight: one compressed matrix resident in HBM plus the descriptor the
C ABI takes.  This is the only place the Python host touches the kernels."""

from __future__ import annotations

import ctypes as C
from typing import Optional

import numpy as np
import torch

from . import _lib
from ._lib import HxqDesc, HXQ_F32, HXQ_F16, HXQ_BF16

_DT = {torch.float32: HXQ_F32, torch.float16: HXQ_F16, torch.bfloat16: HXQ_BF16}

GEMV_MAX_M = 16      # most tokens hxq_gemv takes per call
GEMV_MAX_M_16BIT = 4  # bf16 / fp16 activations: beyond four tokens the tensor-memory kernel is faster


def uses_gemv(M: int, x_dtype: torch.dtype) -> bool:
    """Which product a call of M tokens runs by default: the fp32-accumulate streaming kernel
    (hxq_gemv: one launch per four tokens, every launch re-reading the weights) up to 16 tokens
    of fp32 activations or 4 tokens of 16-bit ones, the tensor-core kernels (bf16 operands) above."""
    return M <= (GEMV_MAX_M if x_dtype == torch.float32 else GEMV_MAX_M_16BIT)


def _dt(t: torch.dtype) -> int:
    try:
        return _DT[t]
    except KeyError:
        raise TypeError(f"Expected float32/float16/bfloat16, got {t}") from None


_workspaces: dict = {}
_status_words: dict = {}


def _workspace(device: torch.device, nbytes: int, kind: str = "gemv") -> Optional[torch.Tensor]:
    """Scratch, one per (device, stream, kernel family); grown on demand.
    hxq_gemv needs its workspace zeroed and leaves it zeroed, so it is cleared
    only when (re)allocated; hxq_gemm uses its own as plain scratch (a bf16 copy
    of the activations) and leaves it dirty - the two are never shared."""
    if nbytes == 0:
        return None
    key = (device.index, torch.cuda.current_stream(device).cuda_stream, kind)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError(
                "hxq kernels need their scratch buffer of this stream allocated (and zeroed) before a CUDA graph "
                "capture starts: run the step once on the capturing stream first, then capture")
        ws = torch.zeros(max(nbytes, 1 << 22), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def _status_word(device: torch.device) -> torch.Tensor:
    sw = _status_words.get(device.index)
    if sw is None:
        sw = torch.zeros(1, dtype=torch.int32, device=device)
        _status_words[device.index] = sw
    return sw


def csr_from_positions(positions: torch.Tensor, out_features: int, in_features: int):
    """Row pointer (int32[out+1]) and local columns (int32[nnz]) of ascending
    flat positions, through the library's host helper."""
    pos = positions.detach().to("cpu", torch.int64).contiguous().numpy()
    rowptr = np.empty(out_features + 1, dtype=np.int32)
    cols = np.empty(max(len(pos), 1), dtype=np.int32)
    st = _lib.lib().hxq_csr_from_positions(pos.ctypes.data, len(pos), out_features, in_features,
                                           rowptr.ctypes.data, cols.ctypes.data)
    if st != 0:
        raise ValueError("sidecar positions must be strictly ascending and inside the matrix")
    return torch.from_numpy(rowptr), torch.from_numpy(cols[:len(pos)].copy())


class HxqWeight:
    """Borrowed views of the module's CUDA buffers + a filled ``hxq_desc``.

    ``indices`` may be a column slice of a wider matrix (row-parallel shard):
    the row stride is taken from the tensor, ``col0`` carries the global column
    of the slice so that affine group ids stay global."""

    def __init__(self, codebook: torch.Tensor, indices: torch.Tensor, *,
                 rowptr: Optional[torch.Tensor] = None, cols: Optional[torch.Tensor] = None,
                 deltas: Optional[torch.Tensor] = None, values: Optional[torch.Tensor] = None,
                 bias: Optional[torch.Tensor] = None,
                 scales: Optional[torch.Tensor] = None, offsets: Optional[torch.Tensor] = None,
                 group_size: int = 0, col0: int = 0):
        if not indices.is_cuda:
            raise RuntimeError("HXQ kernels need CUDA tensors (there is no CPU path)")
        assert indices.dtype == torch.uint8 and indices.ndim == 2, "Expected uint8 [out, in] indices"
        assert indices.stride(1) == 1, "indices must be contiguous along the input dimension"
        assert codebook.dtype == torch.float32 and codebook.numel() == 256 and codebook.is_contiguous(), \
            "Expected a contiguous fp32 codebook of 256 entries"
        self.device = indices.device
        self.out_features, self.in_features = indices.shape
        self.codebook, self.indices = codebook, indices
        self.rowptr, self.cols, self.deltas, self.values = rowptr, cols, deltas, values
        self.bias = None if bias is None else bias.to(torch.float32).contiguous()
        self.scales, self.offsets = scales, offsets
        self.group_size, self.col0 = int(group_size), int(col0)
        if rowptr is not None:
            assert rowptr.dtype == torch.int32 and cols.dtype == torch.int32
            assert rowptr.numel() == self.out_features + 1
        if self.group_size > 0:
            assert scales is not None and offsets is not None
            assert scales.dtype == offsets.dtype and scales.dtype in (torch.float32, torch.float16)
            assert scales.shape == offsets.shape and scales.stride(1) == 1 and offsets.stride() == scales.stride()
        for t in (codebook, rowptr, cols, deltas, values, self.bias, scales, offsets):
            assert t is None or t.device == self.device, "all buffers of one weight live on one device"
        self.desc = self._fill()

    def _fill(self) -> HxqDesc:
        p = lambda t: None if t is None else C.c_void_p(t.data_ptr())
        d = HxqDesc()
        d.out_features, d.in_features = self.out_features, self.in_features
        d.col0, d.group_size = self.col0, self.group_size
        d.ld_idx = self.indices.stride(0)
        d.indices, d.codebook = p(self.indices), p(self.codebook)
        if self.group_size > 0:
            d.scales, d.offsets = p(self.scales), p(self.offsets)
            d.st_dtype = HXQ_F32 if self.scales.dtype == torch.float32 else HXQ_F16
            d.ld_st = self.scales.stride(0)
        d.rowptr, d.cols, d.deltas, d.values = p(self.rowptr), p(self.cols), p(self.deltas), p(self.values)
        d.bias = p(self.bias)
        return d

    # ---- y = x @ W^T (+ sidecar + bias) ------------------------------------
    def matmul(self, x: torch.Tensor, out_dtype: torch.dtype = torch.float32,
               out: Optional[torch.Tensor] = None, force: Optional[str] = None) -> torch.Tensor:
        assert x.is_cuda and x.device == self.device, "x must live on the weight's CUDA device"
        assert x.ndim == 2 and x.shape[1] == self.in_features
        xd = _dt(x.dtype)
        if x.stride(1) != 1:
            x = x.contiguous()
        M = x.shape[0]
        if out is None:
            out = torch.empty(M, self.out_features, device=self.device, dtype=out_dtype)
        if M == 0:
            return out
        L = _lib.lib()
        stream = C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        use_gemv = uses_gemv(M, x.dtype) if force is None else (force == "gemv")
        with torch.cuda.device(self.device):
            if use_gemv:
                y, m0 = out, 0
                while m0 < M:  # hxq_gemv takes at most 16 tokens per call
                    mm = min(GEMV_MAX_M, M - m0)
                    nb = L.hxq_gemv_workspace_bytes(C.byref(self.desc), mm)
                    ws = _workspace(self.device, nb)
                    st = L.hxq_gemv(C.byref(self.desc), C.c_void_p(x[m0:].data_ptr()), xd, mm, x.stride(0),
                                    C.c_void_p(y[m0:].data_ptr()), _dt(out.dtype), out.stride(0),
                                    None if ws is None else C.c_void_p(ws.data_ptr()),
                                    0 if ws is None else ws.numel(), stream)
                    _lib.check(st, "hxq_gemv")
                    m0 += mm
            else:
                nb = L.hxq_gemm_workspace_bytes(C.byref(self.desc), M)
                ws = _workspace(self.device, nb, "gemm")
                sw = _status_word(self.device)
                st = L.hxq_gemm(C.byref(self.desc), C.c_void_p(x.data_ptr()), xd, M, x.stride(0),
                                C.c_void_p(out.data_ptr()), _dt(out.dtype), out.stride(0),
                                None if ws is None else C.c_void_p(ws.data_ptr()),
                                0 if ws is None else ws.numel(), C.c_void_p(sw.data_ptr()), stream)
                _lib.check(st, "hxq_gemm")
        return out

    # ---- dense rows ----------------------------------------------------------
    def dequant(self, row0: int = 0, row1: Optional[int] = None,
                dtype: torch.dtype = torch.float32, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        row1 = self.out_features if row1 is None else row1
        if out is None:
            out = torch.empty(row1 - row0, self.in_features, device=self.device, dtype=dtype)
        assert out.stride(1) == 1
        stream = C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        with torch.cuda.device(self.device):
            st = _lib.lib().hxq_dequant(C.byref(self.desc), row0, row1, C.c_void_p(out.data_ptr()),
                                        _dt(out.dtype), out.stride(0), stream)
        _lib.check(st, "hxq_dequant")
        return out

    def gemm_status(self) -> int:
        """Non-zero if a bounded wait inside the tensor-core kernel gave up
        (synchronises the device)."""
        return int(_status_word(self.device).item())

    def algorithmic_bytes(self, M: int, x_bytes: int, y_bytes: int) -> int:
        """Bytes one product has to move whatever the implementation: indices,
        codebook, scale/offset at fp32, sidecar (int32 col + fp32 delta), row
        pointer, activations in and out."""
        nnz = 0 if self.cols is None else self.cols.numel()
        ng = 0
        if self.group_size > 0:
            ng = (self.col0 + self.in_features - 1) // self.group_size - self.col0 // self.group_size + 1
        return (self.out_features * self.in_features + 1024 + self.out_features * ng * 8 + nnz * 8
                + (self.out_features + 1) * 4 + M * self.in_features * x_bytes
                + M * self.out_features * y_bytes)
