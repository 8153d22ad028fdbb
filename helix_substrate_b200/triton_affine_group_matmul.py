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
    from . import _lib
    with _lib.weights_on_stream():   # dtype conversions / index expansion may still be in flight on this stream
        return _weight(indices, scales, offsets, group_size, bias).matmul(x, out_dtype=torch.float32)


def unpack6(packed: torch.Tensor, out_features: int, in_features: int) -> torch.Tensor:
    """6-bit indices, four values in three bytes (b0 | b1 << 8 | b2 << 16 holds v0..v3 from the low
    bits up, helix_substrate/triton_affine_group_matmul.py:234-238), to one byte per value
    [out_features, in_features].  Plain torch ops, any device."""
    assert packed.dtype == torch.uint8 and in_features % 4 == 0
    assert packed.numel() == out_features * in_features * 3 // 4, "packed size does not match OUT x IN x 3/4"
    b = packed.reshape(out_features, in_features // 4, 3).to(torch.int32)
    w = b[..., 0] | (b[..., 1] << 8) | (b[..., 2] << 16)
    v = torch.stack([(w >> (6 * k)) & 0x3F for k in range(4)], dim=-1)
    return v.reshape(out_features, in_features).to(torch.uint8)


def pack6(indices: torch.Tensor) -> torch.Tensor:
    """Inverse of unpack6 for values < 64 (flat uint8 of OUT * IN * 3 / 4 bytes)."""
    assert indices.dtype == torch.uint8 and indices.ndim == 2 and indices.shape[1] % 4 == 0
    assert int(indices.max()) < 64 if indices.numel() else True
    v = indices.reshape(indices.shape[0], -1, 4).to(torch.int32)
    w = v[..., 0] | (v[..., 1] << 6) | (v[..., 2] << 12) | (v[..., 3] << 18)
    return torch.stack([w & 0xFF, (w >> 8) & 0xFF, (w >> 16) & 0xFF], dim=-1).to(torch.uint8).reshape(-1)


def fused_affine_group_matmul_packed6(x: torch.Tensor, packed_indices: torch.Tensor, scales: torch.Tensor,
                                      offsets: torch.Tensor, out_features: int, in_features: int,
                                      group_size: int = 128, bias: torch.Tensor | None = None) -> torch.Tensor:
    """The reference's 6-bit variant (helix_substrate/triton_affine_group_matmul.py:256-298), any N.
    Up to 16 tokens the packed bytes are unpacked INSIDE the kernel (``hxq_gemv_packed6``: the
    weight stream is 0.75 byte per weight).  More tokens, or shapes that kernel does not take
    (IN or group size not a multiple of 16), expand to one byte per index first (torch ops) and
    run on the ordinary kernels - keep ``unpack6``'s result if you do that repeatedly."""
    import ctypes as C
    from . import _lib
    assert x.is_cuda and packed_indices.is_cuda
    assert x.ndim == 2 and x.shape[1] == in_features
    assert packed_indices.dtype == torch.uint8
    assert packed_indices.numel() == out_features * in_features * 3 // 4, "packed size does not match OUT x IN x 3/4"
    M = x.shape[0]
    dt = {torch.float32: _lib.HXQ_F32, torch.float16: _lib.HXQ_F16, torch.bfloat16: _lib.HXQ_BF16}
    if 0 < M <= 16 and in_features % 16 == 0 and group_size % 16 == 0 and x.dtype in dt:
        assert in_features % group_size == 0, f"IN ({in_features}) must be a multiple of group_size ({group_size})"
        if scales.dtype not in (torch.float16, torch.float32):
            scales, offsets = scales.float(), offsets.float()
        scales, offsets = scales.contiguous(), offsets.to(scales.dtype).contiguous()
        assert scales.shape == (out_features, in_features // group_size) and offsets.shape == scales.shape
        packed = packed_indices.contiguous()
        xc = x if x.stride(1) == 1 else x.contiguous()
        b = None if bias is None else bias.float().contiguous()
        y = torch.empty(M, out_features, device=x.device, dtype=torch.float32)
        with torch.cuda.device(x.device):
            st = _lib.lib().hxq_gemv_packed6(
                C.c_void_p(packed.data_ptr()), out_features, in_features, C.c_void_p(scales.data_ptr()),
                C.c_void_p(offsets.data_ptr()), _lib.HXQ_F32 if scales.dtype == torch.float32 else _lib.HXQ_F16,
                scales.stride(0), group_size, None if b is None else C.c_void_p(b.data_ptr()),
                C.c_void_p(xc.data_ptr()), dt[x.dtype], M, xc.stride(0), C.c_void_p(y.data_ptr()), _lib.HXQ_F32,
                y.stride(0), C.c_void_p(torch.cuda.current_stream(x.device).cuda_stream))
        _lib.check(st, "hxq_gemv_packed6")
        return y
    idx = unpack6(packed_indices, out_features, in_features)
    return fused_affine_group_matmul(x, idx, scales, offsets, group_size=group_size, bias=bias)


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
