"""The decode-step operators between the compressed linears (residual add +
RMSNorm, rotary embedding + KV-cache append, single-query attention, SwiGLU):
thin bf16 wrappers over the C ABI, one launch each (two for attention)."""

from __future__ import annotations

import ctypes as C

import torch

from . import _lib


def _p(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream(dev):
    return C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)


def _bf16_rows(t: torch.Tensor, name: str) -> None:
    if not (t.is_cuda and t.dtype == torch.bfloat16 and t.ndim == 2 and t.stride(1) == 1):
        raise TypeError(f"{name}: expected a CUDA bf16 [rows, n] tensor contiguous along n")


def add_rmsnorm(h: torch.Tensor, delta, weight: torch.Tensor, eps: float, out: torch.Tensor) -> torch.Tensor:
    """``h += delta`` in place (if delta is given), ``out = rmsnorm(h) * weight``."""
    _bf16_rows(h, "h"); _bf16_rows(out, "out")
    if delta is not None:
        _bf16_rows(delta, "delta")
    with torch.cuda.device(h.device):
        st = _lib.lib().hxq_add_rmsnorm(_p(h), _p(delta), _p(weight), _p(out), h.shape[0], h.shape[1], h.stride(0),
                                        0 if delta is None else delta.stride(0), out.stride(0), eps, _stream(h.device))
    _lib.check(st, "hxq_add_rmsnorm")
    return out


def rope_append(qkv: torch.Tensor, pos: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, q_out: torch.Tensor,
                k_cache: torch.Tensor, v_cache: torch.Tensor, nq: int, nkv: int) -> torch.Tensor:
    """qkv [B, (nq + 2 nkv) D] of the new token -> rotated q in q_out [B, nq D]; rotated k and v
    appended at row ``pos`` (int64 device scalar) of the caches [B, nkv, max_len, D]."""
    _bf16_rows(qkv, "qkv"); _bf16_rows(q_out, "q_out")
    B, n_kv, max_len, D = k_cache.shape
    assert n_kv == nkv and v_cache.shape == k_cache.shape and k_cache.is_contiguous() and v_cache.is_contiguous()
    assert k_cache.dtype == torch.bfloat16 and v_cache.dtype == torch.bfloat16
    assert pos.dtype == torch.int64 and pos.is_cuda
    assert cos.dtype == torch.float32 and cos.shape == (max_len, D) and cos.is_contiguous() and sin.shape == cos.shape
    with torch.cuda.device(qkv.device):
        st = _lib.lib().hxq_rope_append(_p(qkv), qkv.stride(0), _p(pos), _p(cos), _p(sin), _p(q_out), q_out.stride(0),
                                        _p(k_cache), _p(v_cache), B, nq, nkv, D, max_len, _stream(qkv.device))
    _lib.check(st, "hxq_rope_append")
    return q_out


_attn_ws: dict = {}


def attn_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, pos: torch.Tensor,
                out: torch.Tensor, nq: int, scale: float) -> torch.Tensor:
    """Attention of one query token per sequence over cache rows 0..pos."""
    _bf16_rows(q, "q"); _bf16_rows(out, "out")
    B, nkv, max_len, D = k_cache.shape
    L = _lib.lib()
    nb = L.hxq_attn_decode_workspace_bytes(B, nq, D, max_len)
    key = (q.device.index, torch.cuda.current_stream(q.device).cuda_stream)
    ws = _attn_ws.get(key)
    if ws is None or ws.numel() < nb:
        ws = torch.empty(nb, dtype=torch.uint8, device=q.device)
        _attn_ws[key] = ws
    with torch.cuda.device(q.device):
        st = L.hxq_attn_decode(_p(q), q.stride(0), _p(k_cache), _p(v_cache), _p(pos), _p(out), out.stride(0),
                               _p(ws), ws.numel(), B, nq, nkv, D, max_len, scale, _stream(q.device))
    _lib.check(st, "hxq_attn_decode")
    return out


def swiglu(gate: torch.Tensor, up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    _bf16_rows(gate, "gate"); _bf16_rows(up, "up"); _bf16_rows(out, "out")
    with torch.cuda.device(gate.device):
        st = _lib.lib().hxq_swiglu(_p(gate), _p(up), _p(out), gate.shape[0], gate.shape[1], gate.stride(0),
                                   up.stride(0), out.stride(0), _stream(gate.device))
    _lib.check(st, "hxq_swiglu")
    return out


DENSE_GEMV_MAX_M = 4      # what the kernel takes
DENSE_GEMV_USE_M = 2      # where it beats a library GEMM (measured: 158 vs 179 us at one token, 230 vs 180 us at four, [152064, 3584])


def dense_gemv(weight: torch.Tensor, x: torch.Tensor, out: torch.Tensor | None = None,
               out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """y = x @ weight.t() for a dense bf16 weight [OUT, IN] and up to four bf16 tokens (lm_head at
    decode time; the reference runs it as _BF16Linear, helix_substrate/basin_runtime.py:181-205)."""
    _bf16_rows(weight, "weight"); _bf16_rows(x, "x")
    M, n_in = x.shape
    n_out = weight.shape[0]
    assert weight.shape[1] == n_in and 0 < M <= DENSE_GEMV_MAX_M
    if out is None:
        out = torch.empty(M, n_out, device=x.device, dtype=out_dtype)
    dt = {torch.float32: _lib.HXQ_F32, torch.float16: _lib.HXQ_F16, torch.bfloat16: _lib.HXQ_BF16}[out.dtype]
    assert out.shape == (M, n_out) and out.stride(1) == 1
    with torch.cuda.device(x.device):
        st = _lib.lib().hxq_dense_gemv(_p(weight), n_out, n_in, weight.stride(0), _p(x), M, x.stride(0), _p(out), dt,
                                       out.stride(0), _stream(x.device))
    _lib.check(st, "hxq_dense_gemv")
    return out
