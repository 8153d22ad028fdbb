"""ctypes binding of libhxq_b200.so.  There is no fallback: if the library is
missing or a call fails, the caller gets an exception."""

from __future__ import annotations

import ctypes as C
from pathlib import Path

import os

# HXQ_B200_LIB points at another build of the same library (e.g. one compiled with different tuning macros)
_LIB_PATH = Path(os.environ.get("HXQ_B200_LIB") or Path(__file__).resolve().parent / "libhxq_b200.so")

HXQ_F32, HXQ_F16, HXQ_BF16 = 0, 1, 2

HXQ_OK = 0
HXQ_E_ARG, HXQ_E_SHAPE, HXQ_E_ALIGN, HXQ_E_DTYPE = -1, -2, -3, -4
HXQ_E_DEVICE, HXQ_E_LAUNCH, HXQ_E_TIMEOUT, HXQ_E_WORKSPACE = -5, -6, -7, -8


class HxqDesc(C.Structure):
    """Mirror of struct hxq_desc (include/hxq_b200.h)."""
    _fields_ = [
        ("out_features", C.c_int32),
        ("in_features", C.c_int32),
        ("col0", C.c_int32),
        ("group_size", C.c_int32),
        ("ld_idx", C.c_int64),
        ("indices", C.c_void_p),
        ("codebook", C.c_void_p),
        ("scales", C.c_void_p),
        ("offsets", C.c_void_p),
        ("st_dtype", C.c_int32),
        ("ld_st", C.c_int32),
        ("rowptr", C.c_void_p),
        ("cols", C.c_void_p),
        ("deltas", C.c_void_p),
        ("values", C.c_void_p),
        ("bias", C.c_void_p),
    ]


class HxqError(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        super().__init__(f"{where}: {strerror(status)} (status {status}). No silent fallback.")


_lib = None


def lib() -> C.CDLL:
    """Load the CUDA library once; raise if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not _LIB_PATH.exists():
        raise RuntimeError(
            f"{_LIB_PATH} is missing: build it with `python -m helix_substrate_b200.build` "
            "(the HXQ path has no CPU or library fallback)")
    L = C.CDLL(str(_LIB_PATH))
    P = C.POINTER(HxqDesc)
    L.hxq_version.restype = C.c_int
    L.hxq_strerror.restype = C.c_char_p
    L.hxq_strerror.argtypes = [C.c_int]
    L.hxq_set_weights_on_stream.restype = None
    L.hxq_set_weights_on_stream.argtypes = [C.c_int]
    L.hxq_dequant.restype = C.c_int
    L.hxq_dequant.argtypes = [P, C.c_int32, C.c_int32, C.c_void_p, C.c_int, C.c_int64, C.c_void_p]
    L.hxq_gemv_workspace_bytes.restype = C.c_size_t
    L.hxq_gemv_workspace_bytes.argtypes = [P, C.c_int32]
    L.hxq_gemv.restype = C.c_int
    L.hxq_gemv.argtypes = [P, C.c_void_p, C.c_int, C.c_int32, C.c_int64, C.c_void_p, C.c_int, C.c_int64,
                           C.c_void_p, C.c_size_t, C.c_void_p]
    L.hxq_gemv_packed6.restype = C.c_int
    L.hxq_gemv_packed6.argtypes = [C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_int, C.c_int32,
                                   C.c_int32, C.c_void_p, C.c_void_p, C.c_int, C.c_int32, C.c_int64, C.c_void_p,
                                   C.c_int, C.c_int64, C.c_void_p]
    L.hxq_gemm_workspace_bytes.restype = C.c_size_t
    L.hxq_gemm_workspace_bytes.argtypes = [P, C.c_int32]
    L.hxq_gemm.restype = C.c_int
    L.hxq_gemm.argtypes = [P, C.c_void_p, C.c_int, C.c_int32, C.c_int64, C.c_void_p, C.c_int, C.c_int64,
                           C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p]
    L.hxq_csr_from_positions.restype = C.c_int
    L.hxq_csr_from_positions.argtypes = [C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]
    L.hxq_add_rmsnorm.restype = C.c_int
    L.hxq_add_rmsnorm.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32,
                                  C.c_int64, C.c_int64, C.c_int64, C.c_float, C.c_void_p]
    L.hxq_rope_append.restype = C.c_int
    L.hxq_rope_append.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64,
                                  C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                  C.c_void_p]
    L.hxq_attn_decode_workspace_bytes.restype = C.c_size_t
    L.hxq_attn_decode_workspace_bytes.argtypes = [C.c_int32, C.c_int32, C.c_int32, C.c_int32]
    L.hxq_attn_decode.restype = C.c_int
    L.hxq_attn_decode.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64,
                                  C.c_void_p, C.c_size_t, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                  C.c_float, C.c_void_p]
    L.hxq_dense_gemv.restype = C.c_int
    L.hxq_dense_gemv.argtypes = [C.c_void_p, C.c_int32, C.c_int32, C.c_int64, C.c_void_p, C.c_int32, C.c_int64, C.c_void_p,
                                 C.c_int, C.c_int64, C.c_void_p]
    L.hxq_swiglu.restype = C.c_int
    L.hxq_swiglu.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int64, C.c_int64,
                             C.c_int64, C.c_void_p]
    L.hxq_allreduce_buffer_bytes.restype = C.c_size_t
    L.hxq_allreduce_buffer_bytes.argtypes = [C.c_int32, C.c_int64]
    L.hxq_allreduce_flag_bytes.restype = C.c_size_t
    L.hxq_allreduce_flag_bytes.argtypes = [C.c_int32]
    L.hxq_allreduce_oneshot.restype = C.c_int
    L.hxq_allreduce_oneshot.argtypes = [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int64, C.c_void_p, C.c_void_p,
                                        C.c_int64, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p]
    L.hxq_allreduce_add_rmsnorm.restype = C.c_int
    L.hxq_allreduce_add_rmsnorm.argtypes = [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int64, C.c_void_p, C.c_int32,
                                            C.c_int32, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_int64, C.c_float,
                                            C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p]
    _lib = L
    return L


class weights_on_stream:
    """``with weights_on_stream():`` around a product whose descriptor buffers (codebook, indices,
    scales, sidecar) were produced by kernels still in flight on the current stream: the decode
    kernels then start only after those kernels have finished (see include/hxq_b200.h)."""

    def __enter__(self):
        lib().hxq_set_weights_on_stream(1)
        return self

    def __exit__(self, *exc):
        lib().hxq_set_weights_on_stream(0)
        return False


def strerror(status: int) -> str:
    try:
        return lib().hxq_strerror(int(status)).decode()
    except Exception:  # library missing: still give a readable message
        return f"status {status}"


def check(status: int, where: str) -> None:
    if status != HXQ_OK:
        raise HxqError(status, where)
