"""The C-ABI library loads on a machine without a GPU and exports every entry
point include/hxq_b200.h declares; argument validation works without a device."""

import ctypes as C
import re
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


def _declared():
    text = (ROOT / "include" / "hxq_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(hxq_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from helix_substrate_b200 import _lib
    L = _lib.lib()
    names = _declared()
    assert {"hxq_version", "hxq_strerror", "hxq_dequant", "hxq_gemv", "hxq_gemm",
            "hxq_gemv_workspace_bytes", "hxq_gemm_workspace_bytes", "hxq_csr_from_positions"} <= set(names)
    for n in names:
        assert hasattr(L, n), f"{n} declared in the header but not exported"
    assert L.hxq_version() >= 100
    assert _lib.strerror(0) == "ok" and "workspace" in _lib.strerror(_lib.HXQ_E_WORKSPACE)


def test_descriptor_layout_matches_header():
    from helix_substrate_b200._lib import HxqDesc
    # 4 x int32, int64, 4 pointers, 2 x int32, 5 pointers
    assert C.sizeof(HxqDesc) == 16 + 8 + 32 + 8 + 40
    assert HxqDesc.ld_idx.offset == 16 and HxqDesc.st_dtype.offset == 56 and HxqDesc.rowptr.offset == 64


def test_argument_validation_without_a_device():
    from helix_substrate_b200 import _lib
    L = _lib.lib()
    d = _lib.HxqDesc()
    assert L.hxq_gemv(C.byref(d), None, 0, 1, 0, None, 0, 0, None, 0, None) == _lib.HXQ_E_ARG
    assert L.hxq_dequant(None, 0, 1, None, 0, 0, None) == _lib.HXQ_E_ARG
    assert L.hxq_gemv_workspace_bytes(C.byref(d), 1) == 0
    # 6-bit packed product: nulls, token count, shapes that are not whole 16-code pieces
    assert L.hxq_gemv_packed6(None, 8, 64, None, None, 0, 1, 64, None, None, 0, 1, 64, None, 0, 8, None) == _lib.HXQ_E_ARG
    buf = np.zeros(64, dtype=np.uint8)
    p = buf.ctypes.data
    assert L.hxq_gemv_packed6(p, 8, 64, p, p, 0, 1, 64, None, p, 0, 17, 64, p, 0, 8, None) == _lib.HXQ_E_ARG
    assert L.hxq_gemv_packed6(p, 8, 60, p, p, 0, 1, 60, None, p, 0, 1, 60, p, 0, 8, None) == _lib.HXQ_E_SHAPE
    assert L.hxq_gemv_packed6(p, 8, 64, p, p, 2, 1, 64, None, p, 0, 1, 64, p, 0, 8, None) == _lib.HXQ_E_DTYPE


def test_csr_helper():
    from helix_substrate_b200 import _lib
    L = _lib.lib()
    pos = np.array([3, 40, 41, 2047], dtype=np.int64)
    rp = np.empty(65, dtype=np.int32)
    cols = np.empty(4, dtype=np.int32)
    assert L.hxq_csr_from_positions(pos.ctypes.data, 4, 64, 32, rp.ctypes.data, cols.ctypes.data) == 0
    assert rp[0] == 0 and rp[1] == 1 and rp[2] == 3 and rp[63] == 3 and rp[64] == 4
    assert cols.tolist() == [3, 8, 9, 31]
    bad = np.array([5, 5], dtype=np.int64)
    assert L.hxq_csr_from_positions(bad.ctypes.data, 2, 64, 32, rp.ctypes.data, cols.ctypes.data) == _lib.HXQ_E_ARG
    assert L.hxq_csr_from_positions(None, 0, 64, 32, rp.ctypes.data, None) == 0 and rp[64] == 0


def test_glue_and_allreduce_entry_points_validate_without_a_device():
    from helix_substrate_b200 import _lib
    L = _lib.lib()
    assert L.hxq_add_rmsnorm(None, None, None, None, 1, 64, 64, 64, 64, 1e-6, None) == _lib.HXQ_E_ARG
    assert L.hxq_rope_append(None, 0, None, None, None, None, 0, None, None, 1, 4, 2, 64, 16, None) == _lib.HXQ_E_ARG
    assert L.hxq_swiglu(None, None, None, 1, 64, 64, 64, 64, None) == _lib.HXQ_E_ARG
    assert L.hxq_dense_gemv(None, 8, 64, 64, None, 1, 64, None, 0, 8, None) == _lib.HXQ_E_ARG
    assert L.hxq_attn_decode(None, 0, None, None, None, None, 0, None, 0, 1, 4, 2, 64, 16, 0.125, None) == _lib.HXQ_E_ARG
    # sizes: 4-byte partial + 2 floats per (sequence, head, 64-row chunk); 2 slots x world x n_max floats
    assert L.hxq_attn_decode_workspace_bytes(2, 28, 128, 2184) == 2 * 28 * 35 * 130 * 4
    assert L.hxq_allreduce_buffer_bytes(4, 3584) == 2 * 4 * 3584 * 4
    assert L.hxq_allreduce_flag_bytes(8) == 2 * 8 * 32 * 4
    assert L.hxq_allreduce_buffer_bytes(9, 3584) == 0 and L.hxq_allreduce_buffer_bytes(2, 0) == 0
    assert L.hxq_allreduce_oneshot(None, None, 0, 2, 64, None, None, 64, None, 0, None, None) == _lib.HXQ_E_ARG


def test_static_scratch_covers_every_qwen25_projection():
    """The header promises that hxq_gemv_static's 2 MiB array is enough for every Qwen2.5-7B / 14B
    projection (also the fused qkv / gate_up ones) at M <= 16: check the sizing function, which
    needs no device (it falls back to 148 SMs)."""
    from helix_substrate_b200 import _lib
    L = _lib.lib()
    dummy = np.zeros(64, dtype=np.uint8)          # never dereferenced by the sizing call
    shapes = [(3584, 3584), (512, 3584), (4608, 3584), (18944, 3584), (37888, 3584), (3584, 18944),
              (5120, 5120), (1024, 5120), (7168, 5120), (13824, 5120), (27648, 5120), (5120, 13824)]
    for n_out, n_in in shapes:
        d = _lib.HxqDesc()
        d.out_features, d.in_features, d.group_size, d.ld_idx = n_out, n_in, 128, n_in
        d.indices = d.codebook = d.scales = d.offsets = dummy.ctypes.data
        d.st_dtype, d.ld_st = _lib.HXQ_F32, n_in // 128
        for M in (1, 2, 4, 16):
            nb = L.hxq_gemv_workspace_bytes(C.byref(d), M)
            assert 0 < nb <= (2 << 20), (n_out, n_in, M, nb)

