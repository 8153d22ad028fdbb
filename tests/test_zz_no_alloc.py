"""hxq_gemv_static: the decode product for hosts that cannot allocate.

Some callers never get to call the CUDA allocator at the point where they need
the product (their process froze its memory plan at start-up, or they are a
plug-in that is only handed inputs and outputs), so they cannot pass hxq_gemv
its scratch buffer.  The library then uses a fixed array of its own.  This
file is named to be collected last: a run that stops at the first failure has
by then run every other test."""

import ctypes as C

import numpy as np
import pytest
import torch

from conftest import rel_l2
from oracle import hxq_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL_F32 = 1e-3


def _entry():
    from helix_substrate_b200 import _lib
    L = _lib.lib()
    f = L.hxq_gemv_static
    f.restype = C.c_int
    f.argtypes = [C.POINTER(_lib.HxqDesc), C.c_void_p, C.c_int, C.c_int32, C.c_int64, C.c_void_p, C.c_int,
                  C.c_int64, C.c_void_p]
    return f


def _case(seed, n_out, n_in, G):
    from helix_substrate_b200.packed import HxqWeight, csr_from_positions
    rng = np.random.default_rng(seed)
    cb = (np.sort(rng.standard_normal(256)) * 0.02).astype(np.float32)
    idx = rng.integers(0, 256, (n_out, n_in), dtype=np.uint8)
    s = (1 + 0.1 * rng.standard_normal((n_out, n_in // G))).astype(np.float32)
    t = (0.002 * rng.standard_normal((n_out, n_in // G))).astype(np.float32)
    nnz = n_out * n_in // 500
    pos = np.sort(rng.choice(n_out * n_in, nnz, replace=False)).astype(np.int64)
    vals = (0.1 * rng.standard_normal(nnz)).astype(np.float16).astype(np.float32)
    bias = rng.standard_normal(n_out).astype(np.float32)
    rows, cols, deltas = O.derive_sidecar(cb, idx, pos, vals, s, t, G)
    rp, cc = csr_from_positions(torch.from_numpy(pos), n_out, n_in)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
    w = HxqWeight(dev(cb), dev(idx), rowptr=rp.to(DEV), cols=cc.to(DEV), deltas=dev(deltas), values=dev(vals),
                  bias=dev(bias), scales=dev(s), offsets=dev(t), group_size=G)
    return w, (cb, idx, rows, cols, deltas, bias, s, t)


@pytest.mark.parametrize("shape,M", [((1000, 3584), 1), ((520, 5120), 4), ((64, 18944), 16)])
def test_static_scratch_entry_matches_workspace_entry(shape, M):
    """Two calls in a row through the C ABI, each against hxq_gemv on the same
    inputs (and against the CPU oracle)."""
    f = _entry()
    w, (cb, idx, rows, cols, deltas, bias, s, t) = _case(shape[0], *shape, 128)
    stream = C.c_void_p(torch.cuda.current_stream(torch.device(DEV)).cuda_stream)
    for call in range(2):
        x = torch.randn(M, shape[1], device=DEV, generator=torch.Generator(device=DEV).manual_seed(call))
        y = torch.full((M, shape[0]), float("nan"), device=DEV)
        st = f(C.byref(w.desc), C.c_void_p(x.data_ptr()), 0, M, x.stride(0), C.c_void_p(y.data_ptr()), 0,
               y.stride(0), stream)
        assert st == 0, f"hxq_gemv_static returned {st} on call {call}"
        ref = w.matmul(x, force="gemv")                 # the existing entry point, caller-provided workspace
        torch.cuda.synchronize()
        assert rel_l2(y.cpu().numpy(), ref.cpu().numpy()) < TOL_F32
        assert torch.equal(y, ref), "same kernels, same partition: the two entry points agree bit for bit"
        ora = O.forward_f64(x.cpu().numpy(), cb, idx, rows, cols, deltas, bias, s, t, 128)
        assert rel_l2(y.cpu().numpy(), ora) < TOL_F32


def test_static_scratch_entry_refuses_what_does_not_fit():
    """A shape needing more scratch than the fixed array holds is turned away
    with HXQ_E_WORKSPACE before any kernel runs (the descriptor below claims far
    more rows than the buffers behind it have: nothing may be read)."""
    from helix_substrate_b200 import _lib
    f = _entry()
    w, _ = _case(1, 64, 1024, 128)
    d = _lib.HxqDesc.from_buffer_copy(w.desc)
    d.out_features = 4_000_000
    need = _lib.lib().hxq_gemv_workspace_bytes(C.byref(d), 4)
    assert need > (2 << 20)
    x = torch.zeros(4, 1024, device=DEV)
    y = torch.zeros(4, 64, device=DEV)
    stream = C.c_void_p(torch.cuda.current_stream(torch.device(DEV)).cuda_stream)
    st = f(C.byref(d), C.c_void_p(x.data_ptr()), 0, 4, 1024, C.c_void_p(y.data_ptr()), 0, 4_000_000, stream)
    assert st == _lib.HXQ_E_WORKSPACE
    assert "workspace" in _lib.strerror(st)
    torch.cuda.synchronize()
    assert float(y.abs().sum()) == 0.0
