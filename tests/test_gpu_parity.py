"""GPU parity: the CUDA path, called through the C ABI, against the CPU oracle
and the golden vectors recorded from the reference.

Tolerances (from the task statement): dequantised weights bit-exact; fp32-
accumulate products rel-L2 <= 1e-3; bf16 tensor-core products rel-L2 <= 1e-2.
"""

import numpy as np
import pytest
import torch

from conftest import load_golden, rel_l2
from oracle import hxq_oracle as O

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
TOL_F32 = 1e-3
TOL_BF16 = 1e-2
CDNA_CASES = ["vq_only_64x32", "vq_sidecar_64x32", "student_t_300x256", "capped_sidecar_48x1024"]


def _t(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
    return t if dtype is None else t.to(dtype)


def _weight(cb, idx, pos=None, vals=None, bias=None, s=None, t=None, G=0, col0=0, idx_view=None):
    """HxqWeight over device copies; sidecar derived by the oracle's rule."""
    from helix_substrate_b200.packed import HxqWeight, csr_from_positions
    kw = {}
    n_out, n_in = idx.shape
    if pos is not None and len(pos):
        rows, cols, deltas = O.derive_sidecar(cb, idx, pos, vals, s, t, G, col0 % G if G else 0)
        rp, cc = csr_from_positions(torch.from_numpy(np.asarray(pos)), n_out, n_in)
        kw = dict(rowptr=rp.to(DEV), cols=cc.to(DEV), deltas=_t(deltas), values=_t(np.asarray(vals, np.float32)))
    if s is not None:
        kw.update(scales=_t(s), offsets=_t(t), group_size=G)
    cbp = np.concatenate([cb, np.repeat(cb[-1:], 256 - len(cb))]).astype(np.float32)
    return HxqWeight(_t(cbp), _t(idx) if idx_view is None else idx_view,
                     bias=None if bias is None else _t(bias), col0=col0, **kw)


def _make(rng, n_out, n_in, G=0, nnz_frac=0.002, st_dtype=np.float32, bias=True):
    cb = (np.sort(rng.standard_normal(256)) * 0.02).astype(np.float32)
    idx = rng.integers(0, 256, (n_out, n_in), dtype=np.uint8)
    s = t = None
    if G:
        ng = -(-n_in // G)
        s = (1.0 + 0.1 * rng.standard_normal((n_out, ng))).astype(st_dtype)
        t = (0.002 * rng.standard_normal((n_out, ng))).astype(st_dtype)
    nnz = int(n_out * n_in * nnz_frac)
    pos = vals = None
    if nnz:
        pos = np.sort(rng.choice(n_out * n_in, nnz, replace=False)).astype(np.int64)
        vals = (0.1 * rng.standard_normal(nnz)).astype(np.float16).astype(np.float32)
    b = rng.standard_normal(n_out).astype(np.float32) if bias else None
    return cb, idx, pos, vals, b, s, t


# --------------------------------------------------------------------------- dequant

@pytest.mark.parametrize("name", CDNA_CASES)
def test_dequant_bit_exact_vs_reference_reconstruct(name):
    g = load_golden(name)
    w = _weight(g["codebook"], g["indices"], g.get("sidecar_positions"), g.get("sidecar_values"))
    assert np.array_equal(w.dequant().cpu().numpy(), g["reconstruct"])
    if "block_rows" in g:
        r0, r1 = (int(v) for v in g["block_rows"])
        assert np.array_equal(w.dequant(r0, r1).cpu().numpy(), g["reconstruct_block"])
    bf = w.dequant(dtype=torch.bfloat16)
    assert torch.equal(bf, _t(g["reconstruct"]).to(torch.bfloat16))


@pytest.mark.parametrize("shape,G,col0", [((40, 256), 128, 0), ((33, 100), 0, 0), ((17, 96), 32, 0),
                                          ((64, 448), 128, 448), ((9, 640), 256, 0), ((24, 50), 25, 0)])
@pytest.mark.parametrize("st", [np.float32, np.float16])
def test_dequant_affine_bit_exact_vs_oracle(shape, G, col0, st):
    rng = np.random.default_rng(hash((shape, G, col0)) & 0xffff)
    n_out, n_in = shape
    cb, idx, pos, vals, b, s, t = _make(rng, n_out, n_in, 0, nnz_frac=0.01)
    if G:
        ng = (col0 + n_in - 1) // G - col0 // G + 1
        s = (1.0 + 0.1 * rng.standard_normal((n_out, ng))).astype(st)
        t = (0.002 * rng.standard_normal((n_out, ng))).astype(st)
    # oracle with global group ids: shift so that local group 0 is col0 // G
    ref = O.reconstruct(cb, idx, pos, vals, s, t, G, col0 - (col0 // G) * G if G else 0)
    w = _weight(cb, idx, pos, vals, None, s, t, G, col0)
    assert np.array_equal(w.dequant().cpu().numpy(), ref)


# --------------------------------------------------------------------------- products

@pytest.mark.parametrize("name", CDNA_CASES)
def test_product_vs_reference_forward(name):
    g = load_golden(name)
    w = _weight(g["codebook"], g["indices"], g.get("sidecar_positions"), g.get("sidecar_values"), g.get("bias"))
    y = w.matmul(_t(g["x"])).cpu().numpy()
    assert rel_l2(y, g["y_naive"]) < TOL_F32
    # the reference's own module-test tolerance also holds at these sizes
    assert np.allclose(y, g["y_naive"], atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("name", ["naive_vq_7x100x50", "naive_vq_1x33x17", "naive_vq_13x200x99",
                                  "naive_vq_16x256x128"])
def test_product_odd_shapes_vs_reference_kernel_test_oracle(name):
    g = load_golden(name)
    w = _weight(g["codebook"], g["indices"], g["sidecar_positions"], g["sidecar_values"], g["bias"])
    y = w.matmul(_t(g["x"])).cpu().numpy()
    # tests/test_triton_vq_matmul.py:34 : rel-max-err < 1e-3
    assert np.abs(y - g["y"]).max() / (np.abs(g["y"]).max() + 1e-8) < 1e-3
    assert rel_l2(y, g["y"]) < TOL_F32


SHAPES = [  # (OUT, IN, G, col0)
    (8, 512, 0, 0), (50, 528, 0, 0), (64, 1024, 128, 0), (100, 3584, 128, 0), (37, 2064, 128, 0),
    (72, 448, 128, 448), (40, 2368, 128, 2368 * 3), (16, 1536, 256, 0), (24, 1536, 1536, 0),
    (300, 160, 32, 0), (19, 77, 0, 0),
    # whole 128-column groups but a short last 512-column chunk: the streaming kernel masks lanes
    # (the shapes of group-aligned tensor-parallel shards: 18944 / 8 -> 2432, 13824 / 8 -> 1792)
    (64, 1792, 128, 0), (24, 640, 128, 0), (40, 2432, 128, 2432), (16, 128, 128, 0), (32, 896, 0, 0),
]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("M", [1, 2, 3, 4, 5, 8, 16])
def test_gemv_vs_oracle(shape, M):
    n_out, n_in, G, col0 = shape
    rng = np.random.default_rng(n_out * 7919 + n_in + M)
    cb, idx, pos, vals, b, s, t = _make(rng, n_out, n_in, 0, nnz_frac=0.003)
    c0 = 0
    if G:
        ng = (col0 + n_in - 1) // G - col0 // G + 1
        s = (1.0 + 0.1 * rng.standard_normal((n_out, ng))).astype(np.float32)
        t = (0.002 * rng.standard_normal((n_out, ng))).astype(np.float32)
        c0 = col0 - (col0 // G) * G
    rows = cols = deltas = None
    if pos is not None:
        rows, cols, deltas = O.derive_sidecar(cb, idx, pos, vals, s, t, G, c0)
    x = rng.standard_normal((M, n_in)).astype(np.float32)
    ref = O.forward_f64(x, cb, idx, rows, cols, deltas, b, s, t, G, c0)
    w = _weight(cb, idx, pos, vals, b, s, t, G, col0)
    y = w.matmul(_t(x), force="gemv")
    assert y.dtype == torch.float32
    assert rel_l2(y.cpu().numpy(), ref) < TOL_F32
    y2 = w.matmul(_t(x), force="gemv")
    assert torch.equal(y, y2), "the product must be bit-identical from run to run"


@pytest.mark.parametrize("xdt,ydt", [(torch.bfloat16, torch.bfloat16), (torch.float16, torch.float32),
                                     (torch.float32, torch.bfloat16), (torch.bfloat16, torch.float32)])
@pytest.mark.parametrize("M", [1, 4, 16])
def test_gemv_dtypes_and_strides(xdt, ydt, M):
    rng = np.random.default_rng(5)
    n_out, n_in, G = 136, 1792, 128
    cb, idx, pos, vals, b, s, t = _make(rng, n_out, n_in, G, st_dtype=np.float16)
    rows, cols, deltas = O.derive_sidecar(cb, idx, pos, vals, s, t, G)
    xbuf = torch.randn(M, n_in + 24, device=DEV).to(xdt)
    off = 4 if M == 4 else 8  # M == 4: rows start off the 16-byte grid -> scalar activation loads
    x = xbuf[:, off:off + n_in]
    ref = O.forward_f64(x.float().cpu().numpy(), cb, idx, rows, cols, deltas, b, s, t, G)
    w = _weight(cb, idx, pos, vals, b, s, t, G)
    y = w.matmul(x, out_dtype=ydt, force="gemv")
    assert y.dtype == ydt
    tol = TOL_F32 if ydt == torch.float32 else 4e-3  # one rounding of the result to bf16
    assert rel_l2(y.float().cpu().numpy(), ref) < tol


def test_gemv_row_parallel_shard_is_zero_copy_slice():
    """A column slice of the full index matrix (row stride = full IN) with
    col0 carrying the global column gives the partial product of that slice."""
    rng = np.random.default_rng(11)
    n_out, n_in, G, tp = 48, 3584, 128, 8
    cb, idx, _, _, _, s, t = _make(rng, n_out, n_in, G, nnz_frac=0)
    x = rng.standard_normal((2, n_in)).astype(np.float32)
    full = O.forward_f64(x, cb, idx, scales=s, offsets=t, group_size=G)
    idx_d, s_d, t_d = _t(idx), _t(s), _t(t)
    from helix_substrate_b200.packed import HxqWeight
    total = torch.zeros(2, n_out, device=DEV, dtype=torch.float64)
    per = n_in // tp  # 448 = 3.5 groups: shards start mid-group
    for r in range(tp):
        c0 = r * per
        g0, g1 = c0 // G, (c0 + per - 1) // G + 1
        w = HxqWeight(_t(cb), idx_d[:, c0:c0 + per], scales=s_d[:, g0:g1], offsets=t_d[:, g0:g1],
                      group_size=G, col0=c0)
        total += w.matmul(_t(x[:, c0:c0 + per]).contiguous(), force="gemv").double()
    assert rel_l2(total.cpu().numpy(), full) < TOL_F32


def test_workspace_is_left_clean():
    from helix_substrate_b200 import packed
    rng = np.random.default_rng(3)
    cb, idx, pos, vals, b, s, t = _make(rng, 64, 2048, 128)
    w = _weight(cb, idx, pos, vals, b, s, t, 128)
    x = torch.randn(4, 2048, device=DEV)
    w.matmul(x, force="gemv")
    torch.cuda.synchronize()
    key = (torch.device(DEV).index, torch.cuda.current_stream(torch.device(DEV)).cuda_stream, "gemv")
    ws = packed._workspaces[key]
    assert int(ws.view(torch.int32).abs().sum()) == 0, "counters and scratch must both be back to zero"


def test_workspace_survives_a_change_of_shape():
    """Two shapes lay counters and scratch out differently inside the same
    workspace; the second must not see leftovers of the first."""
    rng = np.random.default_rng(4)
    outs = []
    for (n_out, n_in) in ((24, 4096), (520, 1536), (24, 4096)):
        cb, idx, pos, vals, b, s, t = _make(np.random.default_rng(n_out), n_out, n_in, 128)
        rows, cols, deltas = O.derive_sidecar(cb, idx, pos, vals, s, t, 128)
        x = np.random.default_rng(1).standard_normal((2, n_in)).astype(np.float32)
        ref = O.forward_f64(x, cb, idx, rows, cols, deltas, b, s, t, 128)
        y = _weight(cb, idx, pos, vals, b, s, t, 128).matmul(_t(x), force="gemv")
        assert rel_l2(y.cpu().numpy(), ref) < TOL_F32
        outs.append(y)
    assert torch.equal(outs[0], outs[2])


# --------------------------------------------------------------------------- full size, property based

@pytest.mark.parametrize("shape", [(18944, 3584), (3584, 18944), (4096, 4096)])
def test_full_size_properties(shape):
    """The benchmark shapes: (i) dequant equals an independent device-side gather,
    (ii) product equals dense fp64 matmul of the dequantised weight on a row
    sample, (iii) linearity in x, (iv) run-to-run bit equality."""
    n_out, n_in = shape
    G = 128
    gen = torch.Generator(device=DEV).manual_seed(n_out)
    idx = torch.randint(0, 256, (n_out, n_in), dtype=torch.uint8, device=DEV, generator=gen)
    cb = (torch.sort(torch.randn(256, device=DEV, generator=gen)).values * 0.02).contiguous()
    s = (1 + 0.1 * torch.randn(n_out, n_in // G, device=DEV, generator=gen)).contiguous()
    t = (0.002 * torch.randn(n_out, n_in // G, device=DEV, generator=gen)).contiguous()
    nnz = n_out * n_in // 1000
    pos = torch.sort(torch.randperm(n_out * n_in, device=DEV, generator=gen)[:nnz]).values
    vals = (0.1 * torch.randn(nnz, device=DEV, generator=gen)).half().float()
    bias = torch.randn(n_out, device=DEV, generator=gen)
    from helix_substrate_b200 import HelixLinear
    mod = HelixLinear(n_in, n_out, cb, idx, pos, vals, bias=bias, group_scales=s, group_offsets=t, group_size=G)
    w_gpu = mod.decode_weight()
    # (i) independent gather + two-rounding affine + overwrite, in torch on the device
    w_chk = cb[idx.long()]
    w_chk = (w_chk.view(n_out, n_in // G, G) * s[:, :, None] + t[:, :, None]).view(n_out, n_in)
    w_chk.view(-1)[pos] = vals
    assert torch.equal(w_gpu, w_chk)
    del w_chk
    # (ii) product on a sample of rows against fp64; decode_weight overwrote, the
    # product adds deltas: identical up to one rounding at the sidecar entries
    for M, xdt in ((1, torch.float32), (4, torch.bfloat16), (16, torch.bfloat16)):
        x = torch.randn(M, n_in, device=DEV, generator=gen).to(xdt)
        y = mod(x)
        assert y.dtype == xdt
        rows = torch.randint(0, n_out, (512,), device=DEV, generator=gen)
        ref = x.double() @ w_gpu[rows].double().t() + bias[rows].double()
        tol = TOL_F32 if xdt == torch.float32 else 4e-3
        assert rel_l2(y[:, rows].double().cpu().numpy(), ref.cpu().numpy()) < tol
        assert torch.equal(y, mod(x))
    # (iii) linearity
    x1 = torch.randn(1, n_in, device=DEV, generator=gen)
    x2 = torch.randn(1, n_in, device=DEV, generator=gen)
    mod.bias = None
    mod._packed = None
    lhs = mod(2.0 * x1 - 3.0 * x2)
    rhs = 2.0 * mod(x1) - 3.0 * mod(x2)
    assert rel_l2(lhs.cpu().numpy(), rhs.cpu().numpy()) < 1e-4


# --------------------------------------------------------------------------- tensor-core path

GEMM_SHAPES = [  # (OUT, IN, G, col0)
    (128, 512, 128, 0), (200, 1024, 128, 0), (64, 3584, 128, 0), (300, 448, 128, 448),
    (136, 1088, 64, 0), (128, 2048, 0, 0), (96, 592, 0, 0),
]


@pytest.mark.parametrize("shape", GEMM_SHAPES)
@pytest.mark.parametrize("M", [17, 64, 100, 256, 300, 600])
def test_gemm_vs_oracle(shape, M):
    n_out, n_in, G, col0 = shape
    rng = np.random.default_rng(n_out * 31 + n_in + M)
    cb, idx, pos, vals, b, s, t = _make(rng, n_out, n_in, 0, nnz_frac=0.004)
    c0 = 0
    if G:
        ng = (col0 + n_in - 1) // G - col0 // G + 1
        s = (1.0 + 0.1 * rng.standard_normal((n_out, ng))).astype(np.float32)
        t = (0.002 * rng.standard_normal((n_out, ng))).astype(np.float32)
        c0 = col0 - (col0 // G) * G
    rows, cols, deltas = O.derive_sidecar(cb, idx, pos, vals, s, t, G, c0)
    x = _t(rng.standard_normal((M, n_in)).astype(np.float32), torch.bfloat16)
    ref = O.forward_f64(x.float().cpu().numpy(), cb, idx, rows, cols, deltas, b, s, t, G, c0)
    w = _weight(cb, idx, pos, vals, b, s, t, G, col0)
    y = w.matmul(x, out_dtype=torch.float32, force="gemm")
    assert w.gemm_status() == 0, "a bounded wait inside the tensor-core kernel gave up"
    assert rel_l2(y.cpu().numpy(), ref) < TOL_BF16
    # the decode kernels agree with it to bf16 precision as well
    y2 = w.matmul(x, out_dtype=torch.float32, force="gemv")
    assert rel_l2(y.cpu().numpy(), y2.cpu().numpy()) < TOL_BF16
    assert torch.equal(y, w.matmul(x, out_dtype=torch.float32, force="gemm"))


@pytest.mark.parametrize("nnz,M", [(2000, 64), (2000, 600), (9000, 24), (9000, 100)])
def test_gemm_sidecar_is_applied(nnz, M):
    """With a zero codebook the product is the sidecar alone: every entry must
    land in the right (row, column) of the dequantised tile.  9000 entries over 256 rows are more
    per 128-row tile than the small-token kernel keeps in shared memory (its cursors then stay on
    global memory)."""
    rng = np.random.default_rng(2)
    n_out, n_in = 256, 1024
    cb = np.zeros(256, np.float32)
    idx = rng.integers(0, 256, (n_out, n_in), dtype=np.uint8)
    pos = np.sort(rng.choice(n_out * n_in, nnz, replace=False)).astype(np.int64)
    vals = rng.standard_normal(nnz).astype(np.float16).astype(np.float32)
    dense = np.zeros(n_out * n_in, np.float32)
    dense[pos] = vals
    x = _t(rng.standard_normal((M, n_in)).astype(np.float32), torch.bfloat16)
    ref = x.float().cpu().numpy().astype(np.float64) @ dense.reshape(n_out, n_in).astype(np.float64).T
    w = _weight(cb, idx, pos, vals)
    y = w.matmul(x, force="gemm")
    assert w.gemm_status() == 0
    assert rel_l2(y.cpu().numpy(), ref) < TOL_BF16


@pytest.mark.parametrize("xdt", [torch.float32, torch.float16])
def test_gemm_converts_other_activation_types(xdt):
    rng = np.random.default_rng(9)
    cb, idx, pos, vals, b, s, t = _make(rng, 128, 1000 // 8 * 8 + 16, 0)
    rows, cols, deltas = O.derive_sidecar(cb, idx, pos, vals)
    x = torch.randn(40, idx.shape[1], device=DEV).to(xdt)
    ref = O.forward_f64(x.float().cpu().numpy(), cb, idx, rows, cols, deltas, b)
    w = _weight(cb, idx, pos, vals, b)
    y = w.matmul(x, out_dtype=torch.bfloat16, force="gemm")
    assert y.dtype == torch.bfloat16 and w.gemm_status() == 0
    assert rel_l2(y.float().cpu().numpy(), ref) < TOL_BF16


@pytest.mark.parametrize("shape,M", [((18944, 3584), 512), ((3584, 18944), 512), ((512, 3584), 2048)])
def test_gemm_full_size_against_dense(shape, M):
    n_out, n_in = shape
    G = 128
    gen = torch.Generator(device=DEV).manual_seed(n_in)
    idx = torch.randint(0, 256, (n_out, n_in), dtype=torch.uint8, device=DEV, generator=gen)
    cb = (torch.sort(torch.randn(256, device=DEV, generator=gen)).values * 0.02).contiguous()
    s = (1 + 0.1 * torch.randn(n_out, n_in // G, device=DEV, generator=gen)).contiguous()
    t = (0.002 * torch.randn(n_out, n_in // G, device=DEV, generator=gen)).contiguous()
    nnz = n_out * n_in // 1000
    pos = torch.sort(torch.randperm(n_out * n_in, device=DEV, generator=gen)[:nnz]).values
    vals = (0.1 * torch.randn(nnz, device=DEV, generator=gen)).half().float()
    bias = torch.randn(n_out, device=DEV, generator=gen)
    from helix_substrate_b200 import HelixLinear
    mod = HelixLinear(n_in, n_out, cb, idx, pos, vals, bias=bias, group_scales=s, group_offsets=t, group_size=G)
    x = torch.randn(M, n_in, device=DEV, generator=gen).bfloat16()
    y = mod(x)
    assert y.dtype == torch.bfloat16 and mod.packed().gemm_status() == 0
    ref = x.double() @ mod.decode_weight().double().t() + bias.double()
    assert rel_l2(y.double().cpu().numpy(), ref.cpu().numpy()) < TOL_BF16
