"""GPU parity on the benchmark configurations exactly as they are stated: the
4096 x 4096 single linear against the reference writer's and forward's recorded
outputs, the Qwen2.5-7B MLP shapes with writer-made (k-means + least-squares
affine) tensors at 1, 4 and 16 tokens, and the tensor-core kernel at its
largest token counts.  All products go through the C ABI.

Tolerances (task statement): dequantised weights bit-exact, fp32-accumulate
products rel-L2 <= 1e-3, bf16 tensor-core products rel-L2 <= 1e-2.
"""

import hashlib

import numpy as np
import pytest
import torch

from conftest import load_golden, rel_l2
from oracle import hxq_oracle as O

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
TOL_F32 = 1e-3
TOL_BF16 = 1e-2


def _config1_weight():
    rng = np.random.default_rng(0)
    w = rng.standard_t(5, size=(4096, 4096)).astype(np.float32)
    w *= np.float32(0.02) / w.std()
    return w.astype(np.float32)


def test_config1_single_linear_as_stated():
    """Student-t(5) seed 0 at std 0.02, the reference writer's codebook and sidecar, indices
    assigned ON THE DEVICE (hash-checked against the reference writer's), no affine,
    x[1, 4096] fp32: dequant bit-exact with reconstruct(), product within 1e-3 of the
    reference HelixLinear forward."""
    from helix_substrate_b200 import HelixLinear
    from helix_substrate_b200.hxq_writer_gpu import assign_indices, find_outliers_percentile
    g = load_golden("config1_4096x4096")
    w = _config1_weight()
    assert hashlib.sha256(w.tobytes()).digest() == bytes(g["weight_sha256"])
    w_d = torch.from_numpy(w).to(DEV)
    cb = torch.from_numpy(g["codebook"]).to(DEV)
    idx = assign_indices(w_d.reshape(-1), cb).view(4096, 4096)
    assert hashlib.sha256(idx.cpu().numpy().tobytes()).digest() == bytes(g["indices_sha256"]), \
        "device-side nearest-centroid assignment differs from the reference writer's"
    pos, vals = find_outliers_percentile(w_d, 99.95)
    assert np.array_equal(pos.cpu().numpy(), g["sidecar_positions"])
    assert np.array_equal(vals.half().float().cpu().numpy(), g["sidecar_values"])
    mod = HelixLinear(4096, 4096, cb, idx, torch.from_numpy(g["sidecar_positions"]).to(DEV),
                      torch.from_numpy(g["sidecar_values"]).to(DEV)).to(DEV)
    assert mod.group_size == 0
    # reconstruct(): recorded rows bit for bit, every row by its fp64 sum
    rows = torch.from_numpy(g["rows"]).to(DEV)
    rec = mod.packed().dequant()
    assert np.array_equal(rec[rows].cpu().numpy(), g["reconstruct_rows"])
    assert np.allclose(rec.double().sum(1).cpu().numpy(), g["reconstruct_row_sums_f64"], rtol=0, atol=1e-9)
    # forward
    x = torch.from_numpy(g["x"]).to(DEV)
    y = mod(x)
    assert y.dtype == torch.float32 and y.shape == (1, 4096)
    assert rel_l2(y.cpu().numpy(), g["y_forward"]) < TOL_F32
    assert rel_l2(y.cpu().numpy(), g["y_naive"]) < TOL_F32
    assert np.allclose(y.cpu().numpy(), g["y_naive"], atol=1e-4, rtol=1e-4)   # the reference's own module tolerance
    assert mod._last_dispatch["dispatch_selected"] == "hxq_gemv_sm100a"
    assert torch.equal(y, mod(x))


@pytest.mark.parametrize("shape", [(18944, 3584), (3584, 18944)])
def test_config2_mlp_shapes_with_writer_made_tensors(shape):
    """Group-128 affine HXQ linears at the Qwen2.5-7B MLP shapes, encoded by the device writer
    from Student-t(5) weights (k-means codebook, nearest-centroid indices, least-squares s/t,
    two-sided 99.95 % sidecar), bf16 activations, 1 / 4 / 16 tokens: (i) dequant bit-exact
    with the oracle on sampled rows, (ii) the product against the oracle's fp64 forward on
    those rows, (iii) compression is faithful to the dense weight."""
    from helix_substrate_b200 import HelixLinear
    from helix_substrate_b200.hxq_writer_gpu import compress_weight, student_t_weight
    n_out, n_in = shape
    w = student_t_weight(shape, 3, DEV)
    enc = compress_weight(w, percentile=99.95, group_size=128)
    mod = HelixLinear(n_in, n_out, **enc).to(DEV)
    gen = torch.Generator(device=DEV).manual_seed(1)
    rows = torch.sort(torch.randperm(n_out, device=DEV, generator=gen)[:256]).values
    # oracle inputs restricted to the sampled rows
    cb = enc["codebook"].cpu().numpy()
    idx_r = enc["indices"][rows].cpu().numpy()
    s_r, t_r = enc["group_scales"][rows].cpu().numpy(), enc["group_offsets"][rows].cpu().numpy()
    pos, vals = enc["sidecar_positions"], enc["sidecar_values"]
    prow = pos // n_in
    keep = torch.isin(prow, rows)
    local_row = torch.searchsorted(rows, prow[keep])
    pos_r = (local_row * n_in + pos[keep] % n_in).cpu().numpy()
    vals_r = vals[keep].cpu().numpy()
    assert np.all(np.diff(pos_r) > 0)
    ref_w = O.reconstruct(cb, idx_r, pos_r, vals_r, s_r, t_r, 128)
    got_w = mod.packed().dequant()[rows]
    assert np.array_equal(got_w.cpu().numpy(), ref_w)
    # the code is a faithful compression of the weight it was made from
    assert rel_l2(got_w.cpu().numpy(), w[rows].cpu().numpy()) < 0.05
    r, c, d = O.derive_sidecar(cb, idx_r, pos_r, vals_r, s_r, t_r, 128)
    for M in (1, 4, 16):
        x = torch.randn(M, n_in, device=DEV, generator=gen).bfloat16()
        y = mod.packed().matmul(x, out_dtype=torch.float32, force="gemv")      # the fp32-accumulate kernel
        ref = O.forward_f64(x.float().cpu().numpy(), cb, idx_r, r, c, d, None, s_r, t_r, 128)
        assert rel_l2(y[:, rows].cpu().numpy(), ref) < TOL_F32, f"M={M}"
        # the module's own choice: that kernel up to 4 tokens of bf16, bf16 tensor-core operands above
        yb = mod(x)
        assert yb.dtype == torch.bfloat16
        assert mod._last_dispatch["dispatch_selected"] == ("hxq_gemv_sm100a" if M <= 4 else "hxq_gemm_sm100a")
        assert rel_l2(yb[:, rows].float().cpu().numpy(), ref) < (4e-3 if M <= 4 else TOL_BF16)
        assert torch.equal(yb, mod(x))


@pytest.mark.parametrize("shape,M", [((512, 3584), 8192), ((3584, 3584), 2048), ((3584, 3584), 8192)])
def test_config3_tensor_core_kernel_at_its_largest_token_counts(shape, M):
    from helix_substrate_b200 import HelixLinear
    from helix_substrate_b200.hxq_writer_gpu import compress_weight, student_t_weight
    n_out, n_in = shape
    enc = compress_weight(student_t_weight(shape, 5, DEV), percentile=99.95, group_size=128)
    bias = torch.randn(n_out, device=DEV) * 0.02
    mod = HelixLinear(n_in, n_out, bias=bias, **enc).to(DEV)
    x = torch.randn(M, n_in, device=DEV, generator=torch.Generator(device=DEV).manual_seed(2)).bfloat16()
    y = mod(x)
    assert y.dtype == torch.bfloat16 and mod.packed().gemm_status() == 0
    assert mod._last_dispatch["dispatch_selected"] == "hxq_gemm_sm100a"
    ref = x.double() @ mod.decode_weight().double().t() + bias.double()
    assert rel_l2(y.double().cpu().numpy(), ref.cpu().numpy()) < TOL_BF16
    assert torch.equal(y, mod(x))


# --------------------------------------------------------------------------- the device-side writer, on the device

def test_device_writer_assignment_and_outliers_match_the_reference_writer():
    """hxq_writer_gpu on CUDA tensors against what the reference writer's _chunked_assign and
    find_outliers_percentile returned (golden 'writer_internals')."""
    from helix_substrate_b200.hxq_writer_gpu import assign_indices, find_outliers_percentile
    g = load_golden("writer_internals")
    data = torch.from_numpy(g["data"]).to(DEV)
    cents = torch.from_numpy(g["centroids"]).to(DEV)
    order = torch.argsort(cents)
    idx_sorted = assign_indices(data, cents[order])
    got = order[idx_sorted.long()].to(torch.uint8)            # index into the reference's (unsorted) centroid list
    want = torch.from_numpy(g["chunked_assign"]).to(DEV)
    same = got == want
    if not bool(same.all()):   # only exact ties between duplicate centroids may differ
        assert torch.equal(cents[got.long()][~same], cents[want.long()][~same])
    pos, vals = find_outliers_percentile(torch.from_numpy(g["outlier_tensor"]).to(DEV), 99.0)
    assert np.array_equal(pos.cpu().numpy(), g["outlier_positions"])
    assert np.array_equal(vals.cpu().numpy(), g["outlier_values"])
