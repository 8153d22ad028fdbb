"""The CPU oracle against the golden vectors recorded from the reference.

This pins the numpy restatement (oracle/hxq_oracle.py) to what the reference's
own CPU code returned on the same seeded inputs (tests/golden/make_golden.py).
"""

import numpy as np
import pytest

from conftest import load_golden, rel_l2
from oracle import hxq_oracle as O

CDNA_CASES = ["vq_only_64x32", "vq_sidecar_64x32", "student_t_300x256", "capped_sidecar_48x1024"]


@pytest.mark.parametrize("name", CDNA_CASES)
def test_reconstruct_bit_exact(name):
    g = load_golden(name)
    w = O.reconstruct(g["codebook"], g["indices"], g.get("sidecar_positions"), g.get("sidecar_values"))
    assert w.dtype == np.float32
    assert np.array_equal(w, g["reconstruct"])


@pytest.mark.parametrize("name", CDNA_CASES)
def test_reconstruct_block_and_tile_bit_exact(name):
    g = load_golden(name)
    if "block_rows" not in g:
        pytest.skip("no block recorded")
    r0, r1 = (int(v) for v in g["block_rows"])
    blk = O.reconstruct_block(g["codebook"], g["indices"], r0, r1,
                              g.get("sidecar_positions"), g.get("sidecar_values"))
    assert np.array_equal(blk, g["reconstruct_block"])
    rows = cols = deltas = None
    if "sidecar_positions" in g:
        rows, cols, deltas = O.derive_sidecar(g["codebook"], g["indices"],
                                              g["sidecar_positions"], g["sidecar_values"])
    tile = O.dequant_tile(g["codebook"], g["indices"], r0, r1, rows, cols, deltas)
    assert np.array_equal(tile, g["dequant_tile"])


@pytest.mark.parametrize("name", [c for c in CDNA_CASES if c != "vq_only_64x32"])
def test_sidecar_derivation(name):
    g = load_golden(name)
    rows, cols, deltas = O.derive_sidecar(g["codebook"], g["indices"],
                                          g["sidecar_positions"], g["sidecar_values"])
    assert np.array_equal(rows, g["sidecar_rows"])
    assert np.array_equal(cols, g["sidecar_cols"])
    assert np.array_equal(deltas, g["sidecar_deltas"])
    # decode_weight() = codebook + delta at the sidecar positions
    full = O.dequant_tile(g["codebook"], g["indices"], 0, g["indices"].shape[0], rows, cols, deltas)
    assert np.array_equal(full.ravel()[g["sidecar_positions"]], g["decode_weight_at_sidecar"])
    rp = O.csr_from_rows(rows, g["indices"].shape[0])
    assert rp[0] == 0 and rp[-1] == len(rows) and np.all(np.diff(rp) >= 0)
    for r in (0, g["indices"].shape[0] // 2, g["indices"].shape[0] - 1):
        assert np.all(rows[rp[r]:rp[r + 1]] == r)


@pytest.mark.parametrize("name", CDNA_CASES)
def test_forward_naive(name):
    g = load_golden(name)
    rows = cols = deltas = None
    if "sidecar_positions" in g:
        rows, cols, deltas = O.derive_sidecar(g["codebook"], g["indices"],
                                              g["sidecar_positions"], g["sidecar_values"])
    y = O.forward_naive(g["x"], g["codebook"], g["indices"], rows, cols, deltas, g.get("bias"))
    # same fp32 arithmetic, different BLAS blocking: tolerance of the reference's
    # own module tests (tests/test_helix_linear.py:92, atol 1e-5)
    assert np.allclose(y, g["y_naive"], atol=1e-5, rtol=1e-5)
    assert np.allclose(y, g["y_forward"], atol=1e-5, rtol=1e-5)
    y64 = O.forward_f64(g["x"], g["codebook"], g["indices"], rows, cols, deltas, g.get("bias"))
    assert rel_l2(g["y_naive"], y64) < 1e-5


@pytest.mark.parametrize("name", ["naive_vq_7x100x50", "naive_vq_1x33x17",
                                  "naive_vq_13x200x99", "naive_vq_16x256x128"])
def test_naive_vq_matmul(name):
    g = load_golden(name)
    y = O.naive_vq_matmul(g["x"], g["codebook"], g["indices"],
                          g["sidecar_positions"], g["sidecar_values"], g["bias"])
    assert np.allclose(y, g["y"], atol=1e-4, rtol=1e-5)
    # delta form (what the kernels use) agrees with the overwrite form
    rows, cols, deltas = O.derive_sidecar(g["codebook"], g["indices"],
                                          g["sidecar_positions"], g["sidecar_values"])
    y2 = O.forward_naive(g["x"], g["codebook"], g["indices"], rows, cols, deltas, g["bias"])
    assert rel_l2(y2, g["y"]) < 1e-5


def test_affine_group_corner():
    g = load_golden("affine_group_96x384")
    G = int(g["group_size"])
    y = O.affine_group_matmul(g["x"], g["indices"], g["scales"], g["offsets"], G, g["bias"])
    assert np.allclose(y, g["y"], atol=1e-4, rtol=1e-5)
    # the superset form with a ramp codebook is the same operator
    ramp = np.arange(256, dtype=np.float32)
    y2 = O.forward_naive(g["x"], ramp, g["indices"], bias=g["bias"],
                         scales=g["scales"], offsets=g["offsets"], group_size=G)
    assert np.allclose(y2, g["y"], atol=1e-4, rtol=1e-5)


def test_block_affine_module():
    g = load_golden("block_affine_64x512")
    w = O.block_affine_weight(g["indices"], g["scales"], g["biases_ab"], 256)
    assert np.array_equal(w, g["decode_weight"])
    y = O.block_affine_forward(g["x"], g["indices"], g["scales"], g["biases_ab"], 256, g["bias"])
    assert np.allclose(y, g["y"], atol=1e-5, rtol=1e-5)


def test_writer_internals():
    g = load_golden("writer_internals")
    cents, assign = O.simple_kmeans(g["data"], 256, max_iters=10)
    assert np.array_equal(cents, g["centroids"])
    assert np.array_equal(assign, g["assignments"])
    assert np.array_equal(O.chunked_assign(g["data"], g["centroids"]), g["chunked_assign"])
    pos, vals = O.find_outliers_percentile(g["outlier_tensor"], 99.0)
    assert np.array_equal(pos, g["outlier_positions"])
    assert np.array_equal(vals, g["outlier_values"])


def test_group_affine_fit_is_least_squares():
    rng = np.random.default_rng(0)
    w = rng.standard_normal((8, 256)).astype(np.float32)
    cb = np.sort(rng.standard_normal(256)).astype(np.float32)
    idx = O.chunked_assign(w.ravel(), cb).reshape(8, 256)
    s, t = O.fit_group_affine(w, cb, idx, 128)
    base = ((w - cb[idx]) ** 2).sum()
    fit = ((w - O.gather_affine(cb, idx, s, t, 128)) ** 2).sum()
    assert fit <= base * (1 + 1e-6)
    # perturbing the fit can only make the residual worse
    for ds, dt in ((1e-3, 0), (0, 1e-3), (-1e-3, 1e-3)):
        worse = ((w - O.gather_affine(cb, idx, s + ds, t + dt, 128)) ** 2).sum()
        assert worse >= fit * (1 - 1e-6)


def test_per_tensor_affine_statement_matches_the_reference(golden):
    """The torch restatement of affine_matmul_reference against what the reference's own returned."""
    import torch
    from helix_substrate_b200.triton_affine_matmul import affine_matmul_reference
    g = golden("per_tensor_affine_80x592")
    y = affine_matmul_reference(torch.from_numpy(g["x"]), torch.from_numpy(g["indices"]), float(g["step"]),
                                float(g["offset"]), torch.from_numpy(g["bias"]))
    assert np.allclose(y.numpy(), g["y"], rtol=1e-5, atol=1e-5)
    w = g["indices"].astype(np.float64) * float(g["step"]) + float(g["offset"])
    assert np.allclose(g["x"].astype(np.float64) @ w.T + g["bias"], g["y"], rtol=1e-4, atol=1e-4)



# --------------------------------------------------------------------------- the 4096 x 4096 benchmark configuration

def _config1_weight():
    rng = np.random.default_rng(0)
    w = rng.standard_t(5, size=(4096, 4096)).astype(np.float32)
    w *= np.float32(0.02) / w.std()
    return w.astype(np.float32)


def test_config1_full_size_against_the_reference_writer_and_forward():
    """The single-linear benchmark configuration as stated (Student-t(5) seed 0, std 0.02,
    k-means codebook, two-sided 99.95 % sidecar, no affine, x[1, 4096] fp32): the reference
    writer's codebook and sidecar are in the golden file, its 16 MB index matrix is pinned by
    hash, and reconstruct() / HelixLinear.forward by rows, row sums and the output."""
    import hashlib
    g = load_golden("config1_4096x4096")
    w = _config1_weight()
    assert hashlib.sha256(w.tobytes()).digest() == bytes(g["weight_sha256"])
    idx = O.assign_sorted(w.ravel(), g["codebook"])
    assert hashlib.sha256(idx.tobytes()).digest() == bytes(g["indices_sha256"])
    rows = g["rows"]
    # the reference's own assignment rule on the recorded rows
    assert np.array_equal(O.chunked_assign(w[rows].ravel(), g["codebook"]), idx.reshape(4096, 4096)[rows].ravel())
    idx = idx.reshape(4096, 4096)
    pos, vals = O.find_outliers_percentile(w, 99.95)
    assert np.array_equal(pos, g["sidecar_positions"])
    assert np.array_equal(O.sidecar_fp16_roundtrip(vals), g["sidecar_values"])
    rec = O.reconstruct(g["codebook"], idx, g["sidecar_positions"], g["sidecar_values"])
    assert np.array_equal(rec[rows], g["reconstruct_rows"])
    assert np.array_equal(rec.astype(np.float64).sum(1), g["reconstruct_row_sums_f64"])
    r, c, d = O.derive_sidecar(g["codebook"], idx, g["sidecar_positions"], g["sidecar_values"])
    y = O.forward_naive(g["x"], g["codebook"], idx, r, c, d)
    assert np.allclose(y, g["y_naive"], atol=1e-5, rtol=1e-5)
    assert rel_l2(y, g["y_forward"]) < 1e-5
