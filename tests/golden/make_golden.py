#!/usr/bin/env python3
"""Generate the golden vectors under tests/golden/ from the REFERENCE itself.

Run once, on a machine that has a checkout of the reference:

    HXQ_REFERENCE_DIR=<reference checkout> python tests/golden/make_golden.py [case ...]

The reference package does not import as shipped (its modules were renamed
cdna* -> hxq* without updating the imports), so this script builds a throw-away
directory of symlinks with the four alias names and imports the reference from
there.  Nothing here is needed at test time: tests read only the .npz files.

Each case records the seeded inputs together with what the reference's own
CPU code returned for them (CDNAv3Reader.reconstruct, HelixLinear forward /
_dequant_tile / decode_weight, affine_group_matmul_reference,
HelixAffineLinear, affine_matmul_reference, the writer's k-means / assignment / outlier selection).
"""

from __future__ import annotations

import os
import sys
import tempfile
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
if "HXQ_REFERENCE_DIR" not in os.environ:
    raise SystemExit("set HXQ_REFERENCE_DIR to a checkout of echo313unfolding/helix-substrate")
REF = Path(os.environ["HXQ_REFERENCE_DIR"])

_ALIASES = {
    "cdna_encoder.py": "hxq_encoder.py",
    "cdnav3_reader.py": "hxq_reader_v3.py",
    "cdnav3_writer.py": "hxq_writer_v3.py",
    "cdna_reader.py": "hxq_reader.py",
}


def _import_reference():
    shim = Path(tempfile.mkdtemp(prefix="hxq_ref_shim_"))
    pkg = shim / "helix_substrate"
    pkg.mkdir()
    for f in (REF / "helix_substrate").glob("*.py"):
        (pkg / f.name).symlink_to(f)
    for alias, real in _ALIASES.items():
        (pkg / alias).symlink_to(REF / "helix_substrate" / real)
    sys.path.insert(0, str(shim))
    sys.path.insert(0, str(REF / "tests"))
    import helix_substrate  # noqa: F401
    return shim


def _student_t(shape, seed):
    rng = np.random.default_rng(seed)
    w = rng.standard_t(5, size=shape).astype(np.float32)
    w *= np.float32(0.02) / w.std()
    return w.astype(np.float32)


def main():
    _import_reference()
    import torch
    from helix_substrate.helix_linear import HelixLinear, load_helix_linear_from_cdnav3
    from helix_substrate.cdnav3_reader import CDNAv3Reader
    from helix_substrate.cdnav3_writer import CDNAv3Writer
    from helix_substrate.tensor_policy import TensorPolicy, TensorClass
    from helix_substrate.generate_sidecars_v3 import find_outliers_percentile
    from helix_substrate.cdna_encoder import _simple_kmeans
    from helix_substrate.triton_affine_group_matmul import affine_group_matmul_reference
    from helix_substrate.helix_affine_linear import HelixAffineLinear, quantize_linear_to_affine
    from test_triton_vq_matmul import _naive_vq_matmul

    torch.set_num_threads(1)
    out = {}
    only = set(sys.argv[1:]) or None   # optional list of case names: write only those files

    def cdna_case(tag, tensor, policy, x, bias=None, block=(0, 0)):
        with tempfile.TemporaryDirectory() as tmp:
            tmp = Path(tmp)
            name = f"model.layers.0.{tag}.weight"
            CDNAv3Writer(tmp).write_tensor(tensor, name, policy=policy)
            tdir = tmp / (name.replace("/", "_").replace(".", "_") + ".cdnav3")
            reader = CDNAv3Reader(tdir)
            w_ref = reader.reconstruct()
            b_t = None if bias is None else torch.from_numpy(bias)
            helix = load_helix_linear_from_cdnav3(tdir, bias=b_t)
            x_t = torch.from_numpy(x)
            y = helix(x_t).numpy()
            y_naive = helix._forward_naive(x_t).numpy()
            rec = {
                "weight": tensor.astype(np.float32),
                "codebook": helix.codebook.numpy(),
                "indices": helix.indices.numpy(),
                "x": x,
                "reconstruct": w_ref.astype(np.float32),
                "y_forward": y,
                "y_naive": y_naive,
                "meta_shape": np.asarray(reader.shape, dtype=np.int64),
            }
            r0, r1 = block
            if r1 > r0:
                rec["block_rows"] = np.asarray([r0, r1], dtype=np.int64)
                rec["reconstruct_block"] = reader.reconstruct_block(r0, r1).astype(np.float32)
                rec["dequant_tile"] = helix._dequant_tile(r0, r1).numpy()
            dw = helix.decode_weight().numpy()
            # decode_weight() adds deltas, reconstruct() overwrites values: they can
            # differ only at sidecar positions, so only those entries are kept.
            if helix.sidecar_positions is None:
                assert np.array_equal(dw, w_ref)
            else:
                p_ = helix.sidecar_positions.numpy()
                chk = dw.copy().ravel()
                chk[p_] = w_ref.ravel()[p_]
                assert np.array_equal(chk.reshape(w_ref.shape), w_ref)
                rec["decode_weight_at_sidecar"] = dw.ravel()[p_]
            if helix.sidecar_positions is not None:
                rec["sidecar_positions"] = helix.sidecar_positions.numpy()
                rec["sidecar_values"] = helix.sidecar_values.numpy()
                rec["sidecar_rows"] = helix._sidecar_rows.numpy()
                rec["sidecar_cols"] = helix._sidecar_cols.numpy()
                rec["sidecar_deltas"] = helix._sidecar_deltas.numpy()
            if bias is not None:
                rec["bias"] = bias
            ms = helix.memory_savings()
            rec["memory_savings"] = np.asarray(
                [ms["dense_bytes"], ms["compressed_bytes"]], dtype=np.int64)
            return rec

    # A. VQ only, the reference's own test tensor (tests/test_helix_linear.py:41-95)
    t = np.random.RandomState(42).randn(64, 32).astype(np.float32)
    pol = TensorPolicy(tensor_class=TensorClass.FFN, storage_mode="codebook", n_clusters=256,
                       sidecar_enabled=False, svd_residual_rank=0)
    x = np.random.RandomState(1).randn(2, 32).astype(np.float32)
    out["vq_only_64x32"] = cdna_case("vq_only", t, pol, x, block=(16, 48))

    # B. VQ + sidecar (tests/test_helix_linear.py:102-140)
    pol = TensorPolicy(tensor_class=TensorClass.ATTENTION_QK, storage_mode="codebook+sidecar",
                       n_clusters=256, sidecar_enabled=True, percentile=99.0, svd_residual_rank=0)
    x = np.random.RandomState(2).randn(4, 32).astype(np.float32)
    out["vq_sidecar_64x32"] = cdna_case("vq_sidecar", t, pol, x, block=(8, 40))

    # C. Student-t(5) at std 0.02 (the benchmark's distribution), two-sided 99.95 %
    #    uncapped sidecar, with bias; rows not a multiple of the 256-row tile.
    t = _student_t((300, 256), seed=0)
    pol = TensorPolicy(tensor_class=TensorClass.FFN, storage_mode="codebook+sidecar",
                       n_clusters=256, use_kmeans=True, sidecar_enabled=True,
                       percentile=99.95, max_corrections=0)
    x = np.random.RandomState(3).randn(3, 256).astype(np.float32)
    bias = np.random.RandomState(4).randn(300).astype(np.float32)
    out["student_t_300x256"] = cdna_case("student_t", t, pol, x, bias=bias, block=(250, 300))

    # D. capped sidecar (reference default policy: max_corrections=512)
    t = _student_t((48, 1024), seed=5)
    pol = TensorPolicy(tensor_class=TensorClass.FFN, storage_mode="codebook+sidecar",
                       n_clusters=256, use_kmeans=True, sidecar_enabled=True,
                       percentile=99.0, max_corrections=64)
    x = np.random.RandomState(6).randn(1, 1024).astype(np.float32)
    out["capped_sidecar_48x1024"] = cdna_case("capped", t, pol, x)

    # E. kernel-test restatement with OVERWRITE sidecar on odd shapes
    #    (tests/test_triton_vq_matmul.py:56-74, shape list :222)
    for (n, n_in, n_out) in [(7, 100, 50), (1, 33, 17), (13, 200, 99), (16, 256, 128)]:
        g = torch.Generator().manual_seed(1000 + n_in)
        cb = torch.randn(256, generator=g)
        idx = torch.randint(0, 256, (n_out, n_in), dtype=torch.uint8, generator=g)
        xx = torch.randn(n, n_in, generator=g)
        nnz = max(1, (n_out * n_in) // 50)
        pos = torch.randperm(n_out * n_in, generator=g)[:nnz].sort().values
        vals = torch.randn(nnz, generator=g)
        b = torch.randn(n_out, generator=g)
        y = _naive_vq_matmul(xx, cb, idx, pos, vals, bias=b.clone())
        out[f"naive_vq_{n}x{n_in}x{n_out}"] = {
            "codebook": cb.numpy(), "indices": idx.numpy(), "x": xx.numpy(),
            "sidecar_positions": pos.numpy(), "sidecar_values": vals.numpy(),
            "bias": b.numpy(), "y": y.numpy(),
        }

    # F. grouped affine corner (triton_affine_group_matmul.py:366-383), fp16 s/t
    g = torch.Generator().manual_seed(77)
    n_out, n_in, G, n = 96, 384, 128, 5
    idx = torch.randint(0, 256, (n_out, n_in), dtype=torch.uint8, generator=g)
    sc = (torch.rand(n_out, n_in // G, generator=g) * 1e-3 + 1e-4).half()
    of = (torch.randn(n_out, n_in // G, generator=g) * 0.05).half()
    xx = torch.randn(n, n_in, generator=g)
    b = torch.randn(n_out, generator=g)
    y = affine_group_matmul_reference(xx, idx, sc, of, G, bias=b)
    out["affine_group_96x384"] = {
        "indices": idx.numpy(), "scales": sc.numpy(), "offsets": of.numpy(), "x": xx.numpy(),
        "bias": b.numpy(), "group_size": np.asarray(G), "y": y.numpy(),
    }

    # G. int8 block-affine module (helix_affine_linear.py:30-139,146-200)
    w = torch.from_numpy(_student_t((64, 512), seed=8))
    idx, sc, bab, _ = quantize_linear_to_affine(w, 256)
    b = torch.from_numpy(np.random.RandomState(9).randn(64).astype(np.float32))
    mod = HelixAffineLinear(512, 64, idx, sc, bab, 256, bias=b)
    xx = torch.from_numpy(np.random.RandomState(10).randn(3, 512).astype(np.float32))
    out["block_affine_64x512"] = {
        "weight": w.numpy(), "indices": idx.numpy(), "scales": sc.numpy(),
        "biases_ab": bab.numpy(), "bias": b.numpy(), "x": xx.numpy(),
        "decode_weight": mod.decode_weight().numpy(), "y": mod(xx).numpy(),
    }

    # H. writer internals (hxq_encoder.py:107-177, hxq_writer_v3.py:446-467,
    #    generate_sidecars_v3.py:18-40)
    data = _student_t((20000,), seed=11)
    cents, assign = _simple_kmeans(data, 256, max_iters=10)
    wr = CDNAv3Writer(Path(tempfile.mkdtemp()))
    idx_full = wr._chunked_assign(data, cents.astype(np.float32))
    t2 = _student_t((40, 250), seed=12)
    pos, vals = find_outliers_percentile(t2, 99.0)
    out["writer_internals"] = {
        "data": data, "centroids": cents.astype(np.float32), "assignments": assign,
        "chunked_assign": idx_full, "outlier_tensor": t2, "outlier_positions": pos,
        "outlier_values": vals,
    }

    # I. per-tensor affine operator, CPU statement (triton_affine_matmul.py:170-187)
    from helix_substrate.triton_affine_matmul import affine_matmul_reference
    rs = np.random.RandomState(13)
    idx = torch.from_numpy(rs.randint(0, 256, size=(80, 592)).astype(np.uint8))
    xx = torch.from_numpy(rs.randn(3, 592).astype(np.float32))
    b = torch.from_numpy(rs.randn(80).astype(np.float32))
    step, offset = 0.00037, -0.047
    out["per_tensor_affine_80x592"] = {
        "indices": idx.numpy(), "x": xx.numpy(), "bias": b.numpy(), "step": np.asarray(step),
        "offset": np.asarray(offset), "y": affine_matmul_reference(xx, idx, step, offset, b).numpy(),
    }

    # J. The 4096 x 4096 single-linear benchmark configuration, exactly as stated: Student-t(5)
    #    seed 0 at std 0.02, reference writer (k-means k=256, two-sided 99.95 % uncapped sidecar,
    #    no affine), x[1, 4096] fp32 ~ N(0,1).  The 16 MB index matrix is not stored: its SHA-256,
    #    per-row sums of the reconstruction, a few full rows and the forward output pin it.
    if only is None or "config1_4096x4096" in only:
        import hashlib
        t = _student_t((4096, 4096), seed=0)
        pol = TensorPolicy(tensor_class=TensorClass.FFN, storage_mode="codebook+sidecar",
                           n_clusters=256, use_kmeans=True, sidecar_enabled=True,
                           percentile=99.95, max_corrections=0)
        x = np.random.default_rng(1).standard_normal((1, 4096)).astype(np.float32)
        full = cdna_case("config1", t, pol, x)
        rows = np.asarray([0, 1, 7, 255, 256, 1023, 2048, 4095], dtype=np.int64)
        out["config1_4096x4096"] = {
            "codebook": full["codebook"], "x": x, "y_forward": full["y_forward"], "y_naive": full["y_naive"],
            "indices_sha256": np.frombuffer(hashlib.sha256(np.ascontiguousarray(full["indices"]).tobytes()).digest(),
                                            dtype=np.uint8).copy(),
            "sidecar_positions": full["sidecar_positions"], "sidecar_values": full["sidecar_values"],
            "rows": rows, "reconstruct_rows": full["reconstruct"][rows],
            "reconstruct_row_sums_f64": full["reconstruct"].astype(np.float64).sum(1),
            "weight_sha256": np.frombuffer(hashlib.sha256(t.tobytes()).digest(), dtype=np.uint8).copy(),
            "memory_savings": full["memory_savings"],
        }

    for name, rec in out.items():
        if only is not None and name not in only:
            continue
        path = HERE / f"{name}.npz"
        np.savez_compressed(path, **rec)
        print(f"{name}: {path.stat().st_size / 1024:.1f} KiB")


if __name__ == "__main__":
    main()
