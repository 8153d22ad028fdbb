"""Host-side logic that needs no GPU: file formats, module plumbing, sharding
arithmetic, the HuggingFace registration and checkpoint round trip."""

import json

import numpy as np
import pytest
import torch
import torch.nn as nn

from conftest import load_golden
from oracle import hxq_oracle as O


def _pol(**kw):
    from helix_substrate_b200.tensor_policy import TensorPolicy, TensorClass
    base = dict(tensor_class=TensorClass.FFN, storage_mode="codebook+sidecar", n_clusters=256, percentile=99.95,
                use_kmeans=True, sidecar_enabled=True, block_rows=16, max_corrections=0)
    base.update(kw)
    return TensorPolicy(**base)


def test_drop_in_package_names():
    import helix_substrate
    from helix_substrate.cdnav3_reader import CDNAv3Reader
    from helix_substrate.hxq_reader_v3 import CDNAv3Reader as R2
    from helix_substrate.cdnav3_writer import CDNAv3Writer
    from helix_substrate.hxq_writer_v3 import CDNAv3Writer as W2
    from helix_substrate.helix_linear import HelixLinear, load_cdna_factors, swap_to_helix  # noqa: F401
    from helix_substrate.triton_vq_matmul import fused_vq_matmul, get_kernel_metadata  # noqa: F401
    from helix_substrate.triton_affine_group_matmul import fused_affine_group_matmul  # noqa: F401
    from helix_substrate.triton_affine_matmul import fused_affine_matmul, affine_matmul_reference  # noqa: F401
    from helix_substrate.hf_integration import HelixQuantizationConfig
    assert R2 is CDNAv3Reader and W2 is CDNAv3Writer
    assert helix_substrate.HelixLinear is HelixLinear
    assert HelixQuantizationConfig(codebook_size=256).n_clusters == 256
    assert get_kernel_metadata()["kernel_impl"] == "libhxq_b200"


def test_writer_reproduces_reference_files(tmp_path):
    """Host encoder = the reference's algorithm: codebook, indices and sidecar
    recorded from the reference writer come out bit for bit."""
    from helix_substrate_b200.cdnav3_writer import CDNAv3Writer
    from helix_substrate_b200.helix_linear import load_helix_linear_from_cdnav3, load_cdna_factors
    g = load_golden("student_t_300x256")
    name = "model.layers.0.mlp.down_proj.weight"
    stats = CDNAv3Writer(tmp_path).write_tensor(g["weight"], name, _pol())
    td = tmp_path / "model_layers_0_mlp_down_proj_weight.cdnav3"
    assert sorted(p.name for p in td.iterdir()) == ["codebook.npy", "indices.bin", "meta.json", "sidecar.npz",
                                                    "stats.json"]
    meta = json.loads((td / "meta.json").read_text())
    assert meta["format_version"] == "cdna_v3" and meta["shape"] == [300, 256] and meta["index_dtype"] == "uint8"
    assert stats["num_outliers"] == len(g["sidecar_positions"])
    mod = load_helix_linear_from_cdnav3(td)
    assert np.array_equal(mod.codebook.numpy()[:256], g["codebook"])
    assert np.array_equal(mod.indices.numpy(), g["indices"])
    assert np.array_equal(mod.sidecar_positions.numpy(), g["sidecar_positions"])
    assert np.array_equal(mod.sidecar_values.numpy(), g["sidecar_values"])
    assert np.array_equal(mod._sidecar_deltas.numpy(), g["sidecar_deltas"])
    CDNAv3Writer(tmp_path).write_tensor(np.ones(300, np.float32), "model.layers.0.mlp.down_proj.bias")
    CDNAv3Writer(tmp_path).write_tensor(np.ones(8, np.float32), "model.norm.weight")
    facs = load_cdna_factors(tmp_path)
    assert list(facs) == ["model.layers.0.mlp.down_proj"] and facs["model.layers.0.mlp.down_proj"].bias is not None
    from helix_substrate_b200.cdnav3_reader import CDNAv3Reader
    r = CDNAv3Reader(td)
    assert r.verify_codebook() and r.shape == (300, 256) and r.has_sidecar


def test_writer_capped_sidecar_and_group_affine(tmp_path):
    from helix_substrate_b200.cdnav3_writer import CDNAv3Writer
    from helix_substrate_b200.helix_linear import load_helix_linear_from_cdnav3
    g = load_golden("capped_sidecar_48x1024")
    CDNAv3Writer(tmp_path).write_tensor(g["weight"], "blk.3.ffn_up.weight", _pol(percentile=99.0, max_corrections=64))
    mod = load_helix_linear_from_cdnav3(tmp_path / "blk_3_ffn_up_weight.cdnav3")
    assert np.array_equal(mod.sidecar_positions.numpy(), g["sidecar_positions"])
    assert np.array_equal(mod.indices.numpy(), g["indices"])
    CDNAv3Writer(tmp_path).write_tensor(g["weight"], "blk.4.ffn_up.weight", _pol(group_size=128))
    mod = load_helix_linear_from_cdnav3(tmp_path / "blk_4_ffn_up_weight.cdnav3")
    assert mod.group_size == 128 and mod.group_scales.shape == (48, 8)
    s, t = O.fit_group_affine(g["weight"], mod.codebook.numpy(), mod.indices.numpy(), 128,
                              mod.sidecar_positions.numpy())
    assert np.allclose(mod.group_scales.numpy(), s, rtol=1e-5) and np.allclose(mod.group_offsets.numpy(), t, atol=1e-7)
    rows, cols, deltas = O.derive_sidecar(mod.codebook.numpy(), mod.indices.numpy(), mod.sidecar_positions.numpy(),
                                          mod.sidecar_values.numpy(), mod.group_scales.numpy(),
                                          mod.group_offsets.numpy(), 128)
    assert np.array_equal(mod._sidecar_deltas.numpy(), deltas)
    assert np.array_equal(mod._csr_rowptr.numpy(), O.csr_from_rows(rows, 48))


def test_tensor_names_and_policy():
    from helix_substrate_b200.helix_linear import _tensor_name_to_module_path as f
    from helix_substrate_b200.tensor_policy import classify_tensor, TensorClass, get_policy
    assert f("model.layers.0.self_attn.q_proj.weight") == "model.layers.0.self_attn.q_proj"
    assert f("blk.7.attn_output.weight") == "model.layers.7.self_attn.o_proj"
    assert f("blk.2.ffn_down.weight") == "model.layers.2.mlp.down_proj"
    assert f("output.weight") == "lm_head" and f("token_embd.weight") == "model.embed_tokens"
    assert classify_tensor("model.layers.1.mlp.gate_proj.weight") == TensorClass.FFN
    assert classify_tensor("model.layers.1.self_attn.k_proj.weight") == TensorClass.ATTENTION_QK
    assert classify_tensor("model.norm.weight", (8,)) == TensorClass.NORM
    assert get_policy("lm_head.weight").max_corrections == 512


def test_gpu_writer_logic_matches_reference_rules_on_cpu():
    from helix_substrate_b200 import hxq_writer_gpu as W
    w = W.student_t_weight((64, 512), 3, "cpu")
    assert abs(float(w.std()) - 0.02) < 1e-6
    enc = W.compress_weight(w, percentile=99.9, group_size=128)
    cb = enc["codebook"].numpy()
    assert np.all(np.diff(cb) >= 0)
    assert np.array_equal(enc["indices"].numpy().ravel(), O.chunked_assign(w.numpy().ravel(), cb))
    pos, vals = O.find_outliers_percentile(w.numpy(), 99.9)
    assert np.array_equal(enc["sidecar_positions"].numpy(), pos)
    assert np.array_equal(enc["sidecar_values"].numpy(), O.sidecar_fp16_roundtrip(vals))
    s, t = O.fit_group_affine(w.numpy(), cb, enc["indices"].numpy(), 128, pos)
    assert np.allclose(enc["group_scales"].numpy(), s, rtol=1e-4, atol=1e-6)
    wh = O.reconstruct(cb, enc["indices"].numpy(), pos, enc["sidecar_values"].numpy(), s, t, 128)
    assert np.linalg.norm(wh - w.numpy()) / np.linalg.norm(w.numpy()) < 0.05


@pytest.mark.parametrize("world", [2, 4, 8])
def test_tp_shards_recompose(world):
    """Column shards concatenate and row shards sum to the unsharded product
    (oracle arithmetic on each shard's own buffers), including shards that
    start mid-group (3584 / 8 = 448 = 3.5 groups of 128)."""
    from helix_substrate_b200 import HelixLinear, hxq_writer_gpu as W
    from helix_substrate_b200.tp import shard_helix_linear
    w = W.student_t_weight((40, 3584), 0, "cpu")
    mod = HelixLinear(3584, 40, bias=torch.randn(40), **W.compress_weight(w, group_size=128, percentile=99.5))
    x = np.random.default_rng(0).standard_normal((2, 3584)).astype(np.float32)

    def fwd(m, xx):
        r = None if m._sidecar_rows is None else m._sidecar_rows.numpy()
        return O.forward_f64(xx, m.codebook.numpy(), m.indices.numpy(), r,
                             None if r is None else m._sidecar_cols.numpy(),
                             None if r is None else m._sidecar_deltas.numpy(),
                             None if m.bias is None else m.bias.numpy(), m.group_scales.numpy(),
                             m.group_offsets.numpy(), 128, m.col0 % 128)
    full = fwd(mod, x)
    tot, nnz = 0, 0
    for r in range(world):
        sh = shard_helix_linear(mod, "row", r, world)
        c0, c1 = sh.tp_slice
        assert sh.col0 == c0 and c0 % 16 == 0
        tot = tot + fwd(sh, x[:, c0:c1])
        nnz += 0 if sh.sidecar_positions is None else sh.sidecar_positions.numel()
    assert nnz == mod.sidecar_positions.numel()
    assert np.abs(tot - full).max() < 1e-9
    cat = np.concatenate([fwd(shard_helix_linear(mod, "column", r, world), x) for r in range(world)], 1)
    assert np.abs(cat - full).max() < 1e-9


def test_hf_round_trip_builds_shells_and_keeps_rope(tmp_path):
    """compress -> one safetensors + quantization_config -> from_pretrained:
    the listed linears come back as HelixLinear with identical buffers, dense
    tensors are untouched and rotary inv_freq keeps the config's theta."""
    transformers = pytest.importorskip("transformers")
    import helix_substrate  # noqa: F401  registers the quantizer
    from helix_substrate_b200 import HelixLinear, hxq_writer_gpu as W, swap_to_helix
    from helix_substrate_b200.convert_safetensors import save_hxq_checkpoint
    cfg = transformers.Qwen2Config(vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                                   num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=64,
                                   rope_theta=1e6, tie_word_embeddings=False)
    torch.manual_seed(0)
    model = transformers.Qwen2ForCausalLM(cfg).eval()
    inv_ref = model.model.rotary_emb.inv_freq.clone()
    facs = {}
    for name, m in model.named_modules():
        if isinstance(m, nn.Linear) and name != "lm_head":
            enc = W.compress_weight(m.weight.data, percentile=99.0, group_size=64 if "mlp" in name else 0)
            facs[name] = HelixLinear(m.in_features, m.out_features, tensor_name=name + ".weight",
                                     bias=None if m.bias is None else m.bias.data.clone(), **enc)
    swap_to_helix(model, facs)
    out = save_hxq_checkpoint(model, tmp_path / "ckpt")
    qc = json.loads((out / "config.json").read_text())["quantization_config"]
    assert qc["quant_method"] == "hxq" and len(qc["compressed_modules"]) == 14
    loaded = transformers.AutoModelForCausalLM.from_pretrained(out)
    n = 0
    for name, m in loaded.named_modules():
        if isinstance(m, HelixLinear):
            src = facs[name]
            n += 1
            for b in ("codebook", "indices", "sidecar_positions", "sidecar_values", "bias", "group_scales",
                      "group_offsets", "_sidecar_deltas", "_csr_rowptr"):
                a, c = getattr(m, b), getattr(src, b)
                assert (a is None) == (c is None), (name, b)
                assert a is None or torch.equal(a, c), (name, b)
            assert m.group_size == src.group_size
    assert n == 14 and isinstance(loaded.lm_head, nn.Linear)
    assert torch.equal(loaded.model.embed_tokens.weight, model.model.embed_tokens.weight)
    assert torch.allclose(loaded.model.rotary_emb.inv_freq, inv_ref)


def test_cdnav3_directory_to_hf_checkpoint_with_completeness_gate(tmp_path):
    """dense model on disk -> CDNAv3Writer folders -> convert_model -> from_pretrained: the compressed
    linears come back as HelixLinear holding exactly what the folders hold (codebook, indices,
    sidecar, group affine), everything the writer skipped is copied from the dense checkpoint in
    its own dtype, and a dense tensor that is neither copied nor replaced stops the conversion."""
    transformers = pytest.importorskip("transformers")
    from safetensors.torch import load_file, save_file
    import helix_substrate  # noqa: F401  registers the quantizer
    from helix_substrate_b200 import HelixLinear
    from helix_substrate_b200.cdnav3_writer import CDNAv3Writer
    from helix_substrate_b200.cdnav3_reader import CDNAv3Reader
    from helix_substrate_b200.convert_safetensors import convert_cdnav3_to_safetensors, convert_model
    from helix_substrate_b200.tensor_policy import TensorClass, TensorPolicy
    cfg = transformers.Qwen2Config(vocab_size=96, hidden_size=64, intermediate_size=128, num_hidden_layers=1,
                                   num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=32,
                                   rope_theta=1e6, tie_word_embeddings=False)
    torch.manual_seed(1)
    dense = transformers.Qwen2ForCausalLM(cfg).eval()
    dense_dir = tmp_path / "dense"
    dense.save_pretrained(dense_dir, safe_serialization=True)
    w = CDNAv3Writer(tmp_path / "cdnav3")
    pol = TensorPolicy(TensorClass.FFN, "codebook+sidecar", percentile=99.0, max_corrections=0, group_size=64)
    pol_plain = TensorPolicy(TensorClass.ATTENTION_QK, "codebook+sidecar", percentile=99.0, max_corrections=0)
    names = []
    for name, m in dense.named_modules():
        if isinstance(m, nn.Linear) and name != "lm_head":
            w.write_tensor(m.weight.detach().numpy(), name + ".weight", pol if "mlp" in name else pol_plain)
            names.append(name)
    w.write_tensor(dense.model.norm.weight.detach().numpy(), "model.norm.weight")      # an exact 1-D tensor
    stats = convert_model(tmp_path / "cdnav3", dense_dir, tmp_path / "hf")
    assert stats["n_compressed"] == len(names) == 7 and stats["n_exact"] == 1 and stats["group_size"] == 64
    assert sorted(stats["compressed_modules"]) == sorted(names)
    ck = load_file(str(tmp_path / "hf" / "model.safetensors"))
    sd = dense.state_dict()
    for k, v in sd.items():        # every dense tensor: itself, or replaced by its parts
        if k[:-len(".weight")] in names and k.endswith(".weight"):
            assert k not in ck and k[:-7] + ".codebook" in ck and ck[k[:-7] + ".indices"].shape == v.shape
        elif k != "model.norm.weight":
            assert torch.equal(ck[k], v), k
    assert ck["model.norm.weight"].dtype == torch.float16          # the writer's exact tensors are fp16
    qc = json.loads((tmp_path / "hf" / "config.json").read_text())["quantization_config"]
    assert qc["quant_method"] == "cdna_v3" and qc["group_size"] == 64 and sorted(qc["compressed_modules"]) == sorted(names)
    assert json.loads((tmp_path / "hf" / "conversion_receipt.json").read_text())["n_total_keys"] == len(ck)
    loaded = transformers.AutoModelForCausalLM.from_pretrained(tmp_path / "hf")
    n = 0
    for name, m in loaded.named_modules():
        if isinstance(m, HelixLinear):
            n += 1
            d = tmp_path / "cdnav3" / (name.replace(".", "_") + "_weight.cdnav3")
            assert torch.equal(m.codebook[: 256], torch.from_numpy(np.load(d / "codebook.npy")))
            assert np.array_equal(m.indices.numpy().ravel(), np.fromfile(d / "indices.bin", dtype=np.uint8))
            assert (m.group_size == 64) == ("mlp" in name)
            if "mlp" in name:
                assert torch.equal(m.group_scales, torch.from_numpy(np.load(d / "group_scales.npy")))
    assert n == 7 and isinstance(loaded.lm_head, nn.Linear)
    assert torch.equal(loaded.model.embed_tokens.weight, dense.model.embed_tokens.weight)
    # the gate: a folder that claims gate_proj but holds a matrix of another shape (a stale folder from
    # another model) and an exact tensor of the wrong size both stop the conversion
    import shutil
    stale = tmp_path / "cdnav3_stale"
    shutil.copytree(tmp_path / "cdnav3", stale)
    shutil.rmtree(stale / "model_layers_0_mlp_gate_proj_weight.cdnav3")
    CDNAv3Writer(stale).write_tensor(np.random.default_rng(0).standard_normal((64, 32)).astype(np.float32),
                                     "model.layers.0.mlp.gate_proj.weight", pol_plain)
    with pytest.raises(RuntimeError, match="completeness gate"):
        convert_cdnav3_to_safetensors(stale, tmp_path / "x.safetensors", dense_dir)
    wrong = tmp_path / "cdnav3_wrong"
    shutil.copytree(tmp_path / "cdnav3", wrong)
    CDNAv3Writer(wrong).write_tensor(np.ones(7, np.float32), "model.norm.weight")
    with pytest.raises(RuntimeError, match="completeness gate"):
        convert_cdnav3_to_safetensors(wrong, tmp_path / "y.safetensors", dense_dir)
    # without a dense checkpoint to compare with, the folders alone convert
    alone = convert_cdnav3_to_safetensors(tmp_path / "cdnav3", tmp_path / "z.safetensors")
    assert alone["n_from_original"] == 0 and alone["n_total_keys"] < len(ck)


def test_per_tensor_affine_reference_formula_on_cpu():
    """affine_matmul_reference (any device) is the dense product with W = idx * step + offset."""
    import numpy as np
    import torch
    from helix_substrate.triton_affine_matmul import affine_matmul_reference, fused_affine_matmul
    rng = np.random.default_rng(5)
    idx = torch.from_numpy(rng.integers(0, 256, (24, 80), dtype=np.uint8))
    x = torch.from_numpy(rng.standard_normal((3, 80)).astype(np.float32))
    b = torch.from_numpy(rng.standard_normal(24).astype(np.float32))
    y = affine_matmul_reference(x, idx, 0.0125, -1.5, b)
    w = idx.double() * 0.0125 - 1.5
    ref = x.double() @ w.t() + b.double()
    assert torch.allclose(y.double(), ref, rtol=1e-4, atol=1e-4)
    import pytest
    with pytest.raises(AssertionError):      # the fused operator is CUDA only, like the reference's
        fused_affine_matmul(x, idx, 0.0125, -1.5)


def test_six_bit_packing_round_trip_and_bit_layout():
    """unpack6 follows the reference kernel's formulas (v0 = b0 & 63, v1 = (b0 >> 6 | b1 << 2) & 63,
    v2 = (b1 >> 4 | b2 << 4) & 63, v3 = b2 >> 2)."""
    import numpy as np
    import torch
    from helix_substrate.triton_affine_group_matmul import pack6, unpack6
    rng = np.random.default_rng(9)
    idx = torch.from_numpy(rng.integers(0, 64, (7, 24), dtype=np.uint8))
    packed = pack6(idx)
    assert packed.dtype == torch.uint8 and packed.numel() == 7 * 24 * 3 // 4
    assert torch.equal(unpack6(packed, 7, 24), idx)
    b = packed.reshape(7, 6, 3).numpy().astype(np.int64)
    b0, b1, b2 = b[..., 0], b[..., 1], b[..., 2]
    ref = np.stack([b0 & 63, ((b0 >> 6) | (b1 << 2)) & 63, ((b1 >> 4) | (b2 << 4)) & 63, (b2 >> 2) & 63], -1)
    assert np.array_equal(ref.reshape(7, 24), idx.numpy())

