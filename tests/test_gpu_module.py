"""Module- and operator-level GPU tests, modelled on the reference's own
tests/test_helix_linear.py, tests/test_fused_parity.py and
tests/test_triton_vq_matmul.py (moved to CUDA: this build has no CPU path)."""

import numpy as np
import pytest
import torch
import torch.nn as nn

from conftest import load_golden, rel_l2
from oracle import hxq_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _module(g, **kw):
    from helix_substrate_b200 import HelixLinear
    t = lambda k: None if k not in g else torch.from_numpy(g[k])
    n_out, n_in = g["indices"].shape
    return HelixLinear(n_in, n_out, t("codebook"), t("indices"), t("sidecar_positions"), t("sidecar_values"),
                       bias=t("bias"), **kw)


@pytest.mark.parametrize("name", ["vq_only_64x32", "vq_sidecar_64x32", "student_t_300x256",
                                  "capped_sidecar_48x1024"])
def test_module_matches_reference(name):
    g = load_golden(name)
    mod = _module(g).to(DEV)
    x = torch.from_numpy(g["x"]).to(DEV)
    y = mod(x)
    assert y.shape == g["y_forward"].shape and y.dtype == torch.float32
    assert np.allclose(y.cpu().numpy(), g["y_forward"], atol=1e-4, rtol=1e-4)
    assert mod._last_dispatch_path == "fused"
    assert mod.dispatch_metadata()["kernel_metadata"]["dispatch_selected"].startswith("hxq_")
    # decode_weight()/_dequant_tile(0, rows) are the same call and equal reconstruct() bit for bit
    assert np.array_equal(mod.decode_weight().cpu().numpy(), g["reconstruct"])
    assert torch.equal(mod._dequant_tile(0, mod.out_features), mod.decode_weight())
    ms = mod.memory_savings()
    assert ms["dense_bytes"] == int(g["memory_savings"][0])
    if "sidecar_positions" in g:
        assert np.array_equal(mod._sidecar_rows.cpu().numpy(), g["sidecar_rows"])
        assert np.array_equal(mod._sidecar_cols.cpu().numpy(), g["sidecar_cols"])
        assert np.array_equal(mod._sidecar_deltas.cpu().numpy(), g["sidecar_deltas"])


def test_subtiles_concat_equals_full():
    g = load_golden("student_t_300x256")
    mod = _module(g).to(DEV)
    full = mod.decode_weight()
    parts = [mod._dequant_tile(a, min(a + 77, 300)) for a in range(0, 300, 77)]
    assert torch.equal(torch.cat(parts), full)


def test_input_ranks_and_dtypes():
    g = load_golden("student_t_300x256")
    mod = _module(g).to(DEV)
    x1 = torch.randn(256, device=DEV)
    x3 = torch.randn(2, 5, 256, device=DEV)
    assert mod(x1).shape == (300,)
    assert mod(x3).shape == (2, 5, 300)
    assert torch.allclose(mod(x3)[1, 2], mod(x3[1, 2]), atol=1e-5)
    for dt in (torch.float32, torch.float16, torch.bfloat16):
        y = mod(x3.to(dt))
        assert y.dtype == dt
    ref = mod(x3)
    assert rel_l2(mod(x3.bfloat16()).float().cpu().numpy(), ref.cpu().numpy()) < 2e-2


def test_cpu_input_raises_and_no_trainable_params():
    g = load_golden("vq_sidecar_64x32")
    mod = _module(g)
    with pytest.raises(RuntimeError, match="No silent fallback"):
        mod(torch.randn(2, 32))
    assert sum(p.numel() for p in mod.parameters() if p.requires_grad) == 0
    mod = mod.to(DEV)
    with pytest.raises(RuntimeError, match="No silent fallback"):
        mod(torch.randn(2, 32))


def test_half_cast_keeps_codebook_exact():
    g = load_golden("student_t_300x256")
    mod = _module(g).to(DEV).to(torch.bfloat16)
    assert mod.codebook.dtype == torch.float32
    assert np.array_equal(mod.decode_weight().cpu().numpy(), g["reconstruct"])


def test_state_dict_round_trip_through_shell():
    from helix_substrate_b200 import HelixLinear
    g = load_golden("student_t_300x256")
    mod = _module(g)
    shell = HelixLinear.from_quantized_config(256, 300, tensor_name="t")
    shell.load_state_dict(mod.state_dict())
    shell._recompute_derived()
    shell = shell.to(DEV)
    x = torch.from_numpy(g["x"]).to(DEV)
    assert torch.equal(shell(x), mod.to(DEV)(x))


def test_sidecar_policy_and_svd_and_channel_scales():
    from helix_substrate_b200 import HelixLinear
    g = load_golden("vq_sidecar_64x32")
    rng = np.random.default_rng(0)
    U = torch.from_numpy(rng.standard_normal((64, 4)).astype(np.float32))
    sv = torch.from_numpy(rng.random(4).astype(np.float32))
    Vt = torch.from_numpy(rng.standard_normal((4, 32)).astype(np.float32))
    cs = torch.from_numpy((0.5 + rng.random(32)).astype(np.float32))
    t = lambda k: torch.from_numpy(g[k])
    mod = HelixLinear(32, 64, t("codebook"), t("indices"), t("sidecar_positions"), t("sidecar_values"),
                      svd_U=U, svd_s=sv, svd_Vt=Vt, channel_scales=cs).to(DEV)
    x = torch.from_numpy(g["x"]).to(DEV)
    w = torch.from_numpy(g["reconstruct"]).to(DEV) + (U.to(DEV) * sv.to(DEV)) @ Vt.to(DEV)
    ref = (x / cs.to(DEV)) @ w.t()
    assert torch.allclose(mod(x), ref, atol=1e-4, rtol=1e-4)
    assert torch.allclose(mod.decode_weight(), w, atol=1e-6)
    mod.set_sidecar_policy("always_off")
    w0 = torch.from_numpy(O.reconstruct(g["codebook"], g["indices"])).to(DEV) + (U.to(DEV) * sv.to(DEV)) @ Vt.to(DEV)
    assert torch.allclose(mod(x), (x / cs.to(DEV)) @ w0.t(), atol=1e-4, rtol=1e-4)
    assert mod.get_sidecar_policy_stats()["skip_count"] == 1
    with pytest.raises(ValueError):
        mod.set_sidecar_policy("sometimes")


@pytest.mark.parametrize("xdt", [torch.bfloat16, torch.float16, torch.float32])
def test_buffered_mode_is_dequant_plus_dense_gemm(xdt):
    """_forward_mode = "buffered" (the reference's default mode, helix_linear.py:556-634): the weight
    materialised by hxq_dequant into the shared 16-bit buffer, then a dense matmul.  Against the fp64
    product of the bit-exact dequantised weight (16-bit operands: rel-L2 <= 1e-2), against the fused
    mode, with a group affine, a sidecar and a bias; the buffer is shared by modules of any size."""
    from helix_substrate_b200 import HelixLinear
    from helix_substrate_b200.hxq_writer_gpu import compress_weight, student_t_weight
    mods = []
    for i, (n_out, n_in) in enumerate([(384, 1024), (200, 512)]):
        enc = compress_weight(student_t_weight((n_out, n_in), 40 + i, DEV), percentile=99.9, group_size=128)
        mods.append(HelixLinear(n_in, n_out, bias=torch.randn(n_out, device=DEV) * 0.02, **enc).to(DEV))
    for mod in mods:
        x = torch.randn(3, 50, mod.in_features, device=DEV).to(xdt)
        ref = x.double() @ mod.decode_weight().double().t() + mod.bias.double()
        y_fused = mod(x)
        mod._forward_mode = "buffered"
        y = mod(x)
        assert mod._last_dispatch_path == "buffered" and mod.dispatch_metadata()["dispatch_path"] == "buffered"
        assert y.shape == (3, 50, mod.out_features) and y.dtype == xdt
        assert rel_l2(y.double().cpu().numpy(), ref.cpu().numpy()) < 1e-2
        assert rel_l2(y.double().cpu().numpy(), y_fused.double().cpu().numpy()) < 1.5e-2
        assert torch.equal(y, mod(x))
        mod._forward_mode = "fused"
        assert torch.equal(mod(x), y_fused)
    assert HelixLinear._shared_buffer_size >= 384 * 1024


def test_swap_to_helix_and_summary(tmp_path):
    from helix_substrate_b200 import swap_to_helix, swap_summary, HelixLinear
    g = load_golden("vq_sidecar_64x32")
    model = nn.Sequential()
    model.add_module("proj", nn.Linear(32, 64, bias=False))
    model.add_module("other", nn.Linear(64, 8))
    swap_to_helix(model, {"proj": _module(g)})
    assert isinstance(model.proj, HelixLinear) and isinstance(model.other, nn.Linear)
    s = swap_summary(model)
    assert s["helix_modules"] == 1 and s["linear_modules"] == 1
    model = model.to(DEV)
    y = model(torch.from_numpy(g["x"]).to(DEV))
    assert y.shape == (4, 8)


# --------------------------------------------------------------------------- operators

@pytest.mark.parametrize("N", [1, 4, 7, 13, 16, 32, 512])
def test_fused_vq_matmul_matches_dense(N):
    from helix_substrate_b200.triton_vq_matmul import fused_vq_matmul
    torch.manual_seed(42)
    IN, OUT = 256, 128
    cb = torch.randn(256, device=DEV)
    idx = torch.randint(0, 256, (OUT, IN), dtype=torch.uint8, device=DEV)
    x = torch.randn(N, IN, device=DEV)
    pos = torch.sort(torch.randperm(OUT * IN, device=DEV)[:200]).values
    vals = torch.randn(200, device=DEV)
    bias = torch.randn(OUT, device=DEV)
    w = cb[idx.long()].reshape(-1).clone()
    w[pos] = vals
    ref = x.double() @ w.reshape(OUT, IN).double().t() + bias.double()
    rows, cols = pos // IN, pos % IN
    deltas = vals - cb[idx.reshape(-1)[pos].long()]
    log = {}
    for kw in (dict(sidecar_rows=rows, sidecar_cols=cols, sidecar_deltas=deltas),
               dict(sidecar_positions=pos, sidecar_values=vals)):
        y = fused_vq_matmul(x, cb, idx, bias=bias, _dispatch_log=log, **kw)
        assert y.dtype == torch.float32 and y.shape == (N, OUT)
        tol = 1e-3 if N <= 16 else 1e-2
        assert rel_l2(y.cpu().numpy(), ref.cpu().numpy()) < tol
    for dt in (torch.float16, torch.bfloat16):
        assert fused_vq_matmul(x.to(dt), cb, idx).dtype == torch.float32  # always fp32 out
    with pytest.raises(AssertionError):
        fused_vq_matmul(x.cpu(), cb, idx)


def test_affine_group_operator_vs_reference():
    from helix_substrate_b200.triton_affine_group_matmul import (
        fused_affine_group_matmul, affine_group_matmul_reference)
    g = load_golden("affine_group_96x384")
    G = int(g["group_size"])
    a = [torch.from_numpy(g[k]).to(DEV) for k in ("x", "indices", "scales", "offsets")]
    bias = torch.from_numpy(g["bias"]).to(DEV)
    y = fused_affine_group_matmul(*a, group_size=G, bias=bias)
    assert y.dtype == torch.float32
    assert np.allclose(y.cpu().numpy(), g["y"], atol=2e-4, rtol=1e-4)
    y1 = fused_affine_group_matmul(a[0][:1], *a[1:], group_size=G, bias=bias)
    assert np.allclose(y1.cpu().numpy(), g["y"][:1], atol=2e-4, rtol=1e-4)
    y2 = affine_group_matmul_reference(*a, group_size=G, bias=bias)
    assert np.allclose(y2.cpu().numpy(), g["y"], atol=2e-4, rtol=1e-4)


def test_block_affine_module_vs_reference():
    from helix_substrate_b200 import HelixAffineLinear, quantize_linear_to_affine
    g = load_golden("block_affine_64x512")
    t = lambda k: torch.from_numpy(g[k])
    mod = HelixAffineLinear(512, 64, t("indices"), t("scales"), t("biases_ab"), 256, bias=t("bias")).to(DEV)
    assert np.array_equal(mod.decode_weight().cpu().numpy(), g["decode_weight"])
    y = mod(t("x").to(DEV))
    assert np.allclose(y.cpu().numpy(), g["y"], atol=1e-4, rtol=1e-4)
    idx, sc, bab, stats = quantize_linear_to_affine(t("weight").to(DEV), 256)
    assert torch.equal(idx.cpu(), t("indices")) and torch.equal(sc.cpu(), t("scales"))
    assert torch.equal(bab.cpu(), t("biases_ab")) and stats["cosine"] > 0.999


@pytest.mark.parametrize("n_out,n_in,M", [(264, 1024, 1), (96, 592, 4), (128, 2048, 40)])
def test_per_tensor_affine_operator(n_out, n_in, M):
    """fused_affine_matmul (reference: helix_substrate/triton_affine_matmul.py:110-167): the byte ramp
    k * step + offset as the codebook of the ordinary kernels."""
    from helix_substrate_b200.triton_affine_matmul import fused_affine_matmul, affine_matmul_reference
    gen = torch.Generator(device=DEV).manual_seed(n_in + M)
    idx = torch.randint(0, 256, (n_out, n_in), dtype=torch.uint8, device=DEV, generator=gen)
    x = torch.randn(M, n_in, device=DEV, generator=gen)
    bias = torch.randn(n_out, device=DEV, generator=gen)
    step, offset = 0.00037, -0.047
    y = fused_affine_matmul(x, idx, step, offset, bias)
    assert y.dtype == torch.float32 and y.shape == (M, n_out)
    ref = x.double() @ (idx.double() * step + offset).t() + bias.double()
    tol = 1e-3 if M <= 16 else 1e-2          # fp32 decode kernels / bf16 tensor-core kernel
    assert rel_l2(y.double().cpu().numpy(), ref.cpu().numpy()) < tol
    assert rel_l2(affine_matmul_reference(x, idx, step, offset, bias).double().cpu().numpy(), ref.cpu().numpy()) < 1e-4


@pytest.mark.parametrize("M", [1, 3, 16, 20])
@pytest.mark.parametrize("shape", [(72, 512, 128), (40, 3584, 128), (9, 208, 16)])
def test_six_bit_packed_affine_group_operator(M, shape):
    """fused_affine_group_matmul_packed6 (reference: N = 1 only): up to 16 tokens the 3-byte groups
    are unpacked inside the kernel, beyond that the unpacked product runs; both against fp64."""
    from helix_substrate_b200.triton_affine_group_matmul import (
        fused_affine_group_matmul, fused_affine_group_matmul_packed6, pack6)
    n_out, n_in, G = shape
    gen = torch.Generator(device=DEV).manual_seed(M)
    idx = torch.randint(0, 64, (n_out, n_in), dtype=torch.uint8, device=DEV, generator=gen)
    s = (0.01 + 0.001 * torch.rand(n_out, n_in // G, device=DEV, generator=gen)).half()
    t = (0.02 * torch.randn(n_out, n_in // G, device=DEV, generator=gen)).half()
    b = torch.randn(n_out, device=DEV, generator=gen)
    w = idx.double() * s.double().repeat_interleave(G, 1) + t.double().repeat_interleave(G, 1)
    for xdt in (torch.float32, torch.bfloat16):
        x = torch.randn(M, n_in, device=DEV, generator=gen).to(xdt)
        y = fused_affine_group_matmul_packed6(x, pack6(idx), s, t, n_out, n_in, G, bias=b)
        assert y.dtype == torch.float32 and y.shape == (M, n_out)
        ref = x.double() @ w.t() + b.double()
        tol = 1e-3 if M <= 16 else 1e-2
        assert rel_l2(y.double().cpu().numpy(), ref.cpu().numpy()) < tol
        y8 = fused_affine_group_matmul(x, idx, s, t, G, bias=b)          # one byte per index, codebook kernels
        # that product runs fp32-accumulate for fp32 activations up to 16 tokens, bf16 tensor-core operands otherwise
        exact = M <= (16 if xdt == torch.float32 else 4)
        assert rel_l2(y.double().cpu().numpy(), y8.double().cpu().numpy()) < (1e-5 if exact else 1e-2)
        assert torch.equal(y, fused_affine_group_matmul_packed6(x, pack6(idx), s, t, n_out, n_in, G, bias=b))


def test_per_tensor_affine_operator_vs_reference_golden():
    from helix_substrate_b200.triton_affine_matmul import fused_affine_matmul
    g = load_golden("per_tensor_affine_80x592")
    t = lambda a: torch.from_numpy(a).to(DEV)
    y = fused_affine_matmul(t(g["x"]), t(g["indices"]), float(g["step"]), float(g["offset"]), t(g["bias"]))
    assert rel_l2(y.cpu().numpy(), g["y"]) < 1e-3



def test_hf_from_pretrained_model_runs_on_the_kernels(tmp_path):
    """The load path a user of the reference takes: compress a (tiny) Qwen2, write ONE
    safetensors checkpoint with its quantization_config, ``import helix_substrate``,
    ``AutoModelForCausalLM.from_pretrained(dir).cuda()`` - and run it.  The loaded model's
    logits must equal those of the model the checkpoint was written from (same kernels, same
    buffers) and agree to bf16 precision with a dense model rebuilt from ``decode_weight()``."""
    transformers = pytest.importorskip("transformers")
    import torch.nn as nn
    import helix_substrate  # noqa: F401  registers the quantizer under the reference's names
    from helix_substrate_b200 import HelixLinear, hxq_writer_gpu as W, swap_to_helix
    from helix_substrate_b200.convert_safetensors import save_hxq_checkpoint
    cfg = transformers.Qwen2Config(vocab_size=256, hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
                                   num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=128,
                                   rope_theta=1e6, tie_word_embeddings=False)
    torch.manual_seed(0)
    model = transformers.Qwen2ForCausalLM(cfg).eval()
    dense = transformers.Qwen2ForCausalLM(cfg).eval()
    dense.load_state_dict(model.state_dict())
    facs = {}
    for name, m in model.named_modules():
        if isinstance(m, nn.Linear) and name != "lm_head":
            enc = W.compress_weight(m.weight.data.to(DEV), percentile=99.5, group_size=128)
            facs[name] = HelixLinear(m.in_features, m.out_features, tensor_name=name + ".weight",
                                     bias=None if m.bias is None else m.bias.data.clone().to(DEV), **enc)
    swap_to_helix(model, facs)
    out = save_hxq_checkpoint(model, tmp_path / "ckpt")
    model = model.to(DEV)
    loaded = transformers.AutoModelForCausalLM.from_pretrained(out).to(DEV).eval()
    n_helix = sum(isinstance(m, HelixLinear) for m in loaded.modules())
    assert n_helix == 14 and isinstance(loaded.lm_head, nn.Linear)
    # the dense twin carries exactly the dequantised weights
    with torch.no_grad():
        for name, m in dense.named_modules():
            if name in facs:
                m.weight.copy_(facs[name].decode_weight().cpu())
    dense = dense.to(DEV)
    for T in (1, 9, 40):    # decode-sized, GEMV-sized and tensor-core-sized token counts
        ids = torch.randint(0, 256, (1, T), device=DEV, generator=torch.Generator(device=DEV).manual_seed(T))
        with torch.no_grad():
            y_loaded = loaded(ids).logits
            y_src = model(ids).logits
            y_dense = dense(ids).logits
        assert torch.equal(y_loaded, y_src), "the reloaded model must be the model that was saved"
        tol = 1e-3 if T <= 16 else 1e-2     # fp32-accumulate kernels / bf16 tensor-core operands
        assert rel_l2(y_loaded.float().cpu().numpy(), y_dense.float().cpu().numpy()) < tol, T
    assert all(m._last_dispatch is not None for m in loaded.modules() if isinstance(m, HelixLinear))
