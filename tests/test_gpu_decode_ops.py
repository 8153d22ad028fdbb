"""Decode-step glue (residual add + RMSNorm, RoPE + KV append, single-query attention,
SwiGLU) against the same operators written in plain torch ops, and the fused one-token
step of the Qwen2-shape decoder against its torch-op step."""

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from conftest import rel_l2

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda:0")


@pytest.mark.parametrize("B,H,with_delta", [(1, 3584, True), (4, 256, True), (2, 5120, False), (3, 1000, True), (2, 1001, True), (1, 11000, True)])
def test_add_rmsnorm(B, H, with_delta):
    from helix_substrate_b200 import decode_ops
    g = torch.Generator(device=_dev()).manual_seed(B * 1000 + H)
    h = torch.randn(B, H, device=_dev(), generator=g).bfloat16()
    d = (torch.randn(B, H, device=_dev(), generator=g) * 0.5).bfloat16() if with_delta else None
    w = (1 + 0.1 * torch.randn(H, device=_dev(), generator=g)).bfloat16()
    h_ref = h + d if with_delta else h.clone()
    xf = h_ref.float()
    ref = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6)).to(torch.bfloat16) * w
    out = torch.empty_like(h)
    decode_ops.add_rmsnorm(h, d, w, 1e-6, out)
    assert torch.equal(h, h_ref), "residual stream must be updated in place with a bf16 add"
    assert rel_l2(out.float().cpu(), ref.float().cpu()) < 4e-3   # one bf16 ulp here and there (rsqrt, summation order)


def _rope_ref(x, cos, sin):
    x1, x2 = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
    return (x.float() * cos + torch.cat([-x2, x1], -1).float() * sin).to(x.dtype)


@pytest.mark.parametrize("B,nq,nkv,D,pos", [(1, 28, 4, 128, 0), (2, 4, 2, 64, 37), (3, 8, 8, 128, 199)])
def test_rope_append(B, nq, nkv, D, pos):
    from helix_substrate_b200 import decode_ops
    dev, max_len = _dev(), 200
    g = torch.Generator(device=dev).manual_seed(pos + D)
    qkv = torch.randn(B, (nq + 2 * nkv) * D, device=dev, generator=g).bfloat16()
    inv = 1.0 / (1e6 ** (torch.arange(0, D, 2, device=dev, dtype=torch.float32) / D))
    ang = torch.arange(max_len, device=dev, dtype=torch.float32)[:, None] * inv[None, :]
    cos, sin = torch.cat([ang.cos(), ang.cos()], -1).contiguous(), torch.cat([ang.sin(), ang.sin()], -1).contiguous()
    kc = torch.zeros(B, nkv, max_len, D, device=dev, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    q_out = torch.empty(B, nq * D, device=dev, dtype=torch.bfloat16)
    p = torch.tensor([pos], device=dev)
    decode_ops.rope_append(qkv, p, cos, sin, q_out, kc, vc, nq, nkv)
    q = qkv[:, : nq * D].view(B, nq, D)
    k = qkv[:, nq * D: (nq + nkv) * D].view(B, nkv, D)
    v = qkv[:, (nq + nkv) * D:].view(B, nkv, D)
    assert rel_l2(q_out.float().cpu(), _rope_ref(q, cos[pos], sin[pos]).reshape(B, -1).float().cpu()) < 3e-3
    assert rel_l2(kc[:, :, pos].float().cpu(), _rope_ref(k, cos[pos], sin[pos]).float().cpu()) < 3e-3
    assert torch.equal(vc[:, :, pos], v)
    mask = torch.ones(max_len, dtype=torch.bool, device=dev)
    mask[pos] = False
    assert not kc[:, :, mask].any() and not vc[:, :, mask].any(), "only row pos may be written"


@pytest.mark.parametrize("B,nq,nkv,D,max_len,pos", [
    (1, 28, 4, 128, 2184, 2047), (1, 28, 4, 128, 300, 0), (2, 4, 2, 64, 200, 63), (2, 4, 2, 64, 200, 64),
    (3, 8, 8, 128, 130, 129), (1, 40, 8, 128, 512, 65), (2, 8, 1, 128, 256, 100)])
def test_attn_decode(B, nq, nkv, D, max_len, pos):
    from helix_substrate_b200 import decode_ops
    dev = _dev()
    g = torch.Generator(device=dev).manual_seed(pos + max_len)
    q = torch.randn(B, nq * D, device=dev, generator=g).bfloat16()
    kc = torch.randn(B, nkv, max_len, D, device=dev, generator=g).bfloat16()
    vc = torch.randn(B, nkv, max_len, D, device=dev, generator=g).bfloat16()
    out = torch.empty_like(q)
    decode_ops.attn_decode(q, kc, vc, torch.tensor([pos], device=dev), out, nq, D ** -0.5)
    G = nq // nkv
    kk = kc[:, :, : pos + 1].double().repeat_interleave(G, 1)
    vv = vc[:, :, : pos + 1].double().repeat_interleave(G, 1)
    s = torch.einsum("bhd,bhpd->bhp", q.view(B, nq, D).double(), kk) * D ** -0.5
    ref = torch.einsum("bhp,bhpd->bhd", s.softmax(-1), vv).reshape(B, nq * D)
    assert rel_l2(out.float().cpu(), ref.cpu()) < 6e-3   # bf16 output rounding


@pytest.mark.parametrize("B,n", [(1, 18944), (4, 1001), (16, 512)])
def test_swiglu(B, n):
    from helix_substrate_b200 import decode_ops
    g = torch.Generator(device=_dev()).manual_seed(n)
    a = (2 * torch.randn(B, n, device=_dev(), generator=g)).bfloat16()
    b = torch.randn(B, n, device=_dev(), generator=g).bfloat16()
    out = torch.empty_like(a)
    decode_ops.swiglu(a, b, out)
    assert rel_l2(out.float().cpu(), (F.silu(a) * b).float().cpu()) < 3e-3


@pytest.mark.parametrize("n_out,n_in,M", [(1000, 3584, 1), (4097, 512, 2), (152064, 3584, 1), (999, 5120, 3), (64, 2056, 4)])
def test_dense_gemv_against_fp64(n_out, n_in, M):
    """hxq_dense_gemv (lm_head at decode time) against the fp64 product of the same bf16 operands:
    fp32 accumulation, so only the summation order differs (rel-L2 <= 1e-5 for fp32 output); bf16
    output is the rounded fp32 result; a padded weight stride and run-to-run equality."""
    from helix_substrate_b200 import decode_ops
    g = torch.Generator(device=_dev()).manual_seed(n_out + M)
    pad = 8 if n_out < 5000 else 0
    wfull = (0.02 * torch.randn(n_out, n_in + pad, device=_dev(), generator=g)).bfloat16()
    w = wfull[:, :n_in]
    x = torch.randn(M, n_in, device=_dev(), generator=g).bfloat16()
    ref = x.double() @ w.double().t()
    y32 = decode_ops.dense_gemv(w, x, out_dtype=torch.float32)
    assert y32.shape == (M, n_out)
    assert rel_l2(y32.double().cpu(), ref.cpu()) < 1e-5
    yb = decode_ops.dense_gemv(w, x)
    assert yb.dtype == torch.bfloat16 and torch.equal(yb, y32.bfloat16())
    assert torch.equal(y32, decode_ops.dense_gemv(w, x, out_dtype=torch.float32))


def test_glue_rejects_bad_arguments():
    from helix_substrate_b200 import _lib, decode_ops
    x = torch.zeros(2, 64, device=_dev(), dtype=torch.float32)
    with pytest.raises(TypeError):
        decode_ops.swiglu(x, x, x)
    q = torch.zeros(1, 9 * 64, device=_dev(), dtype=torch.bfloat16)
    kc = torch.zeros(1, 1, 16, 64, device=_dev(), dtype=torch.bfloat16)
    with pytest.raises(_lib.HxqError):   # nine query heads per KV head: more than the kernel's group limit
        decode_ops.attn_decode(q, kc, kc, torch.zeros(1, device=_dev(), dtype=torch.long), torch.empty_like(q), 9, 0.125)


@pytest.mark.parametrize("fuse_proj", [True, False])
def test_fused_step_matches_the_torch_step(fuse_proj):
    from helix_substrate_b200.qwen2_decode import Qwen2HxqDecoder, Qwen2Shape
    dev = _dev()
    torch.manual_seed(0)
    model = Qwen2HxqDecoder(Qwen2Shape.tiny(), dev, batch=2, max_len=96, fuse_proj=fuse_proj)
    prompt = torch.randint(0, 1024, (2, 70), device=dev)
    with torch.no_grad():
        nxt = model.prefill(prompt)
        pos = torch.tensor([70], device=dev)
        k0, v0 = model.k_cache.clone(), model.v_cache.clone()
        ref = model.forward_tokens(nxt[:, None], pos, pos, None)
        k1, v1 = model.k_cache.clone(), model.v_cache.clone()
        model.k_cache.copy_(k0); model.v_cache.copy_(v0)
        got = model.step_fused(nxt[:, None], pos)
    assert rel_l2(got.float().cpu(), ref.float().cpu()) < 3e-2
    assert rel_l2(model.k_cache.float().cpu(), k1.float().cpu()) < 1e-2
    assert rel_l2(model.v_cache.float().cpu(), v1.float().cpu()) < 1e-2
    # and the captured greedy loop produces tokens
    with torch.no_grad():
        toks = model.greedy_decode(prompt, 8, graphed=True)
    assert toks.shape == (2, 8) and int(toks.min()) >= 0 and int(toks.max()) < 1024


@pytest.mark.parametrize("world", [2, 4])
def test_sharded_decoder_matches_the_unsharded_one_on_one_gpu(world):
    """Tensor-parallel decoding with more ranks than KV heads (14 query / 2 KV heads on 4 ranks: the
    28 / 4 on 8 layout of Qwen2.5-7B), every rank's shard cut from the SAME compressed matrices.
    All ranks run inside this process on one GPU, their row-parallel partials summed where the
    exchange would be: prefill logits, one fused step's logits and the KV caches must agree with
    the unsharded decoder to bf16 precision."""
    from helix_substrate_b200.qwen2_decode import Qwen2HxqDecoder, Qwen2Shape, run_ranks_in_process
    from helix_substrate_b200.tp import head_partition
    dev = _dev()
    shp = Qwen2Shape(hidden=256, inter=640, layers=2, heads=14, kv_heads=2, head_dim=64, vocab=512)
    B, T, max_len = 2, 37, 64
    full = Qwen2HxqDecoder(shp, dev, batch=B, max_len=max_len, build="global")
    ranks = [Qwen2HxqDecoder(shp, dev, batch=B, max_len=max_len, rank=r, world=world, build="global")
             for r in range(world)]
    prompt = torch.randint(0, shp.vocab, (B, T), device=dev, generator=torch.Generator(device=dev).manual_seed(1))
    pos = torch.arange(T, device=dev)
    with torch.no_grad():
        ref = full.forward_tokens(prompt, pos, pos, T)
        outs = run_ranks_in_process([m.blocks_tokens(prompt, pos, pos, T) for m in ranks])
    for o in outs:
        assert torch.equal(o, outs[0]), "every rank must end with the same logits"
    assert rel_l2(outs[0].float().cpu(), ref.float().cpu()) < 3e-2
    parts = head_partition(shp.heads, shp.kv_heads, world)
    for r, m in enumerate(ranks):   # each rank's cache holds exactly its KV heads
        kv0, kv1 = parts[r][2], parts[r][3]
        assert m.k_cache.shape[2] == kv1 - kv0
        assert rel_l2(m.k_cache[:, :, :, :T].float().cpu(), full.k_cache[:, :, kv0:kv1, :T].float().cpu()) < 2e-2
        assert rel_l2(m.v_cache[:, :, :, :T].float().cpu(), full.v_cache[:, :, kv0:kv1, :T].float().cpu()) < 2e-2
    # one fused decode step on top of those caches
    tok = ref.argmax(-1)[:, None]
    p1 = torch.tensor([T], device=dev)
    with torch.no_grad():
        ref_step = full.step_fused(tok, p1)
        outs = run_ranks_in_process([m.blocks_step(tok, p1, fp32_partials=True) for m in ranks])
    for o in outs:
        assert torch.equal(o, outs[0])
    assert rel_l2(outs[0].float().cpu(), ref_step.float().cpu()) < 3e-2
    assert int(outs[0].argmax(-1)[0]) == int(ref_step.argmax(-1)[0]) or \
        rel_l2(outs[0].float().cpu(), ref_step.float().cpu()) < 1e-2
