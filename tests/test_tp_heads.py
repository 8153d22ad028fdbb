"""Tensor-parallel partition of attention heads and MLP columns, checked on the CPU: the
shards every rank builds from the full compressed matrices recompose the unsharded layer
exactly, including the layouts where ranks outnumber the KV heads (28 query / 4 KV heads
on 8 ranks: each KV head on two ranks, its query heads dealt 4 + 3)."""

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from oracle import hxq_oracle as O


def _dense(m):
    """Dequantised weight of a HelixLinear through the oracle (no GPU here)."""
    G = m.group_size
    w = O.reconstruct(m.codebook.numpy(), m.indices.numpy(),
                      None if m.sidecar_positions is None else m.sidecar_positions.numpy(),
                      None if m.sidecar_values is None else m.sidecar_values.numpy(),
                      None if m.group_scales is None else m.group_scales.numpy(),
                      None if m.group_offsets is None else m.group_offsets.numpy(), G, m.col0 % G if G else 0)
    return torch.from_numpy(w).double()


@pytest.mark.parametrize("heads,kv,world,want", [
    (28, 4, 8, [4, 3, 4, 3, 4, 3, 4, 3]), (28, 4, 4, [7] * 4), (28, 4, 2, [14] * 2), (28, 4, 1, [28]),
    (40, 8, 8, [5] * 8), (40, 8, 4, [10] * 4), (40, 8, 2, [20] * 2), (14, 2, 4, [4, 3, 4, 3]),
])
def test_head_partition_covers_every_head_once(heads, kv, world, want):
    from helix_substrate_b200.tp import head_partition
    parts = head_partition(heads, kv, world)
    assert [q1 - q0 for q0, q1, _, _ in parts] == want
    assert [q for q0, q1, _, _ in parts for q in range(q0, q1)] == list(range(heads))
    gq = heads // kv
    for q0, q1, kv0, kv1 in parts:
        assert kv1 > kv0
        for q in range(q0, q1):   # every query head sits with its own KV head
            assert kv0 <= q // gq < kv1


def test_head_partition_refuses_what_it_cannot_split():
    from helix_substrate_b200.tp import head_partition
    with pytest.raises(ValueError):
        head_partition(28, 4, 3)
    with pytest.raises(ValueError):
        head_partition(8, 4, 16)    # 2 query heads per KV head cannot feed 4 ranks


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("fuse", [True, False])
def test_layer_shards_recompose_the_unsharded_layer(world, fuse):
    """A 14-query / 2-KV-head layer (the 7:1 ratio of Qwen2.5-7B) cut for 2 and 4 ranks: dense
    weights of the shards equal the matching rows / columns of the full matrices, and the
    attention + MLP block computed per rank and summed equals the unsharded block."""
    from helix_substrate_b200.qwen2_decode import Qwen2Layer, Qwen2Shape
    from helix_substrate_b200.tp import head_partition, shard_bounds
    shp = Qwen2Shape(hidden=256, inter=640, layers=1, heads=14, kv_heads=2, head_dim=64, vocab=64)
    D, Hq, Hkv, I = shp.head_dim, shp.heads, shp.kv_heads, shp.inter
    full = Qwen2Layer(shp, 0, "cpu", 128, 0, 1, fuse, "global")
    if fuse:
        wqkv, bqkv = _dense(full.qkv_proj), full.qkv_proj.bias.double()
        wq, wk, wv = wqkv[: Hq * D], wqkv[Hq * D: (Hq + Hkv) * D], wqkv[(Hq + Hkv) * D:]
        bq, bk, bv = bqkv[: Hq * D], bqkv[Hq * D: (Hq + Hkv) * D], bqkv[(Hq + Hkv) * D:]
        wgu = _dense(full.gate_up_proj)
        wg, wu = wgu[:I], wgu[I:]
    else:
        wq, wk, wv = _dense(full.q_proj), _dense(full.k_proj), _dense(full.v_proj)
        bq, bk, bv = full.q_proj.bias.double(), full.k_proj.bias.double(), full.v_proj.bias.double()
        wg, wu = _dense(full.gate_proj), _dense(full.up_proj)
    wo, wd = _dense(full.o_proj), _dense(full.down_proj)

    torch.manual_seed(3)
    T = 5
    x = torch.randn(T, shp.hidden, dtype=torch.float64)

    def block(wq, bq, wk, bk, wv, bv, wo, wg, wu, wd, nq, nkv):
        q = (x @ wq.t() + bq).view(T, nq, D).transpose(0, 1)
        k = (x @ wk.t() + bk).view(T, nkv, D).transpose(0, 1)
        v = (x @ wv.t() + bv).view(T, nkv, D).transpose(0, 1)
        a = F.scaled_dot_product_attention(q[None], k[None], v[None], is_causal=True, enable_gqa=True)[0]
        attn = a.transpose(0, 1).reshape(T, nq * D) @ wo.t()
        mlp = (F.silu(x @ wg.t()) * (x @ wu.t())) @ wd.t()
        return attn, mlp

    ref_attn, ref_mlp = block(wq, bq, wk, bk, wv, bv, wo, wg, wu, wd, Hq, Hkv)
    sum_attn, sum_mlp = torch.zeros_like(ref_attn), torch.zeros_like(ref_mlp)
    parts = head_partition(Hq, Hkv, world)
    for r in range(world):
        L = Qwen2Layer(shp, 0, "cpu", 128, r, world, fuse, "global")
        q0, q1, kv0, kv1 = parts[r]
        i0, i1 = shard_bounds(I, r, world, 128)
        assert (L.n_q, L.n_kv, L.inter_local) == (q1 - q0, kv1 - kv0, i1 - i0)
        if fuse:
            w = _dense(L.qkv_proj)
            b = L.qkv_proj.bias.double()
            nq, nkv = L.n_q * D, L.n_kv * D
            sq, sk, sv = w[:nq], w[nq: nq + nkv], w[nq + nkv:]
            sbq, sbk, sbv = b[:nq], b[nq: nq + nkv], b[nq + nkv:]
            g = _dense(L.gate_up_proj)
            sg, su = g[: L.inter_local], g[L.inter_local:]
        else:
            sq, sk, sv = _dense(L.q_proj), _dense(L.k_proj), _dense(L.v_proj)
            sbq, sbk, sbv = L.q_proj.bias.double(), L.k_proj.bias.double(), L.v_proj.bias.double()
            sg, su = _dense(L.gate_proj), _dense(L.up_proj)
        so, sdn = _dense(L.o_proj), _dense(L.down_proj)
        # the shards ARE slices of the full dequantised matrices, bit for bit
        assert torch.equal(sq, wq[q0 * D: q1 * D]) and torch.equal(sk, wk[kv0 * D: kv1 * D])
        assert torch.equal(sv, wv[kv0 * D: kv1 * D]) and torch.equal(sbq, bq[q0 * D: q1 * D])
        assert torch.equal(so, wo[:, q0 * D: q1 * D]) and torch.equal(sdn, wd[:, i0:i1])
        assert torch.equal(sg, wg[i0:i1]) and torch.equal(su, wu[i0:i1])
        assert L.o_proj.col0 == q0 * D and L.down_proj.col0 == i0 and L.down_proj.col0 % 128 == 0
        a, m = block(sq, sbq, sk, sbk, sv, sbv, so, sg, su, sdn, L.n_q, L.n_kv)
        sum_attn += a
        sum_mlp += m
    assert torch.allclose(sum_attn, ref_attn, rtol=1e-10, atol=1e-12)
    assert torch.allclose(sum_mlp, ref_mlp, rtol=1e-10, atol=1e-12)


def test_in_process_rank_driver_sums_in_rank_order_and_rounds_once():
    from helix_substrate_b200.qwen2_decode import run_ranks_in_process

    def gen(r):
        got = yield torch.full((2, 4), 1.0 + r, dtype=torch.float32), "d1"
        got2 = yield got.float() * (r + 1), "d2"
        return got, got2

    res = run_ranks_in_process([gen(r) for r in range(3)])
    for r in range(3):
        a, b = res[r]
        assert a.dtype == torch.bfloat16 and torch.equal(a.float(), torch.full((2, 4), 6.0))
        assert torch.equal(b.float(), torch.full((2, 4), 36.0))
