"""Greedy decode of a Qwen2-architecture decoder whose linears are HelixLinear.

This is the caller around the compressed-linear path (the reference drives HF
models with a Python greedy loop, helix_substrate/basin_runtime.py:358-445, at
one model() call per token): every projection is an HXQ product; the one-token
step runs RMSNorm (+ residual add), RoPE + KV-cache append, single-query
grouped attention and SwiGLU as one launch each (decode_ops: 13 launches per
layer) and is replayed from a CUDA graph; the prompt is prefilled with the same
operators written in plain torch ops (also the parity reference of the step).  Tensor parallel: q/k/v/gate/up are
column-parallel, o/down row-parallel with one sum over ranks each (NCCL, or the one-shot
peer-memory kernel in the fused step).  Attention heads follow ``tp.head_partition``: when the
ranks outnumber the KV heads (Qwen2.5-7B on 8 GPUs: 28 query / 4 KV heads) each KV head lives
on two ranks and its seven query heads are dealt 4 + 3; the MLP is cut on whole 128-column
affine groups.

Weights are random-init (N(0, 0.02)) and compressed on the GPU; lm_head and the
embedding stay dense bf16, as in the reference's policy (tensor_policy.py:199-208).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import decode_ops
from .helix_linear import HelixLinear
from .hxq_writer_gpu import compress_weight
from .tp import head_partition, shard_bounds, take_cols, take_rows


@dataclass
class Qwen2Shape:
    hidden: int = 3584
    inter: int = 18944
    layers: int = 28
    heads: int = 28
    kv_heads: int = 4
    head_dim: int = 128
    vocab: int = 152064
    rope_theta: float = 1e6
    rms_eps: float = 1e-6

    @staticmethod
    def qwen25_7b() -> "Qwen2Shape":
        return Qwen2Shape()

    @staticmethod
    def qwen25_14b() -> "Qwen2Shape":
        return Qwen2Shape(hidden=5120, inter=13824, layers=48, heads=40, kv_heads=8)

    @staticmethod
    def tiny() -> "Qwen2Shape":
        return Qwen2Shape(hidden=256, inter=512, layers=2, heads=4, kv_heads=2, head_dim=64, vocab=1024)


def _compress_random(rows: int, cols: int, seed: int, device, bias: bool, group_size: int, name: str) -> HelixLinear:
    """N(0, 0.02) weights of the given shape, compressed on the device."""
    g = torch.Generator(device=device).manual_seed(seed)
    w = torch.randn(rows, cols, device=device, generator=g) * 0.02
    b = (torch.randn(rows, device=device, generator=g) * 0.02) if bias else None
    enc = compress_weight(w, percentile=99.95, group_size=group_size)
    del w
    return HelixLinear(cols, rows, bias=b, tensor_name=name, **enc)


MLP_CUT = 128   # the intermediate dimension is dealt to ranks in whole affine groups


class Qwen2Layer(nn.Module):
    """One decoder layer's HXQ projections for ``rank`` of ``world``.

    ``build="global"`` compresses each full-size matrix and takes this rank's rows / columns of
    it (exact tensor-parallel semantics: the shards of all ranks recompose the unsharded layer;
    every rank pays for the whole matrix).  ``build="local"`` draws and compresses matrices of the
    shard's own shape (random-init benchmarks: same shapes, 1/world of the encoding work)."""

    def __init__(self, shp: Qwen2Shape, li: int, device, group_size: int, rank: int, world: int, fuse: bool = True,
                 build: str = "local"):
        super().__init__()
        if build not in ("local", "global"):
            raise ValueError(f"build must be 'local' or 'global', got {build!r}")
        H, D, Hq, Hkv, I = shp.hidden, shp.head_dim, shp.heads, shp.kv_heads, shp.inter
        q0, q1, kv0, kv1 = head_partition(Hq, Hkv, world)[rank]
        i0, i1 = shard_bounds(I, rank, world, MLP_CUT if world > 1 else 1)
        if i1 <= i0:
            raise ValueError(f"tensor-parallel {world}: rank {rank} would hold no MLP columns of {I}")
        self.n_q, self.n_kv, self.inter_local = q1 - q0, kv1 - kv0, i1 - i0
        nq, nkv, ni = self.n_q, self.n_kv, self.inter_local
        p, sd = f"model.layers.{li}", 1000 * li
        self.fused = fuse
        glob = build == "global"
        rseed = 0 if glob else 64 + rank       # local builds differ per rank
        mk = lambda rows, cols, k, bias, name: _compress_random(rows, cols, (sd + k) * 128 + rseed, device, bias,
                                                                group_size, f"{p}.{name}.weight")
        if fuse:   # q|k|v and gate|up as one compressed matrix each: 4 products per layer instead of 7
            if glob:
                qkv = mk((Hq + 2 * Hkv) * D, H, 7, True, "self_attn.qkv_proj")
                self.qkv_proj = take_rows(qkv, [(q0 * D, q1 * D), ((Hq + kv0) * D, (Hq + kv1) * D),
                                                ((Hq + Hkv + kv0) * D, (Hq + Hkv + kv1) * D)]).to(device)
                gu = mk(2 * I, H, 8, False, "mlp.gate_up_proj")
                self.gate_up_proj = take_rows(gu, [(i0, i1), (I + i0, I + i1)]).to(device)
                del qkv, gu
            else:
                self.qkv_proj = mk((nq + 2 * nkv) * D, H, 7, True, "self_attn.qkv_proj")
                self.gate_up_proj = mk(2 * ni, H, 8, False, "mlp.gate_up_proj")
        else:
            cut = lambda m, a, b: take_rows(m, [(a, b)]).to(device)
            if glob:
                self.q_proj = cut(mk(Hq * D, H, 0, True, "self_attn.q_proj"), q0 * D, q1 * D)
                self.k_proj = cut(mk(Hkv * D, H, 1, True, "self_attn.k_proj"), kv0 * D, kv1 * D)
                self.v_proj = cut(mk(Hkv * D, H, 2, True, "self_attn.v_proj"), kv0 * D, kv1 * D)
                self.gate_proj = cut(mk(I, H, 4, False, "mlp.gate_proj"), i0, i1)
                self.up_proj = cut(mk(I, H, 5, False, "mlp.up_proj"), i0, i1)
            else:
                self.q_proj = mk(nq * D, H, 0, True, "self_attn.q_proj")
                self.k_proj = mk(nkv * D, H, 1, True, "self_attn.k_proj")
                self.v_proj = mk(nkv * D, H, 2, True, "self_attn.v_proj")
                self.gate_proj = mk(ni, H, 4, False, "mlp.gate_proj")
                self.up_proj = mk(ni, H, 5, False, "mlp.up_proj")
        if glob:
            self.o_proj = take_cols(mk(H, Hq * D, 3, False, "self_attn.o_proj"), q0 * D, q1 * D).to(device)
            self.down_proj = take_cols(mk(H, I, 6, False, "mlp.down_proj"), i0, i1).to(device)
        else:
            self.o_proj = mk(H, nq * D, 3, False, "self_attn.o_proj")
            self.down_proj = mk(H, ni, 6, False, "mlp.down_proj")
        self.ln1 = nn.Parameter(torch.ones(H, device=device, dtype=torch.bfloat16), requires_grad=False)
        self.ln2 = nn.Parameter(torch.ones(H, device=device, dtype=torch.bfloat16), requires_grad=False)


def _drive(gen, reduce):
    """Run a block generator: it yields ``(partial, key)`` wherever a sum over the tensor-parallel
    ranks is due and is sent the summed tensor back."""
    try:
        item = next(gen)
        while True:
            item = gen.send(reduce(*item))
    except StopIteration as e:
        return e.value


def run_ranks_in_process(gens):
    """Drive the block generators of ALL ranks of a tensor-parallel group inside one process, in
    lockstep: at every exchange point the partials are added in rank order in fp32 and rounded
    once to bf16, which is what the one-shot peer-memory kernel does.  This is how the sharded
    decoder is checked against the unsharded one on a single GPU.  Returns each rank's result."""
    results = [None] * len(gens)
    try:
        items = [next(g) for g in gens]
    except StopIteration:
        raise RuntimeError("a rank finished before its first exchange")
    while True:
        total = items[0][0].float().clone()
        for it in items[1:]:
            total += it[0].float()
        total = total.to(torch.bfloat16)
        nxt, done = [], 0
        for r, g in enumerate(gens):
            try:
                nxt.append(g.send(total.clone()))
            except StopIteration as e:
                results[r] = e.value
                done += 1
        if done == len(gens):
            return results
        if done:
            raise RuntimeError("ranks disagree on the number of exchanges")
        items = nxt


class Qwen2HxqDecoder(nn.Module):
    """Static-cache decoder.  ``prefill`` fills the cache from a prompt,
    ``step`` decodes one token per sequence at ``pos`` (a device scalar)."""

    def __init__(self, shp: Qwen2Shape, device, batch: int, max_len: int, group_size: int = 128,
                 rank: int = 0, world: int = 1, group=None, fuse_proj: bool = True, p2p_allreduce: bool = False,
                 build: str = "local"):
        super().__init__()
        self.shp, self.device, self.world, self.group = shp, device, world, group
        self.p2p = bool(p2p_allreduce) and world > 1   # one-shot peer-memory sum instead of NCCL in the fused step
        self.layers = nn.ModuleList(Qwen2Layer(shp, i, device, group_size, rank, world, fuse_proj, build)
                                    for i in range(shp.layers))
        g = torch.Generator(device=device).manual_seed(7)
        self.embed = (torch.randn(shp.vocab, shp.hidden, device=device, generator=g) * 0.02).bfloat16()
        self.lm_head = (torch.randn(shp.vocab, shp.hidden, device=device, generator=g) * 0.02).bfloat16()
        self.norm = torch.ones(shp.hidden, device=device, dtype=torch.bfloat16)
        n_kv = self.layers[0].n_kv
        self.k_cache = torch.zeros(shp.layers, batch, n_kv, max_len, shp.head_dim, device=device, dtype=torch.bfloat16)
        self.v_cache = torch.zeros_like(self.k_cache)
        inv = 1.0 / (shp.rope_theta ** (torch.arange(0, shp.head_dim, 2, device=device, dtype=torch.float32)
                                        / shp.head_dim))
        ang = torch.arange(max_len, device=device, dtype=torch.float32)[:, None] * inv[None, :]
        self.cos = torch.cat([ang.cos(), ang.cos()], -1)
        self.sin = torch.cat([ang.sin(), ang.sin()], -1)
        self.max_len = max_len

    def _rms(self, x, w):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.shp.rms_eps)).to(x.dtype) * w

    @staticmethod
    def _rope(x, cos, sin):
        x1, x2 = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
        return (x.float() * cos + torch.cat([-x2, x1], -1).float() * sin).to(x.dtype)

    def _allreduce(self, t):
        if self.world > 1:
            torch.distributed.all_reduce(t, group=self.group)
        return t

    def forward_tokens(self, ids: torch.Tensor, positions: torch.Tensor, cache_rows: torch.Tensor,
                       attn_len: Optional[int]) -> torch.Tensor:
        """ids [B, T]; positions [T] (absolute); the new K/V go to cache rows
        ``cache_rows`` [T]; attention spans cache[:attn_len] (None = whole cache
        with a position mask, which is what the captured one-token step uses)."""
        return _drive(self.blocks_tokens(ids, positions, cache_rows, attn_len), lambda part, key, *_: self._allreduce(part))

    def blocks_tokens(self, ids: torch.Tensor, positions: torch.Tensor, cache_rows: torch.Tensor,
                      attn_len: Optional[int]):
        """``forward_tokens`` as a generator: yields ``(partial [B, T, hidden], key)`` after o_proj and
        down_proj of every layer and expects the sum over ranks back; returns the logits."""
        B, T = ids.shape
        D = self.shp.head_dim
        h = self.embed[ids]
        cos, sin = self.cos[positions][None, None], self.sin[positions][None, None]
        for li, L in enumerate(self.layers):
            x = self._rms(h, L.ln1)
            if L.fused:
                q, k, v = L.qkv_proj(x).split([L.n_q * D, L.n_kv * D, L.n_kv * D], -1)
            else:
                q, k, v = L.q_proj(x), L.k_proj(x), L.v_proj(x)
            q = q.reshape(B, T, L.n_q, D).transpose(1, 2)
            k = k.reshape(B, T, L.n_kv, D).transpose(1, 2)
            v = v.reshape(B, T, L.n_kv, D).transpose(1, 2)
            q, k = self._rope(q, cos, sin), self._rope(k, cos, sin)
            self.k_cache[li].index_copy_(2, cache_rows, k)
            self.v_cache[li].index_copy_(2, cache_rows, v)
            if attn_len is None:
                kk, vv = self.k_cache[li], self.v_cache[li]
                mask = (torch.arange(self.max_len, device=ids.device)[None, :] <= positions[:, None])[None, None]
            else:
                kk, vv = self.k_cache[li][:, :, :attn_len], self.v_cache[li][:, :, :attn_len]
                mask = (torch.arange(attn_len, device=ids.device)[None, :] <= positions[:, None])[None, None]
            a = F.scaled_dot_product_attention(q, kk, vv, attn_mask=mask, enable_gqa=True)
            a = a.transpose(1, 2).reshape(B, T, L.n_q * D)
            h = h + (yield L.o_proj(a), "d1")
            x = self._rms(h, L.ln2)
            if L.fused:
                gt, up = L.gate_up_proj(x).split([L.inter_local, L.inter_local], -1)
            else:
                gt, up = L.gate_proj(x), L.up_proj(x)
            h = h + (yield L.down_proj(F.silu(gt) * up), "d2")
        h = self._rms(h[:, -1], self.norm)
        return h @ self.lm_head.t()

    def _step_buffers(self, B: int):
        sb = getattr(self, "_sb", None)
        if sb is None or sb["h"].shape[0] != B:
            L0, D, dev = self.layers[0], self.shp.head_dim, self.device
            mk = lambda n: torch.empty(B, n, device=dev, dtype=torch.bfloat16)
            sb = dict(h=mk(self.shp.hidden), x=mk(self.shp.hidden), qkv=mk((L0.n_q + 2 * L0.n_kv) * D),
                      q=mk(L0.n_q * D), a=mk(L0.n_q * D), gu=mk(2 * L0.inter_local), act=mk(L0.inter_local),
                      d1=mk(self.shp.hidden), d2=mk(self.shp.hidden))
            if self.p2p:
                from .tp import OneShotAllReduce
                sb["p32"] = torch.empty(B, self.shp.hidden, device=dev, dtype=torch.float32)
                self._ar = OneShotAllReduce(B * self.shp.hidden, dev, self.group)
            self._sb = sb
        return sb

    def _reduce_step(self, part: torch.Tensor, key: str, w_next: torch.Tensor = None):
        """Sum of one step's row-parallel partial over the ranks.  With the one-shot kernel the residual
        add and the next RMSNorm are folded into the same launch (h and x of the step buffers are
        updated in place) and None is returned; otherwise the bf16 sum is."""
        sb = self._sb
        if self.p2p:
            self._ar.add_rmsnorm(part, sb["h"], w_next, self.shp.rms_eps, sb["x"])
            return None
        return self._allreduce(part)

    def step_fused(self, tok: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        """One decode step for tok [B, 1] at position pos (int64 device tensor [1]): same
        arithmetic as ``forward_tokens(tok, pos, pos, None)`` with the glue between the
        linears in four fused operators.  Returns the logits [B, vocab]."""
        return _drive(self.blocks_step(tok, pos, fp32_partials=self.p2p), self._reduce_step)

    def blocks_step(self, tok: torch.Tensor, pos: torch.Tensor, fp32_partials: bool = False):
        """``step_fused`` as a generator: yields ``(partial [B, hidden], key)`` after o_proj and down_proj
        of every layer (fp32 when the sum is taken by the one-shot kernel or in process, bf16 for NCCL)
        and expects the bf16 sum over ranks back; returns the logits."""
        B = tok.shape[0]
        sb = self._step_buffers(B)
        D, eps = self.shp.head_dim, self.shp.rms_eps
        bf = torch.bfloat16
        h, x = sb["h"], sb["x"]
        h.copy_(self.embed[tok[:, 0]])

        def row_parallel(lin, xin, key):
            if fp32_partials:
                if "p32" not in sb:
                    sb["p32"] = torch.empty(B, self.shp.hidden, device=self.device, dtype=torch.float32)
                return lin.packed().matmul(xin, torch.float32, out=sb["p32"]), key
            return lin.packed().matmul(xin, bf, out=sb[key]), key

        n_layers = len(self.layers)
        decode_ops.add_rmsnorm(h, None, self.layers[0].ln1, eps, x)
        for li, L in enumerate(self.layers):
            nq, nkv = L.n_q, L.n_kv
            qkv, gu, ni = sb["qkv"], sb["gu"], L.inter_local
            if L.fused:
                L.qkv_proj.packed().matmul(x, bf, out=qkv)
            else:
                L.q_proj.packed().matmul(x, bf, out=qkv[:, : nq * D])
                L.k_proj.packed().matmul(x, bf, out=qkv[:, nq * D: (nq + nkv) * D])
                L.v_proj.packed().matmul(x, bf, out=qkv[:, (nq + nkv) * D:])
            decode_ops.rope_append(qkv, pos, self.cos, self.sin, sb["q"], self.k_cache[li], self.v_cache[li], nq, nkv)
            decode_ops.attn_decode(sb["q"], self.k_cache[li], self.v_cache[li], pos, sb["a"], nq, D ** -0.5)
            # the exchange is handed the weight of the norm that follows it: a driver that folds the
            # residual add and that norm into the sum answers None
            delta = yield (*row_parallel(L.o_proj, sb["a"], "d1"), L.ln2)
            if delta is not None:
                decode_ops.add_rmsnorm(h, delta, L.ln2, eps, x)
            if L.fused:
                L.gate_up_proj.packed().matmul(x, bf, out=gu)
            else:
                L.gate_proj.packed().matmul(x, bf, out=gu[:, :ni])
                L.up_proj.packed().matmul(x, bf, out=gu[:, ni:])
            decode_ops.swiglu(gu[:, :ni], gu[:, ni:], sb["act"])
            w_next = self.layers[li + 1].ln1 if li + 1 < n_layers else self.norm
            delta = yield (*row_parallel(L.down_proj, sb["act"], "d2"), w_next)
            if delta is not None:
                decode_ops.add_rmsnorm(h, delta, w_next, eps, x)
        if x.shape[0] <= decode_ops.DENSE_GEMV_USE_M:      # one or two tokens: the streaming kernel; more: a library GEMM
            return decode_ops.dense_gemv(self.lm_head, x)
        return x @ self.lm_head.t()

    @torch.no_grad()
    def prefill(self, prompt: torch.Tensor, chunk: int = 2048) -> torch.Tensor:
        T = prompt.shape[1]
        logits = None
        for a in range(0, T, chunk):
            b = min(a + chunk, T)
            pos = torch.arange(a, b, device=prompt.device)
            logits = self.forward_tokens(prompt[:, a:b], pos, pos, b)
        return logits.argmax(-1)

    @torch.no_grad()
    def make_graphed_step(self, batch: int, fused: bool = True):
        """Capture the one-token step.  Returns (run, tok, pos): write the
        current tokens into ``tok`` [B, 1] and the position into ``pos`` [1],
        call ``run()``, read the next tokens from its result."""
        tok = torch.zeros(batch, 1, device=self.device, dtype=torch.long)
        pos = torch.zeros(1, device=self.device, dtype=torch.long)

        def body():
            if fused:
                return self.step_fused(tok, pos).argmax(-1)
            return self.forward_tokens(tok, pos, pos, None).argmax(-1)

        # warm up on the stream the capture will run on: the kernels' workspaces are kept per
        # stream and must exist (and be zero) before the capture starts
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            for _ in range(2):
                body()
            side.synchronize()
            with torch.cuda.graph(graph, stream=side):
                out = body()
        torch.cuda.current_stream().wait_stream(side)
        self._graph = graph

        def run():
            graph.replay()
            return out
        return run, tok, pos

    @torch.no_grad()
    def greedy_decode(self, prompt: torch.Tensor, new_tokens: int, graphed: bool = True):
        """Prefill, then ``new_tokens`` greedy steps.  Returns the generated
        ids [B, new_tokens] (device tensor)."""
        B, T = prompt.shape
        nxt = self.prefill(prompt)
        outs = [nxt]
        if graphed:
            run, tok, pos = self.make_graphed_step(B)
        for i in range(new_tokens - 1):
            p = T + i
            if graphed:
                tok.copy_(nxt[:, None])
                pos.fill_(p)
                nxt = run().clone()
            else:
                pt = torch.tensor([p], device=prompt.device)
                nxt = self.forward_tokens(nxt[:, None], pt, pt, None).argmax(-1)
            outs.append(nxt)
        return torch.stack(outs, 1)


def run_decode(shape: str, batches, prompt: int, new_tokens: int, device, rank: int = 0, world: int = 1, *,
               layers: int = 0, build: str = "local", allreduce: str = "p2p", fuse_proj: bool = True,
               graph: bool = True, torch_glue: bool = False, fill_cache: bool = False):
    """Build ONE random-init HXQ decoder of the named shape and, for every batch size in ``batches``,
    prefill ``prompt`` tokens per sequence and time ``new_tokens - 1`` greedy steps (CUDA events, max
    over ranks).  ``fill_cache`` replaces the prefill by random K/V rows (decode speed at a given
    context without paying for the prompt).  Returns one dict of measurements per batch size (every
    rank gets the same numbers)."""
    import gc
    import time
    batches = [int(b) for b in ([batches] if isinstance(batches, int) else batches)]
    shp = {"7b": Qwen2Shape.qwen25_7b, "14b": Qwen2Shape.qwen25_14b, "tiny": Qwen2Shape.tiny}[shape]()
    if layers:
        shp.layers = layers
    t0 = time.perf_counter()
    model = Qwen2HxqDecoder(shp, device, max(batches), prompt + new_tokens + 8, rank=rank, world=world,
                            fuse_proj=fuse_proj, p2p_allreduce=(allreduce == "p2p"), build=build)
    torch.cuda.synchronize(device)
    build_s = time.perf_counter() - t0
    k_full, v_full = model.k_cache, model.v_cache
    hxq_mods = [m for m in model.modules() if isinstance(m, HelixLinear)]
    out = []
    for batch in batches:
        model.k_cache, model.v_cache = k_full[:, :batch], v_full[:, :batch]
        for name in ("_graph", "_sb"):
            if hasattr(model, name):
                delattr(model, name)
        ids = torch.randint(0, shp.vocab, (batch, prompt), device=device,
                            generator=torch.Generator(device=device).manual_seed(0))
        prefill_ms = None
        with torch.no_grad():
            if fill_cache:
                g = torch.Generator(device=device).manual_seed(1 + rank)
                for li in range(shp.layers):   # layer by layer: the fp32 temporaries stay small
                    for cache in (model.k_cache, model.v_cache):
                        view = cache[li][:, :, :prompt]
                        view.copy_(torch.randn(view.shape, device=device, generator=g) * 0.5)
                nxt = ids[:, -1].clone()
            else:
                # warm-up call: first-use set-up of every kernel and every workspace the timed call needs (the whole
                # prompt when that is cheap, else enough tokens to reach the large-token kernel)
                model.prefill(ids if batch * prompt <= 4096 else ids[:, : min(prompt, 600)])
                torch.cuda.synchronize(device)
                p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                p0.record()
                nxt = model.prefill(ids)
                p1.record()
                torch.cuda.synchronize(device)
                prefill_ms = p0.elapsed_time(p1)
            run = None
            if graph:
                run, tok, pos = model.make_graphed_step(batch, fused=not torch_glue)
            torch.cuda.synchronize(device)
            e1, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e1.record()
            for i in range(new_tokens - 1):
                p = prompt + i
                if run is not None:
                    tok.copy_(nxt[:, None])
                    pos.fill_(p)
                    nxt = run()
                else:
                    pt = torch.tensor([p], device=device)
                    if torch_glue:
                        nxt = model.forward_tokens(nxt[:, None], pt, pt, None).argmax(-1)
                    else:
                        nxt = model.step_fused(nxt[:, None], pt).argmax(-1)
            e2.record()
            torch.cuda.synchronize(device)
        ms_dec = e1.elapsed_time(e2) / max(1, new_tokens - 1)
        t = torch.tensor([ms_dec, prefill_ms or 0.0], device=device, dtype=torch.float64)
        if world > 1:
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ms_dec, pf = float(t[0].item()), float(t[1].item())
        hxq_bytes = sum(m.packed().algorithmic_bytes(batch, 2, 2) for m in hxq_mods)
        ar_status = None
        if world > 1 and getattr(model, "_ar", None) is not None:
            ar_status = model._ar.check_status()
        out.append({
            "tok_s": batch * 1000.0 / ms_dec, "ms_per_step": ms_dec, "batch": batch, "context": prompt,
            "new_tokens": new_tokens, "shape": shape, "layers": shp.layers, "n_gpus": world,
            "launch": "python" if run is None else "cuda_graph", "glue": "torch" if torch_glue else "fused",
            "projections": "qkv,o,gate_up,down" if fuse_proj else "q,k,v,o,gate,up,down",
            "allreduce": (allreduce if world > 1 else None), "allreduce_status": ar_status,
            "weights": f"random N(0, 0.02), compressed per {'full matrix then sharded' if build == 'global' else 'shard'}",
            "hxq_bytes_per_step_per_gpu": hxq_bytes, "hxq_GBps_per_gpu": hxq_bytes / (ms_dec * 1e-3) / 1e9,
            "prefill_ms": (pf if prefill_ms is not None else None),
            "prefill_tok_s": (batch * prompt / (pf * 1e-3) if prefill_ms is not None else None),
            "kv_cache": "random rows (no prefill)" if fill_cache else "from the prefill",
            "tokens_valid": bool(int(nxt.min()) >= 0 and int(nxt.max()) < shp.vocab), "build_s": build_s,
        })
        run = None
    for name in ("_graph", "_ar", "_sb"):
        if hasattr(model, name):
            delattr(model, name)
    del model, k_full, v_full, hxq_mods
    gc.collect()
    torch.cuda.empty_cache()
    return out


def main(argv=None):
    """``python -m helix_substrate_b200.qwen2_decode --shape 7b --batch 1 --prompt 2048 --new 128``
    (under torchrun for tensor parallel).  Prints one JSON line with decode
    tokens/s, ms per token and the HXQ bytes streamed per token."""
    import argparse
    import json
    import os
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", default="7b", choices=["7b", "14b", "tiny"])
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (0 = the shape's own)")
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--prompt", type=int, default=2048)
    ap.add_argument("--new", type=int, default=128)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--torch-glue", action="store_true", help="run the step's glue in plain torch ops")
    ap.add_argument("--allreduce", default="p2p", choices=["nccl", "p2p"],
                    help="tensor-parallel sum in the fused step: NCCL, or the one-shot peer-memory kernel")
    ap.add_argument("--build", default="local", choices=["local", "global"],
                    help="local: each rank compresses matrices of its shard's shape; global: full matrices, then sharded")
    ap.add_argument("--fill-cache", action="store_true", help="random K/V rows instead of a prefill")
    ap.add_argument("--separate-proj", action="store_true",
                    help="q, k, v and gate, up as separate compressed matrices (7 products per layer instead of 4)")
    args = ap.parse_args(argv)
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        init_tensor_parallel(dev)
    res = run_decode(args.shape, [args.batch], args.prompt, args.new, dev, rank, world, layers=args.layers,
                     build=args.build, allreduce=args.allreduce, fuse_proj=not args.separate_proj,
                     graph=not args.no_graph, torch_glue=args.torch_glue, fill_cache=args.fill_cache)[0]
    if rank == 0:
        print(json.dumps({"metric": "decode_tokens_per_s", "value": res["tok_s"], "unit": "tok/s", **res,
                          "data": "synthetic: N(0,0.02) weights, uniform random prompt ids"}), flush=True)
    if world > 1:
        leave_process_group()


def init_tensor_parallel(device) -> None:
    """NCCL process group for one node, plain peer-to-peer only: no buffer of this process is ever
    bound to an NVLink multicast object (a rank that goes away while bound to one takes its peers'
    GPUs down with it), neither by NCCL (NVLS off) nor by symmetric memory."""
    import os
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    torch.distributed.init_process_group("nccl", device_id=device)


def leave_process_group(*holders) -> None:
    """End a multi-rank run: every rank has finished its GPU work, the captured graphs that hold
    collectives are dropped first (tearing the group down under a live graph blocks), then the
    group is destroyed.  If that still does not return within a minute the process exits anyway -
    after the barrier, with nothing in flight and NVLS off."""
    import gc
    import os
    import sys
    import threading
    torch.cuda.synchronize()
    torch.distributed.barrier()
    torch.cuda.synchronize()
    for h in holders:
        for name in ("_graph", "_ar", "_sb"):
            if hasattr(h, name):
                try:
                    delattr(h, name)
                except AttributeError:
                    pass
    gc.collect()
    sys.stdout.flush()
    sys.stderr.flush()
    t = threading.Timer(60.0, lambda: os._exit(0))
    t.daemon = True
    t.start()
    torch.distributed.destroy_process_group()
    t.cancel()


if __name__ == "__main__":
    main()
