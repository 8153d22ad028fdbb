"""Greedy decode of a Qwen2-architecture decoder whose linears are HelixLinear.

This is the caller around the compressed-linear path (the reference drives HF
models with a Python greedy loop, helix_substrate/basin_runtime.py:358-445, at
one model() call per token): every projection is an HXQ product; the one-token
step runs RMSNorm (+ residual add), RoPE + KV-cache append, single-query
grouped attention and SwiGLU as one launch each (decode_ops: 13 launches per
layer) and is replayed from a CUDA graph; the prompt is prefilled with the same
operators written in plain torch ops (also the parity reference of the step).  Tensor parallel: q/k/v/gate/up are
column-parallel, o/down row-parallel with one all-reduce each (NCCL).

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
from .tp import shard_helix_linear


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


def _hxq_linear(out_f: int, in_f: int, seed: int, device, bias: bool, group_size: int, name: str,
                mode: Optional[str], rank: int, world: int) -> HelixLinear:
    g = torch.Generator(device=device).manual_seed(seed)
    w = torch.randn(out_f, in_f, device=device, generator=g) * 0.02
    b = (torch.randn(out_f, device=device, generator=g) * 0.02) if bias else None
    enc = compress_weight(w, percentile=99.95, group_size=group_size)
    del w
    mod = HelixLinear(in_f, out_f, bias=b, tensor_name=name, **enc)
    if world > 1 and mode is not None:
        mod = shard_helix_linear(mod, mode, rank, world).to(device)
    return mod


def _hxq_fused_columns(outs, in_f: int, seed: int, device, bias: bool, group_size: int, name: str,
                       rank: int, world: int) -> HelixLinear:
    """Several column-parallel projections of one input as ONE compressed matrix (rows concatenated,
    one codebook): this rank's slice of each, generated at its local size."""
    rows = sum(o // world for o in outs)
    g = torch.Generator(device=device).manual_seed(seed * 64 + rank)
    w = torch.randn(rows, in_f, device=device, generator=g) * 0.02
    b = (torch.randn(rows, device=device, generator=g) * 0.02) if bias else None
    enc = compress_weight(w, percentile=99.95, group_size=group_size)
    del w
    return HelixLinear(in_f, rows, bias=b, tensor_name=name, **enc)


class Qwen2Layer(nn.Module):
    def __init__(self, shp: Qwen2Shape, li: int, device, group_size: int, rank: int, world: int, fuse: bool = True):
        super().__init__()
        H, D = shp.hidden, shp.head_dim
        if shp.heads % world or shp.kv_heads % world:
            raise ValueError(f"tensor-parallel {world} does not divide {shp.heads} query / {shp.kv_heads} KV heads")
        p = f"model.layers.{li}"
        mk = lambda o, i, k, bias, name, mode: _hxq_linear(o, i, 1000 * li + k, device, bias, group_size,
                                                           f"{p}.{name}.weight", mode, rank, world)
        self.fused = fuse
        if fuse:   # q|k|v and gate|up as one compressed matrix each: 4 products per layer instead of 7
            self.qkv_proj = _hxq_fused_columns([shp.heads * D, shp.kv_heads * D, shp.kv_heads * D], H, 1000 * li + 7,
                                               device, True, group_size, f"{p}.self_attn.qkv_proj.weight", rank, world)
            self.gate_up_proj = _hxq_fused_columns([shp.inter, shp.inter], H, 1000 * li + 8, device, False, group_size,
                                                   f"{p}.mlp.gate_up_proj.weight", rank, world)
        else:
            self.q_proj = mk(shp.heads * D, H, 0, True, "self_attn.q_proj", "column")
            self.k_proj = mk(shp.kv_heads * D, H, 1, True, "self_attn.k_proj", "column")
            self.v_proj = mk(shp.kv_heads * D, H, 2, True, "self_attn.v_proj", "column")
            self.gate_proj = mk(shp.inter, H, 4, False, "mlp.gate_proj", "column")
            self.up_proj = mk(shp.inter, H, 5, False, "mlp.up_proj", "column")
        self.o_proj = mk(H, shp.heads * D, 3, False, "self_attn.o_proj", "row")
        self.down_proj = mk(H, shp.inter, 6, False, "mlp.down_proj", "row")
        self.inter_local = shp.inter // world
        self.ln1 = nn.Parameter(torch.ones(H, device=device, dtype=torch.bfloat16), requires_grad=False)
        self.ln2 = nn.Parameter(torch.ones(H, device=device, dtype=torch.bfloat16), requires_grad=False)
        self.n_q, self.n_kv = shp.heads // world, shp.kv_heads // world


class Qwen2HxqDecoder(nn.Module):
    """Static-cache decoder.  ``prefill`` fills the cache from a prompt,
    ``step`` decodes one token per sequence at ``pos`` (a device scalar)."""

    def __init__(self, shp: Qwen2Shape, device, batch: int, max_len: int, group_size: int = 128,
                 rank: int = 0, world: int = 1, group=None, fuse_proj: bool = True, p2p_allreduce: bool = False):
        super().__init__()
        self.shp, self.device, self.world, self.group = shp, device, world, group
        self.p2p = bool(p2p_allreduce) and world > 1   # one-shot peer-memory sum instead of NCCL in the fused step
        self.layers = nn.ModuleList(Qwen2Layer(shp, i, device, group_size, rank, world, fuse_proj)
                                    for i in range(shp.layers))
        g = torch.Generator(device=device).manual_seed(7)
        self.embed = (torch.randn(shp.vocab, shp.hidden, device=device, generator=g) * 0.02).bfloat16()
        self.lm_head = (torch.randn(shp.vocab, shp.hidden, device=device, generator=g) * 0.02).bfloat16()
        self.norm = torch.ones(shp.hidden, device=device, dtype=torch.bfloat16)
        n_kv = shp.kv_heads // world
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
            h = h + self._allreduce(L.o_proj(a))
            x = self._rms(h, L.ln2)
            if L.fused:
                gt, up = L.gate_up_proj(x).split([L.inter_local, L.inter_local], -1)
            else:
                gt, up = L.gate_proj(x), L.up_proj(x)
            h = h + self._allreduce(L.down_proj(F.silu(gt) * up))
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

    def _row_parallel(self, lin: HelixLinear, x: torch.Tensor, sb: dict, out_key: str) -> torch.Tensor:
        """Row-parallel product + the sum over ranks, result in bf16 in sb[out_key]."""
        if self.p2p:
            lin.packed().matmul(x, torch.float32, out=sb["p32"])
            return self._ar(sb["p32"], out=sb[out_key])
        return self._allreduce(lin.packed().matmul(x, torch.bfloat16, out=sb[out_key]))

    def step_fused(self, tok: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        """One decode step for tok [B, 1] at position pos (int64 device tensor [1]): same
        arithmetic as ``forward_tokens(tok, pos, pos, None)`` with the glue between the
        linears in four fused operators.  Returns the logits [B, vocab]."""
        B = tok.shape[0]
        sb = self._step_buffers(B)
        D, eps = self.shp.head_dim, self.shp.rms_eps
        bf = torch.bfloat16
        h, x = sb["h"], sb["x"]
        h.copy_(self.embed[tok[:, 0]])
        delta = None
        for li, L in enumerate(self.layers):
            nq, nkv = L.n_q, L.n_kv
            decode_ops.add_rmsnorm(h, delta, L.ln1, eps, x)
            qkv, gu, ni = sb["qkv"], sb["gu"], L.inter_local
            if L.fused:
                L.qkv_proj.packed().matmul(x, bf, out=qkv)
            else:
                L.q_proj.packed().matmul(x, bf, out=qkv[:, : nq * D])
                L.k_proj.packed().matmul(x, bf, out=qkv[:, nq * D: (nq + nkv) * D])
                L.v_proj.packed().matmul(x, bf, out=qkv[:, (nq + nkv) * D:])
            decode_ops.rope_append(qkv, pos, self.cos, self.sin, sb["q"], self.k_cache[li], self.v_cache[li], nq, nkv)
            decode_ops.attn_decode(sb["q"], self.k_cache[li], self.v_cache[li], pos, sb["a"], nq, D ** -0.5)
            delta = self._row_parallel(L.o_proj, sb["a"], sb, "d1")
            decode_ops.add_rmsnorm(h, delta, L.ln2, eps, x)
            if L.fused:
                L.gate_up_proj.packed().matmul(x, bf, out=gu)
            else:
                L.gate_proj.packed().matmul(x, bf, out=gu[:, :ni])
                L.up_proj.packed().matmul(x, bf, out=gu[:, ni:])
            decode_ops.swiglu(gu[:, :ni], gu[:, ni:], sb["act"])
            delta = self._row_parallel(L.down_proj, sb["act"], sb, "d2")
        decode_ops.add_rmsnorm(h, delta, self.norm, eps, x)
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

        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                body()
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            out = body()

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


def main(argv=None):
    """``python -m helix_substrate_b200.qwen2_decode --shape 7b --batch 1 --prompt 2048 --new 128``
    (under torchrun for tensor parallel).  Prints one JSON line with decode
    tokens/s, ms per token and the HXQ bytes streamed per token."""
    import argparse
    import json
    import os
    import time
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
    ap.add_argument("--separate-proj", action="store_true",
                    help="q, k, v and gate, up as separate compressed matrices (7 products per layer instead of 4)")
    args = ap.parse_args(argv)
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.distributed.init_process_group("nccl", device_id=dev)
    shp = {"7b": Qwen2Shape.qwen25_7b, "14b": Qwen2Shape.qwen25_14b, "tiny": Qwen2Shape.tiny}[args.shape]()
    if args.layers:
        shp.layers = args.layers
    t0 = time.perf_counter()
    model = Qwen2HxqDecoder(shp, dev, args.batch, args.prompt + args.new + 8, rank=rank, world=world,
                            fuse_proj=not args.separate_proj, p2p_allreduce=args.allreduce == "p2p")
    torch.cuda.synchronize()
    build_s = time.perf_counter() - t0
    prompt = torch.randint(0, shp.vocab, (args.batch, args.prompt), device=dev,
                           generator=torch.Generator(device=dev).manual_seed(0))
    with torch.no_grad():
        p0, p1, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(4))
        p0.record()
        nxt = model.prefill(prompt)
        p1.record()
        if args.no_graph:
            run = None
        else:
            run, tok, pos = model.make_graphed_step(args.batch, fused=not args.torch_glue)
        torch.cuda.synchronize()
        # timed decode: new-1 graph replays
        e1.record()
        for i in range(args.new - 1):
            p = args.prompt + i
            if run is not None:
                tok.copy_(nxt[:, None])
                pos.fill_(p)
                nxt = run()
            else:
                pt = torch.tensor([p], device=dev)
                if args.torch_glue:
                    nxt = model.forward_tokens(nxt[:, None], pt, pt, None).argmax(-1)
                else:
                    nxt = model.step_fused(nxt[:, None], pt).argmax(-1)
        e2.record()
        torch.cuda.synchronize()
    ms_dec = e1.elapsed_time(e2) / (args.new - 1)
    t = torch.tensor([ms_dec], device=dev, dtype=torch.float64)
    if world > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    ms_dec = float(t.item())
    hxq_bytes = sum(m.packed().algorithmic_bytes(args.batch, 2, 2) for m in model.modules()
                    if isinstance(m, HelixLinear))
    if rank == 0:
        print(json.dumps({
            "metric": "decode_tokens_per_s", "value": args.batch * 1000.0 / ms_dec, "unit": "tok/s",
            "ms_per_token_step": ms_dec, "batch": args.batch, "prompt": args.prompt, "new_tokens": args.new,
            "shape": args.shape, "layers": shp.layers, "n_gpus": world, "launch": "python" if run is None else "cuda_graph",
            "glue": "torch" if args.torch_glue else "fused",
            "projections": "q,k,v,o,gate,up,down" if args.separate_proj else "qkv,o,gate_up,down",
            "allreduce": (args.allreduce if world > 1 else None),
            "hxq_algorithmic_bytes_per_step_per_gpu": hxq_bytes,
            "hxq_GBps_per_gpu_if_all_time_were_linears": hxq_bytes / (ms_dec * 1e-3) / 1e9,
            "prefill_ms": p0.elapsed_time(p1), "build_s": build_s,
            "data": "synthetic: N(0,0.02) weights, uniform random prompt ids",
        }), flush=True)
    if world > 1:   # no process-group teardown while graphs holding its collectives are alive (it blocks)
        import sys
        torch.cuda.synchronize()
        torch.distributed.barrier()
        sys.stdout.flush()
        os._exit(0)


if __name__ == "__main__":
    main()
