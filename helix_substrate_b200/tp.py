"""Tensor-parallel sharding of HelixLinear over the GPUs of one node.

One process per GPU.  Column-parallel layers (q, k, v, gate, up) own a slice of
output rows and need no exchange; row-parallel layers (o, down) own a slice of
input columns and their partial outputs are summed with one all-reduce over
NCCL / NVLink.  The reference has no multi-GPU path; this is the partitioning
that follows from its data layout: sidecar positions are row-major and sorted,
so a row slice is a contiguous run of them, and a column slice keeps ``col0``
so that affine group ids stay global even when the slice starts mid-group.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn as nn

from .helix_linear import HelixLinear


def shard_bounds(n: int, rank: int, world: int, multiple: int = 1) -> Tuple[int, int]:
    """Contiguous slice [a, b) of ``n`` for ``rank``: ``n`` is dealt in units of ``multiple``
    elements as evenly as they go (the first ranks hold one unit more; the last slice ends at n)."""
    units = -(-n // multiple)
    base, extra = divmod(units, world)
    a = (rank * base + min(rank, extra)) * multiple
    b = ((rank + 1) * base + min(rank + 1, extra)) * multiple
    return min(a, n), min(b, n)


def take_rows(mod: HelixLinear, ranges) -> HelixLinear:
    """A new HelixLinear holding the output rows ``[(r0, r1), ...]`` of ``mod``, concatenated in
    the order given (one codebook, so several projections compressed jointly - q|k|v, gate|up -
    shard by picking each one's rows).  Sidecar positions are row-major and sorted, so each range
    is one contiguous run of them."""
    if mod.has_svd or mod.has_channel_scales:
        raise NotImplementedError("SVD residual / channel scales are not sharded")
    n_in, G = mod.in_features, mod.group_size
    ranges = [(int(a), int(b)) for a, b in ranges if b > a]
    idx = torch.cat([mod.indices[a:b] for a, b in ranges]).contiguous()
    kw = {}
    pos, vals = mod.sidecar_positions, mod.sidecar_values
    if pos is not None:
        ps, vs, base = [], [], 0
        for a, b in ranges:
            lo, hi = torch.searchsorted(pos, torch.tensor([a * n_in, b * n_in], device=pos.device)).tolist()
            ps.append(pos[lo:hi] - a * n_in + base * n_in)
            vs.append(vals[lo:hi])
            base += b - a
        kw.update(sidecar_positions=torch.cat(ps).contiguous(), sidecar_values=torch.cat(vs).contiguous())
    if mod.group_scales is not None:
        kw.update(group_scales=torch.cat([mod.group_scales[a:b] for a, b in ranges]).contiguous(),
                  group_offsets=torch.cat([mod.group_offsets[a:b] for a, b in ranges]).contiguous(), group_size=G)
    bias = None if mod.bias is None else torch.cat([mod.bias[a:b] for a, b in ranges]).contiguous()
    out = HelixLinear(n_in, idx.shape[0], mod.codebook, idx, bias=bias, tensor_name=mod.tensor_name,
                      compute_dtype=mod.compute_dtype, **kw)
    out.tp_mode, out.tp_slice = "column", ranges
    return out


def take_cols(mod: HelixLinear, c0: int, c1: int, keep_bias: bool = True) -> HelixLinear:
    """A new HelixLinear over input columns [c0, c1) of ``mod`` (a partial sum of the full
    product).  ``c0`` must be a multiple of 16; the result carries ``col0 = c0`` so that affine
    group ids stay global, and the groups cut by the bounds live on both neighbours."""
    if mod.has_svd or mod.has_channel_scales:
        raise NotImplementedError("SVD residual / channel scales are not sharded")
    if c0 % 16:
        raise ValueError("column shards start on a multiple of 16")
    n_out, n_in, G = mod.out_features, mod.in_features, mod.group_size
    kw = {}
    new_idx = mod.indices[:, c0:c1].contiguous()
    pos, vals = mod.sidecar_positions, mod.sidecar_values
    if pos is not None:
        rows, cols = pos // n_in, pos % n_in
        keep = (cols >= c0) & (cols < c1)
        kw.update(sidecar_positions=(rows[keep] * (c1 - c0) + (cols[keep] - c0)).contiguous(),
                  sidecar_values=vals[keep].contiguous())
    if mod.group_scales is not None:
        g0, g1 = c0 // G, (c1 - 1) // G + 1   # boundary groups are duplicated on both neighbours
        kw.update(group_scales=mod.group_scales[:, g0:g1].contiguous(),
                  group_offsets=mod.group_offsets[:, g0:g1].contiguous(), group_size=G)
    bias = mod.bias if keep_bias else None
    out = HelixLinear.__new__(HelixLinear)
    nn.Module.__init__(out)
    out._init_attrs(c1 - c0, n_out, mod.tensor_name, mod.compute_dtype, 1)
    out.group_size, out.col0 = (G if mod.group_scales is not None else 0), c0
    out.register_buffer("codebook", mod.codebook.clone())
    out.register_buffer("indices", new_idx)
    for name in ("sidecar_positions", "sidecar_values", "group_scales", "group_offsets"):
        out.register_buffer(name, kw.get(name))
    for name in ("svd_U", "svd_s", "svd_Vt", "channel_scales"):
        out.register_buffer(name, None)
    out.register_buffer("bias", None if bias is None else bias.clone())
    for name in ("codebook_f16", "_sidecar_vq_vals", "_sidecar_rows", "_sidecar_cols", "_sidecar_deltas",
                 "_csr_rowptr", "_csr_cols"):
        out.register_buffer(name, None, persistent=False)
    out._derive()
    out.tp_mode, out.tp_slice = "row", (c0, c1)
    return out


def shard_helix_linear(mod: HelixLinear, mode: str, rank: int, world: int,
                       multiple: Optional[int] = None) -> HelixLinear:
    """The shard of ``mod`` that ``rank`` of ``world`` holds.

    ``mode="column"``: rows [r0, r1) of the weight (outputs split).
    ``mode="row"``:   columns [c0, c1) (inputs split, 16-column granularity);
    the result carries ``col0 = c0`` and is a partial sum - use
    RowParallelHelixLinear (or all-reduce yourself).  Bias stays on rank 0.

    ``multiple`` rounds every shard but the last up to that many rows / columns (default 1 for
    rows, 16 for columns).  A column-parallel layer feeding a row-parallel one must be cut with
    the same value; cutting an MLP at ``multiple=128`` keeps every shard of ``down`` on whole
    affine groups, which is the shape the streaming kernel is fastest on."""
    if mode not in ("column", "row"):
        raise ValueError(f"mode must be 'column' or 'row', got {mode!r}")
    if mode == "column":
        r0, r1 = shard_bounds(mod.out_features, rank, world, multiple or 1)
        out = take_rows(mod, [(r0, r1)])
        out.tp_slice = (r0, r1)
        return out
    if multiple is not None and multiple % 16:
        raise ValueError("column shards are cut at multiples of 16")
    c0, c1 = shard_bounds(mod.in_features, rank, world, multiple or 16)
    return take_cols(mod, c0, c1, keep_bias=(rank == 0))


def head_partition(heads: int, kv_heads: int, world: int):
    """Attention heads per tensor-parallel rank: a list of ``(q0, q1, kv0, kv1)``, rank r owning
    query heads [q0, q1) and KV heads [kv0, kv1).

    While ``world`` divides the KV heads every rank gets whole KV groups.  Beyond that
    (``world`` a multiple of the KV heads, e.g. 28 query / 4 KV heads on 8 GPUs) each KV head is
    held by ``world / kv_heads`` ranks and its query heads are dealt over them as evenly as
    they go (7 -> 4 + 3): ranks then differ by one query head, nothing is padded, and the
    row-parallel o_proj sums partials of different input widths."""
    if heads % kv_heads:
        raise ValueError(f"{heads} query heads are not a multiple of {kv_heads} KV heads")
    gq = heads // kv_heads
    if kv_heads % world == 0:
        k = kv_heads // world
        return [(r * k * gq, (r + 1) * k * gq, r * k, (r + 1) * k) for r in range(world)]
    if world % kv_heads:
        raise ValueError(f"tensor-parallel {world} neither divides nor is a multiple of {kv_heads} KV heads")
    rep = world // kv_heads
    if rep > gq:
        raise ValueError(f"{world} ranks for {heads} query heads: some rank would hold none")
    per = -(-gq // rep)
    out = []
    for r in range(world):
        kv, j = r // rep, r % rep
        out.append((kv * gq + min(j * per, gq), kv * gq + min((j + 1) * per, gq), kv, kv + 1))
    return out


class RowParallelHelixLinear(nn.Module):
    """Row-parallel shard + the sum over ranks.  ``x`` is this rank's slice of
    the input features; the result is the full output on every rank.  With
    ``oneshot`` (a OneShotAllReduce sized for tokens x out_features) decode-sized
    calls sum fp32 partials over peer memory; anything larger goes through NCCL."""

    def __init__(self, shard: HelixLinear, group: Optional["torch.distributed.ProcessGroup"] = None,
                 oneshot: Optional["OneShotAllReduce"] = None):
        super().__init__()
        self.shard, self.group, self.oneshot = shard, group, oneshot
        self.in_features, self.out_features = shard.in_features, shard.out_features

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        import torch.distributed as dist
        multi = dist.is_available() and dist.is_initialized() and dist.get_world_size(self.group) > 1
        if multi and self.oneshot is not None and x.is_cuda and x.dtype == torch.bfloat16:
            x2 = x.reshape(-1, self.in_features)
            if x2.shape[0] * self.out_features <= self.oneshot.n_max and x2.shape[0] <= 16:
                part = self.shard.packed().matmul(x2, torch.float32)
                return self.oneshot(part).view(*x.shape[:-1], self.out_features)
        y = self.shard(x)
        if multi:
            dist.all_reduce(y, op=dist.ReduceOp.SUM, group=self.group)
        return y


class OneShotAllReduce:
    """Sum of fp32 partials over the tensor-parallel ranks of one node for decode-sized
    messages (up to 131072 elements): one kernel per rank over peer memory
    (``hxq_allreduce_oneshot``), result in bf16, identical on every rank.

    The receive buffers are symmetric memory (``torch.distributed._symmetric_memory``): the
    same allocation on every GPU, mapped into every process.  ``local_emulation`` builds the
    same object from plain tensors of ONE GPU, for tests that play the other ranks by
    writing their partials and flags into this rank's buffer before the call."""

    def __init__(self, n_max: int, device, group=None, wait_ms: float = 1000.0):
        import os
        import torch.distributed as dist
        # plain peer mappings are all the kernel uses: do not bind the buffer to an NVLink multicast object
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm
        from . import _lib
        group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self._setup_sizes(n_max)
        self.mem = symm.empty(self._nbuf + self._nflag, dtype=torch.uint8, device=device)
        self.mem.zero_()
        hdl = symm.rendezvous(self.mem, group=group)
        self._finish([int(p) for p in hdl.buffer_ptrs], device, wait_ms)
        torch.cuda.synchronize(device)
        dist.barrier(group)      # nobody pushes before everybody's buffer is zero

    def _setup_sizes(self, n_max: int) -> None:
        from . import _lib
        L = _lib.lib()
        self.n_max = -(-int(n_max) // 8) * 8
        self._nbuf = L.hxq_allreduce_buffer_bytes(self.world, self.n_max)
        self._nflag = L.hxq_allreduce_flag_bytes(self.world)
        if self._nbuf == 0 or self._nflag == 0:
            raise ValueError(f"unsupported world size {self.world} (1..8) or message size {n_max}")

    def _finish(self, ptrs, device, wait_ms: float) -> None:
        import ctypes as C
        self._bufs = (C.c_void_p * self.world)(*ptrs)
        self._flags = (C.c_void_p * self.world)(*[p + self._nbuf for p in ptrs])
        self.counters = torch.zeros(32, dtype=torch.int32, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self.wait_cycles = int(wait_ms * 1.9e6)
        self.device = device

    @classmethod
    def local_emulation(cls, world: int, rank: int, n_max: int, device, wait_ms: float = 1000.0):
        self = cls.__new__(cls)
        self.world, self.rank = world, rank
        self._setup_sizes(n_max)
        self.mems = [torch.zeros(self._nbuf + self._nflag, dtype=torch.uint8, device=device) for _ in range(world)]
        self.mem = self.mems[rank]
        self._finish([m.data_ptr() for m in self.mems], device, wait_ms)
        return self

    def views(self, r: int = None):
        """(partials fp32 [2, world, n_max], flags int32 [2, world, 32]) of rank r's buffer
        (only ``local_emulation`` can look at other ranks')."""
        mem = self.mem if r is None or r == self.rank else self.mems[r]
        return (mem[: self._nbuf].view(torch.float32).view(2, self.world, self.n_max),
                mem[self._nbuf:].view(torch.int32).view(2, self.world, 32))

    def __call__(self, partial: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        import ctypes as C
        from . import _lib
        assert partial.is_cuda and partial.dtype == torch.float32 and partial.is_contiguous()
        n = partial.numel()
        if out is None:
            out = torch.empty(partial.shape, dtype=torch.bfloat16, device=partial.device)
        assert out.dtype == torch.bfloat16 and out.is_contiguous() and out.numel() == n
        with torch.cuda.device(self.device):
            st = _lib.lib().hxq_allreduce_oneshot(
                self._bufs, self._flags, self.rank, self.world, self.n_max, C.c_void_p(partial.data_ptr()),
                C.c_void_p(out.data_ptr()), n, C.c_void_p(self.counters.data_ptr()), self.wait_cycles,
                C.c_void_p(self.status.data_ptr()), C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream))
        _lib.check(st, "hxq_allreduce_oneshot")
        return out

    def add_rmsnorm(self, partial: torch.Tensor, h: torch.Tensor, weight: torch.Tensor, eps: float,
                    out: torch.Tensor) -> torch.Tensor:
        """The sum over ranks of ``partial`` [M, H] (fp32) added to the residual stream ``h`` in place
        and RMS-normalised into ``out`` (both bf16 [M, H]) - ``hxq_allreduce_add_rmsnorm``, bit-identical
        to ``self(partial)`` followed by ``decode_ops.add_rmsnorm``.  An object used for this call must not
        also be used for plain sums (one CTA owns rows here, 4096-element slices there)."""
        import ctypes as C
        from . import _lib
        assert partial.is_cuda and partial.dtype == torch.float32 and partial.is_contiguous() and partial.ndim == 2
        M, H = partial.shape
        for t in (h, out):
            assert t.dtype == torch.bfloat16 and t.shape == (M, H) and t.stride(1) == 1
        assert weight.dtype == torch.bfloat16 and weight.numel() == H and weight.is_contiguous()
        with torch.cuda.device(self.device):
            st = _lib.lib().hxq_allreduce_add_rmsnorm(
                self._bufs, self._flags, self.rank, self.world, self.n_max, C.c_void_p(partial.data_ptr()), M, H,
                C.c_void_p(h.data_ptr()), h.stride(0), C.c_void_p(weight.data_ptr()), C.c_void_p(out.data_ptr()),
                out.stride(0), float(eps), C.c_void_p(self.counters.data_ptr()), self.wait_cycles,
                C.c_void_p(self.status.data_ptr()), C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream))
        _lib.check(st, "hxq_allreduce_add_rmsnorm")
        return out

    def check_status(self) -> int:
        """0, or HXQ_E_TIMEOUT if a rank gave up waiting for the others (synchronises)."""
        return int(self.status.item())

