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
    """Contiguous slice [a, b) of ``n`` for ``rank``; every slice but the last
    has ceil(n / world) rounded up to ``multiple`` elements."""
    per = -(-n // world)
    per = -(-per // multiple) * multiple
    return min(rank * per, n), min((rank + 1) * per, n)


def shard_helix_linear(mod: HelixLinear, mode: str, rank: int, world: int) -> HelixLinear:
    """The shard of ``mod`` that ``rank`` of ``world`` holds.

    ``mode="column"``: rows [r0, r1) of the weight (outputs split).
    ``mode="row"``:   columns [c0, c1) (inputs split, 16-column granularity);
    the result carries ``col0 = c0`` and is a partial sum - use
    RowParallelHelixLinear (or all-reduce yourself).  Bias stays on rank 0."""
    if mode not in ("column", "row"):
        raise ValueError(f"mode must be 'column' or 'row', got {mode!r}")
    if mod.has_svd or mod.has_channel_scales:
        raise NotImplementedError("SVD residual / channel scales are not sharded")
    n_out, n_in, G = mod.out_features, mod.in_features, mod.group_size
    idx = mod.indices
    pos, vals = mod.sidecar_positions, mod.sidecar_values
    kw = {}
    if mode == "column":
        r0, r1 = shard_bounds(n_out, rank, world)
        new_idx = idx[r0:r1].contiguous()
        if pos is not None:
            keep = (pos >= r0 * n_in) & (pos < r1 * n_in)
            kw.update(sidecar_positions=(pos[keep] - r0 * n_in).contiguous(), sidecar_values=vals[keep].contiguous())
        if mod.group_scales is not None:
            kw.update(group_scales=mod.group_scales[r0:r1].contiguous(),
                      group_offsets=mod.group_offsets[r0:r1].contiguous(), group_size=G)
        bias = None if mod.bias is None else mod.bias[r0:r1].contiguous()
        out = HelixLinear(n_in, r1 - r0, mod.codebook, new_idx, bias=bias, tensor_name=mod.tensor_name,
                          compute_dtype=mod.compute_dtype, **kw)
        out.tp_mode, out.tp_slice = "column", (r0, r1)
        return out
    c0, c1 = shard_bounds(n_in, rank, world, multiple=16)
    new_idx = idx[:, c0:c1].contiguous()
    if pos is not None:
        rows, cols = pos // n_in, pos % n_in
        keep = (cols >= c0) & (cols < c1)
        kw.update(sidecar_positions=(rows[keep] * (c1 - c0) + (cols[keep] - c0)).contiguous(),
                  sidecar_values=vals[keep].contiguous())
    if mod.group_scales is not None:
        g0, g1 = c0 // G, (c1 - 1) // G + 1   # boundary groups are duplicated on both neighbours
        kw.update(group_scales=mod.group_scales[:, g0:g1].contiguous(),
                  group_offsets=mod.group_offsets[:, g0:g1].contiguous(), group_size=G)
    bias = mod.bias if rank == 0 else None
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


class RowParallelHelixLinear(nn.Module):
    """Row-parallel shard + the sum over ranks.  ``x`` is this rank's slice of
    the input features; the result is the full output on every rank."""

    def __init__(self, shard: HelixLinear, group: Optional["torch.distributed.ProcessGroup"] = None):
        super().__init__()
        self.shard, self.group = shard, group
        self.in_features, self.out_features = shard.in_features, shard.out_features

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        import torch.distributed as dist
        y = self.shard(x)
        if dist.is_available() and dist.is_initialized() and dist.get_world_size(self.group) > 1:
            dist.all_reduce(y, op=dist.ReduceOp.SUM, group=self.group)
        return y
