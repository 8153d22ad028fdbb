"""Tensor-parallel host path with two CPU ranks over gloo: shard descriptors,
the row-parallel all-reduce wrapper and the column-parallel concatenation.  The
per-shard product is done by the CPU oracle here (there is no GPU in this
test); what is under test is the partitioning and the exchange."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import hxq_oracle as O


def _oracle_forward(m, x):
    r = None if m._sidecar_rows is None else m._sidecar_rows.numpy()
    y = O.forward_f64(x.numpy(), m.codebook.numpy(), m.indices.numpy(), r,
                      None if r is None else m._sidecar_cols.numpy(),
                      None if r is None else m._sidecar_deltas.numpy(),
                      None if m.bias is None else m.bias.numpy(),
                      None if m.group_scales is None else m.group_scales.numpy(),
                      None if m.group_offsets is None else m.group_offsets.numpy(), m.group_size,
                      m.col0 % m.group_size if m.group_size else 0)
    return torch.from_numpy(y)


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from helix_substrate_b200 import HelixLinear, hxq_writer_gpu as W
        from helix_substrate_b200.tp import shard_helix_linear, RowParallelHelixLinear
        hidden, inter = 256, 1184  # 1184 / 2 = 592 = 4.625 groups: the split lands mid-group
        torch.manual_seed(0)
        up = HelixLinear(hidden, inter, **W.compress_weight(W.student_t_weight((inter, hidden), 1, "cpu"),
                                                            percentile=99.5, group_size=128))
        down = HelixLinear(inter, hidden, bias=torch.randn(hidden),
                           **W.compress_weight(W.student_t_weight((hidden, inter), 2, "cpu"), percentile=99.5,
                                               group_size=0))
        x = torch.randn(3, hidden, generator=torch.Generator().manual_seed(5))
        full = _oracle_forward(down, _oracle_forward(up, x).float())

        up_s = shard_helix_linear(up, "column", rank, world)
        down_s = shard_helix_linear(down, "row", rank, world)
        assert up_s.tp_slice == down_s.tp_slice, "column slice of up must feed the row slice of down"
        down_s.forward = lambda xx, m=down_s: _oracle_forward(m, xx)   # CPU stand-in for the kernel
        y = RowParallelHelixLinear(down_s)(_oracle_forward(up_s, x).float())  # partial product + all-reduce
        err = float((y - full).abs().max())
        # column-parallel outputs gathered across ranks equal the unsharded layer
        parts = [torch.zeros(3, up_s.out_features, dtype=torch.float64) for _ in range(world)]
        dist.all_gather(parts, _oracle_forward(up_s, x))
        err2 = float((torch.cat(parts, 1) - _oracle_forward(up, x)).abs().max())
        q.put((rank, err, err2, down_s.bias is not None))
    finally:
        dist.destroy_process_group()


def test_two_rank_tensor_parallel_mlp():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    res = sorted(q.get(timeout=5) for _ in range(2))
    for rank, err, err2, has_bias in res:
        assert err < 1e-9 and err2 < 1e-9
        assert has_bias == (rank == 0), "the bias of a row-parallel layer lives on rank 0 only"
