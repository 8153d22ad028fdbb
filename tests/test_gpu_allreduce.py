"""hxq_allreduce_oneshot: on one GPU the other ranks are played by the test (their partials and
flags are written into this rank's receive buffer before the call, so nothing ever waits on
another launch); with two or more GPUs the real exchange runs as child processes against NCCL."""

import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _dev():
    return torch.device("cuda:0")


@pytest.mark.parametrize("n", [3584, 5001, 57344])
def test_single_rank_rounds_its_own_partial(n):
    from helix_substrate_b200.tp import OneShotAllReduce
    ar = OneShotAllReduce.local_emulation(1, 0, n, _dev())
    g = torch.Generator(device=_dev()).manual_seed(n)
    for _ in range(3):   # three calls: both slots, advancing call numbers
        x = torch.randn(n, device=_dev(), generator=g)
        y = ar(x)
        assert torch.equal(y, x.bfloat16())
    assert ar.check_status() == 0


@pytest.mark.parametrize("world,rank,n", [(2, 0, 3584), (4, 2, 5001), (8, 7, 20480)])
def test_sum_in_rank_order_with_the_other_ranks_played_by_the_test(world, rank, n):
    from helix_substrate_b200.tp import OneShotAllReduce
    dev = _dev()
    ar = OneShotAllReduce.local_emulation(world, rank, n, dev)
    data, flags = ar.views()
    g = torch.Generator(device=dev).manual_seed(world * 100 + rank)
    n_cta = -(-n // 4096)
    for call in (1, 2, 3):
        slot = call & 1
        parts = [torch.randn(n, device=dev, generator=g) for _ in range(world)]
        for p in range(world):
            if p != rank:   # what rank p's push would have left here
                data[slot, p, :n] = parts[p]
                flags[slot, p, :n_cta] = call
        torch.cuda.synchronize()
        y = ar(parts[rank])
        ref = torch.zeros(n, device=dev)
        for p in range(world):
            ref = ref + parts[p]
        assert torch.equal(y, ref.bfloat16()), f"call {call}"
        # and this rank's push reached every other rank's buffer, with its flag
        for p in range(world):
            d, f = ar.views(p)
            assert torch.equal(d[slot, rank, :n], parts[rank]) and int(f[slot, rank, 0]) == call
    assert ar.check_status() == 0


@pytest.mark.parametrize("world,rank,M,H", [(1, 0, 1, 3584), (2, 1, 1, 3584), (4, 2, 3, 3584), (8, 5, 24, 5120), (2, 0, 40, 2048), (2, 0, 5, 264)])
def test_sum_with_residual_add_and_rmsnorm_folded_in(world, rank, M, H):
    """hxq_allreduce_add_rmsnorm against the two separate operators it replaces, bit for bit, with the
    other ranks played by the test (one CTA owns whole rows: min(M, 32) flags per source rank)."""
    from helix_substrate_b200 import decode_ops
    from helix_substrate_b200.tp import OneShotAllReduce
    dev = _dev()
    n = M * H
    fused = OneShotAllReduce.local_emulation(world, rank, n, dev)
    plain = OneShotAllReduce.local_emulation(world, rank, n, dev)
    g = torch.Generator(device=dev).manual_seed(world * 1000 + M)
    w = (1.0 + 0.1 * torch.randn(H, device=dev, generator=g)).bfloat16()
    h_f = torch.randn(M, H, device=dev, generator=g).bfloat16()
    h_p = h_f.clone()
    n_cta_rows, n_cta_flat = min(M, 32), -(-n // 4096)
    for call in (1, 2, 3):
        slot = call & 1
        parts = [torch.randn(M, H, device=dev, generator=g) for _ in range(world)]
        for ar, n_cta in ((fused, n_cta_rows), (plain, n_cta_flat)):
            data, flags = ar.views()
            for p in range(world):
                if p != rank:
                    data[slot, p, :n] = parts[p].reshape(-1)
                    flags[slot, p, :n_cta] = call
        torch.cuda.synchronize()
        x_f = torch.empty(M, H, device=dev, dtype=torch.bfloat16)
        fused.add_rmsnorm(parts[rank], h_f, w, 1e-6, x_f)
        delta = plain(parts[rank].reshape(-1)).view(M, H)
        x_p = torch.empty_like(x_f)
        decode_ops.add_rmsnorm(h_p, delta, w, 1e-6, x_p)
        assert torch.equal(h_f, h_p), f"call {call}: residual stream"
        assert torch.equal(x_f, x_p), f"call {call}: normalised row"
        for p in range(world):   # the push reached every rank's buffer, with the flags of all row CTAs
            d, f = fused.views(p)
            assert torch.equal(d[slot, rank, :n], parts[rank].reshape(-1))
            assert bool((f[slot, rank, :n_cta_rows] == call).all())
    assert fused.check_status() == 0


def test_a_wait_that_runs_out_reports_and_leaves_the_context_usable():
    from helix_substrate_b200 import _lib
    from helix_substrate_b200.tp import OneShotAllReduce
    dev = _dev()
    ar = OneShotAllReduce.local_emulation(2, 0, 4096, dev, wait_ms=2.0)   # nobody plays rank 1
    out = torch.full((4096,), 7.0, device=dev, dtype=torch.bfloat16)
    ar(torch.ones(4096, device=dev), out=out)
    assert ar.check_status() == _lib.HXQ_E_TIMEOUT
    assert bool((out == 7.0).all()), "the output must be left untouched"
    assert float((torch.ones(8, device=dev) * 2).sum()) == 16.0


def test_argument_checks():
    import ctypes as C
    from helix_substrate_b200 import _lib
    L = _lib.lib()
    assert L.hxq_allreduce_buffer_bytes(9, 1024) == 0 and L.hxq_allreduce_flag_bytes(0) == 0
    assert L.hxq_allreduce_oneshot(None, None, 0, 1, 8, None, None, 8, None, 0, None, None) == _lib.HXQ_E_ARG


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_against_nccl():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1", PYTHONPATH=str(ROOT))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29531", str(ROOT / "tests" / "allreduce_ranks.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "ALLREDUCE-OK" in r.stdout
