"""Child program of tests/test_gpu_allreduce.py: every rank compares hxq_allreduce_oneshot with
an NCCL all-reduce of the same fp32 partials, eagerly and replayed from a CUDA graph."""

import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    from helix_substrate_b200.tp import OneShotAllReduce
    n = 3584 * 4
    ar = OneShotAllReduce(n, dev)
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    for it in range(20):
        x = torch.randn(n, device=dev, generator=g)
        y = ar(x)
        ref = x.clone()
        dist.all_reduce(ref)
        assert (y.float() - ref).abs().max().item() <= 0.02 * ref.abs().max().item() + 1e-3, f"iteration {it}"
        ys = [torch.empty_like(y) for _ in range(world)]
        dist.all_gather(ys, y)
        assert all(torch.equal(ys[0], t) for t in ys), "ranks must hold identical sums"
    # captured: the call number lives in device memory, so replays stay in step
    x = torch.randn(n, device=dev, generator=g)
    out = torch.empty(n, device=dev, dtype=torch.bfloat16)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        ar(x, out=out)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        ar(x, out=out)
    ref = x.clone()
    dist.all_reduce(ref)
    for _ in range(10):
        out.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert (out.float() - ref).abs().max().item() <= 0.02 * ref.abs().max().item() + 1e-3
    assert ar.check_status() == 0
    # the same exchange with the residual add and the RMSNorm folded in, against NCCL + the separate operator
    from helix_substrate_b200 import decode_ops
    M, H = 4, 3584
    ar2 = OneShotAllReduce(M * H, dev)
    w = (1.0 + 0.1 * torch.randn(H, device=dev, generator=torch.Generator(device=dev).manual_seed(5))).bfloat16()
    h = torch.randn(M, H, device=dev, generator=torch.Generator(device=dev).manual_seed(6)).bfloat16()
    h_ref = h.clone()
    for it in range(5):
        part = torch.randn(M, H, device=dev, generator=g)
        x = torch.empty(M, H, device=dev, dtype=torch.bfloat16)
        ar2.add_rmsnorm(part, h, w, 1e-6, x)
        tot = part.clone()
        dist.all_reduce(tot)
        x_ref = torch.empty_like(x)
        decode_ops.add_rmsnorm(h_ref, tot.bfloat16(), w, 1e-6, x_ref)
        assert (h.float() - h_ref.float()).abs().max().item() <= 0.02 * h_ref.float().abs().max().item() + 1e-3, it
        assert (x.float() - x_ref.float()).abs().max().item() <= 0.05 * x_ref.float().abs().max().item() + 1e-3, it
        h_ref.copy_(h)     # the two sums may differ in the last bit (fixed rank order vs NCCL's): keep them in step
    assert ar2.check_status() == 0
    torch.cuda.synchronize()
    dist.barrier()
    if rank == 0:
        print("ALLREDUCE-OK", flush=True)
    sys.stdout.flush()
    del graph
    from helix_substrate_b200.qwen2_decode import leave_process_group
    leave_process_group()


if __name__ == "__main__":
    main()
