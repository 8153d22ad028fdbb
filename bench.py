#!/usr/bin/env python3
"""Benchmark of the HXQ compressed-linear forward path on B200.

Workload (BASELINE configs[1]): the grouped-affine HXQ linears of a
Qwen2.5-7B MLP - gate/up [18944, 3584] and down [3584, 18944], k=256 codebook,
group-128 fp32 scale/offset, ~0.1 % outlier sidecar - for every one of L layers
with DISTINCT weights, M=1 bf16 activations.  One step = one pass over all 3*L
linears (3*L kernel launches, ~73 MB of indices each, far larger than L2
together).  Metric: algorithmic GB/s of the VQ-GEMV.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--layers L] [--m M]
    python bench.py --impl reference      # the CPU path, timed on the host cores

Prints ONE JSON line on rank 0.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

HIDDEN, INTER, GROUP = 3584, 18944, 128
METRIC = "hxq_vq_gemv_algorithmic_GBps_M1_qwen2.5-7b_mlp"


def _peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.rows, self.proc, self.idx = [], None, gpu_index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.idx}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx = max(mx, float(r[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


def build_layers(n_layers: int, device, seed0: int = 0, tp_rank: int = 0, tp_world: int = 1):
    """Distinct compressed gate/up/down modules per layer (column-parallel
    gate/up and row-parallel down when tp_world > 1)."""
    import torch
    from helix_substrate_b200 import HelixLinear
    from helix_substrate_b200.hxq_writer_gpu import compress_weight, student_t_weight
    from helix_substrate_b200.tp import shard_helix_linear
    layers = []
    for l in range(n_layers):
        mods = {}
        for j, (name, shape) in enumerate((("gate", (INTER, HIDDEN)), ("up", (INTER, HIDDEN)),
                                           ("down", (HIDDEN, INTER)))):
            w = student_t_weight(shape, seed0 + 3 * l + j, device)
            enc = compress_weight(w, percentile=99.95, group_size=GROUP)
            del w
            mod = HelixLinear(shape[1], shape[0], tensor_name=f"model.layers.{l}.mlp.{name}_proj.weight", **enc)
            if tp_world > 1:
                mod = shard_helix_linear(mod, "row" if name == "down" else "column", tp_rank, tp_world)
            mods[name] = mod.to(device)
        layers.append(mods)
        torch.cuda.empty_cache()
    return layers


def algorithmic_bytes(layers, M: int, act_bytes: int) -> int:
    return sum(mod.packed().algorithmic_bytes(M, act_bytes, act_bytes)
               for lay in layers for mod in lay.values())


def cpu_forward_sample(seconds_target: float = 15.0, threads=None):
    """The reference's CPU path (gather, group affine, fp32 matmul in 256-row
    tiles: the oracle's restatement of HelixLinear._forward_naive with
    affine_group_matmul_reference semantics) timed on the host cores for one
    MLP layer's three linears at M=1."""
    import numpy as np
    import torch
    from oracle import hxq_oracle as O
    n_thr = threads or len(os.sched_getaffinity(0))
    torch.set_num_threads(n_thr)
    rng = np.random.default_rng(0)
    cases = []
    for shape in ((INTER, HIDDEN), (INTER, HIDDEN), (HIDDEN, INTER)):
        n_out, n_in = shape
        cb = np.sort(rng.standard_normal(256)).astype(np.float32) * 0.02
        idx = rng.integers(0, 256, shape, dtype=np.uint8)
        s = (1 + 0.1 * rng.standard_normal((n_out, n_in // GROUP))).astype(np.float32)
        t = (0.002 * rng.standard_normal((n_out, n_in // GROUP))).astype(np.float32)
        nnz = n_out * n_in // 1000
        pos = np.sort(rng.choice(n_out * n_in, nnz, replace=False))
        rows, cols = pos // n_in, pos % n_in
        deltas = (0.05 * rng.standard_normal(nnz)).astype(np.float32)
        x = rng.standard_normal((1, n_in)).astype(np.float32)
        cases.append((x, cb, idx, rows, cols, deltas, s, t))
    nbytes = sum(c[2].size + 1024 + c[6].size * 8 + len(c[3]) * 8 + (c[2].shape[0] + 1) * 4
                 + 2 * c[2].shape[1] + 2 * c[2].shape[0] for c in cases)

    def one_pass():
        for (x, cb, idx, rows, cols, deltas, s, t) in cases:
            O.forward_naive_torch(x, cb, idx, rows, cols, deltas, None, s, t, GROUP)

    one_pass()
    t0 = time.perf_counter()
    one_pass()
    dt1 = time.perf_counter() - t0
    reps = max(2, min(50, int(seconds_target / max(dt1, 1e-3))))
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        one_pass()
        times.append(time.perf_counter() - t0)
    times.sort()
    med = times[len(times) // 2]
    return {"value": nbytes / med / 1e9, "unit": "GB/s", "cores": n_thr, "kind": "port",
            "sample": f"1 of the MLP layers (gate+up+down, M=1, fp32), median of {reps} passes, "
                      f"{med * 1e3:.1f} ms per pass", "ms_per_layer": med * 1e3, "bytes": nbytes}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    t0 = time.perf_counter()
    cpu = cpu_forward_sample(seconds_target=max(3.0, 1.5 * args.steps))
    line = {
        "impl": "reference", "metric": METRIC, "value": cpu["value"], "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": cpu["ms_per_layer"] * args.layers,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": "qwen2.5-7b MLP gate/up/down HXQ linears (k=256, group-128 affine, 0.1% sidecar), "
                               "M=1; CPU restatement of the reference's _forward_naive timed on one layer",
                   "layers": args.layers, "m": 1},
        "cpu_baseline": {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": cpu["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "wall_s": time.perf_counter() - t0,
    }
    print(json.dumps(line), flush=True)


PREFILL_SHAPES = (("q", 3584, 3584), ("k", 512, 3584), ("v", 512, 3584), ("o", 3584, 3584),
                  ("gate", 18944, 3584), ("up", 18944, 3584), ("down", 3584, 18944))


def run_prefill(args):
    """Secondary workload (BASELINE configs[2]): the seven Qwen2.5-7B projections as
    HXQ linears at M tokens through the tcgen05 kernel; one step = one pass over all
    seven.  Reports TFLOP/s (2*M*OUT*IN per linear) against the measured bf16 peak."""
    import torch
    from helix_substrate_b200 import HelixLinear
    from helix_substrate_b200.hxq_writer_gpu import compress_weight, student_t_weight
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    M, K, W = args.m if args.m > 16 else 2048, args.steps, max(3, args.warmup)
    mods, xs, ys = [], [], []
    for i, (name, n_out, n_in) in enumerate(PREFILL_SHAPES):
        enc = compress_weight(student_t_weight((n_out, n_in), 100 + i, dev), percentile=99.95, group_size=GROUP)
        bias = torch.randn(n_out, device=dev) * 0.02 if name in ("q", "k", "v") else None
        mods.append(HelixLinear(n_in, n_out, bias=bias, tensor_name=name, **enc).to(dev))
        xs.append(torch.randn(M, n_in, device=dev).bfloat16())
        ys.append(torch.empty(M, n_out, device=dev, dtype=torch.bfloat16))
    flops = sum(2.0 * M * o * i for _, o, i in PREFILL_SHAPES)

    def step():
        for m, x, y in zip(mods, xs, ys):
            m.packed().matmul(x, out=y)

    for _ in range(W):
        step()
    torch.cuda.synchronize()
    per_shape = []
    for (name, o, i), m, x, y in zip(PREFILL_SHAPES, mods, xs, ys):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(K):
            m.packed().matmul(x, out=y)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / K
        per_shape.append({"proj": name, "out": o, "in": i, "ms": ms, "tflops": 2.0 * M * o * i / (ms * 1e-3) / 1e12})
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(dev.index) as clk:
        e0.record()
        for _ in range(K):
            step()
        e1.record()
        torch.cuda.synchronize()
        ms_step = e0.elapsed_time(e1) / K
    status = mods[0].packed().gemm_status()
    peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
    peak = float(peaks.get("bf16_tflops_sustained", 1400.0))
    val = flops / (ms_step * 1e-3) / 1e12
    print(json.dumps({
        "metric": "hxq_prefill_gemm_TFLOPS_qwen2.5-7b_projections", "value": val, "unit": "TFLOP/s", "n_gpus": 1,
        "steps": K, "warmup": W, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"seven Qwen2.5-7B projections as HXQ linears (k=256, group-128 affine, 0.1% sidecar), M={M} bf16 tokens",
                   "m": M, "l2": "weights 0.2 GB + activations larger than L2 per pass"},
        "gpu_launches": 7 * K, "kernel_status_word": status, "per_projection": per_shape,
        "roofline": {"bound": "tensor", "achieved": val, "peak": peak, "unit": "TFLOP/s", "frac": val / peak,
                     "peak_kind": "of measured (sustained bf16 matmul)" if peaks else "of fallback",
                     "kernel": "hxq::gemm::gemm_kernel", "traffic": None},
        "clocks": clk.summary(),
    }), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--layers", type=int, default=28)
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--impl", default="hxq_b200")
    ap.add_argument("--no-graph", action="store_true", help="launch from Python instead of replaying a CUDA graph")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--allreduce", default="p2p", choices=["p2p", "nccl"],
                    help="tensor-parallel sum after down: one-shot peer-memory kernel (default) or NCCL")
    ap.add_argument("--workload", default="gemv", choices=["gemv", "prefill"],
                    help="gemv: the headline decode workload; prefill: tensor-core kernel TFLOP/s (secondary)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.workload == "prefill":
        return run_prefill(args)

    import torch
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    M, L, K, W = args.m, args.layers, args.steps, max(3, args.warmup)
    layers = build_layers(L, dev, tp_rank=rank, tp_world=world)
    act = torch.bfloat16
    hid_local = layers[0]["down"].in_features       # INTER / world (row-parallel input slice)
    x_h = torch.randn(M, HIDDEN, generator=torch.Generator().manual_seed(1)).to(act).pin_memory()
    xd_h = torch.randn(M, hid_local, generator=torch.Generator().manual_seed(2 + rank)).to(act).pin_memory()
    x, xd = x_h.to(dev), xd_h.to(dev)
    outs = [{k: torch.empty(M, m.out_features, device=dev, dtype=act) for k, m in lay.items()} for lay in layers]
    n_launch_per_step = 3 * L * (-(-M // 4) if M > 4 else 1)

    # tensor-parallel sum after `down`: the one-shot peer-memory kernel, or NCCL if asked for / if
    # symmetric memory cannot be set up on every rank (the ranks agree on one of the two)
    oneshot, p32 = None, None
    if world > 1 and args.allreduce == "p2p" and M <= 16:
        from helix_substrate_b200.tp import OneShotAllReduce
        ok = torch.ones(1, device=dev)
        try:
            oneshot = OneShotAllReduce(M * HIDDEN, dev)
        except Exception as e:   # noqa: BLE001 - any set-up failure means "use NCCL", decided together below
            print(f"[bench rank {rank}] one-shot all-reduce unavailable ({type(e).__name__}: {e}); using NCCL", file=sys.stderr)
            ok.zero_()
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if float(ok.item()) < 1.0:
            oneshot = None
        else:
            p32 = torch.empty(M, HIDDEN, device=dev, dtype=torch.float32)
            n_launch_per_step += L
    allreduce_kind = None if world == 1 else ("p2p-oneshot" if oneshot is not None else "nccl")

    def step_kernels():
        """One pass over every linear, straight on the packed weights (C ABI)."""
        for lay, o in zip(layers, outs):
            lay["gate"].packed().matmul(x, out=o["gate"])
            lay["up"].packed().matmul(x, out=o["up"])
            if oneshot is not None:
                lay["down"].packed().matmul(xd, torch.float32, out=p32)
                oneshot(p32, out=o["down"])
            else:
                lay["down"].packed().matmul(xd, out=o["down"])
                if world > 1:
                    dist.all_reduce(o["down"])

    for _ in range(2):
        step_kernels()
    torch.cuda.synchronize()
    graph = None
    if not args.no_graph:
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            step_kernels()
            with torch.cuda.graph(graph, stream=side):
                step_kernels()
        torch.cuda.current_stream().wait_stream(side)
    run = graph.replay if graph is not None else step_kernels

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(W):
        run()
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clk:
        ev0.record()
        for _ in range(K):
            run()
        ev1.record()
        barrier()
        ms = ev0.elapsed_time(ev1)
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_step = float(t.item()) / K
        # keep the sampler alive long enough to see clocks under load; the number of extra passes is
        # derived from the rank-agreed time so that every rank issues the same collectives
        for _ in range(min(2000, int(500.0 / max(ms_step, 1e-3))) if K * ms_step < 400 else 0):
            run()
        torch.cuda.synchronize()

    # ---- end to end through the module API with host buffers ----
    # The public call (HelixLinear.forward per linear) with the step's activations
    # coming from pinned host memory and the last layer's outputs going back to
    # host memory, both inside the timed region; the step is captured once in a
    # CUDA graph (copies included) and the host waits for every step's result.
    xg, xdd = torch.empty_like(x), torch.empty_like(xd)
    out_h = {k: torch.empty(M, m.out_features, dtype=act).pin_memory() for k, m in layers[-1].items()}

    from helix_substrate_b200.tp import RowParallelHelixLinear
    down_mods = {id(lay["down"]): (RowParallelHelixLinear(lay["down"], oneshot=oneshot) if world > 1 else lay["down"])
                 for lay in layers}

    def step_e2e():
        xg.copy_(x_h, non_blocking=True)
        xdd.copy_(xd_h, non_blocking=True)
        g = u = y = None
        for lay in layers:
            g = lay["gate"](xg)
            u = lay["up"](xg)
            y = down_mods[id(lay["down"])](xdd)
        out_h["gate"].copy_(g, non_blocking=True)
        out_h["up"].copy_(u, non_blocking=True)
        out_h["down"].copy_(y, non_blocking=True)

    for _ in range(2):
        step_e2e()
    torch.cuda.synchronize()
    run_e2e = step_e2e
    if not args.no_graph:
        g_e2e = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            step_e2e()
            with torch.cuda.graph(g_e2e, stream=side):
                step_e2e()
        torch.cuda.current_stream().wait_stream(side)
        run_e2e = g_e2e.replay
    for _ in range(3):
        run_e2e()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(K):
        run_e2e()
        torch.cuda.current_stream().synchronize()   # the caller reads the result of every step
    e1.record()
    barrier()
    te = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
    ms_e2e = float(te.item()) / K

    nbytes_rank = algorithmic_bytes(layers, M, 2)
    nb = torch.tensor([float(nbytes_rank)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(nb)
    nbytes = float(nb.item())
    if rank != 0:
        _leave(world)
        return

    peak, peak_kind = _peaks()
    value = nbytes / (ms_step * 1e-3) / 1e9
    per_gpu = value / world
    line = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": "qwen2.5-7b MLP gate/up [18944,3584] + down [3584,18944] HXQ linears "
                               "(k=256 codebook, group-128 fp32 affine, two-sided 99.95% sidecar), distinct "
                               f"weights per layer, M={M} bf16 activations",
                   "layers": L, "m": M, "launch": "python" if graph is None else "cuda_graph",
                   "parallelism": f"tp{world}" if world > 1 else "single", "allreduce": allreduce_kind,
                   "l2": f"inputs larger than L2 ({nbytes_rank / 1e9:.2f} GB of distinct weights per pass)",
                   "algorithmic_bytes_per_step": nbytes},
        "e2e": {"value": nbytes / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": (x_h.numel() + xd_h.numel()) * 2,
                "d2h_bytes_per_step": M * (2 * layers[0]["gate"].out_features + HIDDEN) * 2,
                "api": "HelixLinear.forward per linear; pinned-host activations in and last layer's outputs back "
                       "to pinned host inside the timed region; "
                       + ("python launches" if graph is None else "step captured in a CUDA graph") + ", host sync per step"},
        "gpu_launches": n_launch_per_step * K,
        "roofline": {"bound": "hbm", "achieved": per_gpu, "peak": peak, "unit": "GB/s", "frac": per_gpu / peak,
                     "peak_kind": f"of {peak_kind}", "frac_of_8TBps": per_gpu / 8000.0,
                     # dram__bytes_read + dram__bytes_write per launch from the ncu capture summarised in
                     # profiles/gemv_kernel_m1_qwen7b_mlp.md (gate 73.64 MB, down 73.90 MB; M = 1, one GPU)
                     "traffic": (2 * 73.64e6 + 73.90e6) / 3 if (M == 1 and world == 1 and L > 0) else None,
                     "kernel": "hxq::gemv_lean_kernel<1>" if M == 1 else "hxq::gemv_lean_kernel",
                     "algorithmic_bytes_per_launch": nbytes_rank / (3 * L),
                     "avg_launch_us": ms_step * 1e3 / (3 * L)},
        "clocks": clk.summary(),
    }
    if not args.no_cpu_baseline and world == 1:
        cpu = cpu_forward_sample(seconds_target=12.0)
        line["cpu_baseline"] = {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")}
    print(json.dumps(line), flush=True)
    _leave(world)


def _leave(world: int) -> None:
    """End a multi-rank run.  Tearing the NCCL process group down while CUDA graphs
    that captured its collectives are still alive blocks for ever in this torch /
    NCCL pairing, so ranks meet at a last barrier, flush and exit without the teardown."""
    if world <= 1:
        return
    import torch
    import torch.distributed as dist
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
