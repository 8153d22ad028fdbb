#!/usr/bin/env python3
"""Benchmark of the HXQ compressed-linear forward path on B200.

Headline workload: the grouped-affine HXQ linears of a Qwen2.5-7B MLP - gate/up
[18944, 3584] and down [3584, 18944], k=256 codebook, group-128 fp32
scale/offset, two-sided 99.95 % outlier sidecar - for every one of L layers with
DISTINCT weights, M=1 bf16 activations.  One step = one pass over all 3*L
linears (3*L kernel launches, ~73 MB of indices each, far larger than L2
together).  Metric: algorithmic GB/s of the VQ-GEMV.

The same JSON line carries, from the same run, the rest of what the metric names:
``gemv_m4`` / ``gemv_m16`` (same linears at 4 and 16 tokens), ``prefill`` (the seven
projection shapes on the tensor-core kernel at 512 / 2048 / 8192 tokens, with the
two-pass dequantise-then-dense-GEMM path timed beside it as a labelled baseline)
and ``decode`` (a random-init 28-layer decoder of that shape: prompt 2048, greedy
decode at batch 1 and 32).  ``checked`` says what was compared with the CPU oracle
after the timed region.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--layers L] [--m M] [--blocks a,b,...]
    python bench.py --impl reference      # the CPU path on the same tensors, timed on the host cores
    python bench.py --workload prefill --m 2048 | --workload decode --batch 32 | --workload ceiling

Prints ONE JSON line on rank 0.
"""

from __future__ import annotations

import argparse
import json
import os
import re
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

HIDDEN, INTER, GROUP = 3584, 18944, 128
METRIC = "hxq_vq_gemv_algorithmic_GBps_M1_qwen2.5-7b_mlp"
WORKLOAD = ("qwen2.5-7b MLP gate/up [18944,3584] + down [3584,18944] HXQ linears (k=256 codebook, group-128 fp32 "
            "affine, two-sided 99.95% sidecar), distinct Student-t(5) weights per layer, M=1 bf16 activations")
L2_NOTE = "inputs larger than L2 (distinct weights per layer, 0.22 GB per layer)"
MLP_SHAPES = (("gate", (INTER, HIDDEN)), ("up", (INTER, HIDDEN)), ("down", (HIDDEN, INTER)))
PREFILL_SHAPES = (("q", 3584, 3584), ("k", 512, 3584), ("v", 512, 3584), ("o", 3584, 3584),
                  ("gate", 18944, 3584), ("up", 18944, 3584), ("down", 3584, 18944))


def _measured_peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    return json.loads(p.read_text()) if p.exists() else {}


def _hbm_peak():
    d = _measured_peaks()
    return (float(d["hbm_gbs"]), "measured") if "hbm_gbs" in d else (6650.0, "fallback")


def _profiled_traffic(kernel: str):
    """DRAM bytes per launch of ``kernel`` as one ncu capture recorded them: a line
    ``traffic_bytes_per_launch[<kernel>]: gate=<n> down=<n>`` in a summary under profiles/."""
    for f in sorted((ROOT / "profiles").glob("*.md")):
        m = re.search(r"traffic_bytes_per_launch\[" + re.escape(kernel) + r"\]:\s*gate=(\d+)\s+down=(\d+)", f.read_text())
        if m:
            g, d = int(m.group(1)), int(m.group(2))
            return (2 * g + d) / 3.0, f"profiles/{f.name}"
    return None, None


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


# --------------------------------------------------------------------------- inputs

def encode_mlp_matrix(layer: int, j: int, device, plain: bool = False) -> dict:
    """Compressed tensors of MLP matrix j (gate, up, down) of ``layer``: the same call gives the
    GPU arm, the reference arm and the checks identical tensors."""
    from helix_substrate_b200.hxq_writer_gpu import compress_weight, student_t_weight
    w = student_t_weight(MLP_SHAPES[j][1], 3 * layer + j, device)
    return compress_weight(w, percentile=99.95, group_size=0 if plain else GROUP, sidecar=not plain)


def build_layers(n_layers: int, device, tp_rank: int = 0, tp_world: int = 1, plain: bool = False):
    """Distinct compressed gate/up/down modules per layer (column-parallel gate/up and row-parallel
    down, cut on whole affine groups, when tp_world > 1)."""
    import torch
    from helix_substrate_b200 import HelixLinear
    from helix_substrate_b200.tp import shard_helix_linear
    layers = []
    for l in range(n_layers):
        mods = {}
        for j, (name, shape) in enumerate(MLP_SHAPES):
            enc = encode_mlp_matrix(l, j, device, plain)
            mod = HelixLinear(shape[1], shape[0], tensor_name=f"model.layers.{l}.mlp.{name}_proj.weight", **enc)
            if tp_world > 1:
                mod = shard_helix_linear(mod, "row" if name == "down" else "column", tp_rank, tp_world, multiple=GROUP)
            mods[name] = mod.to(device)
        layers.append(mods)
        torch.cuda.empty_cache()
    return layers


def algorithmic_bytes(layers, M: int, act_bytes: int) -> int:
    return sum(mod.packed().algorithmic_bytes(M, act_bytes, act_bytes)
               for lay in layers for mod in lay.values())


def host_case(enc: dict, x):
    """Host copies of one encoded matrix in the oracle's argument order."""
    import numpy as np
    from oracle import hxq_oracle as O
    cb = enc["codebook"].cpu().numpy()
    idx = enc["indices"].cpu().numpy()
    s = enc["group_scales"].cpu().numpy() if "group_scales" in enc else None
    t = enc["group_offsets"].cpu().numpy() if "group_offsets" in enc else None
    G = int(enc.get("group_size", 0))
    rows = cols = deltas = None
    if "sidecar_positions" in enc:
        rows, cols, deltas = O.derive_sidecar(cb, idx, enc["sidecar_positions"].cpu().numpy(),
                                              enc["sidecar_values"].cpu().numpy(), s, t, G)
    return (np.asarray(x, dtype=np.float32), cb, idx, rows, cols, deltas, s, t, G)


def oracle_check(mod, enc: dict, x, y, n_rows: int = 256) -> float:
    """rel-L2 of ``y`` (the kernel's output for ``x``) against the oracle's fp64 forward on a sample
    of output rows of the matrix encoded in ``enc``."""
    import numpy as np
    import torch
    from oracle import hxq_oracle as O
    n_out, n_in = enc["indices"].shape
    g = torch.Generator().manual_seed(11)
    rows = torch.sort(torch.randperm(n_out, generator=g)[:n_rows]).values
    rows_d = rows.to(enc["indices"].device)
    cb = enc["codebook"].cpu().numpy()
    idx_r = enc["indices"][rows_d].cpu().numpy()
    G = int(enc.get("group_size", 0))
    s_r = enc["group_scales"][rows_d].cpu().numpy() if G else None
    t_r = enc["group_offsets"][rows_d].cpu().numpy() if G else None
    r = c = d = None
    if "sidecar_positions" in enc:
        pos, vals = enc["sidecar_positions"], enc["sidecar_values"]
        prow = pos // n_in
        keep = torch.isin(prow, rows_d)
        local = torch.searchsorted(rows_d, prow[keep])
        pos_r = (local * n_in + pos[keep] % n_in).cpu().numpy()
        r, c, d = O.derive_sidecar(cb, idx_r, pos_r, vals[keep].cpu().numpy(), s_r, t_r, G)
    ref = O.forward_f64(x.float().cpu().numpy(), cb, idx_r, r, c, d, None, s_r, t_r, G)
    got = y[:, rows_d].double().cpu().numpy()
    return float(np.linalg.norm(got - ref) / max(np.linalg.norm(ref), 1e-30))


# --------------------------------------------------------------------------- CPU arm

def cpu_forward_timed(device, steps: int, warmup: int, threads=None, seconds_cap: float = 25.0) -> dict:
    """The reference's CPU forward (``cb[idx.long()]`` per 256-row tile, group affine, in-place
    sidecar add, fp32 ``x @ W.t()``: the oracle's restatement of HelixLinear._forward_naive with the
    reference's own torch calls) timed on the host cores, on EXACTLY the tensors the GPU arm's first
    layer holds and the same activations.  One step = one pass over that layer's gate, up, down."""
    import torch
    from oracle import hxq_oracle as O
    n_thr = threads or len(os.sched_getaffinity(0))
    torch.set_num_threads(n_thr)
    x_h = torch.randn(1, HIDDEN, generator=torch.Generator().manual_seed(1)).bfloat16().float().numpy()
    xd_h = torch.randn(1, INTER, generator=torch.Generator().manual_seed(2)).bfloat16().float().numpy()
    cases, nbytes = [], 0
    for j, (name, shape) in enumerate(MLP_SHAPES):
        enc = encode_mlp_matrix(0, j, device)
        x, cb, idx, rows, cols, deltas, s, t, G = host_case(enc, xd_h if name == "down" else x_h)
        cases.append((x, cb, idx, rows, cols, deltas, s, t, G))
        nbytes += (idx.size + 1024 + s.size * 8 + len(rows) * 8 + (idx.shape[0] + 1) * 4
                   + 2 * idx.shape[1] + 2 * idx.shape[0])
        del enc
    if device is not None and str(device).startswith("cuda"):
        torch.cuda.empty_cache()

    def one_pass():
        for (x, cb, idx, rows, cols, deltas, s, t, G) in cases:
            O.forward_naive_torch(x, cb, idx, rows, cols, deltas, None, s, t, G)

    t0 = time.perf_counter()
    one_pass()
    first = time.perf_counter() - t0
    warm = max(0, min(warmup, int(5.0 / max(first, 1e-3))) - 1)
    for _ in range(warm):
        one_pass()
    reps = max(2, min(steps, int(seconds_cap / max(first, 1e-3))))
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        one_pass()
        times.append(time.perf_counter() - t0)
    mean = sum(times) / len(times)
    return {"value": nbytes / mean / 1e9, "unit": "GB/s", "cores": n_thr, "kind": "port",
            "sample": f"gate+up+down of layer 0 (the GPU arm's tensors and activations, fp32 math), "
                      f"{reps} timed passes after {warm + 1} warm-up, {mean * 1e3:.1f} ms per pass",
            "ms_per_pass": mean * 1e3, "passes": reps, "bytes_per_pass": nbytes}


def run_reference(args):
    """Reference arm: the CPU implementation of the path on the box's host cores (all of them).
    A step is one pass over ONE layer's three linears (layers_timed = 1) of the headline workload."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    import torch
    t0 = time.perf_counter()
    dev = torch.device("cuda", 0) if torch.cuda.is_available() else torch.device("cpu")   # encoder only; the timed path is CPU
    cpu = cpu_forward_timed(dev, steps=args.steps, warmup=max(3, args.warmup))
    line = {
        "impl": "reference", "metric": METRIC, "value": cpu["value"], "unit": "GB/s", "n_gpus": args.gpus,
        "steps": cpu["passes"], "warmup": max(3, args.warmup), "ms_per_step": cpu["ms_per_pass"],
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "layers": args.layers, "m": 1, "l2": L2_NOTE},
        "layers_timed": 1,
        "cpu_baseline": {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": cpu["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "wall_s": time.perf_counter() - t0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- secondary blocks (one GPU)

def _timed_loop(fn, min_s: float, dev, max_iters: int = 20000):
    """Run ``fn`` for at least ``min_s`` seconds of device time (CUDA events), clocks sampled.
    Returns (ms per call, calls, clock summary)."""
    import torch
    for _ in range(3):
        fn()
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    fn()
    e1.record()
    torch.cuda.synchronize(dev)
    n = int(max(3, min(max_iters, min_s * 1e3 / max(e0.elapsed_time(e1), 1e-3))))
    with ClockSampler(dev.index) as clk:
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize(dev)
    return e0.elapsed_time(e1) / n, n, clk.summary()


def block_gemv_m(layers, M: int, dev, min_s: float) -> dict:
    """The headline linears at M tokens (graph replay over all layers)."""
    import torch
    act = torch.bfloat16
    x = torch.randn(M, HIDDEN, device=dev).to(act)
    xd = torch.randn(M, INTER, device=dev).to(act)
    outs = [{k: torch.empty(M, m.out_features, device=dev, dtype=act) for k, m in lay.items()} for lay in layers]

    def step():
        for lay, o in zip(layers, outs):
            lay["gate"].packed().matmul(x, out=o["gate"])
            lay["up"].packed().matmul(x, out=o["up"])
            lay["down"].packed().matmul(xd, out=o["down"])

    graph, side = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()
        side.synchronize()
        with torch.cuda.graph(graph, stream=side):
            step()
    torch.cuda.current_stream().wait_stream(side)
    ms, n, clk = _timed_loop(graph.replay, min_s, dev)
    nbytes = algorithmic_bytes(layers, M, 2)
    peak, kind = _hbm_peak()
    gbs = nbytes / (ms * 1e-3) / 1e9
    from helix_substrate_b200.packed import uses_gemv
    if uses_gemv(M, act):      # fp32-accumulate decode kernel: four tokens per launch
        kernel, launches = "hxq_gemv (gemv_lean_kernel)", 3 * len(layers) * (-(-M // 4))
    else:                         # tensor-memory kernel: one launch per linear, + the split-K sum where the row-tile grid is small (down)
        kernel, launches = "hxq_gemm (gemm_ts_kernel)", 4 * len(layers)
    return {"m": M, "GBps": gbs, "ms_per_step": ms, "steps": n, "us_per_linear": ms * 1e3 / (3 * len(layers)),
            "kernel": kernel, "launches_per_step": launches, "frac_of_hbm_peak": gbs / peak, "peak_kind": f"of {kind}", "clocks": clk}


def block_prefill(Ms, dev, min_s: float) -> dict:
    """The seven projection shapes as HXQ linears on the tensor-core kernel, one pass over all seven
    per step, with the two-pass path (dequantise to a bf16 scratch, then a dense library GEMM: what
    the reference's buffered forward does) timed beside it as a baseline."""
    import torch
    from helix_substrate_b200 import HelixLinear
    from helix_substrate_b200.hxq_writer_gpu import compress_weight, student_t_weight
    mods = []
    for i, (name, n_out, n_in) in enumerate(PREFILL_SHAPES):
        enc = compress_weight(student_t_weight((n_out, n_in), 100 + i, dev), percentile=99.95, group_size=GROUP)
        bias = torch.randn(n_out, device=dev) * 0.02 if name in ("q", "k", "v") else None
        mods.append(HelixLinear(n_in, n_out, bias=bias, tensor_name=name, **enc).to(dev))
    peaks = _measured_peaks()
    peak = float(peaks.get("bf16_tflops_sustained", 1400.0))
    scratch = torch.empty(INTER * HIDDEN, device=dev, dtype=torch.bfloat16)
    out = {"peak_TFLOPs": peak, "peak_kind": "of measured (sustained bf16 matmul)" if peaks else "of fallback", "by_m": []}
    for M in Ms:
        xs = [torch.randn(M, m.in_features, device=dev).bfloat16() for m in mods]
        ys = [torch.empty(M, m.out_features, device=dev, dtype=torch.bfloat16) for m in mods]
        flops = sum(2.0 * M * o * i for _, o, i in PREFILL_SHAPES)

        def fused():
            for m, x, y in zip(mods, xs, ys):
                m.packed().matmul(x, out=y)

        def two_pass():
            for m, x, y in zip(mods, xs, ys):
                w = scratch[: m.out_features * m.in_features].view(m.out_features, m.in_features)
                m.packed().dequant(dtype=torch.bfloat16, out=w)
                if m.bias is not None:
                    torch.addmm(m.bias.to(torch.bfloat16), x, w.t(), out=y)
                else:
                    torch.matmul(x, w.t(), out=y)

        ms, n, clk = _timed_loop(fused, min_s, dev)
        status = mods[0].packed().gemm_status()
        ref = xs[1].double() @ mods[1].decode_weight().double().t() + mods[1].bias.double()
        rel = float(((ys[1].double() - ref).norm() / ref.norm()).item())
        ms2, n2, clk2 = _timed_loop(two_pass, min_s / 2, dev)
        val, val2 = flops / (ms * 1e-3) / 1e12, flops / (ms2 * 1e-3) / 1e12
        out["by_m"].append({"m": M, "TFLOPs": val, "ms_per_step": ms, "steps": n, "frac_of_peak": val / peak,
                            "kernel_status_word": status, "checked_rel_l2_k_proj": rel, "clocks": clk,
                            "two_pass_baseline": {"TFLOPs": val2, "ms_per_step": ms2, "steps": n2, "clocks": clk2,
                                                  "what": "hxq_dequant to a bf16 scratch + torch.matmul per projection"}})
        del xs, ys
    return out


def block_decode(dev, rank, world, batches, shape="7b", prompt=2048, new=128, fill_cache=False, allreduce="p2p") -> dict:
    from helix_substrate_b200.qwen2_decode import run_decode
    peak, kind = _hbm_peak()
    runs = run_decode(shape, batches, prompt, new, dev, rank, world, allreduce=allreduce, fill_cache=fill_cache)
    for r in runs:
        r["frac_of_hbm_peak_per_gpu"] = r["hxq_GBps_per_gpu"] / peak
        r["peak_kind"] = f"of {kind}"
    return {"shape": shape, "runs": runs,
            "note": "random-init decoder, every linear HXQ (k=256, group-128 affine, 99.95% sidecar); embedding and "
                    "lm_head dense bf16; hxq_GBps counts the compressed linears' algorithmic bytes over the whole step time"}


# --------------------------------------------------------------------------- main

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--layers", type=int, default=28)
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--impl", default="hxq_b200")
    ap.add_argument("--no-graph", action="store_true", help="launch from Python instead of replaying a CUDA graph")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--allreduce", default="p2p", choices=["p2p", "nccl"],
                    help="tensor-parallel sum after down: one-shot peer-memory kernel (default) or NCCL")
    ap.add_argument("--workload", default="gemv", choices=["gemv", "prefill", "decode", "ceiling"],
                    help="gemv: the headline line with its secondary blocks; prefill / decode: that block alone; "
                         "ceiling: the headline linears without affine and sidecar (index stream + table lookups + FMA only)")
    ap.add_argument("--blocks", default=None,
                    help="secondary blocks of the gemv workload, comma separated: m,prefill,decode,decode14b "
                         "(default: m,prefill,decode on one GPU; decode on several)")
    ap.add_argument("--block-seconds", type=float, default=2.0, help="minimum timed region of each secondary measurement")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)

    import torch
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        from helix_substrate_b200.qwen2_decode import init_tensor_parallel
        init_tensor_parallel(dev)

    if args.workload in ("prefill", "decode"):
        if args.workload == "prefill":
            blk = block_prefill([args.m if args.m > 16 else 2048], dev, args.block_seconds)
            val, unit, metric = blk["by_m"][0]["TFLOPs"], "TFLOP/s", "hxq_prefill_gemm_TFLOPS_qwen2.5-7b_projections"
        else:
            blk = block_decode(dev, rank, world, [args.batch], allreduce=args.allreduce)
            val, unit, metric = blk["runs"][0]["tok_s"], "tok/s", "hxq_decode_tokens_per_s_qwen2.5-7b_shape"
        if rank == 0:
            print(json.dumps({"metric": metric, "value": val, "unit": unit, "n_gpus": world, "higher_is_better": True,
                              "data": "synthetic", args.workload: blk}), flush=True)
        return _leave(world)

    plain = args.workload == "ceiling"
    M, L, K, W = args.m, args.layers, args.steps, max(3, args.warmup)
    layers = build_layers(L, dev, tp_rank=rank, tp_world=world, plain=plain)
    act = torch.bfloat16
    hid_local = layers[0]["down"].in_features       # this rank's slice of the intermediate dimension
    x_h = torch.randn(M, HIDDEN, generator=torch.Generator().manual_seed(1)).to(act).pin_memory()
    xd_full = torch.randn(M, INTER, generator=torch.Generator().manual_seed(2)).to(act)
    c0 = layers[0]["down"].col0
    xd_h = xd_full[:, c0:c0 + hid_local].contiguous().pin_memory()
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
            side.synchronize()
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
        for _ in range(min(2000, int(700.0 / max(ms_step, 1e-3))) if K * ms_step < 600 else 0):
            run()
        torch.cuda.synchronize()

    # ---- what was timed, checked (outside the timed region) ----
    checked = {"status": 0}
    if True:
        enc0 = encode_mlp_matrix(0, 0, dev, plain)
        if world == 1:
            checked["rel_l2_vs_oracle_gate_layer0"] = oracle_check(layers[0]["gate"], enc0, x, outs[0]["gate"])
            encd = encode_mlp_matrix(0, 2, dev, plain)
            checked["rel_l2_vs_oracle_down_layer0"] = oracle_check(layers[0]["down"], encd, xd, outs[0]["down"])
            checked["tolerance"] = "4e-3 (fp32 accumulate, one rounding of the result to bf16)"
            checked["ok"] = bool(max(checked["rel_l2_vs_oracle_gate_layer0"], checked["rel_l2_vs_oracle_down_layer0"]) < 4e-3)
            del encd
        else:
            # the reduced down output against an NCCL all-reduce of the same fp32 partials, once
            part = layers[0]["down"].packed().matmul(xd, torch.float32)
            dist.all_reduce(part)
            ref = part.to(act).float()
            got = outs[0]["down"].float()
            checked["down_sum_vs_nccl_max_abs"] = float((got - ref).abs().max().item())
            checked["down_sum_vs_nccl_rel_l2"] = float(((got - ref).norm() / ref.norm().clamp_min(1e-30)).item())
            checked["ok"] = bool(checked["down_sum_vs_nccl_rel_l2"] < 1e-2)
            if oneshot is not None:
                checked["status"] = int(oneshot.check_status())
        del enc0

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
    g_e2e = None
    if not args.no_graph:
        g_e2e = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            step_e2e()
            side.synchronize()
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
    if world == 1:
        checked["e2e_output_equals_kernel_output"] = bool(torch.equal(out_h["down"], outs[-1]["down"].cpu()))

    nbytes_rank = algorithmic_bytes(layers, M, 2)
    nb = torch.tensor([float(nbytes_rank), float(nbytes_rank)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(nb[:1])
        dist.all_reduce(nb[1:], op=dist.ReduceOp.MAX)
    nbytes, nbytes_max_rank = float(nb[0].item()), float(nb[1].item())

    # ---- secondary blocks: the rest of the metric, from the same run ----
    default_blocks = "m,prefill,decode" if world == 1 else "decode"
    want = [b for b in (args.blocks if args.blocks is not None else default_blocks).split(",") if b]
    if plain or M != 1:
        want = []
    blocks = {}
    graph = g_e2e = None            # the headline graphs hold collectives: drop them before anything else runs
    run = run_e2e = None
    for name in want:
        try:
            if name == "m" and world == 1:
                blocks["gemv_m4"] = block_gemv_m(layers, 4, dev, args.block_seconds)
                blocks["gemv_m16"] = block_gemv_m(layers, 16, dev, args.block_seconds)
            elif name == "prefill" and world == 1:
                del layers[8:], outs[8:]
                torch.cuda.empty_cache()
                blocks["prefill"] = block_prefill([512, 2048, 8192], dev, args.block_seconds)
            elif name == "decode":
                layers.clear(); outs.clear(); down_mods.clear()
                torch.cuda.empty_cache()
                blocks["decode"] = block_decode(dev, rank, world, [1, 32], allreduce=args.allreduce)
            elif name == "decode14b" and world > 1:
                layers.clear(); outs.clear(); down_mods.clear()
                torch.cuda.empty_cache()
                blocks["decode_14b"] = block_decode(dev, rank, world, [64], shape="14b", prompt=4096, new=64,
                                                    fill_cache=True, allreduce=args.allreduce)
        except Exception as e:   # noqa: BLE001 - a secondary block must not take the headline line with it
            blocks[name] = {"error": f"{type(e).__name__}: {e}"[:400]}
            if world > 1:
                raise
    if rank != 0:
        return _leave(world)

    peak, peak_kind = _hbm_peak()
    value = nbytes / (ms_step * 1e-3) / 1e9
    per_gpu = value / world
    kernel = "hxq::gemv_lean_kernel<1>" if M == 1 else "hxq::gemv_lean_kernel"
    traffic, traffic_src = _profiled_traffic("gemv_lean_kernel<1>") if (M == 1 and world == 1 and not plain) else (None, None)
    line = {
        "metric": METRIC if not plain else METRIC + "_no_affine_no_sidecar", "value": value, "unit": "GB/s",
        "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD if not plain else WORKLOAD.replace("group-128 fp32 affine, two-sided 99.95% sidecar",
                                                                           "no affine, no sidecar"),
                   "layers": L, "m": M, "l2": L2_NOTE,
                   "parallelism": f"tp{world}" if world > 1 else "single"},
        "launch": "python" if args.no_graph else "cuda_graph", "allreduce": allreduce_kind,
        "algorithmic_bytes_per_step": nbytes,
        "e2e": {"value": nbytes / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": (x_h.numel() + xd_h.numel()) * 2,
                "d2h_bytes_per_step": sum(t_.numel() for t_ in out_h.values()) * 2,
                "api": "HelixLinear.forward per linear; pinned-host activations in and last layer's outputs back "
                       "to pinned host inside the timed region; "
                       + ("python launches" if args.no_graph else "step captured in a CUDA graph") + ", host sync per step"},
        "gpu_launches": n_launch_per_step * K,
        "roofline": {"bound": "hbm", "achieved": per_gpu, "peak": peak, "unit": "GB/s", "frac": per_gpu / peak,
                     "peak_kind": f"of {peak_kind}", "frac_of_8TBps": per_gpu / 8000.0,
                     "traffic": traffic, "traffic_source": traffic_src,
                     "kernel": kernel,
                     "algorithmic_bytes_per_launch": nbytes_max_rank / (3 * L),
                     "avg_launch_us": ms_step * 1e3 / (3 * L)},
        "checked": checked,
        "clocks": clk.summary(),
    }
    line.update(blocks)
    if not args.no_cpu_baseline and world == 1 and not plain:
        cpu = cpu_forward_timed(dev, steps=20, warmup=3, seconds_cap=12.0)
        line["cpu_baseline"] = {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")}
    print(json.dumps(line), flush=True)
    _leave(world)


def _leave(world: int) -> None:
    """End a multi-rank run: graphs that captured collectives are gone by now, so the group can be
    torn down (with a timed exit behind it in case the teardown still blocks)."""
    if world <= 1:
        return
    from helix_substrate_b200.qwen2_decode import leave_process_group
    leave_process_group()


if __name__ == "__main__":
    main()
