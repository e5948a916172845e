#!/usr/bin/env python
"""Benchmark of the quantized-linear hot path on B200.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--sweep]

Headline workload (N = 1): the MLX-affine int4 g64 linears of Llama-3.2-3B at decode,
M = 1 — one step streams all 28 layers x (q, k, v, o, gate, up, down) = 196 linears,
1.585 GB of packed weights (far larger than the 126 MB L2, so every step reads HBM).
`value` is algorithmic bytes per second (packed codes + scales + biases + activations in
and out), i.e. the achieved weight-stream bandwidth the metric asks for at M = 1.
`--sweep` adds TFLOP/s for M >= 64 and the fp8 path as extra keys.

With N > 1 every rank runs the same workload on its own GPU (independent replicas, no
data-path collective; weak scaling) and the tensor-parallel 70B-shaped fp8 stack is timed
separately under the `tp` key.

`--impl reference` times the reference project's CPU implementation of the same linears
(its Rust cannot be built here, so this is the C++ restatement in oracle/) on the host
cores; rank 0 only.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from scratchy_b200 import synth  # noqa: E402

N_LAYERS = 28
LAYER_ORDER = ["q", "k", "v", "o", "gate", "up", "down"]
METRIC = "int4_g64_decode_linear_weight_stream"
UNIT = "GB/s"


def affine_alg_bytes(M, N, K):
    """Algorithmic bytes of one int4 g64 linear: codes + bf16 scale/bias per group + x in + y out."""
    return N * K // 2 + 2 * (N * K // 64) * 2 + M * K * 2 + M * N * 2


def fp8_alg_bytes(M, N, K):
    return N * K + 4 * N + 2 * M * K + 2 * M * N


# dram__bytes_read.sum + dram__bytes_write.sum per launch of affine_b4_gemv_kernel at M = 1, by shape, from the ncu
# captures summarised in profiles/affine_b4_gemv_llama3b_m1_full.md (q/o, k/v, down) and
# profiles/affine_b4_gemv_llama3b_gate_m1_full.md (gate/up) (weights cross HBM once; activations come from L2)
GEMV_DRAM_TRAFFIC = {"q": 5335808, "o": 5335808, "k": 1797120, "v": 1797120, "gate": 14208512, "up": 14208512, "down": 14191360}


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "src": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "src": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.p = None
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                       "-i", str(gpu_index), "-lms", "20"], stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.p = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.p is None:
            return out
        time.sleep(0.15)
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except Exception:
            self.p.kill()
        self.f.flush()
        rows = [r.strip().split(", ") for r in open(self.f.name) if r.strip()]
        os.unlink(self.f.name)
        sm, mx, reasons = [], [], set()
        for r in rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except Exception:
                continue
            names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
            for name, v in zip(names, r[5:9]):
                if v.strip().lower().startswith("active"):
                    reasons.add(name)
        if sm:
            out = {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                   "samples": len(sm)}
        return out


# ------------------------------------------------------------------------------------ reference arm
_CPU_DATA = None


def cpu_linears():
    """The 7 int4 linears of one Llama-3.2-3B layer (synthetic, seeded), built once per process."""
    global _CPU_DATA
    import oracle
    if _CPU_DATA is None:
        data = []
        for i, name in enumerate(LAYER_ORDER):
            K, N = synth.LLAMA_3_2_3B[name]
            w, s, b = synth.affine_int4_weights(N, K, 64, 100 + i)
            x = synth.activations_bf16(1, K, 200 + i)
            data.append((w.view(np.uint8).reshape(-1), s, b, x, N, K))
        _CPU_DATA = data
    return oracle, _CPU_DATA


def time_cpu_layer(reps: int, n_lin: int = 7):
    """One 'sample' = the first `n_lin` of the 7 int4 linears of one Llama-3.2-3B layer at M = 1 through the
    oracle; returns (algorithmic GB/s, seconds per sample, threads)."""
    oracle, data = cpu_linears()
    oracle.set_num_threads(os.cpu_count() or 1)       # launchers export OMP_NUM_THREADS=1: use the host's cores all the same
    data = data[:n_lin]
    byts = sum(affine_alg_bytes(1, N, K) for *_, N, K in data)
    oracle.affine_qmm_t_b4(*data[0][:4], 1, data[0][4], data[0][5], 64)    # warm the thread pool
    t0 = time.perf_counter()
    for _ in range(reps):
        for pk, s, b, x, N, K in data:
            oracle.affine_qmm_t_b4(pk, s, b, x, 1, N, K, 64)
    dt = (time.perf_counter() - t0) / reps
    return byts / dt / 1e9, dt, oracle.num_threads()


def run_reference(args):
    """The reference arm: the reference's own CPU arithmetic for the path (the C++/OpenMP restatement — the Rust
    sources cannot be built here) on all host threads.  A step is a bounded sample of the GPU arm's step: the
    first n of one layer's 7 linears, n sized so that warm-up plus K steps stay within about two minutes."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    _, t_layer, _ = time_cpu_layer(1)
    n_lin = max(1, min(7, int(7 * 120.0 / (max(args.steps + args.warmup, 1) * max(t_layer, 1e-3)))))
    for _ in range(max(args.warmup, 1)):
        time_cpu_layer(1, n_lin)
    vals = []
    t_all = 0.0
    for _ in range(args.steps):
        v, dt, cores = time_cpu_layer(1, n_lin)
        vals.append(v)
        t_all += dt
    value = float(np.mean(vals))
    names = ",".join(LAYER_ORDER[:n_lin])
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * t_all / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "llama-3.2-3b int4 g64 linears (q,k,v,o,gate,up,down), M=1",
                   "step": f"{n_lin} linear(s) of one layer ({names}) on the host cores: a bounded sample of the "
                           "28-layer GPU step"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"{n_lin} of one layer's 7 linears per step ({names}), C++/OpenMP restatement of "
                                   "cpu_reference::affine_qmm_t_b4 (the Rust reference cannot be built here)"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ------------------------------------------------------------------------------------ GPU arm
def build_int4_model(device, n_layers, fused=False):
    """The 7 linears of every layer (synthetic, seeded per layer and shape).  With `fused`, also the same weights as
    the reference's fused projections (`load_rows_concat`: q|k|v and gate|up as one matrix each), for the extra
    4-launches-per-layer measurement."""
    import torch
    from scratchy_b200 import AffineQuantLinear
    layers, fused_layers = [], []
    # one set of synthetic checkpoint tensors per shape, re-drawn per layer on the device
    for li in range(n_layers):
        row, raw = [], []
        for name in LAYER_ORDER:
            K, N = synth.LLAMA_3_2_3B[name]
            g = torch.Generator(device=device)
            g.manual_seed(1000 * li + len(row))
            w = torch.randint(-2 ** 31, 2 ** 31 - 1, (N, K // 8), dtype=torch.int32, device=device, generator=g)
            s = (torch.randn((N, K // 64), device=device, generator=g) * 0.02).abs().add(1e-3).to(torch.bfloat16)
            b = (-8.0 * s.float() + torch.randn((N, K // 64), device=device, generator=g) * 1e-3).to(torch.bfloat16)
            row.append(AffineQuantLinear.from_tensors(w, s, b, 64, 4))
            raw.append((w, s, b))
        layers.append(row)
        if fused:
            def cat(idxs):
                return AffineQuantLinear.from_tensors(*(torch.cat([raw[i][j] for i in idxs], 0) for j in range(3)), 64, 4)
            fused_layers.append([cat([0, 1, 2]), row[3], cat([4, 5]), row[6]])
    torch.cuda.synchronize(device)
    return (layers, fused_layers) if fused else layers


def run_gpu(args):
    import torch
    import torch.distributed as dist
    from scratchy_b200 import _lib

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    ctx = _lib.context(local_rank)
    peaks = measured_peaks()

    M = 1
    if world == 1:
        layers, fused_layers = build_int4_model(device, N_LAYERS, fused=True)
    else:
        layers, fused_layers = build_int4_model(device, N_LAYERS), None
    shapes = [synth.LLAMA_3_2_3B[n] for n in LAYER_ORDER]
    step_bytes = N_LAYERS * sum(affine_alg_bytes(M, N, K) for K, N in shapes)
    xs = [torch.randn((M, K), device=device).to(torch.bfloat16) for K, _ in shapes]
    ys = [torch.empty((M, N), dtype=torch.bfloat16, device=device) for _, N in shapes]

    # Dataflow of the reference's Llama forward (crates/models/arch/dsl/llama.py:10-30): q, k and v read
    # the same normed activation and are independent of each other, as are gate and up; o waits for the
    # three, down for the two.  The tape keeps exactly those dependencies: independent linears go to
    # parallel branches of the graph (forked streams at capture), dependent ones join first.
    branch = [torch.cuda.Stream(device) for _ in range(2)]

    from scratchy_b200 import AffineQuantLinear

    def run_group(row, idxs):
        cur = torch.cuda.current_stream(device)
        if len(idxs) == 1 or args.serial:
            for i in idxs:
                row[i].forward(xs[i], out=ys[i])
            return
        if not args.branches:
            # independent linears over the same activation (q, k, v; gate, up): one group launch
            AffineQuantLinear.forward_group([row[i] for i in idxs], xs[idxs[0]], [ys[i] for i in idxs])
            return
        for b, i in enumerate(idxs[1:]):
            branch[b].wait_stream(cur)
            with torch.cuda.stream(branch[b]):
                row[i].forward(xs[i], out=ys[i])
        row[idxs[0]].forward(xs[idxs[0]], out=ys[idxs[0]])
        for b in range(len(idxs) - 1):
            cur.wait_stream(branch[b])

    def step():
        for row in layers:
            run_group(row, [0, 1, 2])      # q, k, v
            run_group(row, [3])            # o
            run_group(row, [4, 5])         # gate, up
            run_group(row, [6])            # down

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    # The decode step is a static tape of launches (as in the reference, whose per-bucket tapes are
    # fixed at build time), so it is captured once into a CUDA graph and replayed per step.
    step()
    barrier()
    side = torch.cuda.Stream(device)
    graph = torch.cuda.CUDAGraph()
    l0 = ctx.launch_count()
    with torch.cuda.graph(graph, stream=side):
        step()
    launches_per_step = ctx.launch_count() - l0

    # ---- device-resident timing (the clock sampler runs from the warm-up on, so that even a short timed
    # region has samples taken under this load beside it)
    sampler = ClockSampler(local_rank) if rank == 0 else None
    for _ in range(args.warmup):
        graph.replay()
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    for _ in range(args.steps):
        graph.replay()
    ev1.record()
    barrier()
    ms = ev0.elapsed_time(ev1)
    launches = launches_per_step * args.steps
    clocks = sampler.stop() if sampler else None

    # ---- extra, not the headline: the same weights as the reference's fused projections, 4 launches per layer
    fused_info = None
    if world == 1:
        fx = [xs[0], xs[3], xs[4], xs[6]]
        fy = [torch.empty((M, l.out_features), dtype=torch.bfloat16, device=device) for l in fused_layers[0]]

        def step_fused():
            for row in fused_layers:
                for i in range(4):
                    row[i].forward_ends(fx[i], fy[i])
        step_fused()
        torch.cuda.synchronize(device)
        graph_f = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph_f, stream=side):
            step_fused()
        for _ in range(max(3, args.warmup)):
            graph_f.replay()
        torch.cuda.synchronize(device)
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record()
        for _ in range(args.steps):
            graph_f.replay()
        f1.record()
        torch.cuda.synchronize(device)
        ms_f = f0.elapsed_time(f1)
        fused_info = {"value": step_bytes * args.steps / (ms_f * 1e-3) / 1e9, "unit": UNIT, "ms_per_step": ms_f / args.steps,
                      "launches_per_step": 4 * N_LAYERS,
                      "workload": "the same 7 linears per layer as q|k|v and gate|up rows-concat fused projections "
                                  "(the reference's load_rows_concat): 4 launches per layer in stream order over concatenated "
                                  "matrices (the headline runs the same 4 launches over the separate matrices)"}
        del graph_f
    fused_layers = None

    # ---- extra, not the headline: the same 196 linears and dependencies as ONE persistent launch (the matvec tape)
    tape_info = None
    if world == 1:
        from scratchy_b200 import AffineTape
        jobs = []
        for li, row in enumerate(layers):
            b = 7 * li
            prev = [b - 1] if li else []
            deps = [prev, prev, prev, [b, b + 1, b + 2], [b + 3], [b + 3], [b + 4, b + 5]]
            jobs += [(row[i], xs[i], ys[i], deps[i]) for i in range(7)]
        tape = AffineTape(jobs, max_rows=M)
        tape.run()
        torch.cuda.synchronize(device)
        graph_t = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph_t, stream=side):
            tape.run()
        for _ in range(max(3, args.warmup)):
            graph_t.replay()
        torch.cuda.synchronize(device)
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(args.steps):
            graph_t.replay()
        t1.record()
        torch.cuda.synchronize(device)
        ctx.device_status(None)
        ms_t = t0.elapsed_time(t1)
        tape_info = {"value": step_bytes * args.steps / (ms_t * 1e-3) / 1e9, "unit": UNIT, "ms_per_step": ms_t / args.steps,
                     "launches_per_step": 1,
                     "workload": "the same 196 linears with the same dependencies inside one persistent cooperative launch "
                                 "(scr_linear_affine_b4_tape)"}
        del graph_t
        tape.close()

    # ---- end to end: host (pinned) activations in, host results out, through the public API.
    # Every linear's input is copied from pinned host memory and its output copied back inside
    # the timed region; the copies are captured in the same graph as the launches.
    # One pinned staging buffer holds the step's activations (one row-set per linear of every
    # layer) and one receives all outputs.  Two H2D and two D2H copies per step on copy streams of their own (graph
    # branches): the first layer's inputs, then everything else while the first layer computes; the outputs of all but
    # the last layer while the last layer computes, then the last layer's.  (A copy per layer was measured slower: 56
    # copy nodes and 56 cross-stream dependencies cost more than the 3 MB they hide.)
    # q, k and v read one activation, gate and up another: a layer has four distinct inputs (`--branches` / `--serial`,
    # where every linear is its own launch, keep one input per linear)
    shared_in = not (args.branches or args.serial)
    in_of = [0, 0, 0, 3, 4, 4, 6] if shared_in else list(range(7))       # linear -> the input it reads
    in_elems = [M * shapes[i][0] if in_of[i] == i else 0 for i in range(7)]
    out_elems = [M * N for _, N in shapes]
    h_in = torch.randn(N_LAYERS * sum(in_elems)).to(torch.bfloat16).pin_memory()
    h_out = torch.empty(N_LAYERS * sum(out_elems), dtype=torch.bfloat16).pin_memory()
    d_in = torch.empty_like(h_in, device=device)
    d_out = torch.empty_like(h_out, device=device)
    h2d = h_in.numel() * 2
    d2h = h_out.numel() * 2
    views = []
    oi = oo = 0
    for li in range(N_LAYERS):
        row, in_views = [], {}
        for i, ((K, N), ne_i, ne_o) in enumerate(zip(shapes, in_elems, out_elems)):
            if in_of[i] == i:
                in_views[i] = d_in[oi:oi + ne_i].view(M, K)
                oi += ne_i
            row.append((in_views[in_of[i]], d_out[oo:oo + ne_o].view(M, N)))
            oo += ne_o
        views.append(row)

    in_per_layer, out_per_layer = sum(in_elems), sum(out_elems)
    copy_in, copy_out = torch.cuda.Stream(device), torch.cuda.Stream(device)

    def step_e2e():
        main = torch.cuda.current_stream(device)
        copy_in.wait_stream(main)
        copy_out.wait_stream(main)
        last = N_LAYERS - 1
        with torch.cuda.stream(copy_in):
            d_in[:in_per_layer].copy_(h_in[:in_per_layer], non_blocking=True)
            first_in = torch.cuda.Event()
            first_in.record(copy_in)
            d_in[in_per_layer:].copy_(h_in[in_per_layer:], non_blocking=True)
            rest_in = torch.cuda.Event()
            rest_in.record(copy_in)
        for li, (row, vrow) in enumerate(zip(layers, views)):
            if li == 0:
                main.wait_event(first_in)
            elif li == 1:
                main.wait_event(rest_in)
            if li == last:                                   # everything before the last layer goes home while it computes
                done = torch.cuda.Event()
                done.record(main)
                copy_out.wait_event(done)
                with torch.cuda.stream(copy_out):
                    h_out[:last * out_per_layer].copy_(d_out[:last * out_per_layer], non_blocking=True)
            for idxs in ([0, 1, 2], [3], [4, 5], [6]):
                cur = torch.cuda.current_stream(device)
                if len(idxs) == 1 or args.serial:
                    for i in idxs:
                        row[i].forward(vrow[i][0], out=vrow[i][1])
                    continue
                if not args.branches:
                    AffineQuantLinear.forward_group([row[i] for i in idxs], vrow[idxs[0]][0], [vrow[i][1] for i in idxs])
                    continue
                for b, i in enumerate(idxs[1:]):
                    branch[b].wait_stream(cur)
                    with torch.cuda.stream(branch[b]):
                        row[i].forward(vrow[i][0], out=vrow[i][1])
                row[idxs[0]].forward(vrow[idxs[0]][0], out=vrow[idxs[0]][1])
                for b in range(len(idxs) - 1):
                    cur.wait_stream(branch[b])
        main.wait_stream(copy_in)
        copy_out.wait_stream(main)
        with torch.cuda.stream(copy_out):
            h_out[last * out_per_layer:].copy_(d_out[last * out_per_layer:], non_blocking=True)
        main.wait_stream(copy_out)

    step_e2e()
    barrier()
    graph_e2e = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph_e2e, stream=side):
        step_e2e()
    for _ in range(max(3, args.warmup // 2)):
        graph_e2e.replay()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        graph_e2e.replay()
        torch.cuda.current_stream(device).synchronize()      # the host reads the step's results
    e1.record()
    barrier()
    ms_e2e = e0.elapsed_time(e1)

    t = torch.tensor([ms, ms_e2e], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms_e2e = float(t[0]), float(t[1])

    value = world * step_bytes * args.steps / (ms * 1e-3) / 1e9
    e2e_value = world * step_bytes * args.steps / (ms_e2e * 1e-3) / 1e9
    per_launch_us = ms * 1e3 / max(launches, 1)
    achieved = step_bytes * args.steps / (ms * 1e-3) / 1e9          # one GPU's kernel stream

    extra = {}
    if fused_info:
        extra["fused_projections"] = fused_info
    if tape_info:
        extra["tape"] = tape_info
    if world == 1:
        extra["config0"] = run_config0(device, peaks)
        extra["prefill"] = run_prefill_extra(device, peaks)
    if world == 1 and not args.no_decode:
        del layers, graph, graph_e2e
        layers = graph = graph_e2e = None
        torch.cuda.empty_cache()
        extra["decode"] = {"workload": "llama-3.2-3b random-init, all linears int4 g64, bf16 paged KV, one CUDA graph per step",
                           "cases": run_decode(device)}
    if args.sweep and rank == 0:
        extra["sweep"] = run_sweep(device, ctx)
    if world > 1 or args.sweep:
        del layers, graph, graph_e2e
        torch.cuda.empty_cache()
        tp_res = run_tp(device, world, rank, fuse_exchange=not args.tp_separate_exchange)
        if rank == 0:
            extra["tp"] = tp_res

    if rank == 0:
        cpu_v, cpu_dt, cores = time_cpu_layer(max(1, int(12.0 / max(time_cpu_layer(1)[1], 1e-3))))
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "llama-3.2-3b int4 g64 linears (q,k,v,o,gate,up,down) x 28 layers, M=1",
                       "bytes_per_step": step_bytes, "l2": "inputs larger than L2 (1.585 GB of distinct weights per step)",
                       "dependencies": "stream order only: the linears of one shape share one input and one output buffer, so a linear "
                                       "waits for its predecessors without consuming their values (a weight-stream measurement)",
                       "replicas": world,
                       "launch": ("one CUDA graph per step; the 7 linears of a layer in 4 launches: q, k, v (one activation) and gate, up "
                                  "(one activation) each as one group launch over the members' own packed buffers "
                                  "(scr_linear_affine_b4_group), o and down on their own") if not (args.serial or args.branches)
                       else ("one CUDA graph of 196 matvec launches per step; q/k/v and gate/up on parallel branches" if args.branches
                             else "one CUDA graph of 196 matvec launches per step, one branch")},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": achieved / peaks["hbm_gbs"],
                         # per launch: the per-shape ncu figures (GEMV_DRAM_TRAFFIC) of a layer's 7 matrices over the
                         # launches that stream them (a group launch streams its members' matrices, each once)
                         "traffic": N_LAYERS * sum(GEMV_DRAM_TRAFFIC[n] for n in LAYER_ORDER) / launches_per_step,
                         "traffic_source": "ncu dram__bytes_read+write per launch, by shape: profiles/affine_b4_gemv_llama3b_m1_full.md, "
                                           "profiles/affine_b4_gemv_llama3b_gate_m1_full.md",
                         "peak_source": peaks["src"],
                         "kernel": "affine_b4_gemv_kernel", "avg_launch_us": per_launch_us,
                         "launches_per_step": launches_per_step,
                         "alg_bytes_per_launch": step_bytes / launches_per_step},
            "cpu_baseline": {"value": cpu_v, "unit": UNIT, "cores": cores, "kind": "port",
                             "sample": f"7 linears of one layer, {cpu_dt * 1e3:.1f} ms per pass, oracle C++/OpenMP"},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": int(launches),
            "clocks": clocks,
        }
        line.update(extra)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def _time_calls(device, calls, replays):
    """One CUDA graph over `calls` (each on its own weight copy), replayed; seconds per call."""
    import torch
    for c in calls[:2]:
        c()
    torch.cuda.synchronize(device)
    side = torch.cuda.Stream(device)
    gr = torch.cuda.CUDAGraph()
    with torch.cuda.graph(gr, stream=side):
        for c in calls:
            c()
    for _ in range(3):
        gr.replay()
    torch.cuda.synchronize(device)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(replays):
        gr.replay()
    b.record()
    torch.cuda.synchronize(device)
    return a.elapsed_time(b) * 1e-3 / (replays * len(calls))


def _int4_copies(device, N, K, copies):
    import torch
    from scratchy_b200 import AffineQuantLinear
    lins = []
    for c in range(copies):
        g = torch.Generator(device=device)
        g.manual_seed(7000 + c)
        w = torch.randint(-2 ** 31, 2 ** 31 - 1, (N, K // 8), dtype=torch.int32, device=device, generator=g)
        s = (torch.randn((N, K // 64), device=device, generator=g) * 0.02).abs().add(1e-3).to(torch.bfloat16)
        b = (-8.0 * s.float() + torch.randn((N, K // 64), device=device, generator=g) * 1e-3).to(torch.bfloat16)
        lins.append(AffineQuantLinear.from_tensors(w, s, b, 64, 4))
    return lins


def run_config0(device, peaks):
    """Benchmark configuration 0 on its own: the single MLX int4 linear M = 1, K = 3072, N = 8192, timed over 29 distinct
    weight copies (411 MB, larger than L2) inside one CUDA graph — no neighbour prefetches for it."""
    import torch
    N, K, M = 8192, 3072, 1
    lins = _int4_copies(device, N, K, 29)
    x = torch.randn((M, K), device=device).to(torch.bfloat16)
    y = torch.empty((M, N), dtype=torch.bfloat16, device=device)
    dt = _time_calls(device, [(lambda l=l: l.forward(x, out=y)) for l in lins], 20)
    byts = affine_alg_bytes(M, N, K)
    return {"workload": "one int4 g64 linear, M=1, K=3072, N=8192, 29 rotating weight copies (larger than L2)", "us": dt * 1e6,
            "alg_bytes": byts, "GBps": byts / dt / 1e9, "frac_hbm_measured": byts / dt / 1e9 / peaks["hbm_gbs"],
            "frac_hbm_nominal_8000": byts / dt / 1e9 / 8000.0}


def run_prefill_extra(device, peaks):
    """A bounded sample of the prefill and fp8 sweeps for the default line: int4 gate at 2048 tokens, fp8 gate at 2048 and
    8192 tokens (quantise + GEMM), fp8 gate at one token.  The fp8 tensor peak is not in the measured-peaks file: fractions are
    quoted against 2 x the measured bf16 burst figure (named as such), against a library fp8 GEMM measured here the same way
    (`torch._scaled_mm`, 8192^3), and against the nominal 4500 TFLOP/s."""
    import torch
    from scratchy_b200 import Fp8Linear
    out = []
    fp8_lib = measure_fp8_peak(device)
    K, N = synth.LLAMA_3_2_3B["gate"]
    lins = _int4_copies(device, N, K, 4)
    M = 2048
    x = torch.randn((M, K), device=device).to(torch.bfloat16)
    y = torch.empty((M, N), dtype=torch.bfloat16, device=device)
    ws = torch.empty(max(16, lins[0].workspace_bytes(M)), dtype=torch.uint8, device=device)
    dt = _time_calls(device, [(lambda l=l: l.forward(x, out=y, workspace=ws)) for l in lins], 5)
    tf = 2.0 * M * N * K / dt / 1e12
    out.append({"kind": "int4", "shape": "gate", "M": M, "N": N, "K": K, "us": dt * 1e6, "TFLOPs": tf,
                "frac_bf16_measured": tf / peaks["bf16_tflops"], "frac_bf16_nominal_2250": tf / 2250.0})
    del lins, x, y, ws
    K, N = synth.QWEN_2_5_7B["gate"]
    copies = 4
    flins = []
    for c in range(copies):
        g = torch.Generator(device=device)
        g.manual_seed(7100 + c)
        w = torch.randint(0, 0x7E, (N, K), dtype=torch.uint8, device=device, generator=g)
        flins.append(Fp8Linear.from_tensors(w, torch.rand(N, device=device, generator=g) * 1e-3 + 1e-4))
    for M in (1, 2048, 8192):
        x = torch.randn((M, K), device=device).to(torch.bfloat16)
        y = torch.empty((M, N), dtype=torch.bfloat16, device=device)
        ws = torch.empty(max(16, flins[0].workspace_bytes(M)), dtype=torch.uint8, device=device)
        dt = _time_calls(device, [(lambda l=l: l.forward(x, out=y, workspace=ws)) for l in flins], 20 if M == 1 else 3)
        tf = 2.0 * M * N * K / dt / 1e12
        row = {"kind": "fp8", "shape": "gate", "M": M, "N": N, "K": K, "us": dt * 1e6}
        if M == 1:
            row.update({"GBps": fp8_alg_bytes(M, N, K) / dt / 1e9, "frac_hbm_measured": fp8_alg_bytes(M, N, K) / dt / 1e9 / peaks["hbm_gbs"],
                        "note": "one launch: the matvec quantises the activation itself; 4 copies x 68 MB rotate (larger than L2)"})
        else:
            row.update({"TFLOPs": tf, "frac_of_2x_bf16_measured": tf / (2.0 * peaks["bf16_tflops"]),
                        "frac_of_scaled_mm_8192": (tf / fp8_lib) if fp8_lib else None, "frac_fp8_nominal_4500": tf / 4500.0,
                        "note": "per-token quantise + GEMM (two launches)"})
        out.append(row)
        del x, y, ws
    out.append({"kind": "peaks", "bf16_tflops_measured": peaks["bf16_tflops"], "fp8_tflops_scaled_mm_8192": fp8_lib,
                "fp8_tflops_nominal": 4500.0, "hbm_gbs_measured": peaks["hbm_gbs"]})
    return out


def measure_fp8_peak(device):
    """Dense fp8 tensor peak, measured the way the bf16 figure in MEASURED_PEAKS.json was: a library
    GEMM (`torch._scaled_mm`, e4m3 x e4m3 -> bf16, 8192^3), best of 10, CUDA events.  None if the
    library call is not available."""
    import torch
    try:
        n = 8192
        a = torch.randn((n, n), device=device).to(torch.float8_e4m3fn)
        b = torch.randn((n, n), device=device).to(torch.float8_e4m3fn).t()
        one = torch.ones((), device=device)
        for _ in range(3):
            torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
        torch.cuda.synchronize(device)
        best = float("inf")
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
            e1.record()
            torch.cuda.synchronize(device)
            best = min(best, e0.elapsed_time(e1))
        return 2.0 * n ** 3 / (best * 1e-3) / 1e12
    except Exception:
        return None


def run_sweep(device, ctx):
    """Extra (not the headline): per-shape timings over M for int4 (3B shapes) and fp8 (7B shapes).
    Each case cycles over enough distinct weight copies that consecutive calls miss L2, captured
    as one CUDA graph of `reps` calls and replayed."""
    import torch
    from scratchy_b200 import AffineQuantLinear, Fp8Linear
    peaks = measured_peaks()
    fp8_peak = measure_fp8_peak(device)
    out = [{"kind": "peak", "fp8_tflops_scaled_mm_8192": fp8_peak, "fp8_tflops_nominal": 4500.0,
            "bf16_tflops_measured": peaks["bf16_tflops"], "hbm_gbs_measured": peaks["hbm_gbs"], "hbm_gbs_nominal": 8000.0}]
    side = torch.cuda.Stream(device)

    def time_graph(calls, replays):
        for c in calls[:2]:
            c()
        torch.cuda.synchronize(device)
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr, stream=side):
            for c in calls:
                c()
        for _ in range(3):
            gr.replay()
        torch.cuda.synchronize(device)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(replays):
            gr.replay()
        b.record()
        torch.cuda.synchronize(device)
        return a.elapsed_time(b) * 1e-3 / (replays * len(calls))

    for name in ["q", "k", "gate", "down"]:
        K, N = synth.LLAMA_3_2_3B[name]
        copies = max(2, int((256 << 20) // (N * K * 9 // 16)) + 1)
        lins = []
        for c in range(copies):
            w = torch.randint(-2 ** 31, 2 ** 31 - 1, (N, K // 8), dtype=torch.int32, device=device)
            s = (torch.randn((N, K // 64), device=device) * 0.02).abs().add(1e-3).to(torch.bfloat16)
            b = (-8.0 * s.float()).to(torch.bfloat16)
            lins.append(AffineQuantLinear.from_tensors(w, s, b))
        for M in [1, 4, 16, 64, 512, 2048]:
            x = torch.randn((M, K), device=device).to(torch.bfloat16)
            y = torch.empty((M, N), dtype=torch.bfloat16, device=device)
            ws = torch.empty(max(16, lins[0].workspace_bytes(M)), dtype=torch.uint8, device=device)
            reps = copies if M <= 64 else min(copies, 8)
            calls = [(lambda l=l: l.forward(x, out=y, workspace=ws)) for l in lins[:reps]]
            dt = time_graph(calls, 5 if M <= 64 else 2)
            out.append({"kind": "int4", "shape": name, "M": M, "N": N, "K": K, "us": dt * 1e6,
                        "GBps": affine_alg_bytes(M, N, K) / dt / 1e9, "TFLOPs": 2.0 * M * N * K / dt / 1e12,
                        "frac_hbm": affine_alg_bytes(M, N, K) / dt / 1e9 / peaks["hbm_gbs"],
                        "frac_bf16": 2.0 * M * N * K / dt / 1e12 / peaks["bf16_tflops"]})
        del lins
    for name in ["q", "k", "gate", "down"]:
        K, N = synth.QWEN_2_5_7B[name]
        copies = max(2, int((256 << 20) // (N * K)) + 1)
        lins = []
        for c in range(copies):
            w = torch.randint(0, 120, (N, K), dtype=torch.uint8, device=device)
            lins.append(Fp8Linear.from_tensors(w, torch.rand(N, device=device) * 1e-3 + 1e-4))
        for M in [1, 16, 256, 2048, 8192]:
            x = torch.randn((M, K), device=device).to(torch.bfloat16)
            y = torch.empty((M, N), dtype=torch.bfloat16, device=device)
            ws = torch.empty(lins[0].workspace_bytes(M), dtype=torch.uint8, device=device)
            reps = copies if M <= 256 else min(copies, 4)
            calls = [(lambda l=l: l.forward(x, out=y, workspace=ws)) for l in lins[:reps]]
            dt = time_graph(calls, 5 if M <= 256 else 2)
            out.append({"kind": "fp8", "shape": name, "M": M, "N": N, "K": K, "us": dt * 1e6,
                        "GBps": fp8_alg_bytes(M, N, K) / dt / 1e9, "TFLOPs": 2.0 * M * N * K / dt / 1e12,
                        "frac_hbm": fp8_alg_bytes(M, N, K) / dt / 1e9 / peaks["hbm_gbs"],
                        "frac_fp8_measured": (2.0 * M * N * K / dt / 1e12 / fp8_peak) if fp8_peak else None,
                        "frac_fp8_nominal": 2.0 * M * N * K / dt / 1e12 / 4500.0,
                        "note": "per-token quantise + contraction (two launches)"})
        del lins
    return out


def run_decode(device, steps=20, batches=(1, 8, 32), context=2048, block_size=16, fuse_rope=True):
    """Benchmark configuration 3: random-init Llama-3.2-3B, every linear MLX int4 g64 (lm_head too), one decode
    step at context `context` with a bf16 paged KV cache, the whole step one CUDA graph.
    tok/s = batch / step time.  The step streams all packed weights (larger than L2) plus the batch's KV."""
    import torch
    from scratchy_b200 import _lib, decode
    peaks = measured_peaks()
    cfg = decode.LLAMA_3_2_3B
    dec = decode.LlamaDecoder(cfg, decode.synthetic_checkpoint_on_device(cfg, device, 0), device, max_pos=context + 64,
                              fuse_rope=fuse_rope)
    ctx = _lib.context(device.index)
    out = []
    blocks_per_seq = (context + 1 + block_size - 1) // block_size
    for batch in batches:
        cache = decode.PagedKvCache(cfg, batch * blocks_per_seq, block_size, device)
        g = torch.Generator(device=device)
        g.manual_seed(batch)
        for t in cache.k + cache.v:
            t.copy_(torch.randn(t.shape, device=device, generator=g).to(torch.bfloat16))
        buf = dec.buffers(batch, blocks_per_seq)
        buf.ids.copy_(torch.randint(0, cfg.vocab, (batch,), device=device, generator=g, dtype=torch.int32))
        buf.positions.fill_(context)
        buf.seq_used_k.fill_(context + 1)
        table = torch.randperm(batch * blocks_per_seq, device=device, generator=g).to(torch.int32)
        buf.block_table.copy_(table.reshape(batch, blocks_per_seq))
        buf.slot_mapping.copy_(buf.block_table[:, context // block_size] * block_size + context % block_size)
        n0 = ctx.launch_count()
        dec.step(buf, cache)
        launches = ctx.launch_count() - n0
        graph = dec.capture(buf, cache)
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize(device)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            graph.replay()
        b.record()
        torch.cuda.synchronize(device)
        dt = a.elapsed_time(b) * 1e-3 / steps
        ctx.device_status(None)
        kv_bytes = batch * (context + 1) * cfg.n_kv_heads * cfg.head_dim * 2 * 2 * cfg.n_layers
        moved = dec.weight_bytes() + kv_bytes
        out.append({"batch": batch, "context": context, "ms_per_step": dt * 1e3, "tok_per_s": batch / dt,
                    "launches_per_step": int(launches), "weight_bytes": dec.weight_bytes(), "kv_bytes": kv_bytes,
                    "GBps": moved / dt / 1e9, "frac_hbm": moved / dt / 1e9 / peaks["hbm_gbs"]})
        del graph, buf, cache
        torch.cuda.empty_cache()
    return out


TP_H, TP_QKV, TP_FF = 8192, 10240, 28672          # Llama-3-70B: hidden, q|k|v rows (64 q + 2 x 8 kv heads of 128), intermediate
TP_CHUNK_ROWS = 1024                              # prefill rows per pipeline chunk (chunk i's exchange overlaps chunk i+1's GEMMs)


def tp_parity_check(device, world, rank, tpw, one, fuse_exchange):
    """In-run value check of the tensor-parallel row-parallel path on the real ranks: a seeded o-projection
    (8192 -> 8192, every rank its K-slice) at M = 1, 32 and 256 through the very calls the timed step makes, rank 0
    against the lockstep oracle (every rank's f32 partial, summed in rank order, rounded once) on a seeded sample of
    output channels.  Returns "ok" or a description of the first failure; every rank takes part."""
    import torch
    import oracle
    from scratchy_b200 import Fp8Linear, tp as tpmod
    H = TP_H
    rng = np.random.default_rng(1234)
    wq = rng.integers(0, 0x7E, size=(H, H), dtype=np.uint8)                 # finite e4m3 patterns
    wsc = (rng.random(H) * 1e-3 + 1e-4).astype(np.float32)
    cols = np.sort(rng.choice(H, 256, replace=False))
    lo, hi = rank * (H // world), (rank + 1) * (H // world)
    lin = Fp8Linear.from_tensors(torch.from_numpy(np.ascontiguousarray(wq[:, lo:hi])).to(device), torch.from_numpy(wsc).to(device))
    comm = tpmod.TpCommunicator(tpw)
    verdict = "ok"
    for M in (1, 32, 256):
        x = synth.activations_bf16(M, H, 77 + M)
        xl = torch.from_numpy(np.ascontiguousarray(x[:, lo:hi]).view(np.int16)).view(torch.bfloat16).to(device)
        if world == 1:
            y = tpmod.partial_to_bf16(lin.forward_partial(xl))
        elif one is not None and fuse_exchange and one.fp8_linear_all_reduce_supported(lin, M):
            y = one.fp8_linear_all_reduce(lin, xl)
        elif one is not None and M * H <= one.max_elems:
            y = one.all_reduce(lin.forward_partial(xl))
        else:
            part = lin.forward_partial(xl)
            comm.all_reduce(part)
            y = tpmod.partial_to_bf16(part)
        torch.cuda.synchronize(device)
        if rank == 0 and verdict == "ok":
            rows = np.arange(M) if M <= 32 else np.sort(rng.choice(M, 16, replace=False))
            parts = []
            for r in range(world):
                sl = slice(r * (H // world), (r + 1) * (H // world))
                _, pf = oracle.fp8_dynamic_linear(np.ascontiguousarray(x[rows][:, sl]), np.ascontiguousarray(wq[cols][:, sl]),
                                                  wsc[cols], len(rows), len(cols), H // world, want_f32=True)
                parts.append(pf)
            want = synth.bf16_bits_to_f32(oracle.f32_to_bf16_bits(oracle.allreduce_rank_order(parts))).astype(np.float64)
            got = y.float().cpu().numpy()[rows][:, cols].astype(np.float64)
            err = float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))
            if not err <= 1e-3:
                verdict = f"M={M}: rel-L2 {err:.3e} against the lockstep oracle"
    return verdict


def run_tp(device, world, rank, fuse_exchange=True):
    """Benchmark configuration 4: Llama-3-70B-shaped fp8 per-channel linears, tensor parallel over `world`
    GPUs: column-parallel qkv and gate/up, row-parallel o and down, each followed by the all-reduce of the f32
    partials [M, 8192] in rank order and one rounding to bf16 — inside the row-parallel matvec's epilogue up to 4
    tokens, the stand-alone peer-memory kernel above (packets, dense one-shot, or — from 16 tokens on — the two-phase
    reduce-scatter + all-gather form, `scr_tp_allreduce_partial`).  Prefill batches run as chunks of 1024 rows on two
    streams, so that one chunk's exchange overlaps the next chunk's GEMMs.  One "layer" = qkv, o, gate_up, down
    (attention and the activation function are outside the path: the row-parallel inputs are fixed buffers of their
    shapes).  Weights are random e4m3 bytes; three layer copies rotate so that small-M steps read HBM, not L2.
    Every rank first times the unsharded (TP = 1) stack on its own GPU: `efficiency` = t(TP=1) / (W * t(TP=W))."""
    import torch
    import torch.distributed as dist
    from scratchy_b200 import Fp8Linear, _lib, tp as tpmod
    tpw = tpmod.TpWorld(world, rank)
    H, QKV, FF = TP_H, TP_QKV, TP_FF
    copies = 3
    Ms = [1, 32, 256, 8192]
    side = [torch.cuda.Stream(device) for _ in range(2)]

    def lin(n, k, seed):
        g = torch.Generator(device=device)
        g.manual_seed(seed)
        w = torch.randint(0, 0x7E, (n, k), dtype=torch.uint8, device=device, generator=g)
        return Fp8Linear.from_tensors(w, torch.rand(n, device=device, generator=g) * 1e-3 + 1e-4)

    def time_run(run, reps, sync_ranks):
        for _ in range(3):
            run()
        if sync_ranks:
            dist.barrier()
        torch.cuda.synchronize(device)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            run()
        b.record()
        torch.cuda.synchronize(device)
        t = torch.tensor([a.elapsed_time(b)], dtype=torch.float64, device=device)
        if sync_ranks:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0]) * 1e3 / (reps * copies)                  # us per layer

    def graph_of(step):
        step()
        torch.cuda.synchronize(device)
        try:
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr, stream=side[0]):
                step()
            return gr.replay, "graph", gr
        except Exception:
            return step, "eager", None

    # ---- the unsharded stack on this GPU (no exchange: the partial is the sum)
    t1 = {}
    if world > 1:
        layers1 = [{"qkv": lin(QKV, H, 10 * c + 1), "o": lin(H, H, 10 * c + 2), "gate_up": lin(2 * FF, H, 10 * c + 3),
                    "down": lin(H, FF, 10 * c + 4)} for c in range(copies)]
        for M in Ms:
            x = torch.randn((M, H), device=device).to(torch.bfloat16)
            act = torch.randn((M, FF), device=device).to(torch.bfloat16)
            ws = torch.empty(max(l.workspace_bytes(M) for l in layers1[0].values()), dtype=torch.uint8, device=device)
            o_qkv = torch.empty((M, QKV), dtype=torch.bfloat16, device=device)
            o_gu = torch.empty((M, 2 * FF), dtype=torch.bfloat16, device=device)
            h = torch.empty((M, H), dtype=torch.bfloat16, device=device)
            y = torch.empty((M, H), dtype=torch.bfloat16, device=device)

            def step1():
                for L in layers1:
                    L["qkv"].forward(x, out=o_qkv, workspace=ws)
                    L["o"].forward(x, out=h, workspace=ws)
                    L["gate_up"].forward(h, out=o_gu, workspace=ws)
                    L["down"].forward(act, out=y, workspace=ws)
            run, _, gr = graph_of(step1)
            t1[M] = time_run(run, 20 if M <= 256 else 3, sync_ranks=False)
            del gr, x, act, ws, o_qkv, o_gu
        del layers1
        torch.cuda.empty_cache()

    # ---- the peer-memory exchange (every rank must take the same path: agree on whether it came up everywhere)
    ones, one_note = [None, None], None
    if world > 1:
        try:
            ones = [tpmod.OneShotAllReduce(tpw, device, max_elems=TP_CHUNK_ROWS * H) for _ in range(2)]    # one per stream
            ok = torch.ones(1, device=device)
        except Exception as exc:                                  # e.g. peer access unavailable between two GPUs
            one_note = f"peer-memory exchange unavailable ({type(exc).__name__}); NCCL used"
            ok = torch.zeros(1, device=device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if float(ok[0]) == 0.0:
            ones = [None, None]
            one_note = one_note or "peer-memory exchange unavailable on another rank; NCCL used"
    one = ones[0]
    comm = tpmod.TpCommunicator(tpw)
    parity = tp_parity_check(device, world, rank, tpw, one, fuse_exchange)

    layers = []
    for c in range(copies):
        layers.append({"qkv": lin(QKV // world, H, 10 * c + 1), "o": lin(H, H // world, 10 * c + 2),
                       "gate_up": lin(2 * FF // world, H, 10 * c + 3), "down": lin(H, FF // world, 10 * c + 4)})
    out = []
    for M in Ms:
        rows = min(M, TP_CHUNK_ROWS)
        n_chunks = M // rows
        lanes = 2 if n_chunks > 1 and one is not None else 1      # pipeline lanes (streams), each with its own buffers
        x = torch.randn((M, H), device=device).to(torch.bfloat16)
        attn = torch.randn((M, H // world), device=device).to(torch.bfloat16)
        act = torch.randn((M, FF // world), device=device).to(torch.bfloat16)
        ws_bytes = max(l.workspace_bytes(rows) for l in layers[0].values())
        lane_bufs = [{"ws": torch.empty(ws_bytes, dtype=torch.uint8, device=device),
                      "qkv": torch.empty((rows, QKV // world), dtype=torch.bfloat16, device=device),
                      "gu": torch.empty((rows, 2 * FF // world), dtype=torch.bfloat16, device=device),
                      "po": torch.empty((rows, H), dtype=torch.float32, device=device),
                      "pd": torch.empty((rows, H), dtype=torch.float32, device=device),
                      "h": torch.empty((rows, H), dtype=torch.bfloat16, device=device),
                      "y": torch.empty((rows, H), dtype=torch.bfloat16, device=device)} for _ in range(lanes)]
        use_peer = one is not None and rows * H <= one.max_elems
        # a few tokens: the row-parallel matvec pushes its partials to the peers and sums in its own epilogue
        fused = (use_peer and fuse_exchange and one.fp8_linear_all_reduce_supported(layers[0]["o"], M)
                 and one.fp8_linear_all_reduce_supported(layers[0]["down"], M))

        def reduce_round(part, dst, lane):
            if world == 1:                       # nothing to exchange: the partial is the sum
                dst.copy_(tpmod.partial_to_bf16(part))
            elif use_peer:
                ones[lane].all_reduce(part, out_bf16=dst)
            else:
                comm.all_reduce(part)
                dst.copy_(tpmod.partial_to_bf16(part))
            return dst

        def chunk_step(L, m0, lane):
            B = lane_bufs[lane]
            L["qkv"].forward(x[m0:m0 + rows], out=B["qkv"], workspace=B["ws"])
            if fused:
                h = ones[lane].fp8_linear_all_reduce(L["o"], attn[m0:m0 + rows], out=B["h"])
            else:
                L["o"].forward_partial(attn[m0:m0 + rows], out=B["po"], workspace=B["ws"])
                h = reduce_round(B["po"], B["h"], lane)
            L["gate_up"].forward(h, out=B["gu"], workspace=B["ws"])
            if fused:
                return ones[lane].fp8_linear_all_reduce(L["down"], act[m0:m0 + rows], out=B["y"])
            L["down"].forward_partial(act[m0:m0 + rows], out=B["pd"], workspace=B["ws"])
            return reduce_round(B["pd"], B["y"], lane)

        def step():
            cur = torch.cuda.current_stream(device)
            for L in layers:
                if lanes == 1:
                    for ci in range(n_chunks):
                        chunk_step(L, ci * rows, 0)
                    continue
                # two lanes: even chunks on the current stream, odd chunks on the second one; every rank issues the
                # calls of a lane's communicator in the same order
                side[1].wait_stream(cur)
                for ci in range(n_chunks):
                    if ci % 2 == 0:
                        chunk_step(L, ci * rows, 0)
                    else:
                        with torch.cuda.stream(side[1]):
                            chunk_step(L, ci * rows, 1)
                cur.wait_stream(side[1])

        run, mode, gr = graph_of(step)
        us_layer = time_run(run, 20 if M <= 256 else 3, sync_ranks=world > 1)
        flops = 2.0 * M * H * (QKV + H + 2 * FF + FF)
        count = rows * H
        form = ("none (one rank)" if world == 1 else
                "pushed and summed in the row-parallel matvec's epilogue over peer memory (one launch with the matvec)" if fused else
                "NCCL all-reduce of the f32 partials, then one rounding kernel" if not use_peer else
                "peer-memory kernel, packets" if count * world <= 32768 else
                "peer-memory kernel, two phases (reduce-scatter + all-gather of bf16)" if count >= 131072 else
                "peer-memory kernel, dense one-shot")
        row = {"M": M, "tp": world, "us_per_layer": us_layer, "layers_per_s": 1e6 / us_layer,
               "tok_per_s_per_layer": M * 1e6 / us_layer, "TFLOPs_all_gpus": flops / us_layer / 1e6,
               "weight_GBps_per_gpu": (H * (QKV + H + 3 * FF) / world) / us_layer / 1e3, "launch": mode,
               "chunks": n_chunks, "lanes": lanes, "allreduce": f"f32 [M,8192] x2 per layer, rank-ordered sum: {form}"}
        if world > 1:
            row["us_per_layer_tp1"] = t1[M]
            row["efficiency"] = t1[M] / (world * us_layer)
        out.append(row)
        del gr, lane_bufs
    try:
        _lib.context(device.index).device_status(None)
    except _lib.ScratchyCudaError as exc:                         # a bounded wait ran out somewhere: the numbers are void
        out.append({"error": str(exc)})
    out.append({"tp_parity": parity, "what": "o-projection 8192 -> 8192 at M = 1, 32, 256 on the real ranks against the lockstep oracle "
                                            "(rank-ordered f32 sum, one rounding) on 256 sampled channels, rel-L2 <= 1e-3"})
    for o in ones:
        if o is not None:
            o.close()
    if one_note:
        out.append({"note": one_note})
    return out


def run_case(args):
    """`--case kind,shape,M`: one linear, timed alone over rotating weight copies (profiling aid; prints one line)."""
    import torch
    from scratchy_b200 import AffineQuantLinear, Fp8Linear
    kind, name, M = args.case.split(",")
    M = int(M)
    device = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    if kind == "attn":
        return run_case_attention(device, batch=int(name), context=M, reps=args.steps)
    # kind "fp8x": the fp8 matvec with the tensor-parallel exchange in its epilogue, on a one-rank communicator
    # (pushes to itself: the whole kernel runs on one GPU)
    # kind "int4c": the int4 matvec through the matvec-ends entry point with no end set (scr_linear_affine_b4_ends)
    K, N = (synth.LLAMA_3_2_3B if kind in ("int4", "int4c") else synth.QWEN_2_5_7B)[name]
    copies = max(2, int((256 << 20) // (N * K)) + 1)
    lins = []
    for c in range(copies):
        if kind in ("int4", "int4c"):
            w = torch.randint(-2 ** 31, 2 ** 31 - 1, (N, K // 8), dtype=torch.int32, device=device)
            s_ = (torch.randn((N, K // 64), device=device) * 0.02).abs().add(1e-3).to(torch.bfloat16)
            lins.append(AffineQuantLinear.from_tensors(w, s_, (-8.0 * s_.float()).to(torch.bfloat16)))
        else:
            w = torch.randint(0, 120, (N, K), dtype=torch.uint8, device=device)
            lins.append(Fp8Linear.from_tensors(w, torch.rand(N, device=device) * 1e-3 + 1e-4))
    x = torch.randn((M, K), device=device).to(torch.bfloat16)
    y = torch.empty((M, N), dtype=torch.bfloat16, device=device)
    ws = torch.empty(max(16, lins[0].workspace_bytes(M)), dtype=torch.uint8, device=device)
    if kind == "fp8x":
        from scratchy_b200 import tp as tpmod
        one = tpmod.OneShotAllReduce(tpmod.TpWorld(1, 0), device, max_elems=(M * N + 3) // 4 * 4)

        def call(l):
            one.fp8_linear_all_reduce(l, x, out=y)
    elif kind == "int4c":
        def call(l):
            l.forward_ends(x, y)
    else:
        def call(l):
            l.forward(x, out=y, workspace=ws)
    for l in lins[:2]:
        call(l)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = args.steps
    a.record()
    for i in range(reps):
        call(lins[i % copies])
    b.record()
    torch.cuda.synchronize()
    dt = a.elapsed_time(b) * 1e-3 / reps
    print(json.dumps({"case": args.case, "us": dt * 1e6, "TFLOPs": 2.0 * M * N * K / dt / 1e12, "N": N, "K": K, "M": M}))


def run_case_attention(device, batch, context, reps, layers=28, block_size=16):
    """`--case attn,<batch>,<context>`: the paged decode attention alone at the Llama-3.2-3B geometry,
    one CUDA graph of `layers` calls over distinct caches (so consecutive calls miss L2), replayed."""
    import torch
    from scratchy_b200 import decode
    cfg = decode.LLAMA_3_2_3B
    blocks_per_seq = (context + block_size - 1) // block_size
    nblk = batch * blocks_per_seq
    shape = (nblk, cfg.n_kv_heads, block_size, cfg.head_dim)
    ks = [torch.randn(shape, device=device).to(torch.bfloat16) for _ in range(layers)]
    vs = [torch.randn(shape, device=device).to(torch.bfloat16) for _ in range(layers)]
    q = torch.randn((batch, cfg.q_dim), device=device).to(torch.bfloat16)
    out = torch.empty_like(q)
    table = torch.randperm(nblk, device=device).to(torch.int32).reshape(batch, blocks_per_seq)
    used = torch.full((batch,), context, dtype=torch.int32, device=device)

    def call(i):
        decode.attention_via_cache(q, ks[i], vs[i], table, used, cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim, block_size,
                                   cfg.head_dim ** -0.5, out=out)
    call(0)
    torch.cuda.synchronize()
    side = torch.cuda.Stream(device)
    gr = torch.cuda.CUDAGraph()
    with torch.cuda.graph(gr, stream=side):
        for i in range(layers):
            call(i)
    for _ in range(3):
        gr.replay()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        gr.replay()
    b.record()
    torch.cuda.synchronize()
    dt = a.elapsed_time(b) * 1e-3 / (reps * layers)
    kv = batch * context * cfg.n_kv_heads * cfg.head_dim * 2 * 2
    print(json.dumps({"case": f"attn,{batch},{context}", "us": dt * 1e6, "kv_bytes": kv, "GBps": kv / dt / 1e9}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--sweep", action="store_true")
    ap.add_argument("--serial", action="store_true", help="one branch: every linear waits for the previous one")
    ap.add_argument("--branches", action="store_true",
                    help="every linear its own launch, q/k/v and gate/up on parallel graph branches (instead of group launches)")
    ap.add_argument("--no-decode", action="store_true", help="skip the whole-decode-step section (config 3)")
    ap.add_argument("--decode-only", action="store_true", help="run only the whole-decode-step section and print it")
    ap.add_argument("--decode-batches", default="1,8,32")
    ap.add_argument("--no-fuse-rope", action="store_true", help="decode step with RoPE + append as a kernel of their own")
    ap.add_argument("--tp-separate-exchange", action="store_true",
                    help="tensor-parallel section: row-parallel matvec and all-reduce as two launches instead of "
                         "scr_linear_fp8_dynamic_allreduce (measured: equal at TP=2, 9 %% slower at TP=8)")
    ap.add_argument("--case", default=None, help="kind,shape,M e.g. int4,gate,2048: time one linear alone")
    args = ap.parse_args()
    if args.case:
        run_case(args)
        return
    if args.decode_only:
        import torch
        device = torch.device("cuda", 0)
        torch.cuda.set_device(device)
        cases = run_decode(device, steps=args.steps, batches=tuple(int(b) for b in args.decode_batches.split(",")),
                           fuse_rope=not args.no_fuse_rope)
        print(json.dumps({"decode": cases}))
        return
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
