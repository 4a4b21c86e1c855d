#!/usr/bin/env python
"""Benchmark of the quantized-linear decode path on B200.

Workload (N = 1): the Llama-2-7B decode layer set of the baseline's second
configuration -- q/k/v/o 4096x4096, gate/up 11008x4096, down 4096x11008, E8-D4
codebook at radius 1.75, 0.2 % critical blocks -- for 32 decoder layers with
distinct synthetic weights (1.66 GB of indices, far larger than the 126 MB L2,
so every step streams from HBM).  One step = one pass over all 224 linears at
batch B (default 1), i.e. the quantized-linear work of one decode token.

  value     algorithmic GB/s with everything resident in HBM (step replayed
            from a CUDA graph of C-ABI calls, CUDA-event timed).  The linears
            have fixed, independent inputs, so the seven linears of a decoder
            layer go into one eptq_linear_forward_group launch (--group 7);
            `one_launch_per_linear` reports the same pass with --group 1.
  e2e       the same GB/s through the Python module API (forward_group over
            EPTQLinear modules) with the activations in pinned HOST memory:
            H2D copy of x, all module calls, D2H copy of the last output inside
            the timed region of every step
  roofline  achieved GB/s of the GEMV launches against the measured HBM peak
  cpu_baseline  the reconstruct-then-matmul CPU path (numpy port of the
            reference's dequantize_layer, torch CPU matmul) on a bounded sample

Further objects on the same line (skipped with --no-extras / --no-decode /
--no-e8): `realistic_grouping` (the four stream-ordered launches per decoder
layer a model can issue), `chained_layer` (the same as one chained launch),
`batch4`, `batch16`, `e8_layer_set`, `gemm` (prefill shapes of the baseline's
fourth configuration against the tensor peak), `decode` (whole-model tokens/s
through the decode engine for both codebooks).

With --gpus N > 1 (torchrun) the linears are sharded tensor-parallel
(q/k/v/gate/up by output rows, o/down by input columns followed by an
all-reduce: the library's one-shot push kernel over peer memory, or NCCL with
--nccl) and the whole-model bytes are divided by the slowest rank's time.
Before anything is timed, `tp_check` compares the sharded, all-reduced outputs
with the unsharded layer; `decode.tp_step_check` does the same for one token of
the tensor-parallel engine, and `decode.llama2_70b_e8` decodes the baseline's
fifth configuration (batches 1, 8 and 64).  A failed check ends the run with
exit code 3 and an error line instead of a result.

`--impl reference` times the CPU path alone, on rank 0.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "dequant_gemv_hbm_gbps"
UNIT = "GB/s"
KIND, RADIUS = "e8_d4", 1.75
N_LAYERS = 32


def algorithmic_bytes(out_f: int, in_f: int, n_masked: int, batch: int, bias: bool = False) -> int:
    """Bytes one GEMV call must move: Q, critical blocks, g, h, x, y (+bias)."""
    M = out_f // 8
    return (2 * M * in_f + 16 * n_masked + 2 * out_f + 2 * in_f
            + 2 * batch * in_f + 2 * batch * out_f + (2 * out_f if bias else 0))


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1])); mx.append(float(r[2]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


# --------------------------------------------------------------------------- CPU path

def host_threads() -> int:
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def cpu_reference_path(batch: int, reps: int, threads: int | None = None):
    """Reference's CPU path on one decoder layer's seven linears: reconstruct once
    (numpy port of dequantize_layer), then steady-state fp32 matmul on the host cores."""
    import numpy as np
    import torch
    import oracle
    from eptq_b200.synthetic import LLAMA2_7B_LINEARS, make_activations, make_layer

    if threads:
        torch.set_num_threads(threads)
    table = oracle.d4_table(RADIUS)
    weights, xs, total_bytes = [], [], 0
    t0 = time.perf_counter()
    for i, (name, (out_f, in_f)) in enumerate(LLAMA2_7B_LINEARS.items()):
        qd = make_layer(out_f, in_f, seed=1000 + i)
        arr = oracle.LayerArrays(Q=qd.Q.numpy(), g=qd.g.numpy(), h=qd.h.numpy(), O=qd.O.numpy())
        weights.append(torch.from_numpy(oracle.dequantize_layer(arr, table)).float())
        xs.append(make_activations(batch, in_f, seed=i).float())
        total_bytes += algorithmic_bytes(out_f, in_f, qd.O.shape[0], batch)
    reconstruct_s = time.perf_counter() - t0
    times = []
    for r in range(reps + 2):
        t = time.perf_counter()
        for W, x in zip(weights, xs):
            _ = x @ W.T
        times.append(time.perf_counter() - t)
    med = statistics.median(times[2:])
    return {"value": total_bytes / med / 1e9, "unit": UNIT, "cores": torch.get_num_threads(),
            "host_cpus": os.cpu_count(), "kind": "port",
            "sample": f"1 of {N_LAYERS} decoder layers (7 linears, batch {batch}), median of {reps} fp32 matmul passes; "
                      f"one-time reconstruct {reconstruct_s:.2f} s excluded",
            "ms_per_layer_set": med * 1e3, "reconstruct_s": reconstruct_s}


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    t0 = time.perf_counter()
    reps = max(min(args.steps, 30), 3)
    # torch.distributed.run exports OMP_NUM_THREADS=1: take the cores this process may run on instead
    res = cpu_reference_path(args.batch, reps, threads=host_threads())
    line = {
        "impl": "reference", "metric": METRIC, "value": res["value"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": res["ms_per_layer_set"] * N_LAYERS,
        "higher_is_better": True, "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": "llama2-7b decode layer set, E8-D4 r=1.75, 0.2% critical blocks",
                   "batch": args.batch, "layers": N_LAYERS, "cpu_sample_layers": 1},
        "cpu_baseline": {k: res[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": res["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "wall_s": time.perf_counter() - t0,
    }
    print(json.dumps(line))


# --------------------------------------------------------------------------- GPU path

def run_gpu_arm(args):
    import torch
    import torch.distributed as dist

    from eptq_b200 import _lib
    from eptq_b200.build import build_library
    from eptq_b200.kernels.linear import EPTQLinear, forward_group
    from eptq_b200.parallel import shard_layer, ROW_PARALLEL
    from eptq_b200.quantizers import E8D4Quantizer
    from eptq_b200.synthetic import LLAMA2_7B_LINEARS, make_layer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
        os.environ["NCCL_DEBUG"] = "WARN"          # keep NCCL's version banner off stdout: one JSON line only
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    if rank == 0:
        build_library()
    if world > 1:
        dist.barrier()
    lib = _lib.load()
    B = args.batch
    n_layers = args.layers
    # Row-parallel partial outputs: this library's one-shot push all-reduce over peer memory, or NCCL.
    comm = None
    comm_note = None
    if world > 1 and not args.nccl:
        from eptq_b200.comm import PushAllReduce
        try:
            comm = PushAllReduce(dist.group.WORLD, B * 8192, dev)
        except RuntimeError as exc:              # raised on every rank alike: fall back to NCCL together
            comm, comm_note = None, str(exc)

    def all_reduce(y):
        if comm is not None and y.numel() <= comm.n_max:
            comm.all_reduce_(y)
        else:
            dist.all_reduce(y)

    if args.codebook == "e8":                       # not the headline: lets the E8 kernel be the profiled workload
        from eptq_b200.quantizers import E8LatticeQuantizer
        qz0 = E8LatticeQuantizer(radius=1.6)
        qz0.remove_last()
        table, kind = qz0.points.to(dev), "e8_lattice"
    else:
        table, kind = E8D4Quantizer(radius=RADIUS).codes.to(dev), KIND
    layers, total_bytes = [], 0
    for li in range(n_layers):
        for i, (name, (out_f, in_f)) in enumerate(LLAMA2_7B_LINEARS.items()):
            qd = make_layer(out_f, in_f, seed=li * 16 + i, device=str(dev))
            total_bytes += algorithmic_bytes(out_f, in_f, qd.O.shape[0], B)
            if world > 1:
                qd = shard_layer(qd, name, rank, world)
            lin = EPTQLinear.from_quantized_data(qd, table, kind)
            lin.tp_row_parallel = world > 1 and name.split(".")[-1] in ROW_PARALLEL
            layers.append((name, lin))
    torch.cuda.synchronize()

    # Device-resident arm: C-ABI calls captured once, replayed per step.  The seven linears of a
    # decoder layer have fixed, independent inputs here, so each decoder layer is one group launch
    # (--group 7); --group 1 issues one launch per linear.
    group = max(1, min(args.group, 32))
    xs = {n: torch.randn(B, n, device=dev).half() for n in {l.in_features for _, l in layers}}
    ys = [torch.empty(B, l.out_features, device=dev, dtype=torch.float16) for _, l in layers]
    descs = [l.descriptor() for _, l in layers]

    def make_calls(gsize):
        calls, need = [], 0
        for i in range(0, len(layers), gsize):
            n = min(gsize, len(layers) - i)
            arr = (_lib.EptqLayer * n)(*descs[i:i + n])
            xp = (C.c_void_p * n)(*[xs[l.in_features].data_ptr() for _, l in layers[i:i + n]])
            yp = (C.c_void_p * n)(*[y.data_ptr() for y in ys[i:i + n]])
            reduce_ys = [ys[i + k] for k in range(n) if layers[i + k][1].tp_row_parallel]
            grouped = lib.eptq_group_workspace_bytes(arr, n, B) > 0 and (gsize > 1)
            need = max(need, lib.eptq_group_workspace_bytes(arr, n, B),
                       *[lib.eptq_workspace_bytes(l.Q.shape[0], l.Q.shape[1], B) for _, l in layers[i:i + n]])
            calls.append((arr, n, xp, yp, reduce_ys, grouped, i))
        return calls, need

    if world > 1:
        dist.barrier()                       # ranks finish building at different times: line them up before the
        torch.cuda.synchronize()             # first reduction, whose device-side wait is bounded
    calls, ws_bytes = make_calls(group)
    calls1, ws_bytes1 = make_calls(1)
    ws = torch.zeros(max(ws_bytes, ws_bytes1), dtype=torch.uint8, device=dev)

    def step_abi(call_list=None):
        stream = torch.cuda.current_stream().cuda_stream
        for arr, n, xp, yp, reduce_ys, grouped, i0 in (calls if call_list is None else call_list):
            if grouped:
                st = lib.eptq_linear_forward_group(arr, n, xp, yp, B, ws.data_ptr(), ws.numel(), stream)
                if st != 0:
                    raise RuntimeError(lib.eptq_strerror(st).decode())
            else:
                for k in range(n):
                    l = layers[i0 + k][1]
                    st = lib.eptq_linear_forward(C.byref(descs[i0 + k]), xs[l.in_features].data_ptr(),
                                                 ys[i0 + k].data_ptr(), B, ws.data_ptr(), ws.numel(), stream)
                    if st != 0:
                        raise RuntimeError(lib.eptq_strerror(st).decode())
            for y in reduce_ys:
                all_reduce(y)

    # Tensor-parallel check before anything is timed: the all-reduced output of the sharded row-parallel layers
    # of decoder layer 0 against the unsharded layer, and the push all-reduce against NCCL on a seeded vector.
    tp_check = None
    if world > 1:
        errs = []
        for i, (name, (out_f, in_f)) in enumerate(LLAMA2_7B_LINEARS.items()):
            if name.split(".")[-1] not in ROW_PARALLEL:
                continue
            full = EPTQLinear.from_quantized_data(make_layer(out_f, in_f, seed=i, device=str(dev)), table, kind)
            xf = torch.randn(1, in_f, device=dev, generator=torch.Generator(device=dev).manual_seed(77)).half()
            want = full(xf).float()
            shard = layers[i][1]
            cols = in_f // world
            part = shard(xf[:, rank * cols:(rank + 1) * cols].contiguous())
            all_reduce(part)
            errs.append(float((part.float() - want).abs().max() / want.abs().max()))
            del full
        v = torch.randn(8192, device=dev, generator=torch.Generator(device=dev).manual_seed(100 + rank)).half()
        ref = v.clone()
        dist.all_reduce(ref)
        got = v.clone()
        all_reduce(got)
        ar_err = float((got.float() - ref.float()).abs().max() / ref.float().abs().max())
        t = torch.tensor([max(errs), ar_err], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        tp_check = {"row_parallel_max_rel": float(t[0]), "allreduce_max_rel": float(t[1]),
                    "ok": bool(float(t[0]) <= 2e-3 and float(t[1]) <= 2e-3)}
        if not tp_check["ok"]:
            if rank == 0:
                print(json.dumps({"metric": METRIC, "error": "tensor-parallel check failed", "tp_check": tp_check}))
            sys.stdout.flush()
            os._exit(3)

    side = torch.cuda.Stream(device=dev)
    with torch.cuda.stream(side):
        step_abi()
        torch.cuda.synchronize()
        before = _lib.launch_count()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            step_abi()
        launches_per_step = _lib.launch_count() - before
    torch.cuda.synchronize()

    def timed(run, steps, warmup):
        for _ in range(warmup):
            run()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(local) as cs:
            e0.record()
            for _ in range(steps):
                run()
            e1.record()
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
                torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, cs.summary()

    ms_dev, clocks = timed(graph.replay, args.steps, args.warmup)
    ms_chain = None
    if group > 1:
        with torch.cuda.stream(side):
            step_abi(calls1)
            torch.cuda.synchronize()
            graph1 = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph1, stream=side):
                step_abi(calls1)
        torch.cuda.synchronize()
        ms_chain, _ = timed(graph1.replay, args.steps, args.warmup)
    if clocks["samples"] < 5:
        # The timed region is shorter than the sampling period: keep the same load running for about
        # 1.5 s.  The replay count is derived from the rank-agreed step time, so that every rank
        # issues the same number of collectives.
        extra = max(20, min(20000, int(1500.0 / max(ms_dev / args.steps, 1e-3))))
        with ClockSampler(local) as cs:
            for i in range(extra):
                graph.replay()
                if i % 50 == 49:
                    torch.cuda.synchronize()
            torch.cuda.synchronize()
        clocks = cs.summary()
        clocks["note"] = f"sampled while replaying the timed step {extra} more times right after the timed region"
    if world > 1:
        dist.barrier()

    # End-to-end arm: public module API, activations start and results end in pinned host memory.
    x_host = {n: torch.randn(B, n).half().pin_memory() for n in xs}
    y_host = torch.empty(B, layers[-1][1].out_features, dtype=torch.float16).pin_memory()
    x_dev = {n: torch.empty_like(v, device=dev) for n, v in x_host.items()}

    def step_module():
        for n in x_dev:
            x_dev[n].copy_(x_host[n], non_blocking=True)
        y = None
        for i in range(0, len(layers), group):
            chunk = [l for _, l in layers[i:i + group]]
            if group > 1 and B <= 16:                     # above 16 rows the linears are GEMMs, one call per layer
                outs = forward_group(chunk, [x_dev[l.in_features] for l in chunk])
            else:
                outs = [l(x_dev[l.in_features]) for l in chunk]
            for l, o in zip(chunk, outs):
                if l.tp_row_parallel:
                    all_reduce(o)
            y = outs[-1]
        y_host.copy_(y, non_blocking=True)

    with torch.cuda.stream(side):
        step_module()
        torch.cuda.synchronize()
        graph2 = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph2, stream=side):
            step_module()
    torch.cuda.synchronize()

    def e2e_step():
        graph2.replay()
        torch.cuda.current_stream().synchronize()     # the host reads the result of every step

    ms_e2e, _ = timed(e2e_step, args.steps, args.warmup)
    h2d = sum(v.numel() * 2 for v in x_host.values())
    d2h = y_host.numel() * 2

    # ---- extra figures on the same weights (one GPU): what a decoder layer can really issue, larger batches
    peak_hbm = measured_peaks()[0]
    realistic, chained_stats, batch_stats = None, None, {}
    if world == 1 and group == 7 and args.codebook == "e8d4" and not args.no_extras:
        names = [n.split(".")[-1] for n, _ in layers[:7]]
        idx = {n: k for k, n in enumerate(names)}
        H, FF = layers[idx["q_proj"]][1].in_features, layers[idx["gate_proj"]][1].out_features
        att = torch.randn(1, H, device=dev).half() * 0.1
        xres = torch.randn(1, H, device=dev).half()
        gbuf = torch.empty(1, FF, device=dev, dtype=torch.float16)
        ubuf = torch.empty_like(gbuf)
        qkv_out = [torch.empty(1, H, device=dev, dtype=torch.float16) for _ in range(3)]

        def ptrs(ts):
            return (C.c_void_p * len(ts))(*[t.data_ptr() for t in ts])

        # (1) the dependent chain of a decoder layer as four group launches: {q,k,v} -> {o} -> {gate,up} -> {down}
        sets = []
        for li in range(n_layers):
            d = descs[li * 7:(li + 1) * 7]
            for members, xin, outs in ((("q_proj", "k_proj", "v_proj"), [xres] * 3, qkv_out),
                                       (("o_proj",), [att], [qkv_out[0]]),
                                       (("gate_proj", "up_proj"), [xres] * 2, [gbuf, ubuf]),
                                       (("down_proj",), [gbuf], [qkv_out[1]])):
                arr = (_lib.EptqLayer * len(members))(*[d[idx[m]] for m in members])
                sets.append((arr, len(members), ptrs(xin), ptrs(outs)))

        def step_realistic():
            stream = torch.cuda.current_stream().cuda_stream
            for arr, n, xp, yp in sets:
                st = lib.eptq_linear_forward_group(arr, n, xp, yp, 1, ws.data_ptr(), ws.numel(), stream)
                if st != 0:
                    raise RuntimeError(lib.eptq_strerror(st).decode())

        def graphed(fn):
            with torch.cuda.stream(side):
                fn()
                torch.cuda.synchronize()
                g_ = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g_, stream=side):
                    fn()
            torch.cuda.synchronize()
            return g_
        g_real = graphed(step_realistic)
        ms_real, _ = timed(g_real.replay, args.steps, args.warmup)
        v = total_bytes / (ms_real / args.steps * 1e-3) / 1e9
        realistic = {"value": v, "unit": UNIT, "ms_per_step": ms_real / args.steps, "frac_of_hbm_peak": v / peak_hbm,
                     "launches_per_step": len(sets),
                     "note": "per decoder layer four stream-ordered group launches {q,k,v} -> {o} -> {gate,up} -> {down}: "
                             "the grouping a model can issue"}
        del g_real

        # (2) the same work as ONE chained launch per decoder layer: o -> gate/up -> down -> q/k/v, with the
        # fused input ops the decode engine uses (residual add, RMSNorm factor, silu*up)
        def fus(x_op=_lib.X_PLAIN, y_op=_lib.Y_STORE, residual=None, x_aux=None):
            f = _lib.EptqFusion()
            f.x_op, f.y_op, f.norm_eps = x_op, y_op, 1e-5
            f.residual = None if residual is None else residual.data_ptr()
            f.x_aux = None if x_aux is None else x_aux.data_ptr()
            return f
        order = ("o_proj", "gate_proj", "up_proj", "down_proj", "q_proj", "k_proj", "v_proj")
        phases = (C.c_int * 7)(0, 1, 1, 2, 3, 3, 3)
        fz = (_lib.EptqFusion * 7)(fus(), fus(_lib.X_RMSNORM), fus(_lib.X_RMSNORM), fus(_lib.X_SILU_MUL, x_aux=ubuf),
                                   fus(_lib.X_RMSNORM), fus(_lib.X_RMSNORM), fus(_lib.X_RMSNORM))
        y_o = torch.empty(1, H, device=dev, dtype=torch.float16)
        y_d = torch.empty(1, H, device=dev, dtype=torch.float16)
        cxs, cys = ptrs([att, y_o, y_o, gbuf, y_d, y_d, y_d]), ptrs([y_o, gbuf, ubuf, y_d] + qkv_out)
        chains = [(_lib.EptqLayer * 7)(*[descs[li * 7 + idx[m]] for m in order]) for li in range(n_layers)]

        def step_chain():
            stream = torch.cuda.current_stream().cuda_stream
            for arr in chains:
                st = lib.eptq_linear_forward_chain(arr, 7, fz, phases, cxs, cys, 1, ws.data_ptr(), ws.numel(), stream)
                if st != 0:
                    raise RuntimeError(lib.eptq_strerror(st).decode())
        try:
            g_chain = graphed(step_chain)
            ms_c, _ = timed(g_chain.replay, args.steps, args.warmup)
            v = total_bytes / (ms_c / args.steps * 1e-3) / 1e9
            chained_stats = {"value": v, "unit": UNIT, "ms_per_step": ms_c / args.steps, "frac_of_hbm_peak": v / peak_hbm,
                             "launches_per_step": len(chains),
                             "note": "one cooperative launch per decoder layer, four dependent phases "
                                     "o -> gate/up -> down(silu*up) -> q/k/v"}
            del g_chain
        except RuntimeError as exc:
            chained_stats = {"unavailable": str(exc)}

        # (3) batches 4 and 16 of the baseline's second configuration, grouped as the headline
        for Bx in (4, 16):
            xb = {n: torch.randn(Bx, n, device=dev).half() for n in xs}
            yb = [torch.empty(Bx, l.out_features, device=dev, dtype=torch.float16) for _, l in layers[:7]]
            bcalls, need = [], 0
            for i in range(0, len(layers), 7):
                arr = (_lib.EptqLayer * 7)(*descs[i:i + 7])
                need = max(need, lib.eptq_group_workspace_bytes(arr, 7, Bx))
                bcalls.append((arr, ptrs([xb[l.in_features] for _, l in layers[i:i + 7]]), ptrs(yb)))
            wsb = ws if need <= ws.numel() else torch.zeros(need, dtype=torch.uint8, device=dev)

            def step_b():
                stream = torch.cuda.current_stream().cuda_stream
                for arr, xp, yp in bcalls:
                    st = lib.eptq_linear_forward_group(arr, 7, xp, yp, Bx, wsb.data_ptr(), wsb.numel(), stream)
                    if st != 0:
                        raise RuntimeError(lib.eptq_strerror(st).decode())
            g_b = graphed(step_b)
            ms_b, _ = timed(g_b.replay, max(3, args.steps // 4), 3)
            per = ms_b / max(3, args.steps // 4)
            bytes_b = total_bytes + sum(2 * (Bx - 1) * (l.in_features + l.out_features) for _, l in layers)
            batch_stats[f"batch{Bx}"] = {"value": bytes_b / (per * 1e-3) / 1e9, "unit": UNIT, "ms_per_step": per,
                                         "frac_of_hbm_peak": bytes_b / (per * 1e-3) / 1e9 / peak_hbm,
                                         "step_time_vs_batch1": per / (ms_dev / args.steps)}
            del g_b, bcalls

    # ---- prefill GEMM, baseline's fourth configuration: Llama-3-8B shapes, group scales qb=128, 2048 tokens
    gemm_stats = None
    if world == 1 and not args.no_extras and args.codebook == "e8d4":
        from eptq_b200.synthetic import LLAMA3_8B_LINEARS
        pk = ROOT / "MEASURED_PEAKS.json"
        tensor_peak = json.loads(pk.read_text())["bf16_tflops"] if pk.exists() else 1590.0
        T = 2048
        gemm_stats = {"tokens": T, "peak_tflops": tensor_peak, "peak_kind": "measured bf16 burst" if pk.exists() else "fallback",
                      "shapes": {}}
        seen, tot_flops, tot_ms = set(), 0.0, 0.0
        for name, (o, i) in LLAMA3_8B_LINEARS.items():
            if (o, i) in seen:
                continue
            seen.add((o, i))
            lin = EPTQLinear.from_quantized_data(make_layer(o, i, seed=42, device=str(dev), qb_size=128), table, KIND)
            xg = torch.randn(T, i, device=dev).half()
            for _ in range(3):
                lin(xg)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(5):
                lin(xg)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / 5
            fl = 2.0 * T * o * i
            count = sum(1 for v in LLAMA3_8B_LINEARS.values() if v == (o, i))
            tot_flops += fl * count
            tot_ms += ms * count
            gemm_stats["shapes"][f"{o}x{i}"] = {"ms": ms, "tflops": fl / ms / 1e9, "frac_of_peak": fl / ms / 1e9 / tensor_peak}
            del lin, xg
        gemm_stats["layer_tflops"] = tot_flops / tot_ms / 1e9
        gemm_stats["layer_frac_of_peak"] = tot_flops / tot_ms / 1e9 / tensor_peak
        torch.cuda.empty_cache()

    # The same layer set with the E8 codebook (radius 1.6) through the same grouped launch: the codebook of the
    # baseline's first, third and fifth configurations.  Reported as an extra figure.
    e8_stats = None
    if not args.no_e8 and world == 1 and group > 1 and args.codebook == "e8d4":
        from eptq_b200.quantizers import E8LatticeQuantizer
        qz = E8LatticeQuantizer(radius=1.6)
        qz.remove_last()
        e8_table = qz.points.to(dev)
        e8_layers = []
        for li in range(n_layers):
            for i, (name, (out_f, in_f)) in enumerate(LLAMA2_7B_LINEARS.items()):
                qd = make_layer(out_f, in_f, seed=9000 + li * 16 + i, device=str(dev))
                e8_layers.append(EPTQLinear.from_quantized_data(qd, e8_table, "e8_lattice"))
        e8_descs = [l.descriptor() for l in e8_layers]
        e8_calls = []
        for i in range(0, len(e8_layers), group):
            n = min(group, len(e8_layers) - i)
            arr = (_lib.EptqLayer * n)(*e8_descs[i:i + n])
            xp = (C.c_void_p * n)(*[xs[l.in_features].data_ptr() for l in e8_layers[i:i + n]])
            yp = (C.c_void_p * n)(*[y.data_ptr() for y in ys[i:i + n]])
            e8_calls.append((arr, n, xp, yp))

        def step_e8():
            stream = torch.cuda.current_stream().cuda_stream
            for arr, n, xp, yp in e8_calls:
                st = lib.eptq_linear_forward_group(arr, n, xp, yp, B, ws.data_ptr(), ws.numel(), stream)
                if st != 0:
                    raise RuntimeError(lib.eptq_strerror(st).decode())
        with torch.cuda.stream(side):
            step_e8()
            torch.cuda.synchronize()
            graph_e8 = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph_e8, stream=side):
                step_e8()
        torch.cuda.synchronize()
        ms_e8, _ = timed(graph_e8.replay, args.steps, args.warmup)
        e8_stats = {"value": total_bytes / (ms_e8 / args.steps * 1e-3) / 1e9, "unit": UNIT,
                    "ms_per_step": ms_e8 / args.steps,
                    "frac_of_hbm_peak": total_bytes / (ms_e8 / args.steps * 1e-3) / 1e9 / measured_peaks()[0],
                    "note": "same layer shapes and launch grouping, E8 codebook r=1.6 (packed table: 219 KB in shared "
                            "memory, 14.6 % of uniform indices read through L2)"}
        del graph_e8, e8_calls, e8_descs, e8_layers
        torch.cuda.empty_cache()

    # Whole-model decode (the baseline's third configuration): random-init Llama-2-7B architecture,
    # 512-token prompt, 128 greedy tokens at batch 1, the step captured in one CUDA graph; tensor-
    # parallel over all ranks.  Reported beside the GEMV figure, not instead of it.
    decode_stats = {}
    if not args.no_decode:
        from eptq_b200.engine import ARCHITECTURES, synthetic_llama_engine
        from eptq_b200.quantizers import E8LatticeQuantizer
        del graph2, graph
        hidden, inter, n_dec, heads, kv, vocab = ARCHITECTURES["llama2-7b"]
        ids = torch.randint(0, vocab, (1, 512), generator=torch.Generator().manual_seed(0)).to(dev)
        for qname in ("e8_d4", "e8_lattice"):
            if qname == "e8_d4":
                tab = E8D4Quantizer(radius=RADIUS).codes.to(dev)
            else:
                qz = E8LatticeQuantizer(radius=1.6)
                qz.remove_last()
                tab = qz.points.to(dev)
            eng = synthetic_llama_engine(hidden, inter, n_dec, heads, kv, vocab, qname, tab, max_len=512 + 128,
                                         batch=1, device=str(dev), tp_rank=rank, tp_size=world,
                                         tp_group=dist.group.WORLD if world > 1 else None, comm=comm)
            eng.decode(ids, 8)
            _, st = eng.decode(ids, 128)
            if world > 1:
                t = torch.tensor([st["decode_s"]], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                st["decode_s"] = float(t.item())
                st["tokens_per_s"] = 127 / st["decode_s"]
                st["ms_per_token"] = 1e3 * st["decode_s"] / 127
            decode_stats[qname] = {"tokens_per_s": st["tokens_per_s"], "ms_per_token": st["ms_per_token"],
                                   "prefill_s": st["prefill_s"]}
            del eng
            torch.cuda.empty_cache()
        decode_stats["config"] = ("llama2-7b architecture, random init, 32 layers, 512-token prompt + 128 greedy "
                                  f"tokens, batch 1, tp{world}, one CUDA graph per token")
        if world > 1 and not args.no_extras:
            # The baseline's fifth configuration: Llama-2-70B architecture, E8 codebook, tensor-parallel over all
            # ranks, batch 1, 1024-token prompt; all 80 decoder layers, 32 new tokens to keep the run short.
            try:
                h70, i70, n70, heads70, kv70, v70 = ARCHITECTURES["llama2-70b"]
                qz = E8LatticeQuantizer(radius=1.6)
                qz.remove_last()
                eng = synthetic_llama_engine(h70, i70, n70, heads70, kv70, v70, "e8_lattice", qz.points.to(dev),
                                             max_len=1024 + 32, batch=1, device=str(dev), tp_rank=rank, tp_size=world,
                                             tp_group=dist.group.WORLD, comm=comm)
                ids70 = torch.randint(0, v70, (1, 1024), generator=torch.Generator().manual_seed(1)).to(dev)
                eng.decode(ids70, 4)
                _, st = eng.decode(ids70, 32)
                t = torch.tensor([st["decode_s"]], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                decode_stats["llama2_70b_e8"] = {"tokens_per_s": 31 / float(t.item()), "ms_per_token": 1e3 * float(t.item()) / 31,
                                                 "prefill_s": st["prefill_s"],
                                                 "config": f"llama2-70b architecture, random init, 80 layers, E8 r=1.6, 1024-token "
                                                           f"prompt + 32 greedy tokens, batch 1, tp{world}"}
                # the same weights at batch 8 (GEMV passes of two rows; reductions of 8 x 8192 values go through NCCL)
                from eptq_b200.engine import LlamaDecodeEngine
                layers70 = eng.layers
                head70 = (eng.embed, eng.final_norm, eng.lm_head, eng.inv_freq, eng.eps, eng.head_dim, eng.n_heads, eng.n_kv_heads)
                eng8 = LlamaDecodeEngine(layers70, *head70, 1024 + 32, batch=8, tp_group=dist.group.WORLD, comm=comm)
                del eng
                ids8 = torch.randint(0, v70, (8, 1024), generator=torch.Generator().manual_seed(2)).to(dev)
                eng8.decode(ids8, 4)
                _, st8 = eng8.decode(ids8, 16)
                t = torch.tensor([st8["decode_s"]], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                decode_stats["llama2_70b_e8"]["batch8"] = {"tokens_per_s": 15 * 8 / float(t.item()),
                                                           "ms_per_step": 1e3 * float(t.item()) / 15}
                del eng8
                torch.cuda.empty_cache()
                # and at batch 64 (the linears take the tensor-core GEMM path), 8 steps
                eng64 = LlamaDecodeEngine(layers70, *head70, 1024 + 16, batch=64, tp_group=dist.group.WORLD, comm=comm)
                ids64 = torch.randint(0, v70, (64, 1024), generator=torch.Generator().manual_seed(3)).to(dev)
                eng64.decode(ids64, 3)
                _, st64 = eng64.decode(ids64, 9)
                t = torch.tensor([st64["decode_s"]], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                decode_stats["llama2_70b_e8"]["batch64"] = {"tokens_per_s": 8 * 64 / float(t.item()),
                                                            "ms_per_step": 1e3 * float(t.item()) / 8}
                del eng64, layers70, head70
            except Exception as exc:                         # noqa: BLE001 -- never lose the bench line over an extra
                decode_stats["llama2_70b_e8"] = {"unavailable": f"{type(exc).__name__}: {exc}"[:200]}
            torch.cuda.empty_cache()
        if world > 1:
            # The tensor-parallel token step (sharded GEMV launches, chained MLP, push all-reduce) against the same
            # model unsharded on this GPU: logits of one decoded token after a 32-token prompt, 2 decoder layers.
            tab = E8D4Quantizer(radius=RADIUS).codes.to(dev)
            kw = dict(max_len=64, batch=1, device=str(dev))
            tp_eng = synthetic_llama_engine(hidden, inter, 2, heads, kv, vocab, "e8_d4", tab, tp_rank=rank, tp_size=world,
                                            tp_group=dist.group.WORLD, comm=comm, **kw)
            one = synthetic_llama_engine(hidden, inter, 2, heads, kv, vocab, "e8_d4", tab, **kw)
            short = ids[:, :32]
            with torch.no_grad():
                tok_tp, tok_one = tp_eng.prefill(short), one.prefill(short)
                pos = torch.tensor([32], device=dev)
                a = tp_eng.forward(tok_one[:, None], pos).float()
                b = one.forward(tok_one[:, None], pos).float()
            t = torch.tensor([float((a - b).abs().max() / b.abs().max())], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            decode_stats["tp_step_check"] = {"logits_max_rel": float(t[0]), "ok": bool(float(t[0]) <= 2e-2)}
            del tp_eng, one
            torch.cuda.empty_cache()
            if not decode_stats["tp_step_check"]["ok"]:
                if rank == 0:
                    print(json.dumps({"metric": METRIC, "error": "tensor-parallel decode step check failed",
                                      "tp_step_check": decode_stats["tp_step_check"]}))
                sys.stdout.flush()
                os._exit(3)

    if comm is not None:
        comm.check()                                   # a device-side wait that ran out would show here
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
    if rank != 0:
        # CUDA graphs that captured NCCL kernels are still alive; tearing the communicator down under
        # them can block, so worker ranks leave without the teardown.
        sys.stdout.flush()
        os._exit(0)

    step_ms = ms_dev / args.steps
    value = total_bytes / (step_ms * 1e-3) / 1e9
    e2e_value = total_bytes / (ms_e2e / args.steps * 1e-3) / 1e9
    peak, peak_kind = measured_peaks()
    n_calls = max(1, int(launches_per_step))
    per_launch_bytes = total_bytes / world / n_calls
    per_launch_us = step_ms * 1e3 / n_calls
    achieved = per_launch_bytes / (per_launch_us * 1e-6) / 1e9
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": step_ms, "higher_is_better": True, "scaling": "strong" if world > 1 else "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": "llama2-7b decode layer set, " + ("E8-D4 r=1.75" if args.codebook == "e8d4" else "E8 r=1.6")
                               + ", 0.2% critical blocks",
                   "batch": B, "layers": n_layers, "linears_per_step": len(layers),
                   "l2_policy": "inputs larger than L2 (1.66 GB of indices per step)" if n_layers >= 8 else "reduced layer count: may be L2-resident",
                   "launch_granularity": f"{group} independent linears per launch" if group > 1 else "one launch per linear",
                   "parallelism": f"tp{world}" if world > 1 else "single",
                   "all_reduce": "none" if world == 1 else ("nccl" if comm is None else "one-shot push kernel over peer memory"),
                   "all_reduce_note": comm_note},
        "decode_tokens_per_s_linears_only": 1e3 / step_ms * B,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": (52291840 if (group == 7 and B == 1 and world == 1 and args.codebook == "e8d4") else None),
                     "traffic_source": "dram read+write of one 7-linear launch of gemv_stream_kernel, ncu capture summarised in profiles/gemv_stream_kernel_llama7b_layer_set.md",
                     "peak_kind": f"{peak_kind} copy bandwidth",
                     "per_launch_bytes": per_launch_bytes, "per_launch_us": per_launch_us},
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": ms_e2e / args.steps},
        "gpu_launches": int(launches_per_step * args.steps),
        "one_launch_per_linear": None if ms_chain is None else {
            "value": total_bytes / (ms_chain / args.steps * 1e-3) / 1e9, "unit": UNIT,
            "ms_per_step": ms_chain / args.steps,
            "note": "the same pass through eptq_linear_forward, one launch per linear, each ordered after the previous"},
        "clocks": clocks,
        "decode": decode_stats or None,
        "e8_layer_set": e8_stats,
        "realistic_grouping": realistic,
        "chained_layer": chained_stats,
        "batch4": batch_stats.get("batch4"),
        "batch16": batch_stats.get("batch16"),
        "gemm": gemm_stats,
        "tp_check": tp_check,
    }
    if not args.no_cpu_baseline and world == 1:
        res = cpu_reference_path(B, 10, threads=host_threads())
        line["cpu_baseline"] = {k: res[k] for k in ("value", "unit", "cores", "kind", "sample")}
    print(json.dumps(line))
    if world > 1:
        sys.stdout.flush()
        os._exit(0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--layers", type=int, default=N_LAYERS)
    ap.add_argument("--group", type=int, default=7,
                    help="independent linears per launch (7 = one decoder layer's linears, 1 = one launch each)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-decode", action="store_true", help="skip the whole-model decode tokens/s arm")
    ap.add_argument("--no-e8", action="store_true", help="skip the E8-codebook layer-set figure")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the realistic-grouping, chained-layer, batch 4/16 and prefill-GEMM figures")
    ap.add_argument("--nccl", action="store_true", help="tensor-parallel runs: NCCL all-reduce instead of the push kernel")
    ap.add_argument("--codebook", default="e8d4", choices=["e8d4", "e8"],
                    help="codebook of the timed layer set (the headline is e8d4)")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
