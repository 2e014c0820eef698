#!/usr/bin/env python
"""Benchmark of the quantized-linear hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--m M]

Workload (the configuration the headline metric is quoted on): the four
Llama-3-8B projection shapes in Q4_K -- 4096->6144 (QKV), 4096->4096 (O), 4096->28672 (gate|up),
14336->4096 (down) -- at decode batch M (default 1), for 32 layers with distinct weights.  One step
is one pass over all 128 linears (3.93 GB of packed weights, far larger than the 126 MB L2, so every
step streams from HBM).  Weights are N(0, 0.02) quantized with the package encoder, activations
N(0, 1) bf16, all seeded and synthetic.

Metric: Q4_K dequant-GEMV GB/s = algorithmic bytes (packed weights + x + y) / time.
N > 1 (torchrun, one rank per GPU): each linear is tensor-parallel -- QKV and gate|up split by
output rows, O and down by input columns followed by an NCCL all-reduce -- total work fixed
("strong" scaling).

`--impl reference` times the reference's CPU implementation of the same operator on the host cores:
ATen linear on dequantized bf16 weights (what Linear.forward, linear.nim:45-57, calls), on a bounded
sample of the workload (one layer per step).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SHAPES = [("qkv", 4096, 6144), ("o", 4096, 4096), ("gate_up", 4096, 28672), ("down", 14336, 4096)]
N_LAYERS = 32
Q4K_BYTES_PER_256 = 144


def algorithmic_bytes(m: int, k: int, n: int, x_bytes: int = 2, y_bytes: int = 2) -> int:
    return n * (k // 256) * Q4K_BYTES_PER_256 + m * k * x_bytes + m * n * y_bytes


class ClockSampler:
    """Polls NVML for SM clock and throttle reasons while the timed region runs (read-only)."""

    REASONS = {
        0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
        0x80: "hw_power_brake_slowdown",
    }

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._nv = None

    def _run(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
                mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._h))
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.005)

    def start(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()
        med = int(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def visible_physical_index(local_index: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_index])
        except (ValueError, IndexError):
            pass
    return local_index


# --------------------------------------------------------------------------------------------------
# reference arm / CPU baseline: ATen linear on the host cores (and the packed-bytes CPU port)
# --------------------------------------------------------------------------------------------------
def cpu_layer_sample(m: int, seed: int = 2000):
    """One layer's four linears: dequantized bf16 weights (reference path) and packed blocks (port)."""
    import oracle  # CPU checker; used here only to decode blocks for the CPU baseline

    from tattletale_b200 import quantize as Q

    layers = []
    for idx, (_, k, n) in enumerate(SHAPES):
        g = torch.Generator().manual_seed(seed + idx)
        w = torch.randn(n, k, generator=g) * 0.02
        blocks = Q.quantize(Q.FMT_Q4_K, w).numpy()
        w_deq = torch.from_numpy(oracle.dequantize(oracle.Q4_K, blocks)).to(torch.bfloat16)
        x = torch.randn(m, k, generator=g).to(torch.bfloat16)
        layers.append((k, n, blocks, w_deq, x))
    return layers


def time_cpu_reference(m: int, steps: int, warmup: int, budget_s: float = 25.0):
    """Returns (GB/s of the metric, ms per step, cores, port GB/s) for one-layer steps on the host."""
    import oracle

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    layers = cpu_layer_sample(m)
    step_bytes = sum(algorithmic_bytes(m, k, n) for k, n, *_ in layers)

    def aten_step():
        for _, _, _, w_deq, x in layers:
            torch.nn.functional.linear(x, w_deq)

    def port_step():
        for _, _, blocks, _, x in layers:
            oracle.linear(oracle.Q4_K, blocks, x.view(torch.int16).numpy().view(np.uint16), oracle.BF16, fast=True)

    def run(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        t0 = time.perf_counter()
        done = 0
        for _ in range(steps):
            fn()
            done += 1
            if time.perf_counter() - t0 > budget_s:
                break
        return (time.perf_counter() - t0) / done, done

    t_aten, done = run(aten_step, steps, warmup)
    t_port, _ = run(port_step, max(3, min(steps, 10)), 1)
    return step_bytes / t_aten / 1e9, t_aten * 1e3, cores, step_bytes / t_port / 1e9, done


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # exactly the requested warm-up and step counts (a step is one layer, ~3 ms: hundreds of steps stay within seconds;
    # the time budget only guards against a pathological host)
    gbs, ms, cores, port_gbs, done = time_cpu_reference(args.m, args.steps, args.warmup, budget_s=240.0)
    sample = (f"one Llama-3-8B layer (4 linears, M={args.m}) per step, {done} steps; ATen linear on "
              f"dequantized bf16 weights, {cores} threads")
    line = {
        "impl": "reference", "metric": "Q4_K dequant-GEMV GB/s", "value": round(gbs, 3), "unit": "GB/s",
        "n_gpus": args.gpus, "steps": done, "warmup": args.warmup, "ms_per_step": round(ms, 4),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args.m, args.gpus),
        "cpu_baseline": {"value": round(gbs, 3), "unit": "GB/s", "cores": cores, "kind": "reference",
                         "sample": sample, "port_value": round(port_gbs, 3)},
        "e2e": {"value": round(gbs, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_config(m: int, gpus: int):
    return {
        "workload": f"Llama-3-8B projection shapes, Q4_K, M={m} decode GEMV, {N_LAYERS} layers x 4 linears",
        "shapes_k_to_n": [[k, n] for _, k, n in SHAPES], "M": m, "layers": N_LAYERS,
        "parallelism": "single GPU" if gpus == 1 else f"tp{gpus} (column/row split; row-parallel sum fused into the GEMV "
                       "over NVLink peer memory for M <= 16, NCCL all-reduce otherwise)",
        "l2": f"{N_LAYERS * 122683392 / 1e9:.2f} GB of weights per step, larger than L2: every step streams from HBM",
    }


# --------------------------------------------------------------------------------------------------
# our arm
# --------------------------------------------------------------------------------------------------
def build_layers(ttq, ctx, dev, rank, world, m):
    """Quantize on the device, repack through the C ABI.  Returns per-layer lists of (linear, x, y)."""
    from tattletale_b200 import quantize as Q

    layers = []
    for layer in range(N_LAYERS):
        entry = []
        for idx, (name, k, n) in enumerate(SHAPES):
            g = torch.Generator(device=dev).manual_seed(2000 + idx + 16 * layer)
            if world == 1:
                nl, kl = n, k
            elif name in ("qkv", "gate_up"):
                nl, kl = n // world, k
            else:
                nl, kl = n, k // world
            # every rank draws its own slice; the full matrix is never materialised
            w = torch.randn(nl, kl, generator=g, device=dev) * 0.02
            blocks = Q.quantize(Q.FMT_Q4_K, w)
            lin = ttq.QuantLinear(ctx, ttq.FMT_Q4_K, blocks, kl)
            del w, blocks
            x = torch.randn(m, kl, generator=g, device=dev).to(torch.bfloat16)
            y = torch.empty(m, nl, dtype=torch.bfloat16, device=dev)
            entry.append((name, lin, x, y))
        layers.append(entry)
    return layers


def ours_arm(args):
    import tattletale_b200 as ttq

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the quantized-linear path has no CPU implementation")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)
    m = args.m
    ctx = ttq.Context(local_rank)
    layers = build_layers(ttq, ctx, dev, rank, world, m)
    torch.cuda.synchronize()
    comm = None
    if world > 1 and not args.nccl_allreduce:
        from tattletale_b200 import tp

        comm = tp.Communicator(ctx, n_cap=4096, m_cap=16)  # row-parallel outputs are [M, 4096]

    def step():
        for entry in layers:
            for name, lin, x, y in entry:
                if world > 1 and name in ("o", "down"):
                    if comm is not None:
                        lin.forward_allreduce(x, comm, out=y)  # all-reduce fused into the linear (peer memory)
                    else:
                        lin.forward(x, out=y)
                        dist.all_reduce(y)
                else:
                    lin.forward(x, out=y)

    # launches per step, counted on an eager step
    torch.cuda.synchronize()
    c0 = ctx.launch_count
    step()
    torch.cuda.synchronize()
    launches_per_step = ctx.launch_count - c0

    graph = None
    if not args.no_graph:
        try:
            stream = torch.cuda.Stream()
            stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(stream):
                step()
            torch.cuda.current_stream().wait_stream(stream)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step()
        except Exception as exc:  # capture refused (e.g. a collective that cannot be captured): run eagerly
            print(f"[bench] CUDA graph capture failed, running eagerly: {exc}", file=sys.stderr)
            graph = None
            torch.cuda.synchronize()
    run_step = graph.replay if graph is not None else step

    for _ in range(max(args.warmup, 3)):
        run_step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    sampler = ClockSampler(visible_physical_index(local_rank))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler.start()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(args.steps):
        run_step()
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    if world > 1:
        dist.barrier()
    ms_total = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms_total], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_step = ms_total / args.steps
    step_bytes = N_LAYERS * sum(algorithmic_bytes(m, k, n) for _, k, n in SHAPES)  # whole job, all ranks
    value = step_bytes / (ms_step * 1e-3) / 1e9

    # ---- the same linears as ONE recorded batch on the device buffers (ttq_host_batch_*): the activations of all linears are
    # converted by one launch and the linears, independent of each other, run side by side on forked streams.  Reported
    # beside `value`, which stays the chain of stand-alone calls (what a decoder, whose linears depend on each other, gets).
    batched = None
    if world == 1 and m <= 2:
        items = [(lin, x, y) for entry in layers for name, lin, x, y in entry]
        batch = ttq.HostBatch(ctx, items)
        reps = max(3, min(args.steps, 100))
        for _ in range(3):
            batch.run()
        t0 = time.perf_counter()
        for _ in range(reps):
            batch.run()  # returns after its own synchronisation
        b_s = (time.perf_counter() - t0) / reps
        batch.close()
        batched = {"value": round(step_bytes / b_s / 1e9, 2), "unit": "GB/s", "ms_per_step": round(b_s * 1e3, 5), "steps": reps,
                   "timing": "wall clock around ttq_host_batch_run (each call ends with its own synchronisation)",
                   "api": "ttq_host_batch_create / _run on the device buffers: one batched activation pass, then the 128 GEMV launches on four forked streams"}

    # ---- end to end: host buffers through the C-ABI host entry point, copies inside the timed region
    e2e = None
    h2d = d2h = 0
    if world == 1 and not args.no_e2e:
        host = []
        for entry in layers:
            for name, lin, x, y in entry:
                xh = x.cpu().pin_memory()
                yh = torch.empty(y.shape, dtype=y.dtype).pin_memory()
                host.append((lin, xh, yh))
                h2d += xh.numel() * xh.element_size()
                d2h += yh.numel() * yh.element_size()
        e2e_steps = max(3, min(args.steps, 50))

        def e2e_time(wait_per_call: bool) -> float:
            calls = [lin.host_call(xh, yh, wait=wait_per_call) for lin, xh, yh in host]  # arguments bound once

            def one_step():
                for call in calls:
                    call()
                if not wait_per_call:
                    ctx.host_sync()  # the step's results are in host memory when this returns
            one_step()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(e2e_steps):
                one_step()
            torch.cuda.synchronize()
            return (time.perf_counter() - t0) / e2e_steps

        per_call_s = e2e_time(True)
        enqueue_s = e2e_time(False)
        batch = ttq.HostBatch(ctx, host)  # the step recorded once: one foreign call and one wait per step
        batch.run()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            batch.run()
        e2e_s = (time.perf_counter() - t0) / e2e_steps
        batch.close()
        e2e = {"value": round(step_bytes / e2e_s / 1e9, 3), "unit": "GB/s", "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "ms_per_step": round(e2e_s * 1e3, 4), "steps": e2e_steps,
               "api": "ttq_host_batch_run: the step's 128 host-buffer linears recorded once (ttq_host_batch_create) on pinned buffers; every step one kernel converts the activations of all linears straight from the host buffers (batched activation pass), the linears write y through the buffers' device mappings, and the call returns when all results are in host memory; failure flag in mapped host memory",
               "enqueue_then_wait": {"value": round(step_bytes / enqueue_s / 1e9, 3), "ms_per_step": round(enqueue_s * 1e3, 4),
                                     "api": "ttq_linear_forward_host_async per linear + one ttq_host_sync per step"},
               "wait_per_call": {"value": round(step_bytes / per_call_s / 1e9, 3), "ms_per_step": round(per_call_s * 1e3, 4),
                                 "api": "ttq_linear_forward_host: one wait per linear (the reference's synchronous forward)"}}

    if world > 1 and not args.no_e2e:
        # every rank feeds its shard from pinned host memory and reads its result back: per linear one host -> device
        # copy of the activations, the (row-parallel: fused-exchange) linear, one device -> host copy of the output;
        # one synchronisation per step; wall clock, maximum over ranks
        host = []
        in_place = comm is not None
        for entry in layers:
            for name, lin, x, y in entry:
                xh, yh = x.cpu().pin_memory(), torch.empty(y.shape, dtype=y.dtype).pin_memory()
                xa = ya = None
                if in_place:
                    # the kernels read x and write y in the pinned buffers themselves, through their device addresses
                    xa, ya = _device_alias(xh, dev), _device_alias(yh, dev)
                    in_place = xa is not None and ya is not None
                host.append((name, lin, xh, x, y, yh, xa, ya))
                h2d += x.numel() * x.element_size()
                d2h += y.numel() * y.element_size()

        def e2e_step():
            for name, lin, xh, x, y, yh, xa, ya in host:
                if in_place:
                    if name in ("o", "down"):
                        lin.forward_allreduce(xa, comm, out=ya)
                    else:
                        lin.forward(xa, out=ya)
                    continue
                x.copy_(xh, non_blocking=True)
                if name in ("o", "down"):
                    if comm is not None:
                        lin.forward_allreduce(x, comm, out=y)
                    else:
                        lin.forward(x, out=y)
                        dist.all_reduce(y)
                else:
                    lin.forward(x, out=y)
                yh.copy_(y, non_blocking=True)
            torch.cuda.synchronize()

        e2e_steps = max(3, min(args.steps, 50))
        e2e_step()
        # in place, the step is a fixed sequence of launches on fixed buffers: recorded once, replayed per step (the
        # wait stays outside the recording)
        e2e_graph = None
        if in_place and not args.no_graph:
            try:
                def e2e_launches():
                    for name, lin, xh, x, y, yh, xa, ya in host:
                        if name in ("o", "down"):
                            lin.forward_allreduce(xa, comm, out=ya)
                        else:
                            lin.forward(xa, out=ya)
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    e2e_launches()
                torch.cuda.current_stream().wait_stream(side)
                torch.cuda.synchronize()
                dist.barrier()
                e2e_graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(e2e_graph):
                    e2e_launches()
                torch.cuda.synchronize()
            except Exception as exc:  # pragma: no cover - depends on the runtime
                print(f"[bench] end-to-end graph capture failed, launching eagerly: {exc}", file=sys.stderr)
                e2e_graph = None
        if e2e_graph is not None:
            def e2e_step():  # noqa: F811 - the recorded form of the same step
                e2e_graph.replay()
                torch.cuda.synchronize()
            e2e_step()
        dist.barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step()
        t = torch.tensor([(time.perf_counter() - t0) / e2e_steps], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
        e2e = {"value": round(step_bytes / e2e_s / 1e9, 3), "unit": "GB/s", "h2d_bytes_per_step": h2d * world,
               "d2h_bytes_per_step": d2h * world, "ms_per_step": round(e2e_s * 1e3, 4), "steps": e2e_steps,
               "api": ("per rank and linear: QuantLinear.forward / forward_allreduce on the rank's shard with x and y in pinned host "
                       "memory (the kernels read and write them in place over the host link); the step's launches "
                       + ("replayed as a CUDA graph" if e2e_graph is not None else "issued eagerly") + "; one sync per step; bytes summed over ranks")
                      if in_place else
                      ("per rank and linear: pinned host -> device copy of x, QuantLinear.forward / forward_allreduce on the "
                       "rank's shard, device -> pinned host copy of y; one sync per step; bytes summed over ranks")}

    # ---- per-shape breakdown (device-resident, cold L2: the 32 layers' copies are rotated)
    per_shape = {}
    if world == 1 and not args.no_e2e:
        for idx, (name, k, n) in enumerate(SHAPES):
            items = [layers[l][idx] for l in range(N_LAYERS)]
            for _, lin, x, y in items:
                lin.forward(x, out=y)
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps = 4
            a.record()
            for _ in range(reps):
                for _, lin, x, y in items:
                    lin.forward(x, out=y)
            b.record()
            torch.cuda.synchronize()
            us = a.elapsed_time(b) * 1e3 / (reps * N_LAYERS)
            per_shape[f"{k}x{n}"] = {"us": round(us, 3), "gbs": round(algorithmic_bytes(m, k, n) / us / 1e3, 1)}

    # ---- batched rows: M = 2 .. 2048 on every shape.  One launch per layer's weight (32 distinct matrices per shape,
    # 0.3 - 2.1 GB: cold L2 for the memory-bound sizes), replayed as a CUDA graph so that host launch time stays out
    sweep = {}
    if world == 1 and not args.no_e2e and not args.no_sweep:
        for ms in (2, 4, 8, 16, 64, 256, 2048):
            for idx, (name, k, n) in enumerate(SHAPES):
                lins = [layers[l][idx][1] for l in range(N_LAYERS if ms <= 64 else min(N_LAYERS, 4))]
                g = torch.Generator(device=dev).manual_seed(2100 + ms)
                xs = torch.randn(ms, k, generator=g, device=dev).to(torch.bfloat16)
                ys = torch.empty(ms, n, dtype=torch.bfloat16, device=dev)

                def sweep_step():
                    for lin in lins:
                        lin.forward(xs, out=ys)

                us = _time_graph(sweep_step, reps=4) / len(lins)
                sweep[f"M{ms}_{k}x{n}"] = {"us": round(us, 2), "tflops": round(2.0 * ms * n * k / us / 1e6, 1),
                                            "gbs": round(algorithmic_bytes(ms, k, n) / us / 1e3, 1)}
                del xs, ys
        # the decode-batch sizes again as recorded batches of independent linears (ttq_host_batch_* on the device buffers):
        # per shape the same 32 weights, wall clock around the synchronous run call
        for ms in (2, 4, 8, 16):
            for idx, (name, k, n) in enumerate(SHAPES):
                lins = [layers[l][idx][1] for l in range(N_LAYERS)]
                g = torch.Generator(device=dev).manual_seed(2100 + ms)
                xs = torch.randn(ms, k, generator=g, device=dev).to(torch.bfloat16)
                ybuf = [torch.empty(ms, n, dtype=torch.bfloat16, device=dev) for _ in lins]
                torch.cuda.synchronize()
                batch = ttq.HostBatch(ctx, [(lin, xs, y) for lin, y in zip(lins, ybuf)])
                for _ in range(2):
                    batch.run()
                t0 = time.perf_counter()
                for _ in range(4):
                    batch.run()
                us = (time.perf_counter() - t0) / 4 / len(lins) * 1e6
                batch.close()
                sweep[f"M{ms}_{k}x{n}"]["batched_us"] = round(us, 2)
                sweep[f"M{ms}_{k}x{n}"]["batched_gbs"] = round(algorithmic_bytes(ms, k, n) / us / 1e3, 1)
                del xs, ybuf
        ctx.check_device_status()

    # ---- the other half of the metric: decode tokens/s of the full decoder stack (one GPU)
    decode_stack = None
    if world == 1 and not args.no_e2e and not args.no_decode_stack:
        decode_stack = _decode_stack_numbers(ttq, ctx, dev, layers)

    # ---- N > 1: the configurations where sharding has more to give than at M = 1 -- the decoder stack at batch 1 and
    # 32 (tokens/s) and trellis-coded linears on the Llama-3-70B shapes at M = 16, all tensor-parallel over the ranks
    tp_extras = None
    if world > 1 and not args.no_e2e:
        tp_extras = _tp_extras(ttq, ctx, dev, rank, world, comm, dist)

    if rank != 0:
        _finish_distributed(dist, world)
        return

    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))
    peak_kind = "measured (MEASURED_PEAKS.json hbm_gbs)" if "hbm_gbs" in peaks else "fallback 6650"
    gemv_launches = N_LAYERS * len(SHAPES)
    roofline = {
        "bound": "hbm", "achieved": round(value / world, 2), "peak": peak, "unit": "GB/s",
        "frac": round(value / world / peak, 4),
        # dram read + write per launch, measured by ncu on a 2-layer case of the same kernels and shapes (the traffic of a
        # launch does not depend on the layer count); other batch sizes and shards have no capture
        "traffic": _measured_traffic("gemv_q4k_m1_llama8b_per_launch") if (m == 1 and world == 1) else None,
        "traffic_source": "ncu capture of a 2-layer case, mean over one layer's four launches" if (m == 1 and world == 1) else None,
        "peak_source": peak_kind,
        "kernel": _linear_kernel_name(m),
        "avg_launch_us": round(ms_step * 1e3 / gemv_launches, 3),
        "algorithmic_bytes_per_launch": step_bytes // gemv_launches,
        "frac_of_nominal_8TBs": round(value / world / 8000.0, 4),
    }
    cpu_baseline = None
    if world == 1 and not args.no_cpu_baseline:
        gbs, ms, cores, port_gbs, done = time_cpu_reference(m, 20, 2, budget_s=12.0)
        cpu_baseline = {"value": round(gbs, 3), "unit": "GB/s", "cores": cores, "kind": "reference",
                        "sample": f"one layer (4 linears, M={m}) x {done} steps, ATen linear on dequantized bf16 weights",
                        "port_value": round(port_gbs, 3), "port_kind": "oracle fused dequant-dot on packed blocks"}
    line = {
        "metric": "Q4_K dequant-GEMV GB/s", "value": round(value, 2), "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms_step, 5),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8", "arithmetic": "u8|s8 x s8 -> s32 tensor-core dot per sub-block, fp32 scales",
        "data": "synthetic", "config": workload_config(m, world), "roofline": roofline, "cpu_baseline": cpu_baseline,
        "e2e": e2e, "gpu_launches": int(launches_per_step * args.steps), "launches_per_step": int(launches_per_step),
        "cuda_graph": graph is not None, "clocks": clocks, "per_shape": per_shape,
        "decode_linears_tokens_per_s": round(m / (ms_step * 1e-3), 1),
    }
    if batched:
        batched["frac_of_hbm_peak"] = round(batched["value"] / peak, 4)
        line["batched_independent"] = batched
        # the same kernel without the dependent hand-over between launches: what separates `frac` from the kernel's own rate
        roofline["achieved_batched_independent"] = batched["value"]
        roofline["frac_batched_independent"] = batched["frac_of_hbm_peak"]
    if decode_stack:
        line["decode_stack"] = decode_stack
    if tp_extras:
        line["tensor_parallel"] = tp_extras
    if sweep:
        best = max(v["tflops"] for key, v in sweep.items() if key.startswith("M2048_"))
        tpeak = float(peaks.get("bf16_tflops", 1590.0))
        line["sweep"] = sweep
        line["roofline_gemm"] = {"bound": "tensor", "achieved": best, "peak": tpeak, "unit": "TFLOP/s",
                                 "frac": round(best / tpeak, 4), "kernel": "gemm_q4k_pair_kernel (tcgen05 cta_group::2) or gemm_q4k_kernel, chosen per call by the library's cost model; fp16 operands, fp32 accumulate",
                                 "workload": "best of the four Q4_K shapes at M=2048 (graph replay over 4 layers' weights, includes the activation pass)",
                                 "peak_source": "MEASURED_PEAKS.json bf16_tflops (burst)" if "bf16_tflops" in peaks else "fallback 1590"}
    print(json.dumps(line), flush=True)
    _finish_distributed(dist, world)


class _PinnedView:
    """The CUDA array interface of a pinned host tensor's bytes (16-bit elements)."""

    def __init__(self, t):
        self.keep = t
        self.__cuda_array_interface__ = {"data": (t.data_ptr(), False), "shape": tuple(t.shape), "typestr": "<i2", "version": 2,
                                         "strides": None}


def _device_alias(t, dev):
    """A CUDA tensor over the memory of pinned host tensor `t` (unified addressing: the device address of page-locked
    memory allocated by the runtime is its host address), or None when that cannot be had."""
    if t.element_size() != 2 or not t.is_pinned() or not t.is_contiguous():
        return None
    try:
        alias = torch.as_tensor(_PinnedView(t), device=dev).view(t.dtype)
        return alias if alias.data_ptr() == t.data_ptr() else None
    except Exception:
        return None


def _linear_kernel_name(m: int) -> str:
    """The kernels a Q4_K linear of `m` rows runs (the library's dispatch by row count)."""
    if m <= 2:
        return "xprep_kernel + gemv_kernel<Q4_K> (activation planes bulk-copied from scratch)"
    if m <= 16:
        return "q4k_decode_kernel (one launch, integer-exact fp16 mma.sync)"
    return "xh_prep_kernel + gemm_q4k_kernel / gemm_q4k_pair_kernel (tcgen05, tensor memory)"


def _time_graph(step, reps: int = 4, warm: int = 2) -> float:
    """Microseconds of one `step()` replayed as a CUDA graph (capture on a side stream, `warm` untimed replays)."""
    step()
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    for _ in range(warm):
        graph.replay()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        graph.replay()
    b.record()
    torch.cuda.synchronize()
    del graph
    return a.elapsed_time(b) * 1e3 / reps


def _decode_stack_numbers(ttq, ctx, dev, layers=None):
    """Decode tokens/s of the Llama-3-8B decoder stack (configs[2]: 32 layers, Q4_K linears, Q6_K vocabulary
    projection over the full 128256-row table, context 2048) at batch 1, 8 and 32 on this GPU."""
    from tattletale_b200.decoder import DecoderConfig, DecoderStack

    cfg = DecoderConfig()
    peaks = _peaks()
    peak = float(peaks.get("hbm_gbs", 6650.0))
    torch.manual_seed(3000)
    stack = DecoderStack(ctx, cfg, 32)
    out = {}
    for batch in (1, 8, 32):
        g = torch.Generator(device=dev).manual_seed(3100 + batch)
        ids = torch.randint(0, cfg.vocab, (batch,), generator=g, device=dev)
        us = _time_graph(lambda: stack.step(ids), reps=10, warm=3)
        kv_bytes = 2 * cfg.n_layers * batch * cfg.n_kv_heads * cfg.context * cfg.head_dim * 2
        gbs = (stack.weight_bytes + kv_bytes) / us / 1e3
        out[str(batch)] = {"tokens_per_s": round(batch / (us * 1e-6), 1), "ms_per_step": round(us / 1e3, 4),
                           "hbm_gbs": round(gbs, 1), "frac_of_hbm_peak": round(gbs / peak, 4),
                           "bytes_per_step": {"weights": int(stack.weight_bytes), "kv_cache": int(kv_bytes)}}
    ctx.check_device_status()
    del stack
    torch.cuda.empty_cache()
    return out


def _max_over_ranks(us: float, dev, dist) -> float:
    t = torch.tensor([us], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _tp_extras(ttq, ctx, dev, rank, world, comm, dist):
    """Tensor-parallel numbers beside the headline (device-timed, max over ranks): decoder stack tokens/s at batch 1 and
    32 (QKV and gate|up split by rows, O and down by columns with the sum over ranks fused into the linear up to 16
    rows and through NCCL beyond), and one layer of trellis-coded 3-bit linears on the Llama-3-70B shapes at M = 16
    (column split for QKV and gate|up, row split + NCCL all-reduce for O and down)."""
    from tattletale_b200 import formats, tp
    from tattletale_b200._lib import SHARD_COLUMN, SHARD_ROW
    from tattletale_b200.decoder import DecoderConfig, DecoderStack

    out = {}
    cfg = DecoderConfig()
    torch.manual_seed(3000 + rank)
    stack = DecoderStack(ctx, cfg, 32, rank, world, comm=comm)
    for batch in (1, 32):
        g = torch.Generator(device=dev).manual_seed(3100 + batch)
        ids = torch.randint(0, cfg.vocab, (batch,), generator=g, device=dev)
        dist.barrier()
        try:
            us = _time_graph(lambda: stack.step(ids), reps=10, warm=3)
            graph = True
        except Exception:  # a collective that cannot be captured: time eager steps
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            for _ in range(3):
                stack.step(ids)
            a.record()
            for _ in range(10):
                stack.step(ids)
            b.record()
            torch.cuda.synchronize()
            us, graph = a.elapsed_time(b) * 1e3 / 10, False
        us = _max_over_ranks(us, dev, dist)
        out[f"decode_batch{batch}"] = {"tokens_per_s": round(batch / (us * 1e-6), 1), "ms_per_step": round(us / 1e3, 4), "cuda_graph": graph}
    del stack
    torch.cuda.empty_cache()
    # trellis-coded linears, random code bits (the kernels' speed does not depend on the bit values)
    shapes = [("qkv", 8192, 10240, SHARD_COLUMN), ("o", 8192, 8192, SHARD_ROW), ("gate_up", 8192, 57344, SHARD_COLUMN),
              ("down", 28672, 8192, SHARD_ROW)]
    m = 16
    lins = []
    for idx, (name, k, n, kind) in enumerate(shapes):
        g = torch.Generator(device="cpu").manual_seed(4000 + idx)
        packed = torch.randint(0, 256, (formats.packed_bytes(ttq.FMT_TQ3, n, k),), generator=g, dtype=torch.uint8)
        sc = (torch.randn(n, generator=g) * 0.015).to(torch.float16)
        packed[n * k * 3 // 8: n * k * 3 // 8 + 2 * n] = sc.view(torch.uint8)
        local, nl, kl = tp.shard_trellis(packed, n, k, kind, rank, world)
        lin = ttq.QuantLinear(ctx, ttq.FMT_TQ3, local.contiguous().to(dev), kl, out_features=nl)
        x = torch.randn(m, kl, device=dev).to(torch.bfloat16)
        lins.append((kind, lin, x))

    def trellis_step():
        for kind, lin, x in lins:
            if kind == SHARD_ROW:
                lin.forward_reduce(x)
            else:
                lin.forward(x)

    dist.barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(3):
        trellis_step()
    a.record()
    for _ in range(10):
        trellis_step()
    b.record()
    torch.cuda.synchronize()
    us = _max_over_ranks(a.elapsed_time(b) * 1e3 / 10, dev, dist)
    out["trellis_m16_llama70b_layer"] = {"us_per_layer": round(us, 1), "shapes_k_to_n": [[k, n] for _, k, n, _ in shapes]}
    ctx.check_device_status()
    return out


def _peaks():
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        return {}


def _measured_traffic(key: str):
    """DRAM read + write bytes per launch from the committed ncu capture of this kernel (a `key = bytes` line of
    profiles/ncu_traffic.txt, written when the capture is summarised); None when no capture covers the case."""
    try:
        for ln in open(os.path.join(ROOT, "profiles", "ncu_traffic.txt")):
            ln = ln.split("#", 1)[0].strip()
            if "=" in ln:
                name, val = (t.strip() for t in ln.split("=", 1))
                if name == key:
                    return int(float(val))
    except Exception:
        pass
    return None


def decode_arm(args):
    """Full Llama-3-8B decoder stack (random init), one decode step at context 2048."""
    import tattletale_b200 as ttq
    from tattletale_b200.decoder import DecoderConfig, DecoderStack

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)
    cfg = DecoderConfig(n_layers=args.layers)
    ctx = ttq.Context(local_rank)
    torch.manual_seed(3000 + rank)
    comm = None
    if world > 1 and not args.nccl_allreduce:
        from tattletale_b200 import tp

        comm = tp.Communicator(ctx, n_cap=cfg.hidden, m_cap=16)
    stack = DecoderStack(ctx, cfg, args.batch, rank, world, comm=comm, fused_glue=not args.torch_glue)
    g = torch.Generator(device=dev).manual_seed(3100)
    ids = torch.randint(0, cfg.vocab, (args.batch,), generator=g, device=dev)
    out = stack.step(ids)
    torch.cuda.synchronize()
    c0 = ctx.launch_count
    out = stack.step(ids)
    torch.cuda.synchronize()
    launches_per_step = ctx.launch_count - c0
    graph = None
    if not args.no_graph:
        try:
            st = torch.cuda.Stream()
            st.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(st):
                stack.step(ids)
            torch.cuda.current_stream().wait_stream(st)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                out = stack.step(ids)
        except Exception as exc:
            print(f"[bench] CUDA graph capture failed, running eagerly: {exc}", file=sys.stderr)
            graph = None
            torch.cuda.synchronize()
    run = graph.replay if graph is not None else (lambda: stack.step(ids))
    for _ in range(max(args.warmup, 3)):
        run()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    sampler = ClockSampler(visible_physical_index(local_rank))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler.start()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(args.steps):
        run()
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms_total = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms_total], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_step = ms_total / args.steps
    ctx.check_device_status()
    if rank == 0:
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except Exception:
            pass
        peak = float(peaks.get("hbm_gbs", 6650.0))
        kv_bytes = 2 * cfg.n_layers * args.batch * cfg.n_kv_heads * cfg.context * cfg.head_dim * 2
        w_bytes = stack.weight_bytes * world
        gbs = (w_bytes + kv_bytes) / (ms_step * 1e-3) / 1e9
        line = {
            "metric": "decode tokens/s", "value": round(args.batch / (ms_step * 1e-3), 1), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms_step, 4), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
            "config": {"workload": f"Llama-3-8B decoder stack, {cfg.n_layers} layers, Q4_K linears + Q6_K lm_head, decode batch "
                                   f"{args.batch} at context {cfg.context}", "batch": args.batch, "context": cfg.context,
                       "parallelism": "single GPU" if world == 1 else f"tp{world}",
                       "glue": ("RMSNorm, RoPE, KV cache and attention are torch ops" if args.torch_glue else
                                "residual + RMSNorm, RoPE + KV append and single-query attention are libttq kernels; "
                                "embedding lookup and argmax are torch ops")},
            "roofline": {"bound": "hbm", "achieved": round(gbs / world, 1), "peak": peak, "unit": "GB/s", "frac": round(gbs / world / peak, 4),
                         "traffic": None, "bytes_per_step": {"weights": int(w_bytes), "kv_cache": int(kv_bytes)}},
            "gpu_launches": int(launches_per_step * args.steps), "launches_per_step": int(launches_per_step),
            "cuda_graph": graph is not None, "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    _finish_distributed(dist, world)


def moe_arm(args):
    """Mixture-of-experts layer, Qwen3-30B-A3B-like: hidden 2048, 128 experts of FFN 768 (gated), top-8
    routing from N(0,1) router logits, 4096 tokens, Q4_K experts ~N(0, 0.02).  N > 1: expert parallel (each rank
    holds E/N experts and T/N tokens; NCCL all-to-all dispatch and combine around the local grouped GEMM)."""
    import torch.distributed as dist

    import tattletale_b200 as ttq
    from tattletale_b200 import quantize as Q
    from tattletale_b200 import tp

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    H, I, E, K, T = 2048, 768, 128, 8, args.tokens
    assert E % world == 0 and T % world == 0
    epr, tl = E // world, T // world
    ctx = ttq.Context(local_rank)
    gu, dn = [], []
    for e in range(rank * epr, (rank + 1) * epr):
        g = torch.Generator(device=dev).manual_seed(5000 + e)
        gu.append(Q.quantize(ttq.FMT_Q4_K, torch.randn(2 * I, H, generator=g, device=dev) * 0.02))
        dn.append(Q.quantize(ttq.FMT_Q4_K, torch.randn(H, I, generator=g, device=dev) * 0.02))
    g = torch.Generator(device=dev).manual_seed(6000 + rank)
    x = torch.randn(tl, H, generator=g, device=dev).to(torch.bfloat16)
    logits = torch.randn(tl, E, generator=g, device=dev)
    wts, ids = torch.softmax(logits, dim=-1).topk(K, dim=-1)
    wts = (wts / wts.sum(dim=-1, keepdim=True)).float().contiguous()
    ids = ids.to(torch.int32).contiguous()
    if world == 1:
        layer = ttq.MoELayer(ctx, ttq.FMT_Q4_K, gu, dn, H, I, top_k=K, max_tokens=T)
        y = torch.empty_like(x)
        step = lambda: layer.forward(x, ids, wts, out=y)
    else:
        local = ttq.MoELayer(ctx, ttq.FMT_Q4_K, gu, dn, H, I, top_k=1, max_tokens=3 * tl * K)
        ep = tp.ExpertParallelMoE.from_layer(local)
        step = lambda: ep.forward(x, ids, wts)
    del gu, dn
    step()
    torch.cuda.synchronize()
    c0 = ctx.launch_count
    step()
    torch.cuda.synchronize()
    launches_per_step = ctx.launch_count - c0
    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    steps = min(args.steps, 200)
    sampler = ClockSampler(visible_physical_index(local_rank))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler.start()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms_total = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms_total], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_step = ms_total / steps
    ctx.check_device_status()
    if rank == 0:
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except Exception:
            pass
        peak = float(peaks.get("bf16_tflops", 1590.0))
        flops = 2.0 * T * K * (2 * I * H + H * I)
        tf = flops / (ms_step * 1e-3) / 1e12
        w_bytes = E * ((2 * I) * (H // 256) + H * (I // 256)) * Q4K_BYTES_PER_256
        line = {
            "metric": "MoE expert-GEMM TFLOP/s", "value": round(tf, 1), "unit": "TFLOP/s", "n_gpus": world, "steps": steps,
            "warmup": max(args.warmup, 3), "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f16", "arithmetic": "Q4_K expanded to fp16 in shared memory, tcgen05 f16 MMA, fp32 accumulation",
            "data": "synthetic",
            "config": {"workload": f"Qwen3-30B-A3B-like MoE layer: hidden {H}, {E} experts of FFN {I} (gated), top-{K}, {T} tokens, Q4_K",
                       "tokens": T, "parallelism": "single GPU" if world == 1 else f"ep{world} (NCCL all-to-all dispatch / combine)",
                       "l2": f"{w_bytes / 1e6:.0f} MB of expert weights + {T * K * (H + 2 * I + I + H) * 2 / 1e6:.0f} MB of routed "
                             "intermediates per step, larger than L2",
                       "includes": "routing, activation conversion, both grouped GEMMs, silu*up, weighted combine"},
            "tokens_per_s": round(T / (ms_step * 1e-3), 1),
            "roofline": {"bound": "tensor", "achieved": round(tf / world, 1), "peak": peak, "unit": "TFLOP/s",
                         "frac": round(tf / world / peak, 4), "traffic": None,
                         "peak_source": "measured (MEASURED_PEAKS.json bf16_tflops)" if "bf16_tflops" in peaks else "fallback"},
            "gpu_launches": int(launches_per_step * steps), "launches_per_step": int(launches_per_step), "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    _finish_distributed(dist, world)


def trellis_arm(args):
    """Trellis-coded 3-bit linears on the Llama-3-70B projection shapes: 8192->10240,
    8192->8192, 8192->57344, 28672->8192 at M = --m rows, weights N(0, 0.015) coded by the package's beam-search
    encoder (or uniformly random code bits with --trellis-codes random: the kernels' speed does not depend on
    the bit values).  One step = one pass over --layers layers of four linears."""
    import tattletale_b200 as ttq
    from tattletale_b200 import formats
    from tattletale_b200 import quantize as Q

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    ctx = ttq.Context(0)
    shapes = [(8192, 10240), (8192, 8192), (8192, 57344), (28672, 8192)]
    n_layers = args.layers if args.layers != 32 else 2
    m = args.m
    lins = []
    t_enc = time.perf_counter()
    for layer in range(n_layers):
        for idx, (k, n) in enumerate(shapes):
            g = torch.Generator(device=dev).manual_seed(4000 + 16 * layer + idx)
            if args.trellis_codes == "random":
                packed = torch.randint(0, 256, (formats.packed_bytes(ttq.FMT_TQ3, n, k),), generator=g, device=dev, dtype=torch.uint8)
                sc = (torch.randn(n, generator=g, device=dev) * 0.015).to(torch.float16)
                packed[n * k * 3 // 8: n * k * 3 // 8 + 2 * n] = sc.view(torch.uint8)
            else:
                w = torch.randn(n, k, generator=g, device=dev) * 0.015
                packed = Q.quantize_tq3(w, seed=4000 + idx, beam=4, tile_chunk=1 << 16)
                del w
            lins.append((k, n, ttq.QuantLinear(ctx, ttq.FMT_TQ3, packed, k, out_features=n)))
            del packed
    torch.cuda.synchronize()
    t_enc = time.perf_counter() - t_enc
    xs = {k: torch.randn(m, k, device=dev).to(torch.bfloat16) for k in (8192, 28672)}
    ys = {n: torch.empty(m, n, dtype=torch.bfloat16, device=dev) for n in (10240, 8192, 57344)}

    def step():
        for k, n, lin in lins:
            lin.forward(xs[k], out=ys[n])

    step()
    torch.cuda.synchronize()
    c0 = ctx.launch_count
    step()
    torch.cuda.synchronize()
    launches_per_step = ctx.launch_count - c0
    graph = None
    if not args.no_graph:
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                step()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step()
        except Exception as exc:
            print(f"[bench] CUDA graph capture failed, running eagerly: {exc}", file=sys.stderr)
            graph = None
            torch.cuda.synchronize()
    run = graph.replay if graph is not None else step
    for _ in range(max(args.warmup, 3)):
        run()
    steps = min(args.steps, 100)
    sampler = ClockSampler(visible_physical_index(0))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler.start()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(steps):
        run()
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms_step = e0.elapsed_time(e1) / steps
    ctx.check_device_status()
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    w_bytes = sum(formats.packed_bytes(ttq.FMT_TQ3, n, k) for k, n, _ in lins)
    io_bytes = sum(m * k * 2 + m * n * 2 for k, n, _ in lins)
    flops = sum(2.0 * m * n * k for k, n, _ in lins)
    gbs = (w_bytes + io_bytes) / (ms_step * 1e-3) / 1e9
    tf = flops / (ms_step * 1e-3) / 1e12
    hbm_bound = m <= 32
    roof = ({"bound": "hbm", "achieved": round(gbs, 1), "peak": float(peaks.get("hbm_gbs", 6650.0)), "unit": "GB/s"} if hbm_bound else
            {"bound": "tensor", "achieved": round(tf, 1), "peak": float(peaks.get("bf16_tflops", 1590.0)), "unit": "TFLOP/s"})
    roof["frac"] = round(roof["achieved"] / roof["peak"], 4)
    roof["traffic"] = None
    roof["kernel"] = "tq3_gemv_kernel (decode-and-multiply)" if hbm_bound else "tq3_decode_kernel (expansion) + gemm kernel (plain mode)"
    line = {
        "metric": "trellis 3-bit linear GB/s" if hbm_bound else "trellis 3-bit linear TFLOP/s",
        "value": round(gbs, 1) if hbm_bound else round(tf, 1), "unit": "GB/s" if hbm_bound else "TFLOP/s", "n_gpus": 1,
        "steps": steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32" if hbm_bound else "f16", "data": "synthetic",
        "config": {"workload": f"Llama-3-70B projection shapes, trellis-coded 3.0 bits/weight, M={m}, {n_layers} layers x 4 linears",
                   "shapes_k_to_n": [[k, n] for k, n in shapes], "M": m, "layers": n_layers, "codes": args.trellis_codes,
                   "l2": f"{w_bytes / 1e6:.0f} MB of packed weights per step, larger than L2", "encode_seconds": round(t_enc, 1)},
        "roofline": roof, "gpu_launches": int(launches_per_step * steps), "launches_per_step": int(launches_per_step),
        "cuda_graph": graph is not None, "clocks": clocks,
    }
    print(json.dumps(line), flush=True)


def _finish_distributed(dist, world):
    """Leave a multi-rank run without tearing NCCL down: a captured graph still references the communicator,
    and destroying the process group under it has been seen to block; the process simply exits."""
    if world > 1:
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def main():
    global N_LAYERS
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=500)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--m", type=int, default=1, help="decode batch (rows of x)")
    ap.add_argument("--workload", default="linears", choices=["linears", "decode", "moe", "trellis"],
                    help="linears: the headline Q4_K GEMV pass (default); decode: full decoder stack, tokens/s; "
                         "moe: one mixture-of-experts layer, TFLOP/s; trellis: trellis-coded 3-bit linears on 70B shapes")
    ap.add_argument("--trellis-codes", default="encoded", choices=["encoded", "random"],
                    help="trellis workload: code bits from the beam-search encoder or uniformly random")
    ap.add_argument("--tokens", type=int, default=4096, help="moe workload: tokens per step (all ranks together)")
    ap.add_argument("--batch", type=int, default=1, help="decode workload: sequences decoded together")
    ap.add_argument("--torch-glue", action="store_true",
                    help="decode workload: run norm / RoPE / attention as torch ops instead of the library's decode-step kernels")
    ap.add_argument("--no-graph", action="store_true", help="launch eagerly instead of replaying a CUDA graph")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--nccl-allreduce", action="store_true", help="N > 1: use NCCL for the row-parallel sums instead of the fused exchange")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg")
    ap.add_argument("--no-sweep", action="store_true", help="skip the M = 2..2048 sweep")
    ap.add_argument("--no-decode-stack", action="store_true", help="skip the decoder-stack tokens/s numbers of the default line")
    ap.add_argument("--layers", type=int, default=32,
                    help="layers in the pass (default 32; smaller values are for profiler captures only)")
    args = ap.parse_args()
    N_LAYERS = args.layers
    if args.impl == "reference":
        reference_arm(args)
    elif args.workload == "decode":
        decode_arm(args)
    elif args.workload == "moe":
        moe_arm(args)
    elif args.workload == "trellis":
        trellis_arm(args)
    else:
        ours_arm(args)


if __name__ == "__main__":
    main()
