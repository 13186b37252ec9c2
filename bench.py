#!/usr/bin/env python3
"""Update-step throughput of the CUDA executor.

    python bench.py [--config 4] --gpus N --steps K --warmup W      (N > 1: under torchrun)
    python bench.py --impl reference ...                            the reference CPU executor

--config picks the workload (default 4, the int8-weight decoder the headline
metric is quoted on):
    1  feed-forward plan, 256 -> 1024 -> 64, batch 32, f32                (samples/s)
    2  isolated GEMM training step, S^3, f32 and bf16, S = 512 .. 8192     (rows/s; a sweep table)
    3  small f32 decoder, 4 layers d256 seq 128, 32 sequences               (tokens/s)
    4  int8-weight decoder, 12 layers d768 seq 512, 64 sequences, dp over N (tokens/s)
    5  causal attention forward + backward, B8 H16 d64/128, S = 256 .. 4096 (a sweep table)

One JSON line on stdout (rank 0).  `value` times K steps with the batch already
resident in HBM; `e2e` times the same K steps through the public call sequence
with HOST buffers (stage_batch -> train -> read_loss), copies inside the timed
region.  `roofline` is the dominant kernel: algorithmic work of every launch of
it in a profiled step divided by the CUDA-event time of those launches, against
the measured peak.  `hbm_kernels` lists the bandwidth-bound opcodes of the same
profiled step the same way against the measured copy bandwidth.
`cpu_baseline` times the reference CPU executor beside it; `parity` compares
the first step's loss and gradient block of the two, outside any timed region.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from see_ai_b200 import plan as P  # noqa: E402
from see_ai_b200 import workloads as W  # noqa: E402

NCU_TRAFFIC_BYTES = 71.5e6
NCU_TRAFFIC_NOTE = ("ncu, one 32768x768x768 launch with its low-rank blocks and the bf16 operand copy of its result as "
                    "the only store (the most frequent form of the step's tensor-core GEMM launches): 60.2 MB read + "
                    "11.3 MB written; algorithmic 109 MB (A bf16 50 MB, low-rank operand 8 MB, W 1 MB, bf16 result "
                    "50 MB), most of the result is still in L2 when the kernel ends")
METRIC = "update_step_tokens_per_s"


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], bf16_tflops=p["bf16_tflops"],
                    bf16_tflops_sustained=p.get("bf16_tflops_sustained", p["bf16_tflops"]),
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "20", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                  "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def unit_metric(wl) -> str:
    return METRIC if wl.unit == "tokens" else "update_step_samples_per_s"


# ---- the reference arm: the reference's own CPU executor ------------------------------------

def cpu_executor():
    import oracle
    kind = "reference" if oracle.have_ref() else "port"
    if kind == "port" and not oracle.have_oracle():
        oracle.build("oracle")
    ex = oracle.RefExecutor() if kind == "reference" else oracle.OracleExecutor()
    cores = 1
    if kind == "reference":
        ex.set_threads(os.cpu_count() or 1)
        cores = ex.threads()
    return ex, kind, int(cores)


def cpu_plan_sample(config: int, steps: int, warmup: int):
    """Steps of the configuration's plan through the reference CPU executor with
    every host thread.  Configurations 1 and 3 at their stated size; the int8
    decoder at ONE sequence (512 tokens) per step instead of 64 (a full step
    takes minutes on a CPU; its tokens/s does not depend on the batch).
    Returns (units/s, info)."""
    import oracle
    from see_ai_b200 import dp, synth
    wl = W.plan_workload(config)
    if config == 4:
        blob = synth.build_decoder_plan(W.int8_decoder_config(1))
        sample = "optimizer step(s) of the same 12-layer plan at 1 sequence (512 tokens) instead of 64"
    else:
        blob = wl.build(1)
        sample = "optimizer step(s) of the same plan at its stated size"
    plan = P.Plan(blob)
    h = plan.header
    arena = plan.stage_arena()
    ex, kind, cores = cpu_executor()
    ex.bind(arena, np.frombuffer(plan.rodata, dtype=np.uint8).copy())
    batches = wl.batches(h["batch"], 2, seed=11)
    _bwd, opt_begin = dp.scan_phases(plan.train)
    g_off, g_bytes = dp.gradient_block(plan)
    times, first = [], {}
    for s in range(warmup + steps):
        x, y = batches[s % 2]
        t0 = time.perf_counter()
        xb, yb = x.view(np.uint8).reshape(-1), y.view(np.uint8).reshape(-1)
        arena[h["input_ref"]:h["input_ref"] + xb.size] = xb
        arena[h["label_ref"]:h["label_ref"] + yb.size] = yb
        sp = oracle.StepParams(h["lr"], h["beta1"], h["beta2"], h["eps"], h["weight_decay"], 0, s + 1)
        if s == 0:   # the first step in two ranges, so that its loss and gradient block can be kept
            ex.run(plan.train, sp, 0, opt_begin)
            first = dict(loss=float(arena[h["loss_ref"]:h["loss_ref"] + 4].view(np.float32)[0]),
                         grad=arena[g_off:g_off + g_bytes].view(np.float32).copy(), batch=(x, y), blob=blob)
            ex.run(plan.train, sp, opt_begin, len(plan.train))
        else:
            ex.run(plan.train, sp)
        if s >= warmup:
            times.append(time.perf_counter() - t0)
    sec = sum(times) / len(times)
    return h["batch"] / sec, dict(kind=kind, cores=cores, seconds_per_step=sec, first=first,
                                  sample=f"{len(times)} {sample}", same_config=config != 4)


def run_reference(args):
    if int(os.environ.get("RANK", "0")) != 0:
        return
    if args.config in (2, 5):
        return run_sweep(args, reference_only=True)
    wl = W.plan_workload(args.config)
    if args.config == 1:
        steps, warmup = min(args.steps * 50, 2000), min(args.warmup * 10, 100)   # a step is a fraction of a millisecond
    else:
        steps, warmup = min(args.steps, 60), min(args.warmup, 10)                  # a step is 2-10 s of host time
    ups, info = cpu_plan_sample(args.config, steps, warmup)
    emit({
        "impl": "reference", "metric": unit_metric(wl), "value": ups, "unit": wl.unit + "/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup,
        "ms_per_step": info["seconds_per_step"] * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": wl.description, "timed": info["sample"]},
        "cpu_baseline": {"value": ups, "unit": wl.unit + "/s", "cores": info["cores"],
                         "kind": info["kind"], "sample": info["sample"]},
        "e2e": {"value": ups, "unit": wl.unit + "/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    })


def gpu_vs_cpu_first_step(first: dict, device: int, graphs: bool, tolerance: float) -> dict:
    """Outside every timed region: the engine exactly as the timed loop drives it
    (graphs, fusions, tensor-core kernels) on the CPU sample's plan and first
    batch, its loss and gradient block against the reference CPU executor's."""
    from see_ai_b200.engine import Engine
    eng = Engine(device)
    eng.load(first["blob"])
    eng.set_use_graphs(graphs)
    x, y = first["batch"]
    eng.stage_batch(x, y)
    eng.train_forward_backward(True)
    loss = eng.read_loss()
    off, nbytes = eng.gradient_block()
    got = eng.read_arena(off, nbytes).view(np.float32).astype(np.float64)
    eng.close()
    want = first["grad"].astype(np.float64)
    rms = float(np.sqrt(np.mean((got - want) ** 2)) / np.sqrt(np.mean(want ** 2)))
    worst = float(np.abs(got - want).max() / np.abs(want).max())
    return {"plan": "the CPU sample's plan, first step, same batch on both sides",
            "loss_gpu": loss, "loss_cpu": first["loss"],
            "loss_rel_err": abs(loss - first["loss"]) / abs(first["loss"]),
            "gradient_block_rel_rms": rms, "gradient_block_max_err_over_max": worst,
            "tolerance": tolerance,
            "within_tolerance": bool(worst <= tolerance and abs(loss - first["loss"]) <= tolerance * abs(first["loss"]))}


# ---- plan workloads on the engine (configurations 1, 3, 4) ------------------------------------

def run_plan(args):
    import torch
    import torch.distributed as dist
    from see_ai_b200 import dp
    from see_ai_b200.engine import Engine

    wl = W.plan_workload(args.config)
    reduced = args.config == 4 and (args.layers or args.batch_seqs)
    if reduced:   # same kernels on a case small enough to sit under a profiler; never a headline number
        wl = W.Int8DecoderWorkload(layers=args.layers or 12, batch_seqs=args.batch_seqs or 64)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit("bench.py --gpus N > 1 must be launched with torch.distributed.run")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    units = wl.global_units // wl.seq
    if units % world:
        raise SystemExit(f"{units} {'sequences' if wl.seq > 1 else 'rows'} do not split over {world} ranks")
    blob = wl.build(world)
    plan = P.Plan(blob)
    rows = plan.header["batch"]
    train = plan.section("train")

    stream = torch.cuda.Stream()
    eng = Engine(local_rank)
    with torch.cuda.stream(stream):
        eng.backend.set_stream(stream.cuda_stream)
        eng.load(blob)
        del blob
        eng.set_horizon(plan.header["default_steps"])
        exchange = dp.GradientExchange(eng) if world > 1 else None
        batches = wl.batches(rows, 4, seed=1000 + rank)
        ex0 = torch.cuda.Event(enable_timing=True)
        ex1 = torch.cuda.Event(enable_timing=True)
        exchange_ms = []

        def step(stage: bool, i: int, time_exchange: bool = False) -> None:
            if stage:
                eng.stage_batch(*batches[i % len(batches)])
            eng.train_forward_backward(True)
            if exchange:
                if time_exchange:
                    ex0.record(stream)
                exchange.exchange()
                if time_exchange:
                    ex1.record(stream)
            eng.train_optimizer()
            if exchange and time_exchange:
                ex1.synchronize()
                exchange_ms.append(ex0.elapsed_time(ex1))

        # -- one profiled eager step: per-instruction CUDA events (the profiler hook) --
        # (after one unprofiled step, so one-time weight conversion and module loading are not in it)
        eng.stage_batch(*batches[0])
        step(False, 0)
        eng.backend.set_profiling(True)
        c0 = eng.backend.counters()
        step(False, 0)
        loss0 = eng.read_loss()
        prof8 = eng.backend.take_profile(with_absorbed=True)
        eng.backend.set_profiling(False)
        c1 = eng.backend.counters()
        launches_per_step = c1.kernel_launches - c0.kernel_launches
        tensor = [(m, n, k, kms, absorbed) for (_op, _i, _ms, m, n, k, kms, absorbed) in prof8 if kms > 0]
        gemm_flops = sum(2.0 * m * n * k for (m, n, k, _t, _a) in tensor)
        gemm_ms = sum(t for (*_s, t, _a) in tensor)
        plain = [(m, n, k, t) for (m, n, k, t, a) in tensor if a == 0]
        plain_flops = sum(2.0 * m * n * k for (m, n, k, _t) in plain)
        plain_ms = sum(t for (*_s, t) in plain)
        by_op, hbm = {}, {}
        # The records of the two ranges (forward + backward, optimizer) in program order.  A kernel
        # that also did following instructions (an absorbed add, the loss backward inside the loss
        # forward's row pass) is credited with their bytes too and listed as "<opcode>+absorbed";
        # the absorbed instructions launch nothing (their records hold event overhead only).
        hold = None   # the last bandwidth-bound record that absorbed others, still collecting their bytes
        for rec, ins in zip(prof8, train):
            op, ms, absorbed = rec[0], rec[2], rec[7]
            name = P.OP_NAMES.get(op, str(op))
            by_op[name] = by_op.get(name, 0.0) + ms
            _fl, nbytes = W.algorithmic_work(ins)
            if nbytes <= 0 or ms <= 0:
                continue
            launched = nbytes / 1e9 / (ms * 1e-3) < 1.5 * peaks()["hbm_gbs"]
            if not launched:
                if hold is not None and hold[1] > 0:
                    hold[0][1] += nbytes
                    hold[1] -= 1
                continue
            e = hbm.setdefault(name + ("+absorbed" if absorbed else ""), [0.0, 0.0, 0])
            e[0] += ms; e[1] += nbytes; e[2] += 1
            hold = [e, absorbed] if absorbed else None
        profiled_ms = sum(by_op.values())
        if args.dump_profile and rank == 0:
            with open(args.dump_profile, "w") as f:
                json.dump([{"index": i, "op": P.OP_NAMES.get(r[0], str(r[0])), "ms": r[2], "m": r[3], "n": r[4],
                            "k": r[5], "tensor_kernel_ms": r[6], "absorbed": r[7]} for i, r in enumerate(prof8)], f)
        for _ in range(3 if exchange else 0):
            step(False, 0, time_exchange=True)

        eng.set_use_graphs(not args.no_graphs)
        for i in range(args.warmup):
            step(False, i)
        eng.read_loss()

        def timed(stage: bool):
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            sampler = ClockSampler(local_rank)
            if rank == 0:
                sampler.start()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            last = 0.0
            for i in range(args.steps):
                step(stage, i)
                if stage:
                    last = eng.read_loss()   # the device->host read of the step's result
            e1.record(stream)
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            ms = e0.elapsed_time(e1)
            clocks = sampler.stop() if rank == 0 else None
            if world > 1:
                t = torch.tensor([ms], device="cuda")
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t.item())
            return ms, clocks, last

        ms_resident, clocks, _ = timed(False)
        ms_e2e, _, last_loss = timed(True)
        final_loss = eng.read_loss()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    pk = peaks()
    value = wl.global_units * args.steps / (ms_resident * 1e-3)
    e2e = wl.global_units * args.steps / (ms_e2e * 1e-3)
    x0, y0 = batches[0]
    h2d = x0.nbytes + y0.nbytes
    line = {
        "metric": unit_metric(wl), "value": value, "unit": wl.unit + "/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_resident / args.steps, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
        "config": {"workload": wl.description, "rows_per_gpu": rows, "parallelism": f"dp{world}",
                   "l2_policy": ("inputs larger than L2 (the step streams >10 GB through HBM)" if args.config == 4 else
                                 "a step's working set is rewritten every step; no separate flush"),
                   "cuda_graphs": not args.no_graphs, **({"reduced_case_for_profiling": True} if reduced else {})},
        "e2e": {"value": e2e, "unit": wl.unit + "/s", "h2d_bytes_per_step": h2d * world,
                "d2h_bytes_per_step": 4 * world, "ms_per_step": ms_e2e / args.steps},
        "gpu_launches": int(launches_per_step * args.steps),
        "clocks": clocks,
        "profile_ms_per_step": {k: round(v, 3) for k, v in sorted(by_op.items(), key=lambda kv: -kv[1])},
        "profiled_step_ms": profiled_ms,
        "hbm_kernels": {k: {"launches": n, "ms": round(ms, 4), "algorithmic_GB": round(b / 1e9, 4),
                            "GB_per_s": round(b / 1e9 / (ms * 1e-3), 1),
                            "frac_of_measured_copy": round(b / 1e9 / (ms * 1e-3) / pk["hbm_gbs"], 3)}
                        for k, (ms, b, n) in sorted(hbm.items(), key=lambda kv: -kv[1][0])},
        "loss": {"first": loss0, "last": final_loss},
        "counters": {"relaxed_executions_per_step": int(c1.relaxed_executions - c0.relaxed_executions),
                     "split_executions_per_step": int(c1.split_executions - c0.split_executions),
                     "fused_dispatches_per_step": int(c1.fused_dispatches - c0.fused_dispatches)},
    }
    if exchange_ms:
        line["exchange_ms_per_step"] = statistics.median(exchange_ms)
    achieved = gemm_flops / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else 0.0
    if args.config == 4:
        peak = pk["bf16_tflops_sustained"]
        plain_achieved = plain_flops / (plain_ms * 1e-3) / 1e12 if plain_ms > 0 else 0.0
        line["roofline"] = {
            "bound": "tensor", "kernel": "UmmaGemmPersistentKernel (tcgen05 bf16, relaxed frozen-weight GEMMs)",
            "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak if peak else None,
            "peak_source": pk["source"] + " (bf16 sustained)",
            # dram__bytes_read.sum + dram__bytes_write.sum of one launch of the most frequent shape
            # (ncu capture summarised under profiles/); a constant, not measured here.
            "traffic": NCU_TRAFFIC_BYTES, "traffic_note": NCU_TRAFFIC_NOTE,
            "launches_per_step": len(tensor), "kernel_ms_per_step": gemm_ms,
            # The headline figure counts every launch, including those whose epilogue also does a
            # following GELU / GELU backward / add, or carries an adapter's low-rank term (extra
            # traffic, instructions and K blocks, no extra credited FLOPs).  `plain` is the same
            # ratio over the launches that carry nothing else.
            "plain": {"launches_per_step": len(plain), "kernel_ms_per_step": plain_ms, "achieved": plain_achieved,
                      "frac": plain_achieved / peak if peak and plain_achieved else None}}
    elif args.config == 3:
        peak = pk["bf16_tflops_sustained"] / 6.0
        line["roofline"] = {
            "bound": "tensor", "kernel": "UmmaGemmKernel / UmmaGemmPersistentKernel over bf16 pieces (exact f32 products "
                                         "as six bf16 piece products)",
            "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak if peak else None,
            "peak_source": pk["source"] + " (bf16 sustained / 6: six piece products per f32 product)",
            "traffic": None, "launches_per_step": len(tensor), "kernel_ms_per_step": gemm_ms}
    else:
        # 25 instructions of a few KB to a few hundred KB each: the step is launch latency.
        total_bytes = sum(W.algorithmic_work(i)[1] for i in train) + \
            sum(4.0 * (i.out[0] * i.out[2] + i.out[2] * i.out[1] + i.out[0] * i.out[1]) for i in train
                if W.algorithmic_work(i)[0] > 0)
        ach = total_bytes / 1e9 / (ms_resident / args.steps * 1e-3)
        line["roofline"] = {
            "bound": "hbm", "kernel": "the whole step (every kernel of it moves kilobytes: launch latency, not "
                                      "bandwidth, is what is measured)",
            "achieved": ach, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": ach / pk["hbm_gbs"],
            "peak_source": pk["source"] + " (copy)", "traffic": None, "launches_per_step": int(launches_per_step)}
    if world == 1 and not args.no_cpu_baseline and not reduced:
        ups, info = cpu_plan_sample(args.config, 200 if args.config == 1 else 3, 20 if args.config == 1 else 1)
        line["cpu_baseline"] = {"value": ups, "unit": wl.unit + "/s", "cores": info["cores"],
                                "kind": info["kind"], "sample": info["sample"]}
        line["parity"] = gpu_vs_cpu_first_step(info["first"], local_rank, not args.no_graphs,
                                               2e-2 if args.config == 4 else 1e-5)
    emit(line)
    if world > 1:
        dist.destroy_process_group()


# ---- the two sweeps (configurations 2 and 5) through the backend seam -------------------------

def _device_ms(be, prog, rounds: int):
    """Median over `rounds` of the summed per-instruction device times of one run."""
    totals, per_op = [], {}
    for _ in range(rounds):
        be.set_profiling(True)
        be.run(prog)
        recs = be.take_profile(with_absorbed=True)
        be.set_profiling(False)
        totals.append(sum(r[2] for r in recs))
        per_op = {}
        for r in recs:
            per_op[P.OP_NAMES.get(r[0], str(r[0]))] = per_op.get(P.OP_NAMES.get(r[0], str(r[0])), 0.0) + r[2]
    return statistics.median(totals), per_op


def _cpu_ms(prog_instrs, arena, rodata, rounds: int = 1):
    ex, kind, cores = cpu_executor()
    a = arena.copy()
    ex.bind(a, rodata)
    best = None
    for _ in range(rounds):
        t0 = time.perf_counter()
        ex.run(prog_instrs)
        dt = (time.perf_counter() - t0) * 1e3
        best = dt if best is None else min(best, dt)
    return best, kind, cores, a


def run_sweep(args, reference_only: bool = False):
    from see_ai_b200 import backend as B
    if int(os.environ.get("RANK", "0")) != 0:
        return
    pk = peaks()
    rows = []
    cpu_info = None
    if args.config == 2:
        sizes = [int(s) for s in args.sizes.split(",")] if args.sizes else [512, 1024, 2048, 4096, 8192]
        dtypes = args.dtypes.split(",") if args.dtypes else ["f32", "bf16"]
        cases = [(S, dt) for S in sizes for dt in dtypes]
    else:
        seqs = [int(s) for s in args.sizes.split(",")] if args.sizes else [256, 512, 1024, 2048, 4096]
        dims = [int(d) for d in args.head_dims.split(",")] if args.head_dims else [64, 128]
        cases = [(S, d) for d in dims for S in seqs]
    headline = None
    clocks = None
    for case in cases:
        if args.config == 2:
            S, dt = case
            prog = W.gemm_step_program(S, relaxed=dt == "bf16")
            units, label = S, {"S": S, "dtype": dt}
            cpu_prog, cpu_units_scale = prog, 1.0
        else:
            S, d = case
            prog = W.attention_chain_program(8, S, 16, d, relaxed=True)
            units, label = 8 * S, {"S": S, "head_dim": d, "batch": 8, "heads": 16}
            # the CPU arm on a (batch, head) subset: units are independent per (b, h)
            sub_b, sub_h = (1, 2) if S <= 1024 else (1, 1)
            cpu_prog = W.attention_chain_program(sub_b, S, sub_h, d, relaxed=False)
            cpu_units_scale = (8 * 16) / (sub_b * sub_h)
        cpu_ok = S <= args.cpu_max_size
        row = dict(label)
        row["algorithmic_gflop"] = round(prog.flops / 1e9, 3)
        if not reference_only:
            be = B.CudaBackend(0)
            be.set_coherence(B.COHERENCE_LAZY)
            be.bind(prog.arena, prog.rodata)
            for _ in range(max(1, args.warmup)):
                be.run(prog.instrs)
            sampler = ClockSampler(0)
            sampler.start()
            ms, per_op = _device_ms(be, prog.instrs, max(3, args.steps))
            # end to end: the step's host inputs uploaded, one result word read back, wall clock
            first = "A" if args.config == 2 else "q"
            nbytes = (4 * S * S) if args.config == 2 else 4 * 8 * S * 16 * case[1]
            n_e2e = max(2, min(args.steps, 5))
            t0 = time.perf_counter()
            for _ in range(n_e2e):
                be.host_wrote(prog.refs[first], nbytes)
                be.run(prog.instrs)
                be.host_needs(prog.refs["dA" if args.config == 2 else "dv"], 4)
            e2e_ms = (time.perf_counter() - t0) * 1e3 / n_e2e
            clocks = sampler.stop()
            c = be.counters()
            be.close()
            tflops = prog.flops / (ms * 1e-3) / 1e12
            peak = pk["bf16_tflops_sustained"] / (6.0 if (args.config == 2 and case[1] == "f32") else 1.0)
            row.update(ms=round(ms, 4), tflops=round(tflops, 2), frac_of_peak=round(tflops / peak, 4),
                       units_per_s=units / (ms * 1e-3), e2e_ms=round(e2e_ms, 3), h2d_bytes=nbytes,
                       per_opcode_ms={k: round(v, 4) for k, v in per_op.items()},
                       tensor_core_instructions=int(c.relaxed_executions + c.split_executions))
            headline = (row, peak, units, nbytes)
        if cpu_ok and not args.no_cpu_baseline:
            cms, kind, cores, _a = _cpu_ms(cpu_prog.instrs, cpu_prog.arena, cpu_prog.rodata)
            cms *= cpu_units_scale
            row.update(cpu_ms=round(cms, 2), cpu_units_per_s=units / (cms * 1e-3))
            cpu_info = dict(kind=kind, cores=cores)
            if "ms" in row:
                row["speedup_vs_cpu"] = round(cms / row["ms"], 1)
        rows.append(row)
    what = ("isolated GEMM training step around a frozen S x S weight with a rank-8 adapter (C = A W, dA = dC W^T, "
            "A^T dC and the six rank-8 products), f32 (exact opcodes) and bf16 (relaxed permission)") if args.config == 2 \
        else "causal attention forward + backward (tiled family, relaxed permission), batch 8, 16 heads"
    if reference_only:
        timed_rows = [r for r in rows if "cpu_ms" in r]
        if not timed_rows:
            emit({"impl": "reference", "unavailable": "no sweep case within --cpu-max-size"})
            return
        last = timed_rows[-1]
        emit({"impl": "reference", "metric": METRIC, "value": last["cpu_units_per_s"], "unit": "tokens/s",
              "n_gpus": args.gpus, "steps": 1, "warmup": 0, "ms_per_step": last["cpu_ms"], "higher_is_better": True,
              "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
              "config": {"workload": what, "timed": f"the largest case the CPU arm runs: {last}"},
              "cpu_baseline": {"value": last["cpu_units_per_s"], "unit": "tokens/s", "cores": cpu_info["cores"],
                               "kind": cpu_info["kind"], "sample": "one step per case; attention on a (batch, head) "
                                                                   "subset scaled to the full batch"},
              "e2e": {"value": last["cpu_units_per_s"], "unit": "tokens/s", "h2d_bytes_per_step": 0,
                      "d2h_bytes_per_step": 0}, "sweep": rows})
        return
    row, peak, units, nbytes = headline
    line = {
        "metric": METRIC, "value": row["units_per_s"], "unit": "tokens/s", "n_gpus": 1, "steps": max(3, args.steps),
        "warmup": max(1, args.warmup), "ms_per_step": row["ms"], "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": what, "headline_case": {k: row[k] for k in row if k in ("S", "dtype", "head_dim")},
                   "l2_policy": "operands larger than L2 at the headline case; a step rewrites its working set",
                   "timing": "sum of per-instruction CUDA-event times of one step (median over steps)"},
        "e2e": {"value": units / (row["e2e_ms"] * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": nbytes,
                "d2h_bytes_per_step": 4, "ms_per_step": row["e2e_ms"]},
        "gpu_launches": None, "clocks": clocks,
        "roofline": {"bound": "tensor", "kernel": "tcgen05 GEMM" if args.config == 2 else "tcgen05 attention",
                     "achieved": row["tflops"], "peak": peak, "unit": "TFLOP/s", "frac": row["frac_of_peak"],
                     "peak_source": pk["source"] + " (bf16 sustained)", "traffic": None},
        "sweep": rows,
    }
    if cpu_info:
        with_cpu = [r for r in rows if "cpu_ms" in r]
        line["cpu_baseline"] = {"value": with_cpu[-1]["cpu_units_per_s"], "unit": "tokens/s", "cores": cpu_info["cores"],
                                "kind": cpu_info["kind"],
                                "sample": f"one step of each case up to S = {args.cpu_max_size} (see sweep)"}
    emit(line)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", type=int, default=4, choices=[1, 2, 3, 4, 5])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="cuda", choices=["cuda", "reference"])
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--sizes", default="", help="configs 2 and 5: comma-separated S values")
    ap.add_argument("--dtypes", default="", help="config 2: f32,bf16")
    ap.add_argument("--head-dims", default="", help="config 5: 64,128")
    ap.add_argument("--cpu-max-size", type=int, default=1024, help="configs 2 and 5: largest S the CPU arm runs")
    ap.add_argument("--dump-profile", default="", help="config 4: write the profiled step's per-instruction records here")
    ap.add_argument("--layers", type=int, default=0, help="config 4 only: a REDUCED case for profiler captures")
    ap.add_argument("--batch-seqs", type=int, default=0, help="config 4 only: a REDUCED case for profiler captures")
    args = ap.parse_args()
    # stdout carries exactly one JSON line.  Libraries underneath (NCCL's version
    # banner, for one) write to file descriptor 1 behind Python's back, so the
    # descriptor itself is pointed at stderr for the run and the line goes to a
    # saved copy of the real stdout.
    global _RESULT_FD
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)
    if args.impl == "reference":
        run_reference(args)
    elif args.config in (2, 5):
        run_sweep(args)
    else:
        run_plan(args)


_RESULT_FD = None


def emit(line: dict) -> None:
    data = (json.dumps(line) + "\n").encode()
    os.write(_RESULT_FD if _RESULT_FD is not None else 1, data)


if __name__ == "__main__":
    main()
