#!/usr/bin/env python3
"""Update-step throughput of the CUDA executor on the int8-weight decoder
(12 layers, d_model 768, 12 heads, FFN 3072, vocab 32000, seq 512, global batch
64 sequences, LoRA r16 on Q/K/V/O, relaxed bf16 frozen-weight GEMMs, AdamW).

    python bench.py --gpus N --steps K --warmup W          (N > 1: under torchrun)
    python bench.py --impl reference ...                   the reference CPU executor

One JSON line on stdout (rank 0).  `value` times K steps with the batch already
resident in HBM; `e2e` times the same K steps through the engine's public call
sequence with HOST buffers (stage_batch -> train -> read_loss), copies inside
the timed region.  `roofline` is the tensor-core GEMM kernel (the dominant
kernel): algorithmic 2*M*N*K FLOPs of every launch in a profiled step divided by
the CUDA-event time of those launches, against the measured bf16 peak.
`cpu_baseline` times the reference CPU executor on a bounded sample of the same
plan (one sequence instead of sixty-four).
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
from see_ai_b200 import synth  # noqa: E402

NCU_TRAFFIC_BYTES = 95.6e6
NCU_TRAFFIC_NOTE = ("ncu, one 32768x768x768 launch (93 of the step's 143 tensor-core GEMM launches): 51.7 MB read "
                    "+ 43.9 MB written; algorithmic 152 MB (A bf16 50 MB, W 1 MB, C f32 101 MB), part of C is "
                    "still in L2 when the kernel ends")
GLOBAL_SEQS = 64
SEQ = 512
METRIC = "update_step_tokens_per_s"
WORKLOAD = ("int8-weight decoder LoRA update: 12 layers, d_model 768, 12 heads, FFN 3072, vocab 32000, "
            "seq 512, global batch 64 sequences, LoRA r16 alpha 32 on Q/K/V/O, relaxed bf16 GEMMs, AdamW")


def decoder_config(batch_seqs: int) -> synth.DecoderConfig:
    return synth.DecoderConfig(layers=12, d_model=768, heads=12, ffn=3072, vocab=32000, seq=SEQ,
                               batch_seqs=batch_seqs, rank=16, alpha=32.0,
                               targets=("q", "k", "v", "o"), quantized=True, attention="tiled",
                               lr=1e-3, steps=1000, seed=7)


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


def synthetic_batches(rows: int, vocab: int, count: int, seed: int):
    rng = np.random.default_rng(seed)
    out = []
    for _ in range(count):
        rec = rng.integers(0, vocab, size=(rows // SEQ, SEQ + 1), dtype=np.int32)
        out.append((np.ascontiguousarray(rec[:, :-1]).reshape(-1), np.ascontiguousarray(rec[:, 1:]).reshape(-1)))
    return out


# ---- the reference arm: the reference's own CPU executor on a bounded sample --------

def cpu_sample(steps: int, warmup: int):
    """Steps of the same 12-layer plan at ONE sequence (512 tokens) through the
    reference CPU executor with every host thread.  Returns (tokens/s, info)."""
    import oracle
    kind = "reference" if oracle.have_ref() else "port"
    if kind == "port" and not oracle.have_oracle():
        oracle.build("oracle")
    cfg = decoder_config(1)
    plan = P.Plan(synth.build_decoder_plan(cfg))
    h = plan.header
    arena = plan.stage_arena()
    ex = oracle.RefExecutor() if kind == "reference" else oracle.OracleExecutor()
    cores = os.cpu_count() or 1
    if kind == "reference":
        ex.set_threads(cores)
        cores = ex.threads()
    else:
        cores = 1
    ex.bind(arena, np.frombuffer(plan.rodata, dtype=np.uint8).copy())
    batches = synthetic_batches(h["batch"], cfg.vocab, 2, seed=11)
    from see_ai_b200 import dp
    _bwd, opt_begin = dp.scan_phases(plan.train)
    g_off, g_bytes = dp.gradient_block(plan)
    times = []
    first = {}
    for s in range(warmup + steps):
        x, y = batches[s % 2]
        t0 = time.perf_counter()
        arena[h["input_ref"]:h["input_ref"] + x.nbytes] = x.view(np.uint8)
        arena[h["label_ref"]:h["label_ref"] + y.nbytes] = y.view(np.uint8)
        sp = oracle.step_params(lr=cfg.lr, step=s + 1)
        if s == 0:   # the first step in two ranges, so that its loss and gradient block can be kept
            ex.run(plan.train, sp, 0, opt_begin)
            first = dict(loss=float(arena[h["loss_ref"]:h["loss_ref"] + 4].view(np.float32)[0]),
                         grad=arena[g_off:g_off + g_bytes].view(np.float32).copy(), batch=(x, y))
            ex.run(plan.train, sp, opt_begin, len(plan.train))
        else:
            ex.run(plan.train, sp)
        if s >= warmup:
            times.append(time.perf_counter() - t0)
    sec = sum(times) / len(times)
    loss = float(arena[h["loss_ref"]:h["loss_ref"] + 4].view(np.float32)[0])
    return h["batch"] / sec, dict(kind=kind, cores=int(cores), seconds_per_step=sec, loss=loss, first=first,
                                  sample=f"{len(times)} optimizer step(s) of the same 12-layer plan at "
                                         f"1 sequence ({h['batch']} tokens) instead of {GLOBAL_SEQS}")


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, warmup = min(args.steps, 60), min(args.warmup, 10)   # a step is about 2-10 s of host time
    tps, info = cpu_sample(steps, warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": tps, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup,
        "ms_per_step": info["seconds_per_step"] * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "timed": info["sample"]},
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": info["cores"],
                         "kind": info["kind"], "sample": info["sample"]},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    emit(line)


def gpu_vs_cpu_first_step(first: dict, device: int, graphs: bool) -> dict:
    """Outside every timed region: the engine exactly as the timed loop drives it
    (graphs, fusions, tensor-core kernels) on the CPU sample's plan and first
    batch, its loss and gradient block against the reference CPU executor's."""
    from see_ai_b200.engine import Engine
    cfg = decoder_config(1)
    eng = Engine(device)
    eng.load(synth.build_decoder_plan(cfg))
    eng.set_horizon(cfg.steps)
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
    return {"plan": "the benchmark's plan at 1 sequence, first step, same batch on both sides",
            "loss_gpu": loss, "loss_cpu": first["loss"],
            "loss_rel_err": abs(loss - first["loss"]) / abs(first["loss"]),
            "gradient_block_rel_rms": rms, "gradient_block_max_err_over_max": worst,
            "tolerance": 2e-2, "within_tolerance": bool(rms <= 2e-2 and abs(loss - first["loss"]) <= 2e-2 * abs(first["loss"]))}


# ---- our arm ---------------------------------------------------------------------------

def run_cuda(args):
    import torch
    import torch.distributed as dist
    from see_ai_b200 import dp
    from see_ai_b200.engine import Engine

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("bench.py --gpus N > 1 must be launched with torch.distributed.run")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    if GLOBAL_SEQS % world:
        raise SystemExit("global batch of 64 sequences does not split over this many ranks")
    cfg = decoder_config(GLOBAL_SEQS // world)
    blob = synth.build_decoder_plan(cfg)
    rows = cfg.rows

    stream = torch.cuda.Stream()
    eng = Engine(local_rank)
    with torch.cuda.stream(stream):
        eng.backend.set_stream(stream.cuda_stream)
        eng.load(blob)
        del blob
        eng.set_horizon(cfg.steps)
        exchange = dp.GradientExchange(eng) if world > 1 else None
        batches = synthetic_batches(rows, cfg.vocab, 4, seed=1000 + rank)

        def step(stage: bool, i: int) -> None:
            if stage:
                eng.stage_batch(*batches[i % len(batches)])
            eng.train_forward_backward(True)
            if exchange:
                exchange.exchange()
            eng.train_optimizer()

        # -- one profiled eager step: per-instruction CUDA events (the profiler hook) --
        # (after one unprofiled step, so one-time weight conversion and module loading are not in it)
        eng.stage_batch(*batches[0])
        step(False, 0)
        eng.backend.set_profiling(True)
        c0 = eng.backend.counters()
        step(False, 0)
        loss0 = eng.read_loss()
        prof8 = eng.backend.take_profile(with_absorbed=True)
        prof = [r[:7] for r in prof8]
        eng.backend.set_profiling(False)
        launches_per_step = eng.backend.counters().kernel_launches - c0.kernel_launches
        gemm_flops = sum(2.0 * m * n * k for (_op, _i, _ms, m, n, k, kms) in prof if kms > 0)
        gemm_ms = sum(kms for (*_r, kms) in prof if kms > 0)
        gemm_launches = sum(1 for (*_r, kms) in prof if kms > 0)
        # The same over the launches whose epilogue carries no absorbed instruction
        # (an absorbed GELU or add is HBM work the FLOP count does not see).
        plain = [(m, n, k, kms) for (_op, _i, _ms, m, n, k, kms, absorbed) in prof8 if kms > 0 and absorbed == 0]
        plain_flops = sum(2.0 * m * n * k for (m, n, k, _t) in plain)
        plain_ms = sum(t for (*_s, t) in plain)
        by_op = {}
        for (op, _i, ms, *_rest) in prof:
            by_op[P.OP_NAMES.get(op, str(op))] = by_op.get(P.OP_NAMES.get(op, str(op)), 0.0) + ms
        profiled_ms = sum(by_op.values())

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
    tokens = GLOBAL_SEQS * SEQ
    value = tokens * args.steps / (ms_resident * 1e-3)
    e2e = tokens * args.steps / (ms_e2e * 1e-3)
    achieved = gemm_flops / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else 0.0
    plain_achieved = plain_flops / (plain_ms * 1e-3) / 1e12 if plain_ms > 0 else 0.0
    peak = pk["bf16_tflops_sustained"]
    h2d = 2 * rows * 4
    line = {
        "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_resident / args.steps, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "rows_per_gpu": rows, "parallelism": f"dp{world}",
                   "l2_policy": "inputs larger than L2 (the step streams >10 GB through HBM)",
                   "cuda_graphs": not args.no_graphs},
        "e2e": {"value": e2e, "unit": "tokens/s", "h2d_bytes_per_step": h2d * world,
                "d2h_bytes_per_step": 4 * world, "ms_per_step": ms_e2e / args.steps},
        "gpu_launches": int(launches_per_step * args.steps),
        "clocks": clocks,
        "roofline": {"bound": "tensor", "kernel": "UmmaGemmPersistentKernel (tcgen05 bf16, relaxed frozen-weight GEMMs)",
                     "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                     "frac": achieved / peak if peak else None,
                     "peak_source": pk["source"] + " (bf16 sustained)",
                     # dram__bytes_read.sum + dram__bytes_write.sum of one launch of the most frequent
                     # shape (ncu capture summarised under profiles/); a constant, not measured here.
                     "traffic": NCU_TRAFFIC_BYTES, "traffic_note": NCU_TRAFFIC_NOTE,
                     "launches_per_step": gemm_launches, "kernel_ms_per_step": gemm_ms,
                     # The headline figure counts every launch, including those whose epilogue
                     # also does a following GELU / GELU backward / add (extra HBM traffic and
                     # instructions, no extra FLOPs).  `plain` is the same ratio over the
                     # launches that carry nothing else.
                     "plain": {"launches_per_step": len(plain), "kernel_ms_per_step": plain_ms,
                               "achieved": plain_achieved,
                               "frac": plain_achieved / peak if peak and plain_achieved else None}},
        "profile_ms_per_step": {k: round(v, 3) for k, v in sorted(by_op.items(), key=lambda kv: -kv[1])},
        "profiled_step_ms": profiled_ms,
        "loss": {"first": loss0, "last": final_loss},
    }
    if world == 1 and not args.no_cpu_baseline:
        tps, info = cpu_sample(4, 1)   # about 10-25 s of host time
        line["cpu_baseline"] = {"value": tps, "unit": "tokens/s", "cores": info["cores"],
                                "kind": info["kind"], "sample": info["sample"]}
        line["parity"] = gpu_vs_cpu_first_step(info["first"], local_rank, not args.no_graphs)
    emit(line)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="cuda", choices=["cuda", "reference"])
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
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
    else:
        run_cuda(args)


_RESULT_FD = None


def emit(line: dict) -> None:
    data = (json.dumps(line) + "\n").encode()
    os.write(_RESULT_FD if _RESULT_FD is not None else 1, data)


if __name__ == "__main__":
    main()
