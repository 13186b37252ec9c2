"""Micro-benchmark of one frozen-weight GEMM instruction through the backend.

    python -m see_ai_b200.probe_gemm --m 32768 --n 3072 --k 768 [--kind nn_q8|nt_q8|nn_f32]
                                      [--exact] [--iters 20]

Builds a one-instruction program (the instruction the compiler emits for a
quantised projection: kGemmNNQ8 / kGemmNTQ8 with per-column scales and the
relaxed permission, or an f32 kGemmNN), runs it `iters` times with the
per-instruction CUDA-event profile on, and prints one JSON line: time of the
whole instruction, time of the tensor-core kernel alone, TFLOP/s of each.
Small enough to sit under a profiler; the same launch the engine makes.
"""

from __future__ import annotations

import argparse
import json

import numpy as np

from . import backend as B
from . import plan as P


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=3072)
    ap.add_argument("--k", type=int, default=768)
    ap.add_argument("--kind", default="nn_q8", choices=["nn_q8", "nt_q8", "nn_f32"])
    ap.add_argument("--exact", action="store_true", help="withhold the relaxed permission")
    ap.add_argument("--iters", type=int, default=20)
    args = ap.parse_args()
    M, N, K = args.m, args.n, args.k
    rng = np.random.default_rng(1)

    def al(n):
        return (n + 63) // 64 * 64

    a_off, c_off = 0, al(4 * M * K)
    arena = np.zeros(c_off + al(4 * M * N), dtype=np.uint8)
    arena[:4 * M * K] = rng.standard_normal(M * K, dtype=np.float32).view(np.uint8)
    flags = 0 if args.exact else P.FLAG_RELAXED
    if args.kind == "nn_f32":
        w = (rng.standard_normal((K, N), dtype=np.float32) * np.float32(0.02))
        ro = w.view(np.uint8).reshape(-1)
        ins = P.Instr(P.Op.GEMM_NN, flags, 0, (a_off, P.RODATA_BIT, c_off, P.NULL_REF), (M, N, K))
    else:
        q = rng.integers(-127, 128, size=K * N, dtype=np.int8)
        scales = (rng.random(N if args.kind == "nn_q8" else K) * 0.01 + 1e-3).astype(np.float32)
        s_off = al(q.size)
        ro = np.zeros(s_off + scales.nbytes, dtype=np.uint8)
        ro[:q.size] = q.view(np.uint8)
        ro[s_off:] = scales.view(np.uint8)
        op = P.Op.GEMM_NN_Q8 if args.kind == "nn_q8" else P.Op.GEMM_NT_Q8
        ins = P.Instr(op, flags | P.FLAG_Q8_COL_SCALE, 0,
                      (a_off, P.RODATA_BIT, c_off, P.RODATA_BIT | s_off), (M, N, K))

    be = B.CudaBackend(0)
    be.set_coherence(B.COHERENCE_LAZY)
    be.bind(arena, ro)
    prog = [ins] * args.iters
    be.run(prog[:2])            # converts the weight once; warms the kernel
    be.set_profiling(True)
    be.run(prog)
    recs = be.take_profile()
    c = be.counters()
    be.close()
    ms = sorted(r[2] for r in recs)
    kms = sorted(r[6] for r in recs if r[6] > 0)
    flops = 2.0 * M * N * K
    med = ms[len(ms) // 2]
    out = {"m": M, "n": N, "k": K, "kind": args.kind, "relaxed": not args.exact,
           "instruction_ms_median": med, "instruction_tflops": flops / (med * 1e-3) / 1e12,
           "relaxed_executions": int(c.relaxed_executions)}
    if kms:
        kmed = kms[len(kms) // 2]
        out.update(kernel_ms_median=kmed, kernel_tflops=flops / (kmed * 1e-3) / 1e12)
    print(json.dumps(out))


if __name__ == "__main__":
    main()
