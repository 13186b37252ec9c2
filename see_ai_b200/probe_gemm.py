"""Micro-benchmark of one frozen-weight GEMM instruction through the backend.

    python -m see_ai_b200.probe_gemm --m 32768 --n 3072 --k 768 [--kind nn_q8|nt_q8|nn_f32]
                                      [--exact] [--iters 20] [--absorb gelu|gelu_bwd|add]

Builds a one-instruction program (the instruction the compiler emits for a
quantised projection: kGemmNNQ8 / kGemmNTQ8 with per-column scales and the
relaxed permission, or an f32 kGemmNN), runs it `iters` times with the
per-instruction CUDA-event profile on, and prints one JSON line: time of the
whole instruction, time of the tensor-core kernel alone, TFLOP/s of each.
Small enough to sit under a profiler; the same launch the engine makes.

With --absorb the instruction is followed by the one its epilogue can do in lazy
coherence (a GELU whose output only a second relaxed GEMM reads, a GELU backward
likewise, an elementwise add), so the timed kernel is the product WITH the
absorbed work; `fused_dispatches` in the output says that it was.
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
    ap.add_argument("--absorb", default="none", choices=["none", "gelu", "gelu_bwd", "add"])
    args = ap.parse_args()
    M, N, K = args.m, args.n, args.k
    rng = np.random.default_rng(1)

    def al(n):
        return (n + 63) // 64 * 64

    a_off, c_off = 0, al(4 * M * K)
    x_off = c_off + al(4 * M * N)          # second operand of an absorbed GELU backward / add
    g_off = x_off + al(4 * M * N)          # the absorbed instruction's output
    o_off = g_off + al(4 * M * N)          # the consumer GEMM's output [M, 64]
    extra = args.absorb != "none"
    arena = np.zeros((o_off + al(4 * M * 64)) if extra else (c_off + al(4 * M * N)), dtype=np.uint8)
    arena[:4 * M * K] = rng.standard_normal(M * K, dtype=np.float32).view(np.uint8)
    if extra:
        arena[x_off:x_off + 4 * M * N] = rng.standard_normal(M * N, dtype=np.float32).view(np.uint8)
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

    unit, tail = [ins], []
    if extra:
        if args.kind == "nn_f32":
            raise SystemExit("--absorb wants a quantised kind")
        # The consumer of the absorbed instruction's output: a transposed int8 GEMM [M, 64, N].
        q2 = rng.integers(-127, 128, size=64 * N, dtype=np.int8)
        s2 = (rng.random(N) * 0.01 + 1e-3).astype(np.float32)
        q2_off = al(ro.size)
        s2_off = q2_off + al(q2.size)
        ro2 = np.zeros(s2_off + s2.nbytes, dtype=np.uint8)
        ro2[:ro.size] = ro
        ro2[q2_off:q2_off + q2.size] = q2.view(np.uint8)
        ro2[s2_off:] = s2.view(np.uint8)
        ro = ro2
        consumer = P.Instr(P.Op.GEMM_NT_Q8, P.FLAG_RELAXED | P.FLAG_Q8_COL_SCALE, 0,
                           (g_off, P.RODATA_BIT | q2_off, o_off, P.RODATA_BIT | s2_off), (M, 64, N))
        fill = lambda off: P.Instr(P.Op.FILL, 0, 0, (off, P.f32_bits(0.0)), (M * N, 0, 0))
        if args.absorb == "gelu":
            unit += [P.Instr(P.Op.GELU_FWD, 0, 0, (c_off, g_off), (M * N, 0, 0)), consumer]
            tail = [fill(g_off)]
        elif args.absorb == "gelu_bwd":
            unit += [P.Instr(P.Op.GELU_BWD, 0, 0, (c_off, x_off, g_off, P.NULL_REF), (M * N, 0, 0)), consumer]
            tail = [fill(c_off), fill(g_off)]
        else:
            unit += [P.Instr(P.Op.ADD_EW, 0, 0, (x_off, c_off, g_off, P.NULL_REF), (M * N, 0, 0))]
            tail = [fill(c_off)]

    be = B.CudaBackend(0)
    be.set_coherence(B.COHERENCE_LAZY)
    be.bind(arena, ro)
    prog = unit * args.iters + tail   # an intermediate is dead once the next round (or the tail) rewrites it
    be.run(unit * 2 + tail)     # converts the weights once; warms the kernels
    c0 = be.counters()
    be.set_profiling(True)
    be.run(prog)
    recs = [r for r in be.take_profile() if r[0] == ins.opcode and (r[3], r[4], r[5]) == (M, N, K)]
    c = be.counters()
    be.close()
    ms = sorted(r[2] for r in recs)
    kms = sorted(r[6] for r in recs if r[6] > 0)
    flops = 2.0 * M * N * K
    med = ms[len(ms) // 2]
    out = {"m": M, "n": N, "k": K, "kind": args.kind, "relaxed": not args.exact,
           "instruction_ms_median": med, "instruction_tflops": flops / (med * 1e-3) / 1e12,
           "relaxed_executions": int(c.relaxed_executions), "absorb": args.absorb,
           "fused_dispatches": int(c.fused_dispatches - c0.fused_dispatches)}
    if kms:
        kmed = kms[len(kms) // 2]
        out.update(kernel_ms_median=kmed, kernel_tflops=flops / (kmed * 1e-3) / 1e12)
    print(json.dumps(out))


if __name__ == "__main__":
    main()
