"""Micro-benchmark of the six rank-r adapter products of one LoRA projection
(t = x A, y += s t B, dT = s dY B^T, dX += dT A^T, dA = x^T dT, dB = s t^T dY) as
the plan carries them (exact opcodes kGemmNN / kGemmNT / kGemmTN), through the
backend's C ABI.

    python -m see_ai_b200.probe_adapters [--rows 32768] [--width 768] [--rank 16] [--rounds 3]

Runs the six instructions `rounds` times, the last round with the
per-instruction CUDA-event profile on, and prints one line per product.  Small
enough to sit under a profiler.
"""

from __future__ import annotations

import argparse

import numpy as np

from . import backend as B
from . import plan as P


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=32768)
    ap.add_argument("--width", type=int, default=768)
    ap.add_argument("--rank", type=int, default=16)
    ap.add_argument("--rounds", type=int, default=3)
    args = ap.parse_args()
    M, D, r = args.rows, args.width, args.rank
    rng = np.random.default_rng(0)

    def al(n):
        return (n + 63) // 64 * 64

    offs, size = {}, 0
    for name, n in [("x", M * D), ("dy", M * D), ("y", M * D), ("dx", M * D), ("t", M * r), ("dt", M * r),
                    ("A", D * r), ("B", r * D), ("gA", D * r), ("gB", r * D)]:
        offs[name] = size
        size = al(size + 4 * n)
    arena = np.zeros(size, dtype=np.uint8)
    for name in ("x", "dy", "y", "dx"):
        arena[offs[name]:offs[name] + 4 * M * D] = rng.standard_normal(M * D, dtype=np.float32).view(np.uint8)
    for name in ("A", "B"):
        arena[offs[name]:offs[name] + 4 * D * r] = \
            (rng.standard_normal(D * r, dtype=np.float32) * np.float32(0.03)).view(np.uint8)
    f, o = P.f32_bits, offs
    prog = [
        P.Instr(P.Op.GEMM_NN, 0, 0, (o["x"], o["A"], o["t"], P.NULL_REF), (M, r, D)),
        P.Instr(P.Op.GEMM_NN, P.FLAG_GEMM_ADDEND, f(2.0), (o["t"], o["B"], o["y"], o["y"]), (M, D, r)),
        P.Instr(P.Op.GEMM_NT, 0, f(2.0), (o["dy"], o["B"], o["dt"], P.NULL_REF), (M, r, D)),
        P.Instr(P.Op.GEMM_NT, P.FLAG_GEMM_ADDEND, 0, (o["dt"], o["A"], o["dx"], o["dx"]), (M, D, r)),
        P.Instr(P.Op.GEMM_TN, 0, 0, (o["x"], o["dt"], o["gA"], P.NULL_REF), (D, r, M)),
        P.Instr(P.Op.GEMM_TN, 0, f(2.0), (o["t"], o["dy"], o["gB"], P.NULL_REF), (r, D, M)),
    ]
    names = ["t = x A", "y += s t B", "dT = s dY B^T", "dX += dT A^T", "dA = x^T dT", "dB = s t^T dY"]
    be = B.CudaBackend(0)
    be.set_coherence(B.COHERENCE_LAZY)
    be.bind(arena, np.zeros(64, dtype=np.uint8))
    for _ in range(max(0, args.rounds - 1)):
        be.run(prog)
    be.set_profiling(True)
    be.run(prog)
    for name, rec in zip(names, be.take_profile()):
        print("%-14s %-8s M=%d N=%d K=%d  %.1f us" % (name, P.OP_NAMES[rec[0]], rec[3], rec[4], rec[5], rec[2] * 1e3))
    be.close()


if __name__ == "__main__":
    main()
