"""Micro-benchmark of the tiled attention opcodes (forward, dQ, dK, dV) with the
relaxed permission, i.e. the tensor-core kernels, through the backend's C ABI.

    python -m see_ai_b200.probe_attention [--batch 64] [--seq 512] [--heads 12] [--head-dim 64] [--rounds 3]

Runs the chain `rounds` times, the last round with the per-instruction
CUDA-event profile on (operand packing is part of an instruction's time), and
prints one line per opcode.  Small enough to sit under a profiler.
"""

from __future__ import annotations

import argparse

import numpy as np

from . import backend as B
from . import plan as P


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--seq", type=int, default=512)
    ap.add_argument("--heads", type=int, default=12)
    ap.add_argument("--head-dim", type=int, default=64)
    ap.add_argument("--rounds", type=int, default=3)
    args = ap.parse_args()
    Bq, S, H, d = args.batch, args.seq, args.heads, args.head_dim
    td = Bq * S * H * d
    rng = np.random.default_rng(0)

    def al(n):
        return (n + 63) // 64 * 64

    offs, size = {}, 0
    for name in ("q", "k", "v", "do", "o", "dq", "dk", "dv"):
        offs[name] = size
        size = al(size + 4 * td)
    offs["stats"] = size
    size = al(size + 16 * Bq * H * S)
    arena = np.zeros(size, dtype=np.uint8)
    for name in ("q", "k", "v", "do"):
        arena[offs[name]:offs[name] + 4 * td] = \
            (rng.standard_normal(td, dtype=np.float32) * np.float32(0.5)).view(np.uint8)
    o = offs
    bs, hd, geo = P.pack2(Bq, S), P.pack2(H, d), P.pack_attn_geometry(Bq, S, H, d)
    rel = P.FLAG_RELAXED
    prog = [
        P.Instr(P.Op.ATTN_FWD_TILED, rel, 0, (o["q"], o["k"], o["v"], o["o"]), (o["stats"], bs, hd)),
        P.Instr(P.Op.ATTN_DQ_TILED, rel, 0, (o["q"], o["k"], o["v"], o["do"]), (o["stats"], o["dq"], geo)),
        P.Instr(P.Op.ATTN_DK_TILED, rel, 0, (o["q"], o["k"], o["v"], o["do"]), (o["stats"], o["dk"], geo)),
        P.Instr(P.Op.ATTN_DV_TILED, rel, 0, (o["q"], o["k"], o["v"], o["do"]), (o["stats"], o["dv"], geo)),
    ]
    be = B.CudaBackend(0)
    be.set_coherence(B.COHERENCE_LAZY)
    be.bind(arena, np.zeros(64, dtype=np.uint8))
    for _ in range(max(0, args.rounds - 1)):
        be.run(prog)
    be.set_profiling(True)
    be.run(prog)
    for rec in be.take_profile()[:4]:
        print("%-16s %.1f us" % (P.OP_NAMES[rec[0]], rec[2] * 1e3))
    print("relaxed executions:", be.counters().relaxed_executions)
    be.close()


if __name__ == "__main__":
    main()
