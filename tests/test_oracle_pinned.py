"""Pins the CPU checkers.

(a) Our C restatement (oracle/see_oracle.c) reproduces, bit for bit, every
    extent of every instruction in the write traces the reference's own probe
    recorded for eight plans compiled by the reference compiler.
(b) The reference executor built from the reference's sources (oracle/_ref),
    when present, reproduces the same traces — which validates the shim — and
    agrees bit for bit with the restatement on seeded instruction programs that
    reach opcodes and edge shapes the compiled plans do not.
"""

import numpy as np
import pytest

import oracle
from see_ai_b200 import plan as P
from tests.util import CASES, Case

Op = P.Op


def setup_module(_m):
    oracle.build("oracle")


def _replay(executor_cls, case: Case):
    ex = executor_cls()
    arena = case.plan.stage_arena()
    ex.bind(arena, case.rodata, case.source)
    mismatches = []
    for run in case.runs:
        case.stage_batch(arena, run)
        prog = case.plan.section(run["section"])
        sp = case.step_params(oracle.StepParams, run["step"])
        for (idx, op, _rel, extents) in run["trace"]:
            ex.run(prog, sp, idx, idx + 1)
            for off, want in extents:
                if arena[off:off + len(want)].tobytes() != want:
                    mismatches.append((run["section"], idx, P.OP_NAMES[op], off))
    assert np.array_equal(arena, case.final_arena)
    return mismatches


@pytest.mark.parametrize("name", CASES)
def test_restatement_reproduces_reference_traces(name):
    assert _replay(oracle.OracleExecutor, Case(name)) == []


@pytest.mark.parametrize("name", CASES)
def test_reference_build_reproduces_its_own_traces(name):
    if not oracle.have_ref():
        pytest.skip("oracle/_ref is not built (reference tree absent)")
    assert _replay(oracle.RefExecutor, Case(name)) == []


# ---- seeded instruction programs: restatement vs the reference executor ---------

class Arena:
    """Bump allocator over a byte arena and a rodata blob (64-byte aligned)."""

    def __init__(self, rng):
        self.rng = rng
        self.parts = []
        self.size = 0
        self.ro = bytearray()

    def alloc(self, n_floats, init=None, dtype=np.float32, scale=1.0):
        off = self.size
        if init is None:
            data = np.zeros(n_floats, dtype=dtype)
        elif isinstance(init, str) and init == "normal":
            data = (self.rng.standard_normal(n_floats) * scale).astype(np.float32)
        else:
            data = np.asarray(init, dtype=dtype).reshape(-1)
        self.parts.append((off, data.view(np.uint8).reshape(-1).copy()))
        self.size = (off + data.nbytes + 63) // 64 * 64
        return off

    def ro_alloc(self, data):
        off = (len(self.ro) + 63) // 64 * 64
        self.ro.extend(b"\0" * (off - len(self.ro)))
        self.ro.extend(np.ascontiguousarray(data).tobytes())
        return off | P.RODATA_BIT

    def build(self):
        arena = np.zeros(self.size + 64, dtype=np.uint8)
        for off, b in self.parts:
            arena[off:off + b.size] = b
        ro = np.frombuffer(bytes(self.ro) + b"\0" * 64, dtype=np.uint8).copy()
        return arena, ro


def seeded_programs():
    """-> list of (name, program, arena, rodata).  Shapes cross the kernels'
    blocking boundaries (K % 4 and K % 8 tails, odd row counts, single rows)."""
    out = []
    rng = np.random.default_rng(20261125)
    f = P.f32_bits

    # GEMM family over odd shapes, every flag the opcodes admit.
    for (M, N, K) in [(1, 1, 1), (3, 5, 7), (37, 29, 131), (8, 64, 13), (65, 33, 66),
                      (300, 16, 70), (12, 300, 70),
                      # the adapter-product shapes: narrow outputs over a long K, rank-K expansions
                      (300, 16, 80), (260, 8, 608), (257, 4, 64), (70, 64, 12), (100, 96, 16), (64, 128, 8),
                      # enough rows for each of the three block geometries of the narrow-output kernels
                      (20000, 16, 80), (9000, 8, 64)]:
        a = Arena(rng)
        A = a.alloc(M * K, "normal"); At = a.alloc(K * M, "normal")
        B = a.alloc(K * N, "normal"); Bt = a.alloc(N * K, "normal")
        D = a.alloc(M * N, "normal"); bias = a.alloc(N, "normal")
        q = rng.integers(-127, 128, size=K * N, dtype=np.int8)
        Bq = a.ro_alloc(q); Bqt = a.ro_alloc(rng.integers(-127, 128, size=N * K, dtype=np.int8))
        csn = a.ro_alloc((rng.random(N) * 0.02 + 1e-3).astype(np.float32))
        csk = a.ro_alloc((rng.random(K) * 0.02 + 1e-3).astype(np.float32))
        bf = (rng.standard_normal(K * N).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
        Bbf = a.ro_alloc(bf); Bbft = a.ro_alloc(bf[:N * K])
        outs = [a.alloc(M * N) for _ in range(16)]
        acc = a.alloc(M * N, "normal")
        dims = (M, N, K)
        prog = [
            P.Instr(Op.GEMM_NN, 0, 0, (A, B, outs[0], P.NULL_REF), dims),
            P.Instr(Op.GEMM_NN, P.FLAG_EPILOGUE_BIAS | (P.ACT_RELU << 1), 0, (A, B, outs[1], bias), dims),
            P.Instr(Op.GEMM_NN, P.FLAG_EPILOGUE_BIAS | (P.ACT_GELU << 1), 0, (A, B, outs[2], bias), dims),
            P.Instr(Op.GEMM_NN, P.ACT_SILU << 1, 0, (A, B, outs[3], P.NULL_REF), dims),
            P.Instr(Op.GEMM_NN, P.FLAG_GEMM_ADDEND, f(0.3), (A, B, outs[4], D), dims),
            P.Instr(Op.GEMM_NT, 0, f(1.7), (A, Bt, outs[5], P.NULL_REF), dims),
            P.Instr(Op.GEMM_NT, P.FLAG_GEMM_ADDEND, 0, (A, Bt, outs[6], D), dims),
            P.Instr(Op.GEMM_TN, 0, f(2.0), (At, B, outs[7], P.NULL_REF), dims),
            P.Instr(Op.GEMM_TN, P.FLAG_GEMM_ADDEND, 0, (At, B, outs[8], D), dims),
            P.Instr(Op.GEMM_ACC_NN, 0, 0, (A, B, acc, f(0.25)), dims),
            P.Instr(Op.GEMM_NN_Q8, 0, 0, (A, Bq, outs[9], f(0.0123)), dims),
            P.Instr(Op.GEMM_NN_Q8, P.FLAG_Q8_COL_SCALE | (P.ACT_RELU << 1), 0, (A, Bq, outs[10], csn), dims),
            P.Instr(Op.GEMM_NT_Q8, 0, 0, (A, Bqt, outs[11], f(0.0123)), dims),
            P.Instr(Op.GEMM_NT_Q8, P.FLAG_Q8_COL_SCALE, 0, (A, Bqt, outs[12], csk), dims),
            P.Instr(Op.GEMM_NN_BF16, P.FLAG_EPILOGUE_BIAS, 0, (A, Bbf, outs[13], bias), dims),
            P.Instr(Op.GEMM_NT_BF16, 0, 0, (A, Bbft, outs[14], P.NULL_REF), dims),
        ]
        out.append((f"gemm_{M}x{N}x{K}", prog, *a.build()))

    # Elementwise, fused map, reductions, losses, optimizers, clips.
    for n_rows, n_cols in [(1, 1), (5, 3), (33, 130), (300, 17), (9, 4100), (3, 32000)]:
        a = Arena(rng)
        n = n_rows * n_cols
        x = a.alloc(n, "normal"); y = a.alloc(n, "normal"); z = a.alloc(n, "normal")
        b = a.alloc(n_cols, "normal")
        labels = a.alloc(n_rows, rng.integers(0, n_cols, size=n_rows), np.int32)
        mlabels = rng.integers(0, n_cols, size=n_rows).astype(np.int32)
        mlabels[::3] = -1
        mlab = a.alloc(n_rows, mlabels, np.int32)
        seed = a.alloc(1, [1.0]); loss = a.alloc(4)
        o = [a.alloc(n) for _ in range(24)]
        colsum = a.alloc(n_cols)
        p = a.alloc(n, "normal"); m = a.alloc(n, "normal", scale=0.01)
        v = a.alloc(n, np.abs(rng.standard_normal(n)).astype(np.float32) * 1e-4)
        p2 = a.alloc(n, "normal"); g2 = a.alloc(n, "normal")
        accslot = a.alloc(1, [0.5])
        stages = (P.Op.NOP,)
        st = lambda kind, arg=0, right=False: kind | (arg << 4) | (0x80 if right else 0)
        chain = st(1, 1) | (st(3, 1) << 8) | (st(5) << 16) | (st(2, 2, True) << 24)
        prog = [
            P.Instr(Op.ADD_EW, 0, 0, (x, y, o[0], P.NULL_REF), (n, 0, 0)),
            P.Instr(Op.MUL_EW, 0, 0, (x, y, o[1], P.NULL_REF), (n, 0, 0)),
            P.Instr(Op.ADD_BIAS, 0, 0, (x, b, o[2], P.NULL_REF), (n_rows, n_cols, 0)),
            P.Instr(Op.RELU_FWD, 0, 0, (x, o[3]), (n, 0, 0)),
            P.Instr(Op.RELU_BWD, 0, 0, (y, x, o[4], P.NULL_REF), (n, 0, 0)),
            P.Instr(Op.GELU_FWD, 0, 0, (x, o[5]), (n, 0, 0)),
            P.Instr(Op.GELU_BWD, 0, 0, (y, x, o[6], P.NULL_REF), (n, 0, 0)),
            P.Instr(Op.SILU_FWD, 0, 0, (x, o[7]), (n, 0, 0)),
            P.Instr(Op.SILU_BWD, 0, 0, (y, x, o[8], P.NULL_REF), (n, 0, 0)),
            P.Instr(Op.SCALE, 0, 0, (x, o[9], f(-0.37)), (n, 0, 0)),
            P.Instr(Op.COPY, 0, 0, (x, o[10]), (n, 0, 0)),
            P.Instr(Op.FILL, 0, 0, (o[11], f(2.5)), (n, 0, 0)),
            P.Instr(Op.ACCUMULATE, 0, 0, (o[11], y), (n, 0, 0)),
            P.Instr(Op.REDUCE_ROWS, 0, 0, (x, colsum), (n_rows, n_cols, 0)),
            P.Instr(Op.FUSED_MAP, 0, 0, (x, y, z, o[12]), (n, chain, f(0.5) | (f(1.5) << 32))),
            P.Instr(Op.XENT_FWD, 0, 0, (x, labels, loss, o[13]), (n_rows, n_cols, 0)),
            P.Instr(Op.XENT_BWD, 0, 0, (o[13], labels, seed, o[14]), (n_rows, n_cols, 0)),
            P.Instr(Op.XENT_MASKED_FWD, 0, 0, (x, mlab, loss + 4, o[15]), (n_rows, n_cols, 0)),
            P.Instr(Op.XENT_MASKED_BWD, 0, 0, (o[15], mlab, seed, o[16]), (n_rows, n_cols, 0)),
            P.Instr(Op.MSE_FWD, 0, 0, (x, y, loss + 8, P.NULL_REF), (n, 0, 0)),
            P.Instr(Op.MSE_BWD, 0, 0, (x, y, seed, o[17]), (n, 0, 0)),
            P.Instr(Op.KL_FWD, 0, 0, (x, y, loss + 12, o[18]),
                    (o[19], P.pack2(n_rows, n_cols), f(2.0) | (f(4.0) << 32))),
            P.Instr(Op.KL_BWD, 0, 0, (o[18], o[19], seed, o[20]),
                    (P.pack2(n_rows, n_cols), f(2.0) | (f(4.0) << 32), 0)),
            P.Instr(Op.LAYERNORM_FWD, 0, f(1e-6), (x, b, b, o[21]),
                    (P.pack2(n_rows, n_cols), o[22], o[22] + 4 * n_rows)),
            P.Instr(Op.LAYERNORM_BWD, 0, 0, (y, x, b, o[23]),
                    (o[22], o[22] + 4 * n_rows, P.pack2(n_rows, n_cols))),
            P.Instr(Op.ADAMW_STEP, 0, 0, (p, x, m, v), (n, 0, 0)),
            P.Instr(Op.ADAMW_STEP, 0, 0, (p, y, m, v), (n, f(0.5), 0)),
            P.Instr(Op.SGD_STEP, 0, 0, (p2, g2), (n, f(0.25), 0)),
            P.Instr(Op.CLIP_NORM, 0, 0, (g2, f(0.1)), (n, 0, 0)),
            P.Instr(Op.SQNORM_ACCUM, 0, 0, (g2, accslot), (n, 0, 0)),
            P.Instr(Op.CLIP_GLOBAL, 0, 0, (z, accslot, f(0.2)), (n, 0, 0)),
        ]
        out.append((f"elementwise_{n_rows}x{n_cols}", prog, *a.build()))

    # Attention families, RoPE, segment mask.
    for (B, S, H, d) in [(1, 1, 1, 2), (2, 9, 3, 8), (1, 40, 2, 16)]:
        a = Arena(rng)
        td = B * S * H * d
        pn = B * H * S * S
        q = a.alloc(td, "normal"); k = a.alloc(td, "normal"); v = a.alloc(td, "normal")
        do = a.alloc(td, "normal")
        o1 = a.alloc(td); o2 = a.alloc(td); o3 = a.alloc(td); o4 = a.alloc(td)
        Pm = a.alloc(pn); Pseg = a.alloc(pn); dP = a.alloc(pn); dS = a.alloc(pn)
        dq = a.alloc(td); dk = a.alloc(td); dv = a.alloc(td)
        dq2 = a.alloc(td); dk2 = a.alloc(td); dv2 = a.alloc(td)
        dq3 = a.alloc(td); dk3 = a.alloc(td); dv3 = a.alloc(td)
        stats = a.alloc(B * H * S * 4); stats2 = a.alloc(B * H * S * 4)
        toks = rng.integers(0, 4, size=B * S).astype(np.int32)
        tk = a.alloc(B * S, toks, np.int32); starts = a.alloc(B * S, None, np.int32)
        table = a.alloc(S * d); r1 = a.alloc(td); r2 = a.alloc(td); r3 = a.alloc(td)
        bs, hd = P.pack2(B, S), P.pack2(H, d)
        geo = P.pack_attn_geometry(B, S, H, d)
        prog = [
            P.Instr(Op.ROPE_TABLE, 0, 0, (table,), (P.pack2(S, d), f(10000.0), 0)),
            P.Instr(Op.ROPE_FWD, 0, 0, (q, r1, table), (bs, hd, f(10000.0))),
            P.Instr(Op.ROPE_FWD, 0, 0, (q, r2, P.NULL_REF), (bs, hd, f(500000.0))),
            P.Instr(Op.ROPE_BWD, 0, 0, (do, r3, P.NULL_REF), (bs, hd, f(10000.0))),
            P.Instr(Op.ATTN_FWD, 0, 0, (q, k, v, o1), (Pm, bs, hd)),
            P.Instr(Op.ATTN_DP, 0, 0, (do, v, dP, P.NULL_REF), (bs, hd, 0)),
            P.Instr(Op.ATTN_DV, 0, 0, (Pm, do, dv, P.NULL_REF), (bs, hd, 0)),
            P.Instr(Op.SOFTMAX_ROWS_BWD, 0, 0, (Pm, dP, dS, P.NULL_REF), (P.pack2(B * H * S, S), 0, 0)),
            P.Instr(Op.ATTN_DQ, 0, 0, (dS, k, dq, P.NULL_REF), (bs, hd, 0)),
            P.Instr(Op.ATTN_DK, 0, 0, (dS, q, dk, P.NULL_REF), (bs, hd, 0)),
            P.Instr(Op.ATTN_FWD_TILED, 0, 0, (q, k, v, o2), (stats, bs, hd)),
            P.Instr(Op.ATTN_DQ_TILED, 0, 0, (q, k, v, do), (stats, dq2, geo)),
            P.Instr(Op.ATTN_DK_TILED, 0, 0, (q, k, v, do), (stats, dk2, geo)),
            P.Instr(Op.ATTN_DV_TILED, 0, 0, (q, k, v, do), (stats, dv2, geo)),
            P.Instr(Op.SEGMENT_STARTS, 0, 0, (tk, starts), (bs, 1, 0)),
            P.Instr(Op.ATTN_FWD_SEG, 0, 0, (q, k, v, o3), (Pseg, geo, starts)),
            P.Instr(Op.ATTN_FWD_TILED_SEG, 0, 0, (q, k, v, o4), (stats2, geo, starts)),
            P.Instr(Op.ATTN_DQ_TILED, 0, 0, (q, k, v, do), (stats2, dq3, geo)),
            P.Instr(Op.ATTN_DK_TILED, 0, 0, (q, k, v, do), (stats2, dk3, geo)),
            P.Instr(Op.ATTN_DV_TILED, 0, 0, (q, k, v, do), (stats2, dv3, geo)),
        ]
        out.append((f"attention_B{B}S{S}H{H}d{d}", prog, *a.build()))
    return out


PROGRAMS = seeded_programs()


@pytest.mark.parametrize("entry", PROGRAMS, ids=[p[0] for p in PROGRAMS])
def test_restatement_equals_reference_on_seeded_programs(entry):
    if not oracle.have_ref():
        pytest.skip("oracle/_ref is not built (reference tree absent)")
    name, prog, arena, ro = entry
    a1, a2 = arena.copy(), arena.copy()
    ref, ours = oracle.RefExecutor(), oracle.OracleExecutor()
    ref.bind(a1, ro); ours.bind(a2, ro)
    sp = oracle.step_params(lr=1e-2, step=3)
    for i, ins in enumerate(prog):
        ref.run(prog, sp, i, i + 1)
        ours.run(prog, sp, i, i + 1)
        assert np.array_equal(a1, a2), f"{name}: instruction {i} ({P.OP_NAMES[ins.opcode]}) differs"


def test_thread_count_does_not_change_reference_bits():
    if not oracle.have_ref():
        pytest.skip("oracle/_ref is not built")
    name, prog, arena, ro = PROGRAMS[2]
    outs = []
    for threads in (1, 3, 8):
        a = arena.copy()
        ref = oracle.RefExecutor()
        ref.set_threads(threads)
        ref.bind(a, ro)
        ref.run(prog, oracle.step_params(step=2))
        outs.append(a)
    ref.set_threads(0)
    assert np.array_equal(outs[0], outs[1]) and np.array_equal(outs[0], outs[2])
