"""Producer-side bf16 conversion.  The instruction that writes a tensor a relaxed
GEMM reads next may emit the GEMM's bf16 operand itself; the GEMM then skips its
own conversion pass.  The copy must be the one that pass would have made, so the
chain run as ONE range (copies handed from producer to consumer) has to give the
same bits as the chain run one instruction per range (every range starts with no
cached copies, so each GEMM converts for itself) — and must launch fewer kernels."""

import numpy as np
import pytest

from see_ai_b200 import backend as B
from see_ai_b200 import plan as P
from tests.test_gpu_umma import bf16_round
from tests.test_oracle_pinned import Arena

pytestmark = pytest.mark.gpu
Op = P.Op
f = P.f32_bits
REL = P.FLAG_RELAXED


def _chain(rng):
    """LayerNorm -> q8 GEMM; GELU -> q8 GEMM; add -> transposed q8 GEMM with a
    per-k scale; GELU backward -> transposed q8 GEMM; xent backward -> transposed
    q8 GEMM; tiled attention forward -> q8 GEMM; attention dQ -> transposed q8 GEMM."""
    M, D, F, V = 256, 128, 256, 4096
    Bq, S, H, d = 1, 256, 2, 64          # M == Bq * S, D == H * d
    a = Arena(rng)
    x = a.alloc(M * D, "normal"); gamma = a.alloc(D, "normal"); beta = a.alloc(D, "normal")
    ln = a.alloc(M * D); mean = a.alloc(M); rstd = a.alloc(M)
    wq = a.ro_alloc(rng.integers(-127, 128, size=D * F, dtype=np.int8))
    sc_f = a.ro_alloc((rng.random(F) * 0.01 + 1e-3).astype(np.float32))
    sc_d = a.ro_alloc((rng.random(D) * 0.01 + 1e-3).astype(np.float32))
    sc_v = a.ro_alloc((rng.random(V) * 0.01 + 1e-3).astype(np.float32))
    h1 = a.alloc(M * F); g1 = a.alloc(M * F)
    w2 = a.ro_alloc(rng.integers(-127, 128, size=F * D, dtype=np.int8))
    h2 = a.alloc(M * D)
    r = a.alloc(M * D, "normal"); s1 = a.alloc(M * D)
    wt = a.ro_alloc(rng.integers(-127, 128, size=F * D, dtype=np.int8))   # [N=F][K=D]
    dx1 = a.alloc(M * F)
    dyf = a.alloc(M * F, "normal"); gb = a.alloc(M * F)
    wt2 = a.ro_alloc(rng.integers(-127, 128, size=D * F, dtype=np.int8))  # [N=D][K=F]
    dx2 = a.alloc(M * D)
    probs = rng.random((M, V)).astype(np.float32)
    probs /= probs.sum(axis=1, keepdims=True)
    pr = a.alloc(M * V, probs); labels = a.alloc(M, rng.integers(0, V, size=M), np.int32)
    seed = a.alloc(1, [1.0]); dlog = a.alloc(M * V)
    wv = a.ro_alloc(rng.integers(-127, 128, size=D * V, dtype=np.int8))   # [N=D][K=V]
    dx3 = a.alloc(M * D)
    q = a.alloc(M * D, bf16_round(rng.standard_normal(M * D).astype(np.float32)))
    k = a.alloc(M * D, bf16_round(rng.standard_normal(M * D).astype(np.float32)))
    v = a.alloc(M * D, bf16_round(rng.standard_normal(M * D).astype(np.float32)))
    do = a.alloc(M * D, bf16_round(rng.standard_normal(M * D).astype(np.float32)))
    o = a.alloc(M * D); stats = a.alloc(Bq * H * S * 4); dq = a.alloc(M * D)
    wo = a.ro_alloc(rng.integers(-127, 128, size=D * D, dtype=np.int8))
    po = a.alloc(M * D); dxq = a.alloc(M * D)
    bs, hd, geo = P.pack2(Bq, S), P.pack2(H, d), P.pack_attn_geometry(Bq, S, H, d)
    CS = P.FLAG_Q8_COL_SCALE
    prog = [
        P.Instr(Op.LAYERNORM_FWD, 0, f(1e-5), (x, gamma, beta, ln), (P.pack2(M, D), mean, rstd)),
        P.Instr(Op.GEMM_NN_Q8, REL | CS, 0, (ln, wq, h1, sc_f), (M, F, D)),
        P.Instr(Op.GELU_FWD, 0, 0, (h1, g1), (M * F, 0, 0)),
        P.Instr(Op.GEMM_NN_Q8, REL | CS, 0, (g1, w2, h2, sc_d), (M, D, F)),
        P.Instr(Op.ADD_EW, 0, 0, (h2, r, s1, P.NULL_REF), (M * D, 0, 0)),
        P.Instr(Op.GEMM_NT_Q8, REL | CS, 0, (s1, wt, dx1, sc_d), (M, F, D)),
        P.Instr(Op.GELU_BWD, 0, 0, (dyf, dx1, gb, P.NULL_REF), (M * F, 0, 0)),
        P.Instr(Op.GEMM_NT_Q8, REL | CS, 0, (gb, wt2, dx2, sc_f), (M, D, F)),
        P.Instr(Op.XENT_BWD, 0, 0, (pr, labels, seed, dlog), (M, V, 0)),
        P.Instr(Op.GEMM_NT_Q8, REL | CS, 0, (dlog, wv, dx3, sc_v), (M, D, V)),
        P.Instr(Op.ATTN_FWD_TILED, REL, 0, (q, k, v, o), (stats, bs, hd)),
        P.Instr(Op.GEMM_NN_Q8, REL | CS, 0, (o, wo, po, sc_d), (M, D, D)),
        P.Instr(Op.ATTN_DQ_TILED, REL, 0, (q, k, v, do), (stats, dq, geo)),
        P.Instr(Op.GEMM_NT_Q8, REL | CS, 0, (dq, wo, dxq, sc_d), (M, D, D)),
    ]
    arena, ro = a.build()
    return prog, arena, ro


def test_producer_made_copies_are_the_conversion_pass_bit_for_bit():
    prog, arena0, ro = _chain(np.random.default_rng(11))
    sp = B.StepParams(1e-3, 0.9, 0.999, 1e-8, 0.01, 0, 1)

    fused = arena0.copy()
    be = B.CudaBackend(0)
    be.bind(fused, ro)
    be.run(prog, sp)
    c_fused = be.counters()
    be.close()

    split = arena0.copy()
    be = B.CudaBackend(0)
    be.bind(split, ro)
    be.set_program(prog)
    for i in range(len(prog)):
        be.run(None, sp, i, i + 1)     # a range of one: nothing is handed over
    c_split = be.counters()
    be.close()

    assert c_fused.relaxed_executions == c_split.relaxed_executions == 9
    assert np.array_equal(fused, split)
    assert np.isfinite(fused.view(np.float32)).all()
    # Seven GEMMs found their operand already converted, and the attention
    # backward found the forward's three packed operands.
    assert c_split.kernel_launches - c_fused.kernel_launches == 7 + 3
