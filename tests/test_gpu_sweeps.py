"""Parity at the sizes of the GEMM and attention sweeps, through properties that
do not need the CPU oracle to redo the whole problem:

* GEMM S x S x S (S = 4096, persistent tensor-core kernel; S = 1024, exact
  kernels): the CPU GEMM is row-independent, so sampled rows are recomputed in
  float64 and held to the reference's scaled metric
  (|got - want| / (1 + sum|a_k b_k|) < 2e-6; reference:
  test/runtime/executor/kernels_test.cc:1803-1822); exact opcodes must also
  match the oracle bit for bit on the sampled row block.
* Tiled attention chain with the relaxed permission at S = 2048 (d = 64) and
  S = 1024 (d = 128): units are independent per (sequence, head), so the oracle
  runs the exact tiled family on the same few units; 1e-2 of each tensor's scale.
"""

import numpy as np
import pytest

import oracle
from see_ai_b200 import backend as B
from see_ai_b200 import plan as P
from tests.test_gpu_umma import bf16_round
from tests.test_oracle_pinned import Arena

pytestmark = pytest.mark.gpu
Op = P.Op
REL = P.FLAG_RELAXED


def setup_module(_m):
    if not oracle.have_oracle():
        oracle.build("oracle")


def _run_gpu(prog, arena, ro):
    be = B.CudaBackend(0)
    be.bind(arena, ro)
    be.run(prog)
    c = be.counters()
    be.close()
    return c


def test_relaxed_gemm_4096_cubed_sampled_rows():
    S = 4096
    rng = np.random.default_rng(4096)
    a = Arena(rng)
    A_np = bf16_round(rng.standard_normal((S, S)).astype(np.float32))
    q = rng.integers(-127, 128, size=(S, S), dtype=np.int8)
    cs = (rng.random(S) * 0.02 + 1e-3).astype(np.float32)
    A = a.alloc(S * S, A_np)
    C_nn = a.alloc(S * S); C_nt = a.alloc(S * S)
    Wq = a.ro_alloc(q); Cs = a.ro_alloc(cs)
    csk = (2.0 ** rng.integers(-8, -3, size=S)).astype(np.float32)   # powers of two: A*s stays bf16
    Csk = a.ro_alloc(csk)
    prog = [P.Instr(Op.GEMM_NN_Q8, REL | P.FLAG_Q8_COL_SCALE, 0, (A, Wq, C_nn, Cs), (S, S, S)),
            P.Instr(Op.GEMM_NT_Q8, REL | P.FLAG_Q8_COL_SCALE, 0, (A, Wq, C_nt, Csk), (S, S, S))]
    arena, ro = a.build()
    c = _run_gpu(prog, arena, ro)
    assert c.relaxed_executions == 2
    rows = rng.choice(S, size=48, replace=False)
    A64 = A_np[rows].astype(np.float64)
    q64 = q.astype(np.float64)
    got_nn = arena[C_nn:C_nn + 4 * S * S].view(np.float32).reshape(S, S)[rows].astype(np.float64)
    want_nn = (A64 @ q64) * cs.astype(np.float64)
    mag_nn = (np.abs(A64) @ np.abs(q64)) * cs.astype(np.float64)
    assert (np.abs(got_nn - want_nn) / (1.0 + mag_nn)).max() < 2e-6
    As = A64 * csk.astype(np.float64)            # C = (A * s_k) . W^T with W = q as [N][K]
    got_nt = arena[C_nt:C_nt + 4 * S * S].view(np.float32).reshape(S, S)[rows].astype(np.float64)
    want_nt = As @ q64.T
    mag_nt = np.abs(As) @ np.abs(q64.T)
    assert (np.abs(got_nt - want_nt) / (1.0 + mag_nt)).max() < 2e-6


def test_exact_gemm_1024_cubed_is_the_oracles_bits_on_a_row_block():
    S, R0, R = 1024, 512, 40
    rng = np.random.default_rng(1024)
    a = Arena(rng)
    A = a.alloc(S * S, "normal"); Bm = a.alloc(S * S, "normal")
    C1 = a.alloc(S * S); C2 = a.alloc(S * S); C3 = a.alloc(S * S)
    prog = [P.Instr(Op.GEMM_NN, 0, P.f32_bits(0.5), (A, Bm, C1, P.NULL_REF), (S, S, S)),
            P.Instr(Op.GEMM_NT, 0, 0, (A, Bm, C2, P.NULL_REF), (S, S, S)),
            P.Instr(Op.GEMM_TN, 0, 0, (A, Bm, C3, P.NULL_REF), (S, S, S))]
    arena, ro = a.build()
    gpu = arena.copy()
    _run_gpu(prog, gpu, ro)
    # The oracle on rows [R0, R0 + R) only: NN and NT are row-independent in A;
    # for TN (C = A^T B) a row block of C is a column block of A.
    A_np = arena[A:A + 4 * S * S].view(np.float32).reshape(S, S)
    B_np = arena[Bm:Bm + 4 * S * S].view(np.float32).reshape(S, S)
    b = Arena(rng)
    a_rows = b.alloc(R * S, A_np[R0:R0 + R]); a_cols = b.alloc(S * R, np.ascontiguousarray(A_np[:, R0:R0 + R]))
    bm = b.alloc(S * S, B_np)
    o1 = b.alloc(R * S); o2 = b.alloc(R * S); o3 = b.alloc(R * S)
    sub = [P.Instr(Op.GEMM_NN, 0, P.f32_bits(0.5), (a_rows, bm, o1, P.NULL_REF), (R, S, S)),
           P.Instr(Op.GEMM_NT, 0, 0, (a_rows, bm, o2, P.NULL_REF), (R, S, S)),
           P.Instr(Op.GEMM_TN, 0, 0, (a_cols, bm, o3, P.NULL_REF), (R, S, S))]
    cpu, cro = b.build()
    ref = oracle.OracleExecutor()
    ref.bind(cpu, cro)
    ref.run(sub)
    for full, part in ((C1, o1), (C2, o2), (C3, o3)):
        got = gpu[full:full + 4 * S * S].view(np.float32).reshape(S, S)[R0:R0 + R]
        want = cpu[part:part + 4 * R * S].view(np.float32).reshape(R, S)
        assert np.array_equal(got, want)


@pytest.mark.parametrize("geom", [(1, 2048, 2, 64), (1, 1024, 2, 128)], ids=["S2048d64", "S1024d128"])
def test_relaxed_tiled_attention_at_sweep_lengths(geom):
    Bq, S, H, d = geom
    rng = np.random.default_rng(S + d)
    a = Arena(rng)
    td = Bq * S * H * d
    t = {}
    for name in ("q", "k", "v", "do"):
        t[name] = a.alloc(td, bf16_round(rng.standard_normal(td).astype(np.float32) * 0.7))
    for name in ("o", "dq", "dk", "dv"):
        t[name] = a.alloc(td)
    stats = a.alloc(Bq * H * S * 4)
    bs, hd, geo = P.pack2(Bq, S), P.pack2(H, d), P.pack_attn_geometry(Bq, S, H, d)

    def prog(flags):
        return [
            P.Instr(Op.ATTN_FWD_TILED, flags, 0, (t["q"], t["k"], t["v"], t["o"]), (stats, bs, hd)),
            P.Instr(Op.ATTN_DQ_TILED, flags, 0, (t["q"], t["k"], t["v"], t["do"]), (stats, t["dq"], geo)),
            P.Instr(Op.ATTN_DK_TILED, flags, 0, (t["q"], t["k"], t["v"], t["do"]), (stats, t["dk"], geo)),
            P.Instr(Op.ATTN_DV_TILED, flags, 0, (t["q"], t["k"], t["v"], t["do"]), (stats, t["dv"], geo)),
        ]
    arena, ro = a.build()
    cpu, gpu = arena.copy(), arena.copy()
    ref = oracle.OracleExecutor()
    ref.bind(cpu, ro)
    ref.run(prog(0))
    c = _run_gpu(prog(REL), gpu, ro)
    assert c.relaxed_executions == 4
    for name in ("o", "dq", "dk", "dv"):
        got = gpu[t[name]:t[name] + 4 * td].view(np.float32)
        want = cpu[t[name]:t[name] + 4 * td].view(np.float32)
        assert np.isfinite(got).all(), name
        err = np.max(np.abs(got - want)) / np.max(np.abs(want))
        assert err < 1e-2, f"{name}: {err:.3g} of scale"
