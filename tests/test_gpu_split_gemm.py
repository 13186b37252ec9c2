"""Exact f32 products on the tensor cores as six bf16 piece products.

Held to the reference's own value test for its GEMMs: every output within 2e-6
of a float64 product, scaled by 1 + sum_k |a_k b_k| (reference:
test/runtime/executor/kernels_test.cc:1786-1822) — for the NN, NT and TN forms
with alpha, addend, bias and activation, at shapes that cross every tile
boundary of the kernel (ragged M, N % 256, K % 64) and at the sweep's sizes
through sampled rows.  Shapes below the size threshold, or with widths the
kernel does not take, must still run on the exact kernels, bit for bit.
"""

import numpy as np
import pytest

import oracle
from see_ai_b200 import backend as B
from see_ai_b200 import plan as P
from tests.test_oracle_pinned import Arena

pytestmark = pytest.mark.gpu
Op = P.Op


def setup_module(_m):
    if not oracle.have_oracle():
        oracle.build("oracle")


def _run(prog, arena0, ro, mode):
    arena = arena0.copy()
    be = B.CudaBackend(0)
    be.set_split_gemm(mode)
    be.bind(arena, ro)
    be.run(prog)
    c = be.counters()
    be.close()
    return arena, c


def _f64(arena, off, rows, cols):
    return arena[off:off + 4 * rows * cols].view(np.float32).astype(np.float64).reshape(rows, cols)


SHAPES = [(384, 256, 768), (515, 260, 1028), (131, 516, 2052), (1024, 1024, 1024), (4096, 256, 256)]


@pytest.mark.parametrize("shape", SHAPES, ids=[f"{m}x{n}x{k}" for m, n, k in SHAPES])
def test_split_products_match_a_float64_product(shape):
    M, N, K = shape
    rng = np.random.default_rng(M * 7 + N * 3 + K)
    a = Arena(rng)
    A = a.alloc(M * K, "normal"); At = a.alloc(K * M, "normal")
    Bm = a.alloc(K * N, "normal"); Bt = a.alloc(N * K, "normal")
    W = a.ro_alloc(rng.standard_normal((K, N)).astype(np.float32))       # a frozen f32 weight (cached pieces)
    D = a.alloc(M * N, "normal")
    bias = a.ro_alloc(rng.standard_normal(N).astype(np.float32))
    outs = [a.alloc(M * N) for _ in range(5)]
    alpha = 0.375
    prog = [
        P.Instr(Op.GEMM_NN, P.FLAG_GEMM_ADDEND, P.f32_bits(alpha), (A, Bm, outs[0], D), (M, N, K)),
        P.Instr(Op.GEMM_NT, 0, P.f32_bits(alpha), (A, Bt, outs[1], P.NULL_REF), (M, N, K)),
        P.Instr(Op.GEMM_TN, 0, P.f32_bits(alpha), (At, Bm, outs[2], P.NULL_REF), (M, N, K)),
        P.Instr(Op.GEMM_NN, P.FLAG_EPILOGUE_BIAS | (P.ACT_RELU << 1), 0, (A, W, outs[3], bias), (M, N, K)),
        P.Instr(Op.GEMM_NN, 0, 0, (A, W, outs[4], P.NULL_REF), (M, N, K)),   # the cached pieces again
    ]
    arena0, ro = a.build()
    got, c = _run(prog, arena0, ro, 1)
    assert c.split_executions == len(prog), c.split_executions
    exact, c0 = _run(prog, arena0, ro, 0)
    assert c0.split_executions == 0
    Am, Atm = _f64(arena0, A, M, K), _f64(arena0, At, K, M)
    Bmm, Btm = _f64(arena0, Bm, K, N), _f64(arena0, Bt, N, K)
    Wm = np.frombuffer(ro.tobytes()[W & ~P.RODATA_BIT:(W & ~P.RODATA_BIT) + 4 * K * N], np.float32) \
        .astype(np.float64).reshape(K, N)
    bv = np.frombuffer(ro.tobytes()[bias & ~P.RODATA_BIT:(bias & ~P.RODATA_BIT) + 4 * N], np.float32).astype(np.float64)
    Dm = _f64(arena0, D, M, N)
    wants = [
        (alpha * (Am @ Bmm) + Dm, alpha * (np.abs(Am) @ np.abs(Bmm)) + np.abs(Dm)),
        (alpha * (Am @ Btm.T), alpha * (np.abs(Am) @ np.abs(Btm.T))),
        (alpha * (Atm.T @ Bmm), alpha * (np.abs(Atm.T) @ np.abs(Bmm))),
        (np.maximum(Am @ Wm + bv, 0.0), np.abs(Am) @ np.abs(Wm) + np.abs(bv)),
        (Am @ Wm, np.abs(Am) @ np.abs(Wm)),
    ]
    worst = []
    for off, (want, mag) in zip(outs, wants):
        g = _f64(got, off, M, N)
        assert np.isfinite(g).all()
        worst.append(float((np.abs(g - want) / (1.0 + mag)).max()))
    assert max(worst) < 2e-6, worst
    for off, (want, mag) in zip(outs, wants):
        # the exact kernels meet the same bound: the two agree to twice it
        e = _f64(exact, off, M, N)
        assert (np.abs(e - want) / (1.0 + mag)).max() < 2e-6
    assert not np.array_equal(got[outs[1]:outs[1] + 4 * M * N], exact[outs[1]:outs[1] + 4 * M * N])


def test_small_and_narrow_products_keep_the_exact_kernels():
    rng = np.random.default_rng(5)
    a = Arena(rng)
    A = a.alloc(256 * 128, "normal"); Bm = a.alloc(128 * 128, "normal")     # 2^22 multiply-adds: below the threshold
    A2 = a.alloc(4096 * 768, "normal"); B2 = a.alloc(768 * 16, "normal")     # a rank-16 product: too narrow
    A3 = a.alloc(512 * 514, "normal"); B3 = a.alloc(514 * 512, "normal")     # K % 4 != 0
    o1, o2, o3 = a.alloc(256 * 128), a.alloc(4096 * 16), a.alloc(512 * 512)
    prog = [P.Instr(Op.GEMM_NN, 0, 0, (A, Bm, o1, P.NULL_REF), (256, 128, 128)),
            P.Instr(Op.GEMM_NN, 0, 0, (A2, B2, o2, P.NULL_REF), (4096, 16, 768)),
            P.Instr(Op.GEMM_NN, 0, 0, (A3, B3, o3, P.NULL_REF), (512, 512, 514))]
    arena0, ro = a.build()
    got, c = _run(prog, arena0, ro, 1)
    cpu = arena0.copy()
    ref = oracle.OracleExecutor()
    ref.bind(cpu, ro)
    ref.run(prog)
    assert c.split_executions == 0
    assert np.array_equal(got, cpu)


@pytest.mark.parametrize("S", [2048, 8192])
def test_sweep_sizes_through_sampled_rows(S):
    """The isolated-GEMM sweep's sizes: NN at S^3, checked on 48 sampled rows
    against float64 (rows of a product are independent)."""
    rng = np.random.default_rng(S)
    A_np = rng.standard_normal((S, S)).astype(np.float32)
    B_np = rng.standard_normal((S, S)).astype(np.float32)
    arena = np.zeros(3 * 4 * S * S + 64, dtype=np.uint8)
    arena[:4 * S * S] = A_np.view(np.uint8).reshape(-1)
    arena[4 * S * S:8 * S * S] = B_np.view(np.uint8).reshape(-1)
    out = 8 * S * S
    be = B.CudaBackend(0)
    be.set_split_gemm(1)
    be.set_coherence(B.COHERENCE_LAZY)
    be.bind(arena, None)
    be.run([P.Instr(Op.GEMM_NN, 0, 0, (0, 4 * S * S, out, P.NULL_REF), (S, S, S))])
    assert be.counters().split_executions == 1
    rows = np.sort(rng.choice(S, size=48, replace=False))
    be.host_needs(out, 4 * S * S)
    be.flush()
    be.close()
    C = arena[out:out + 4 * S * S].view(np.float32).reshape(S, S)
    A64, B64 = A_np[rows].astype(np.float64), B_np.astype(np.float64)
    want = A64 @ B64
    mag = np.abs(A64) @ np.abs(B64)
    err = np.abs(C[rows].astype(np.float64) - want) / (1.0 + mag)
    assert err.max() < 2e-6, err.max()
