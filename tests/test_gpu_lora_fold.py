"""An adapter's rank-r expand product folded into the frozen product it adds to.

Three instruction patterns the planner recognises (forward: product, down
product, expand; backward with the product first; backward with the expand
first and the sum by a kAddEW), each with and without a following kAddEW, on
the one-tile and the persistent tensor-core kernel.  A program run as ONE range
(folded) is compared with the same program run one instruction per range (every
instruction its own kernels): the frozen product is the same bf16 computation
both ways, so the two differ only by the arithmetic of the low-rank term and of
the sums — held to 2e-6 of 1 + |base| + s * sum|t_k||b_k| per element, the
reference's own bound for a GEMM's summation error (reference:
test/runtime/executor/kernels_test.cc:1803-1822).  The down product's output
t is written by the same exact kernel both ways: bit for bit.
"""

import numpy as np
import pytest

from see_ai_b200 import backend as B
from see_ai_b200 import plan as P
from tests.test_oracle_pinned import Arena

pytestmark = pytest.mark.gpu
Op = P.Op
REL, CS, ADDEND = P.FLAG_RELAXED, P.FLAG_Q8_COL_SCALE, P.FLAG_GEMM_ADDEND
SIZES = [(256, 128, 192), (4864, 128, 2048)]   # (M, K, N): one-tile; 38 x 8 wide tiles > 2 x 148 -> persistent


def _run(prog, arena0, ro, one_range, fold=True):
    arena = arena0.copy()
    be = B.CudaBackend(0)
    be.set_coherence(B.COHERENCE_LAZY)
    be.set_lora_fold(fold)
    be.bind(arena, ro)
    be.set_program(prog)
    if one_range:
        be.run(None)
    else:
        for i in range(len(prog)):
            be.run(None, None, i, i + 1)
    be.host_needs(0, arena.size)
    be.flush()
    c = be.counters()
    be.close()
    return arena, c


def _f32(arena, off, n):
    return arena[off:off + 4 * n].view(np.float32).astype(np.float64)


def _check(fused, split, out, M, N, t, w_mat, scale, base_mag):
    got, want = _f32(fused, out, M * N).reshape(M, N), _f32(split, out, M * N).reshape(M, N)
    assert np.isfinite(got).all()
    mag = 1.0 + base_mag + abs(scale) * (np.abs(t) @ np.abs(w_mat))
    err = np.abs(got - want) / mag
    assert err.max() < 2e-6, err.max()
    assert not np.array_equal(got, want) or M * N < 4, "identical bits: did the fold run?"


@pytest.mark.parametrize("size", SIZES, ids=["one-tile", "persistent"])
@pytest.mark.parametrize("with_add", [False, True], ids=["plain", "then-add"])
@pytest.mark.parametrize("r", [8, 16])
def test_forward_pattern(size, with_add, r):
    M, K, N = size
    rng = np.random.default_rng(M + r)
    a = Arena(rng)
    x = a.alloc(M * K, "normal")
    w = a.ro_alloc(rng.integers(-127, 128, size=K * N, dtype=np.int8))
    sc = a.ro_alloc((rng.random(N) * 0.01 + 1e-3).astype(np.float32))
    A = a.alloc(K * r, "normal", scale=1.0 / np.sqrt(K))
    Bm = a.alloc(r * N, "normal", scale=0.05)
    res = a.alloc(M * N, "normal")
    base = a.alloc(M * N); t = a.alloc(M * r); out = a.alloc(M * N); x1 = a.alloc(M * N)
    s = 2.0
    prog = [
        P.Instr(Op.GEMM_NN_Q8, REL | CS, 0, (x, w, base, sc), (M, N, K)),
        P.Instr(Op.GEMM_NN, 0, 0, (x, A, t, P.NULL_REF), (M, r, K)),
        P.Instr(Op.GEMM_NN, ADDEND, P.f32_bits(s), (t, Bm, out, base), (M, N, r)),
    ]
    if with_add:
        prog.append(P.Instr(Op.ADD_EW, 0, 0, (res, out, x1, P.NULL_REF), (M * N, 0, 0)))
        prog.append(P.Instr(Op.FILL, 0, 0, (out, P.f32_bits(0.0)), (M * N, 0, 0)))
    prog.append(P.Instr(Op.FILL, 0, 0, (base, P.f32_bits(0.0)), (M * N, 0, 0)))
    arena0, ro = a.build()
    fused, c_fused = _run(prog, arena0, ro, True)
    split, c_split = _run(prog, arena0, ro, False)
    assert c_fused.fused_dispatches == (3 if with_add else 2), c_fused.fused_dispatches
    assert np.array_equal(fused[t:t + 4 * M * r], split[t:t + 4 * M * r])
    tv = _f32(split, t, M * r).reshape(M, r)
    bm = _f32(arena0, Bm, r * N).reshape(r, N)
    final = x1 if with_add else out
    # |base| from the unfused run: out - s t B (- res)
    lr = s * (tv @ bm)
    base_mag = np.abs(_f32(split, final, M * N).reshape(M, N) - lr)
    _check(fused, split, final, M, N, tv, bm, s, base_mag)
    # with the fold switched off the single range gives the unfused bits (the older fusions are bit-exact)
    plain, c_plain = _run(prog, arena0, ro, True, fold=False)
    assert np.array_equal(plain[final:final + 4 * M * N], split[final:final + 4 * M * N])


@pytest.mark.parametrize("size", SIZES, ids=["one-tile", "persistent"])
@pytest.mark.parametrize("with_add", [False, True], ids=["plain", "then-add"])
def test_backward_pattern_product_first(size, with_add):
    M, K, N = size           # dy [M, K] through W^T [N = k_in, K]
    r = 16
    rng = np.random.default_rng(M + 7)
    a = Arena(rng)
    dy = a.alloc(M * K, "normal")
    wt = a.ro_alloc(rng.integers(-127, 128, size=N * K, dtype=np.int8))      # [N, K]
    sk = a.ro_alloc((rng.random(K) * 0.01 + 1e-3).astype(np.float32))
    dt = a.alloc(M * r, "normal")
    A = a.alloc(N * r, "normal", scale=0.05)                                  # [N, r]
    res = a.alloc(M * N, "normal")
    base = a.alloc(M * N); out = a.alloc(M * N); s2 = a.alloc(M * N)
    prog = [
        P.Instr(Op.GEMM_NT_Q8, REL | CS, 0, (dy, wt, base, sk), (M, N, K)),
        P.Instr(Op.GEMM_NT, ADDEND, 0, (dt, A, out, base), (M, N, r)),
    ]
    if with_add:
        prog.append(P.Instr(Op.ADD_EW, 0, 0, (out, res, s2, P.NULL_REF), (M * N, 0, 0)))
        prog.append(P.Instr(Op.FILL, 0, 0, (out, P.f32_bits(0.0)), (M * N, 0, 0)))
    prog.append(P.Instr(Op.FILL, 0, 0, (base, P.f32_bits(0.0)), (M * N, 0, 0)))
    arena0, ro = a.build()
    fused, c_fused = _run(prog, arena0, ro, True)
    split, c_split = _run(prog, arena0, ro, False)
    assert c_fused.fused_dispatches == (2 if with_add else 1), c_fused.fused_dispatches
    tv = _f32(arena0, dt, M * r).reshape(M, r)
    am = _f32(arena0, A, N * r).reshape(N, r).T
    final = s2 if with_add else out
    base_mag = np.abs(_f32(split, final, M * N).reshape(M, N) - tv @ am)
    _check(fused, split, final, M, N, tv, am, 1.0, base_mag)


@pytest.mark.parametrize("size", SIZES, ids=["one-tile", "persistent"])
@pytest.mark.parametrize("between", [1, 2], ids=["one-between", "two-between"])
def test_backward_pattern_expand_first(size, between):
    M, K, N = size
    r = 16
    rng = np.random.default_rng(M + 11)
    a = Arena(rng)
    dy = a.alloc(M * K, "normal")
    wt = a.ro_alloc(rng.integers(-127, 128, size=N * K, dtype=np.int8))
    sk = a.ro_alloc((rng.random(K) * 0.01 + 1e-3).astype(np.float32))
    dt = a.alloc(M * r, "normal")
    A = a.alloc(N * r, "normal", scale=0.05)
    acc = a.alloc(M * N, "normal")
    xin = a.alloc(M * N, "normal")
    part = a.alloc(M * N); out = a.alloc(M * N); s2 = a.alloc(M * N); gA = a.alloc(N * r); junk = a.alloc(64)
    prog = [P.Instr(Op.GEMM_NT, ADDEND, 0, (dt, A, part, acc), (M, N, r)),
            P.Instr(Op.GEMM_TN, 0, 0, (xin, dt, gA, P.NULL_REF), (N, r, M))]
    if between == 2:
        prog.append(P.Instr(Op.FILL, 0, 0, (junk, P.f32_bits(1.0)), (16, 0, 0)))
    prog += [
        P.Instr(Op.GEMM_NT_Q8, REL | CS, 0, (dy, wt, out, sk), (M, N, K)),
        P.Instr(Op.ADD_EW, 0, 0, (part, out, s2, P.NULL_REF), (M * N, 0, 0)),
        P.Instr(Op.FILL, 0, 0, (part, P.f32_bits(0.0)), (M * N, 0, 0)),
        P.Instr(Op.FILL, 0, 0, (out, P.f32_bits(0.0)), (M * N, 0, 0)),
    ]
    arena0, ro = a.build()
    fused, c_fused = _run(prog, arena0, ro, True)
    split, c_split = _run(prog, arena0, ro, False)
    assert c_fused.fused_dispatches == 2, c_fused.fused_dispatches    # the kAddEW and the expand
    assert np.array_equal(fused[gA:gA + 4 * N * r], split[gA:gA + 4 * N * r])
    tv = _f32(arena0, dt, M * r).reshape(M, r)
    am = _f32(arena0, A, N * r).reshape(N, r).T
    base_mag = np.abs(_f32(split, s2, M * N).reshape(M, N) - tv @ am)   # |acc + product|
    _check(fused, split, s2, M, N, tv, am, 1.0, base_mag + np.abs(_f32(arena0, acc, M * N).reshape(M, N)))


def test_pattern_is_left_alone_when_an_intermediate_is_read_later():
    M, K, N = SIZES[0]
    r = 16
    rng = np.random.default_rng(3)
    a = Arena(rng)
    x = a.alloc(M * K, "normal")
    w = a.ro_alloc(rng.integers(-127, 128, size=K * N, dtype=np.int8))
    sc = a.ro_alloc((rng.random(N) * 0.01 + 1e-3).astype(np.float32))
    A = a.alloc(K * r, "normal"); Bm = a.alloc(r * N, "normal")
    base = a.alloc(M * N); t = a.alloc(M * r); out = a.alloc(M * N); keep = a.alloc(M * N)
    prog = [
        P.Instr(Op.GEMM_NN_Q8, REL | CS, 0, (x, w, base, sc), (M, N, K)),
        P.Instr(Op.GEMM_NN, 0, 0, (x, A, t, P.NULL_REF), (M, r, K)),
        P.Instr(Op.GEMM_NN, ADDEND, 0, (t, Bm, out, base), (M, N, r)),
        P.Instr(Op.COPY, 0, 0, (base, keep), (M * N, 0, 0)),      # the un-adapted product is still wanted
        P.Instr(Op.FILL, 0, 0, (base, P.f32_bits(0.0)), (M * N, 0, 0)),
    ]
    arena0, ro = a.build()
    fused, c_fused = _run(prog, arena0, ro, True)
    split, c_split = _run(prog, arena0, ro, False)
    assert c_fused.fused_dispatches == 0
    assert np.array_equal(fused, split)


def test_adapter_products_with_contracted_multiply_adds():
    """In lazy coherence the rank-r products run with fused multiply-adds (same
    kernels and reduction order, one rounding per term instead of two).  Held to
    the reference's bound for its own GEMMs against a float64 sum, |got - sum| /
    (1 + sum|a_k b_k|) < 2e-6; identical run to run; and with the knob off the
    bits of the strict seam."""
    M, K, r = 4096, 768, 16
    rng = np.random.default_rng(99)
    a = Arena(rng)
    x = a.alloc(M * K, "normal")
    dy = a.alloc(M * K, "normal")
    A = a.alloc(K * r, "normal", scale=0.05)        # [K, r]
    Bt = a.alloc(r * K, "normal", scale=0.05)       # [r, K]: B of an adapter whose width is K
    t = a.alloc(M * r); dt = a.alloc(M * r); gB = a.alloc(r * K); gA = a.alloc(K * r)
    s = 2.0
    prog = [
        P.Instr(Op.GEMM_NN, 0, 0, (x, A, t, P.NULL_REF), (M, r, K)),                      # t = x A
        P.Instr(Op.GEMM_NT, 0, P.f32_bits(s), (dy, Bt, dt, P.NULL_REF), (M, r, K)),       # dT = s dY B^T
        P.Instr(Op.GEMM_TN, 0, P.f32_bits(s), (t, dy, gB, P.NULL_REF), (r, K, M)),        # dB = s t^T dY
        P.Instr(Op.GEMM_TN, 0, 0, (x, dt, gA, P.NULL_REF), (K, r, M)),                    # dA = x^T dT
    ]
    arena0, ro = a.build()

    def run(coherence, fma):
        arena = arena0.copy()
        be = B.CudaBackend(0)
        be.set_coherence(coherence)
        be.set_adapter_fma(fma)
        be.bind(arena, ro)
        be.run(prog)
        be.host_needs(0, arena.size)
        be.flush()
        be.close()
        return arena

    strict = run(B.COHERENCE_STRICT, True)
    fast1 = run(B.COHERENCE_LAZY, True)
    fast2 = run(B.COHERENCE_LAZY, True)
    lazy_exact = run(B.COHERENCE_LAZY, False)
    assert np.array_equal(fast1, fast2)
    assert np.array_equal(lazy_exact, strict)
    X = _f32(arena0, x, M * K).reshape(M, K); DY = _f32(arena0, dy, M * K).reshape(M, K)
    Am = _f32(arena0, A, K * r).reshape(K, r); Bm = _f32(arena0, Bt, r * K).reshape(r, K)
    T = _f32(fast1, t, M * r).reshape(M, r); DT = _f32(fast1, dt, M * r).reshape(M, r)
    cases = [
        ("t", T, X @ Am, np.abs(X) @ np.abs(Am)),
        ("dT", DT, s * (DY @ Bm.T), s * (np.abs(DY) @ np.abs(Bm.T))),
        ("dB", _f32(fast1, gB, r * K).reshape(r, K), s * (T.T @ DY), s * (np.abs(T.T) @ np.abs(DY))),
        ("dA", _f32(fast1, gA, K * r).reshape(K, r), X.T @ DT, np.abs(X.T) @ np.abs(DT)),
    ]
    differs = False
    for name, got, want, mag in cases:
        err = np.abs(got - want) / (1.0 + mag)
        assert err.max() < 2e-6, (name, err.max())
    for off, n in ((t, M * r), (dt, M * r), (gB, r * K), (gA, K * r)):
        differs = differs or not np.array_equal(fast1[off:off + 4 * n], strict[off:off + 4 * n])
    assert differs, "the contracted kernels gave the exact kernels' bits: did they run?"


@pytest.mark.parametrize("shape", [(4096, 768, 16), (4100, 768, 8), (1000, 256, 8), (8200, 768, 16), (16400, 768, 16)],
                         ids=["4096x768r16", "4100x768r8-ragged", "1000x256r8", "8200x768r16-four-warps-a-tile",
                              "16400x768r16-two-warps-a-tile"])
def test_one_pass_adapter_backward_and_tensor_core_down_product(shape):
    """In lazy coherence the down product t = x A runs as 3xTF32 on the tensor cores,
    and the three backward products of a site — dT = a dY B^T, dB = a t^T dY,
    dA = x^T dT, three instructions that each stream an activation — run as one
    pass over dY and x.  Held to 2e-6 of 1 + sum|a_k b_k| against float64 (the
    reference's bound for its own GEMMs); identical run to run; the strict seam
    keeps the exact kernels' bits.  The row counts cover the down product's forms for a
    data-parallel rank's share of the rows (16, 8, 4 and 2 warps sharing a 16-row tile)."""
    M, D, r = shape
    rng = np.random.default_rng(M + r)
    a = Arena(rng)
    x = a.alloc(M * D, "normal"); dy = a.alloc(M * D, "normal")
    A = a.alloc(D * r, "normal", scale=0.05); Bm = a.alloc(r * D, "normal", scale=0.05)
    acc = a.alloc(M * D, "normal")
    t = a.alloc(M * r); dt = a.alloc(M * r); gB = a.alloc(r * D); gA = a.alloc(D * r); part = a.alloc(M * D)
    s = 2.0
    prog = [
        P.Instr(Op.GEMM_NN, 0, 0, (x, A, t, P.NULL_REF), (M, r, D)),
        P.Instr(Op.GEMM_NT, 0, P.f32_bits(s), (dy, Bm, dt, P.NULL_REF), (M, r, D)),
        P.Instr(Op.GEMM_TN, 0, P.f32_bits(s), (t, dy, gB, P.NULL_REF), (r, D, M)),
        P.Instr(Op.GEMM_NT, ADDEND, 0, (dt, A, part, acc), (M, D, r)),          # what a plan puts in between
        P.Instr(Op.GEMM_TN, 0, 0, (x, dt, gA, P.NULL_REF), (D, r, M)),
    ]
    arena0, ro = a.build()

    def run(coherence, fma=True):
        arena = arena0.copy()
        be = B.CudaBackend(0)
        be.set_coherence(coherence)
        be.set_adapter_fma(fma)
        be.bind(arena, ro)
        be.run(prog)
        be.host_needs(0, arena.size)
        be.flush()
        c = be.counters()
        be.close()
        return arena, c

    strict, _ = run(B.COHERENCE_STRICT)
    fast1, c1 = run(B.COHERENCE_LAZY)
    fast2, _ = run(B.COHERENCE_LAZY)
    plain, c0 = run(B.COHERENCE_LAZY, fma=False)
    assert c1.fused_dispatches == 2 and c0.fused_dispatches == 0
    assert np.array_equal(fast1, fast2)
    assert np.array_equal(plain, strict)
    X = _f32(arena0, x, M * D).reshape(M, D); DY = _f32(arena0, dy, M * D).reshape(M, D)
    Am = _f32(arena0, A, D * r).reshape(D, r); Bmm = _f32(arena0, Bm, r * D).reshape(r, D)
    T = _f32(fast1, t, M * r).reshape(M, r); DT = _f32(fast1, dt, M * r).reshape(M, r)
    cases = [
        ("t", T, X @ Am, np.abs(X) @ np.abs(Am)),
        ("dT", DT, s * (DY @ Bmm.T), s * (np.abs(DY) @ np.abs(Bmm.T))),
        ("dB", _f32(fast1, gB, r * D).reshape(r, D), s * (T.T @ DY), s * (np.abs(T.T) @ np.abs(DY))),
        ("dA", _f32(fast1, gA, D * r).reshape(D, r), X.T @ DT, np.abs(X.T) @ np.abs(DT)),
    ]
    worst = {name: float((np.abs(got - want) / (1.0 + mag)).max()) for name, got, want, mag in cases}
    assert max(worst.values()) < 2e-6, worst
    # the expand product in between saw the dT the fused pass wrote
    want_part = _f32(arena0, acc, M * D).reshape(M, D) + DT @ Am.T
    got_part = _f32(fast1, part, M * D).reshape(M, D)
    assert np.abs(got_part - want_part).max() < 1e-4


def test_adapter_backward_on_tcgen05_and_on_the_legacy_instruction_agree():
    """A site of rank 16 with widths that are multiples of 128 takes its three backward
    products on the tcgen05 tensor cores (bf16 pieces: two of the streamed operands, three
    of the small ones); the process-wide switch sends it to the legacy tensor
    instruction's 3xTF32 kernel instead.  Both are held to 2e-6 of 1 + sum|a_k b_k|
    against float64, agree with each other to that, are each identical run to run, and
    differ in bits (which shows that the switch chose between them).  8200 rows: a ragged
    last tile for both."""
    M, D, r = 8200, 768, 16
    rng = np.random.default_rng(4242)
    a = Arena(rng)
    x = a.alloc(M * D, "normal"); dy = a.alloc(M * D, "normal")
    A = a.alloc(D * r, "normal", scale=0.05); Bm = a.alloc(r * D, "normal", scale=0.05)
    t = a.alloc(M * r); dt = a.alloc(M * r); gB = a.alloc(r * D); gA = a.alloc(D * r)
    s = 2.0
    prog = [
        P.Instr(Op.GEMM_NN, 0, 0, (x, A, t, P.NULL_REF), (M, r, D)),
        P.Instr(Op.GEMM_NT, 0, P.f32_bits(s), (dy, Bm, dt, P.NULL_REF), (M, r, D)),
        P.Instr(Op.GEMM_TN, 0, P.f32_bits(s), (t, dy, gB, P.NULL_REF), (r, D, M)),
        P.Instr(Op.GEMM_TN, 0, 0, (x, dt, gA, P.NULL_REF), (D, r, M)),
    ]
    arena0, ro = a.build()

    def run(tensor_backward):
        arena = arena0.copy()
        be = B.CudaBackend(0)
        be.set_adapter_tensor_backward(tensor_backward)
        try:
            be.set_coherence(B.COHERENCE_LAZY)
            be.bind(arena, ro)
            be.run(prog)
            be.host_needs(0, arena.size)
            be.flush()
        finally:
            be.set_adapter_tensor_backward(True)
            be.close()
        return arena

    new1, new2, old1, old2 = run(True), run(True), run(False), run(False)
    assert np.array_equal(new1, new2) and np.array_equal(old1, old2)
    X = _f32(arena0, x, M * D).reshape(M, D); DY = _f32(arena0, dy, M * D).reshape(M, D)
    Bmm = _f32(arena0, Bm, r * D).reshape(r, D)
    differs = False
    for got in (new1, old1):
        T = _f32(got, t, M * r).reshape(M, r); DT = _f32(got, dt, M * r).reshape(M, r)
        cases = [
            ("dT", DT, s * (DY @ Bmm.T), s * (np.abs(DY) @ np.abs(Bmm.T))),
            ("dB", _f32(got, gB, r * D).reshape(r, D), s * (T.T @ DY), s * (np.abs(T.T) @ np.abs(DY))),
            ("dA", _f32(got, gA, D * r).reshape(D, r), X.T @ DT, np.abs(X.T) @ np.abs(DT)),
        ]
        worst = {name: float((np.abs(g - want) / (1.0 + mag)).max()) for name, g, want, mag in cases}
        assert max(worst.values()) < 2e-6, worst
    for off, n in ((dt, M * r), (gB, r * D), (gA, D * r)):
        differs = differs or not np.array_equal(new1[off:off + 4 * n], old1[off:off + 4 * n])
    assert differs, "the switch made no difference: did both kernels run?"
