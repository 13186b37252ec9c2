"""The tensor-core (tcgen05) GEMM path against the CPU oracle.

Operands are pre-rounded to bf16-representable values, so the relaxed kernel
(activation rounded to bf16, weight exact, f32 accumulate) and the exact CPU
kernels see identical numbers and differ only in summation order.  The bound is
the reference's own scaled metric for its GEMMs (reference:
test/runtime/executor/kernels_test.cc:1803-1822): |got - want| / (1 + sum|a_k b_k|)
below 2e-6.  A second test feeds unrounded activations and holds the result to
the relaxed tolerance the plan format promises (2e-2 of the tensor's scale).
"""

import numpy as np
import pytest

import oracle
from see_ai_b200 import backend as B
from see_ai_b200 import plan as P
from tests.test_oracle_pinned import Arena

pytestmark = pytest.mark.gpu
Op = P.Op
REL = P.FLAG_RELAXED


def setup_module(_m):
    if not oracle.have_oracle():
        oracle.build("oracle")


def bf16_round(x: np.ndarray) -> np.ndarray:
    b = x.astype(np.float32).view(np.uint32).astype(np.uint64)
    b = (b + 0x7FFF + ((b >> 16) & 1)) & 0xFFFF0000
    return b.astype(np.uint32).view(np.float32)


# (CTA pairs, which need a far larger product, are held to the single-CTA bits by a test below.)
# The last three are shard-sized: too few 128 x 256 tiles for every SM, so the persistent kernel
# takes them on 128-wide tiles (or on one wide tile per CTA), ragged edges included.
SHAPES = [(64, 16, 64), (128, 128, 64), (256, 384, 512), (200, 132, 72), (512, 768, 768),
          (130, 260, 200), (1000, 64, 3072), (4096, 768, 768), (2500, 780, 320), (9000, 520, 192)]


def build_case(rng, M, N, K, pre_round=True):
    a = Arena(rng)
    A_np = rng.standard_normal((M, K)).astype(np.float32)
    if pre_round:
        A_np = bf16_round(A_np)
    A = a.alloc(M * K, A_np)
    D_np = rng.standard_normal((M, N)).astype(np.float32)
    D = a.alloc(M * N, D_np)
    Wf = bf16_round(rng.standard_normal((K, N)).astype(np.float32) * 0.05)
    Wft = np.ascontiguousarray(Wf.T)
    q = rng.integers(-127, 128, size=(K, N), dtype=np.int8)
    qt = np.ascontiguousarray(q.T)
    csn = (rng.random(N) * 0.02 + 1e-3).astype(np.float32)
    csk = (2.0 ** rng.integers(-8, -3, size=K)).astype(np.float32)  # powers of two: A*s stays bf16
    bias_np = rng.standard_normal(N).astype(np.float32)
    r = dict(Wf=a.ro_alloc(Wf), Wft=a.ro_alloc(Wft), q=a.ro_alloc(q), qt=a.ro_alloc(qt),
             csn=a.ro_alloc(csn), csk=a.ro_alloc(csk), bias=a.ro_alloc(bias_np),
             bf=a.ro_alloc((Wf.view(np.uint32) >> 16).astype(np.uint16)),
             bft=a.ro_alloc((Wft.view(np.uint32) >> 16).astype(np.uint16)))
    outs = [a.alloc(M * N) for _ in range(8)]
    dims = (M, N, K)
    f = P.f32_bits
    variants = [
        ("nn.f32+bias+relu", Op.GEMM_NN, P.FLAG_EPILOGUE_BIAS | (P.ACT_RELU << 1), (A, r["Wf"], outs[0], r["bias"])),
        ("nn.f32+addend", Op.GEMM_NN, P.FLAG_GEMM_ADDEND, (A, r["Wf"], outs[1], D)),
        ("nt.f32", Op.GEMM_NT, 0, (A, r["Wft"], outs[2], P.NULL_REF)),
        ("nn.q8.tensor", Op.GEMM_NN_Q8, 0, (A, r["q"], outs[3], f(0.0078125))),
        ("nn.q8.cols+gelu", Op.GEMM_NN_Q8, P.FLAG_Q8_COL_SCALE | (P.ACT_GELU << 1), (A, r["q"], outs[4], r["csn"])),
        ("nt.q8.cols", Op.GEMM_NT_Q8, P.FLAG_Q8_COL_SCALE, (A, r["qt"], outs[5], r["csk"])),
        ("nn.bf16+bias", Op.GEMM_NN_BF16, P.FLAG_EPILOGUE_BIAS, (A, r["bf"], outs[6], r["bias"])),
        ("nt.bf16", Op.GEMM_NT_BF16, 0, (A, r["bft"], outs[7], P.NULL_REF)),
    ]
    absA = np.abs(A_np.astype(np.float64))
    mags = {
        "f32": absA @ np.abs(Wf.astype(np.float64)),
        "q8t": absA @ np.abs(q.astype(np.float64)) * 0.0078125,
        "q8n": absA @ np.abs(q.astype(np.float64)) * csn.astype(np.float64),
        "q8k": (absA * csk.astype(np.float64)) @ np.abs(q.astype(np.float64)),
    }
    mag_of = {"nn.f32+bias+relu": "f32", "nn.f32+addend": "f32", "nt.f32": "f32",
              "nn.q8.tensor": "q8t", "nn.q8.cols+gelu": "q8n", "nt.q8.cols": "q8k",
              "nn.bf16+bias": "f32", "nt.bf16": "f32"}
    arena, ro = a.build()
    return variants, dims, outs, arena, ro, mags, mag_of


@pytest.mark.parametrize("shape", SHAPES, ids=[f"{m}x{n}x{k}" for m, n, k in SHAPES])
def test_tensor_core_gemm_matches_oracle_on_identical_operands(shape):
    M, N, K = shape
    rng = np.random.default_rng(M * 1000003 + N * 1009 + K)
    variants, dims, outs, arena, ro, mags, mag_of = build_case(rng, M, N, K)
    exact_prog = [P.Instr(op, fl, 0, ins, dims) for (_n, op, fl, ins) in variants]
    relaxed_prog = [P.Instr(op, fl | REL, 0, ins, dims) for (_n, op, fl, ins) in variants]
    cpu, gpu = arena.copy(), arena.copy()
    ref = oracle.OracleExecutor()
    ref.bind(cpu, ro)
    ref.run(exact_prog)
    be = B.CudaBackend(0)
    be.bind(gpu, ro)
    be.run(relaxed_prog)
    c = be.counters()
    be.close()
    assert c.relaxed_executions == len(variants), "the tensor-core path did not take these shapes"
    for (name, _op, _fl, _ins), off in zip(variants, outs):
        got = gpu[off:off + 4 * M * N].view(np.float32).astype(np.float64).reshape(M, N)
        want = cpu[off:off + 4 * M * N].view(np.float32).astype(np.float64).reshape(M, N)
        scaled = np.abs(got - want) / (1.0 + mags[mag_of[name]])
        assert np.isfinite(got).all(), name
        assert scaled.max() < 2e-6, f"{name}: scaled error {scaled.max():.3g}"


def test_cta_pair_tiles_give_the_single_cta_bits():
    """A product large enough for CTA pairs (two SMs per 256 x 256 tile) computes the same products in the
    same order as one CTA per 128 x 256 tile: identical bits, ragged edges in both directions included."""
    M, N, K = 10300, 1028, 1600
    rng = np.random.default_rng(99)
    variants, dims, outs, arena, ro, _mags, _mag_of = build_case(rng, M, N, K)
    prog = [P.Instr(op, fl | REL, 0, ins, dims) for (_n, op, fl, ins) in variants]
    images = []
    for pairs in (True, False):
        img = arena.copy()
        be = B.CudaBackend(0)
        be.set_cta_pairs(pairs)
        be.bind(img, ro)
        be.run(prog)
        c = be.counters()
        be.set_cta_pairs(True)
        be.close()
        assert c.relaxed_executions == len(variants)
        images.append(img)
    for (name, _op, _fl, _ins), off in zip(variants, outs):
        assert np.array_equal(images[0][off:off + 4 * M * N], images[1][off:off + 4 * M * N]), name


def test_relaxed_rounding_stays_within_plan_tolerance():
    """Unrounded activations: the relaxed result differs from the exact one by
    the bf16 rounding of A, within 2e-2 of the output's scale."""
    M, N, K = 384, 256, 1024
    rng = np.random.default_rng(5)
    variants, dims, outs, arena, ro, _mags, _ = build_case(rng, M, N, K, pre_round=False)
    exact_prog = [P.Instr(op, fl, 0, ins, dims) for (_n, op, fl, ins) in variants]
    relaxed_prog = [P.Instr(op, fl | REL, 0, ins, dims) for (_n, op, fl, ins) in variants]
    cpu, gpu, gpu_exact = arena.copy(), arena.copy(), arena.copy()
    ref = oracle.OracleExecutor()
    ref.bind(cpu, ro)
    ref.run(exact_prog)
    be = B.CudaBackend(0)
    be.bind(gpu, ro)
    be.run(relaxed_prog)
    assert be.counters().relaxed_executions == len(variants)
    # the permission is not a demand: with it withheld the exact kernels run, bit for bit
    be2 = B.CudaBackend(0)
    be2.set_relaxed_allowed(False)
    be2.bind(gpu_exact, ro)
    be2.run(relaxed_prog)
    assert be2.counters().relaxed_executions == 0
    for (name, op, fl, _ins), off in zip(variants, outs):
        got = gpu[off:off + 4 * M * N].view(np.float32)
        want = cpu[off:off + 4 * M * N].view(np.float32)
        err = np.max(np.abs(got - want)) / np.max(np.abs(want))
        assert err < 2e-2, f"{name}: {err}"
        assert err > 0, f"{name}: relaxed path produced the exact bits — did it run?"
        if ((fl & P.FLAG_ACT_MASK) >> 1) < 2:
            assert np.array_equal(gpu_exact[off:off + 4 * M * N], cpu[off:off + 4 * M * N]), name
    be.close()
    be2.close()


def test_activation_copy_is_invalidated_by_writes():
    """Two relaxed GEMMs read the same arena range with a write in between: the
    second must see the new values (the cached bf16 copy is dropped)."""
    M, N, K = 128, 128, 128
    rng = np.random.default_rng(9)
    a = Arena(rng)
    A = a.alloc(M * K, bf16_round(rng.standard_normal(M * K).astype(np.float32)))
    A2 = a.alloc(M * K, bf16_round(rng.standard_normal(M * K).astype(np.float32)))
    W = a.ro_alloc(bf16_round(rng.standard_normal((K, N)).astype(np.float32)))
    o1, o2, o3 = a.alloc(M * N), a.alloc(M * N), a.alloc(M * N)
    prog = [
        P.Instr(Op.GEMM_NN, REL, 0, (A, W, o1, P.NULL_REF), (M, N, K)),
        P.Instr(Op.GEMM_NN, REL, 0, (A, W, o2, P.NULL_REF), (M, N, K)),   # cached copy reused
        P.Instr(Op.COPY, 0, 0, (A2, A), (M * K, 0, 0)),                   # overwrite A
        P.Instr(Op.GEMM_NN, REL, 0, (A, W, o3, P.NULL_REF), (M, N, K)),
    ]
    arena, ro = a.build()
    cpu, gpu = arena.copy(), arena.copy()
    ref = oracle.OracleExecutor()
    ref.bind(cpu, ro)
    ref.run([P.Instr(i.opcode, i.flags & ~REL, i.imm, i.ins, i.out) for i in prog])
    be = B.CudaBackend(0)
    be.bind(gpu, ro)
    be.run(prog)
    be.close()
    for off in (o1, o2, o3):
        got = gpu[off:off + 4 * M * N].view(np.float32)
        want = cpu[off:off + 4 * M * N].view(np.float32)
        assert np.max(np.abs(got - want)) < 1e-3 * np.max(np.abs(want))
    assert np.array_equal(gpu[o1:o1 + 4 * M * N], gpu[o2:o2 + 4 * M * N])
    assert not np.array_equal(gpu[o1:o1 + 4 * M * N], gpu[o3:o3 + 4 * M * N])


@pytest.mark.parametrize("K", [768, 3072])
def test_transposed_int8_product_with_real_reduction_axis_scales(K):
    """dX = (dY * s_k) W^T with per-column scales as a quantiser produces them
    (max|col| / 127 of N(0, 0.02) weights: not powers of two).  The tensor-core
    path folds s_k into its bf16 weight copy, w = bf16(W[n,k] * s[k]), a
    rounding the exact kernels do not have: the result must still stay within the
    relaxed tolerance of the exact one, and well inside it in the mean."""
    M, N = 256, 384
    rng = np.random.default_rng(K)
    a = Arena(rng)
    A_np = rng.standard_normal((M, K)).astype(np.float32)
    A = a.alloc(M * K, A_np)
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)        # [N, K]: W^T rows; column k of W is w[:, k]
    scale = (np.abs(w).max(axis=0) / np.float32(127.0)).astype(np.float32)
    q = np.clip(np.round(w / scale), -127, 127).astype(np.int8)
    qt = a.ro_alloc(q)
    csk = a.ro_alloc(scale)
    out = a.alloc(M * N)
    ins = (A, qt, out, csk)
    arena, ro = a.build()
    cpu, gpu = arena.copy(), arena.copy()
    ref = oracle.OracleExecutor()
    ref.bind(cpu, ro)
    ref.run([P.Instr(Op.GEMM_NT_Q8, P.FLAG_Q8_COL_SCALE, 0, ins, (M, N, K))])
    be = B.CudaBackend(0)
    be.bind(gpu, ro)
    be.run([P.Instr(Op.GEMM_NT_Q8, P.FLAG_Q8_COL_SCALE | REL, 0, ins, (M, N, K))])
    assert be.counters().relaxed_executions == 1
    be.close()
    got = gpu[out:out + 4 * M * N].view(np.float32).astype(np.float64)
    want = cpu[out:out + 4 * M * N].view(np.float32).astype(np.float64)
    worst = np.abs(got - want).max() / np.abs(want).max()
    rms = np.sqrt(np.mean((got - want) ** 2)) / np.sqrt(np.mean(want ** 2))
    assert worst < 2e-2, worst
    assert rms < 5e-3, rms   # two independent bf16 roundings (activation, scaled weight): about 2^-9 each
