"""Twin test (the reference's RunTwin pattern, test/runtime/executor/
metal_backend_test.cc:365-404): the same instruction list over the same arena
and rodata bytes on the CPU oracle and on the CUDA backend, one instruction at
a time from the oracle's bytes.  Covers opcodes, flags and ragged shapes the
compiled golden plans do not reach (MSE, KL, masked cross-entropy, fused map,
segment mask, scale, copy, reduce-rows, 1x1x1 and K%4 / K%8 tails)."""

import numpy as np
import pytest

import oracle
from see_ai_b200 import backend as B
from see_ai_b200 import plan as P
from tests.test_oracle_pinned import PROGRAMS
from tests.util import BIT_EXACT, GEMM_OPS, compare

pytestmark = pytest.mark.gpu


def setup_module(_m):
    if not oracle.have_oracle():
        oracle.build("oracle")


@pytest.mark.parametrize("entry", PROGRAMS, ids=[p[0] for p in PROGRAMS])
def test_twin_lockstep(entry):
    name, prog, arena0, ro = entry
    cpu, gpu = arena0.copy(), arena0.copy()
    ref = oracle.OracleExecutor()
    ref.bind(cpu, ro)
    be = B.CudaBackend(0)
    be.bind(gpu, ro)
    be.set_program(prog)
    sp_c = oracle.step_params(lr=1e-2, step=3)
    sp_g = B.StepParams(1e-2, 0.9, 0.999, 1e-8, 0.01, 0, 3)
    be.begin_range(0, len(prog))
    failures = []
    for i, ins in enumerate(prog):
        ref.run(prog, sp_c, i, i + 1)
        be.execute(i, sp_g)
        be.flush()
        act = (ins.flags & P.FLAG_ACT_MASK) >> P.FLAG_ACT_SHIFT
        exact = ins.opcode in BIT_EXACT and not (ins.opcode in GEMM_OPS and act >= 2)
        if exact:
            if not np.array_equal(cpu, gpu):
                bad = np.flatnonzero(cpu != gpu)
                failures.append(f"[{i}] {P.OP_NAMES[ins.opcode]}: bits differ at byte {bad[0]}")
        else:
            diff = np.flatnonzero(cpu != gpu)
            if diff.size:
                lo, hi = diff[0] // 4 * 4, diff[-1] // 4 * 4 + 4
                ok, ratio = compare(gpu[lo:hi].tobytes(), cpu[lo:hi].tobytes(), 1e-5, 1e-7)
                if not ok:
                    failures.append(f"[{i}] {P.OP_NAMES[ins.opcode]}: err/bound {ratio:.3g}")
        gpu[:] = cpu  # adopt the oracle's bytes
        be.host_wrote(0, gpu.size)
    be.close()
    assert not failures, "\n".join(failures)


def test_refusals_match_reference_wording():
    """Non-finite gradient norm under a clip: the step is refused, parameters and
    moments untouched, same words as the CPU executor (reference:
    runtime/executor/backend.h:72-80)."""
    rng = np.random.default_rng(3)
    n = 100
    arena = np.zeros(4096, dtype=np.uint8)
    f32 = arena.view(np.float32)
    f32[0:n] = rng.standard_normal(n)          # p
    f32[128:128 + n] = rng.standard_normal(n)  # g
    f32[128 + 5] = np.inf
    f32[256:256 + n] = 0.01                    # m
    f32[384:384 + n] = 0.001                   # v
    prog = [P.Instr(P.Op.ADAMW_STEP, 0, 0, (0, 512, 1024, 1536), (n, P.f32_bits(1.0), 0))]
    cpu, gpu = arena.copy(), arena.copy()
    ref = oracle.OracleExecutor()
    ref.bind(cpu, None)
    with pytest.raises(RuntimeError) as e_cpu:
        ref.run(prog, oracle.step_params())
    be = B.CudaBackend(0)
    be.bind(gpu, None)
    with pytest.raises(B.Refusal) as e_gpu:
        be.run(prog, B.StepParams(1e-3, 0.9, 0.999, 1e-8, 0.01, 0, 1))
    assert "gradient norm is not finite" in str(e_gpu.value)
    assert str(e_gpu.value).split(": ", 1)[-1] in str(e_cpu.value) or \
        "gradient norm is not finite" in str(e_cpu.value)
    assert np.array_equal(cpu, arena) and np.array_equal(gpu, arena)
    # the flag clears after it is reported: a finite step then runs
    gpu.view(np.float32)[128 + 5] = 0.5
    be.host_wrote(0, gpu.size)
    be.run(prog, B.StepParams(1e-3, 0.9, 0.999, 1e-8, 0.01, 0, 1))
    assert not np.array_equal(gpu[:400], arena[:400])
    # a bad clip threshold is refused before anything is launched
    bad = [P.Instr(P.Op.CLIP_NORM, 0, 0, (512, P.f32_bits(-1.0)), (n, 0, 0))]
    with pytest.raises(B.Refusal) as e2:
        be.run(bad, B.StepParams(1e-3, 0.9, 0.999, 1e-8, 0.01, 0, 1))
    assert "clip threshold" in str(e2.value)
    be.close()


def test_unknown_opcode_and_out_of_bounds_are_errors_not_faults():
    arena = np.zeros(4096, dtype=np.uint8)
    be = B.CudaBackend(0)
    be.bind(arena, None)
    with pytest.raises(B.BackendError):
        be.run([P.Instr(99, 0, 0, (0, 0, 0, 0), (1, 0, 0))])
    with pytest.raises(B.BackendError):  # count runs past the arena
        be.run([P.Instr(P.Op.ADD_EW, 0, 0, (0, 64, 128, P.NULL_REF), (4096, 0, 0))])
    with pytest.raises(B.BackendError):  # rodata ref with no rodata bound
        be.run([P.Instr(P.Op.COPY, 0, 0, (P.RODATA_BIT, 0), (4, 0, 0))])
    be.run([P.Instr(P.Op.NOP)])  # and the backend is still usable
    be.close()


def test_split_k_adapter_gradients_fixed_order():
    """Transposed-A products with a small output and a long reduction (the LoRA
    dA / dB shapes: K = batch rows) run split over K in fixed 256-row chunks.
    Not the CPU's bits, but held to the reference's own GEMM accuracy metric
    (|got - want| / (1 + sum|a_k b_k|) < 2e-6; reference:
    test/runtime/executor/kernels_test.cc:1803-1822) and identical run to run."""
    rng = np.random.default_rng(77)
    from tests.test_oracle_pinned import Arena
    for (M, N, K) in [(16, 96, 4096), (200, 16, 3000), (8, 8, 1024), (16, 64, 1027), (70, 12, 1030)]:
        a = Arena(rng)
        At = a.alloc(K * M, "normal"); Bm = a.alloc(K * N, "normal"); D = a.alloc(M * N, "normal")
        o1, o2 = a.alloc(M * N), a.alloc(M * N)
        prog = [P.Instr(P.Op.GEMM_TN, 0, P.f32_bits(2.0), (At, Bm, o1, P.NULL_REF), (M, N, K)),
                P.Instr(P.Op.GEMM_TN, P.FLAG_GEMM_ADDEND, 0, (At, Bm, o2, D), (M, N, K))]
        arena, ro = a.build()
        cpu = arena.copy()
        ref = oracle.OracleExecutor()
        ref.bind(cpu, ro)
        ref.run(prog)
        runs = []
        for _ in range(2):
            gpu = arena.copy()
            be = B.CudaBackend(0)
            be.bind(gpu, ro)
            be.run(prog)
            be.close()
            runs.append(gpu)
        assert np.array_equal(runs[0], runs[1])
        A_np = arena[At:At + 4 * K * M].view(np.float32).astype(np.float64).reshape(K, M)
        B_np = arena[Bm:Bm + 4 * K * N].view(np.float32).astype(np.float64).reshape(K, N)
        mag = np.abs(A_np).T @ np.abs(B_np)
        for off, scale in ((o1, 2.0), (o2, 1.0)):
            got = runs[0][off:off + 4 * M * N].view(np.float32).astype(np.float64).reshape(M, N)
            want = cpu[off:off + 4 * M * N].view(np.float32).astype(np.float64).reshape(M, N)
            assert (np.abs(got - want) / (1.0 + scale * mag)).max() < 2e-6
