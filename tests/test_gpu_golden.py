"""Parity of the CUDA executor with the reference CPU executor on the golden
plans (compiled by the reference compiler, traced by the reference probe).

Lockstep: every instruction runs on the GPU from the reference's own bytes (the
arena is reset to the oracle's state after each instruction), and each written
extent is compared with the reference trace — bit for bit for the opcodes in
BIT_EXACT, within rtol 1e-5 of the extent's scale otherwise (2e-2 where an
instruction ran on the bf16 tensor-core path).

Free run: the same sections run back to back with no resets; the persistent
segment, the loss and the merged deltas are compared at the end.
"""

import numpy as np
import pytest

from see_ai_b200 import backend as B
from see_ai_b200 import plan as P
from tests.util import BIT_EXACT, CASES, GEMM_OPS, Case, compare

pytestmark = pytest.mark.gpu

RTOL_F32 = 1e-5
RTOL_RELAXED = 2e-2
ATOL = 1e-7


def _lockstep(case: Case, relaxed_allowed: bool):
    be = B.CudaBackend(0)
    be.set_relaxed_allowed(relaxed_allowed)
    arena = case.plan.stage_arena()
    be.bind(arena, case.rodata)
    if case.source is not None:
        be.bind_source(case.source)
    failures, worst = [], {}
    for run in case.runs:
        for off, n in case.stage_batch(arena, run):
            be.host_wrote(off, n)
        prog = case.plan.section(run["section"])
        be.set_program(prog)
        sp = case.step_params(B.StepParams, run["step"])
        be.begin_range(0, len(prog))
        for (idx, op, _rel, extents) in run["trace"]:
            before = be.counters().relaxed_executions
            be.execute(idx, sp)
            be.flush()
            ran_relaxed = be.counters().relaxed_executions > before
            ins = prog[idx]
            act = (ins.flags & P.FLAG_ACT_MASK) >> P.FLAG_ACT_SHIFT
            exact = op in BIT_EXACT and not ran_relaxed and not (op in GEMM_OPS and act >= 2)
            for off, want in extents:
                got = arena[off:off + len(want)].tobytes()
                if exact:
                    if got != want:
                        ok, ratio = compare(got, want, RTOL_F32, ATOL)
                        failures.append(f"{run['section']}[{idx}] {P.OP_NAMES[op]} @{off:#x}: "
                                        f"bits differ (err/bound {ratio:.3g})")
                else:
                    rtol = RTOL_RELAXED if ran_relaxed else RTOL_F32
                    ok, ratio = compare(got, want, rtol, ATOL)
                    key = P.OP_NAMES[op] + ("*" if ran_relaxed else "")
                    worst[key] = max(worst.get(key, 0.0), ratio)
                    if not ok:
                        failures.append(f"{run['section']}[{idx}] {P.OP_NAMES[op]} @{off:#x}: "
                                        f"err/bound {ratio:.3g}")
                # adopt the oracle's bytes so the next instruction starts from them
                arena[off:off + len(want)] = np.frombuffer(want, dtype=np.uint8)
                be.host_wrote(off, len(want))
        be.end_range()
    be.close()
    return failures, worst


@pytest.mark.parametrize("name", CASES)
def test_lockstep_exact_kernels(name):
    failures, worst = _lockstep(Case(name), relaxed_allowed=False)
    print(name, "worst err/bound per opcode:", {k: round(v, 4) for k, v in worst.items()})
    assert not failures, "\n".join(failures[:20])


def test_lockstep_relaxed_tensor_core_path():
    failures, worst = _lockstep(Case("gpt_tiny_q8_relaxed"), relaxed_allowed=True)
    print("relaxed worst err/bound:", {k: round(v, 4) for k, v in worst.items()})
    assert not failures, "\n".join(failures[:20])


@pytest.mark.parametrize("name", CASES)
def test_free_run_matches_reference_final_state(name):
    case = Case(name)
    be = B.CudaBackend(0)
    be.set_relaxed_allowed(False)
    arena = case.plan.stage_arena()
    be.bind(arena, case.rodata)
    if case.source is not None:
        be.bind_source(case.source)
    for run in case.runs:
        for off, n in case.stage_batch(arena, run):
            be.host_wrote(off, n)
        be.run(case.plan.section(run["section"]), case.step_params(B.StepParams, run["step"]))
    be.close()
    h = case.header
    ref = case.final_arena
    # loss slot (of the eval run) and the persistent segment (adapters + moments)
    ok, ratio = compare(arena[h["loss_ref"]:h["loss_ref"] + 4].tobytes(),
                        ref[h["loss_ref"]:h["loss_ref"] + 4].tobytes(), 1e-5, 1e-7)
    assert ok, f"loss err/bound {ratio}"
    ok, ratio = compare(arena[:h["persistent_size"]].tobytes(),
                        ref[:h["persistent_size"]].tobytes(), 1e-3, 1e-7)
    assert ok, f"persistent segment err/bound {ratio}"
    for e in case.plan.emit:
        ok, ratio = compare(arena[e.arena_offset:e.arena_offset + e.byte_size].tobytes(),
                            ref[e.arena_offset:e.arena_offset + e.byte_size].tobytes(), 1e-3, 1e-7)
        assert ok, f"merged delta err/bound {ratio}"
