"""Tensor-core (tcgen05) tiled attention against the CPU oracle's exact tiled
family.  The chain is the one a plan carries: kAttnFwdTiled, then kAttnDQTiled
(writes delta), kAttnDKTiled (reads delta), kAttnDVTiled, all with the relaxed
permission.  Q, K, V and dO are bf16-representable, so the two sides see the
same operands; what differs is P and dS rounded to bf16 for their second
product and the f32 summation order.  Each output tensor is held to 1e-2 of its
own scale (the plan format promises 2e-2 for relaxed instructions)."""

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

GEOMS = [(2, 128, 1, 64), (2, 256, 3, 64), (1, 384, 2, 128), (1, 200, 2, 64), (1, 512, 12, 64)]


def setup_module(_m):
    if not oracle.have_oracle():
        oracle.build("oracle")


def build(rng, Bq, S, H, d):
    a = Arena(rng)
    td = Bq * S * H * d
    t = {}
    for name in ("q", "k", "v", "do"):
        t[name] = a.alloc(td, bf16_round(rng.standard_normal(td).astype(np.float32)))
    for name in ("o", "dq", "dk", "dv"):
        t[name] = a.alloc(td)
    t["stats"] = a.alloc(Bq * H * S * 4)
    bs, hd = P.pack2(Bq, S), P.pack2(H, d)
    geo = P.pack_attn_geometry(Bq, S, H, d)

    def prog(flags):
        return [
            P.Instr(Op.ATTN_FWD_TILED, flags, 0, (t["q"], t["k"], t["v"], t["o"]), (t["stats"], bs, hd)),
            P.Instr(Op.ATTN_DQ_TILED, flags, 0, (t["q"], t["k"], t["v"], t["do"]), (t["stats"], t["dq"], geo)),
            P.Instr(Op.ATTN_DK_TILED, flags, 0, (t["q"], t["k"], t["v"], t["do"]), (t["stats"], t["dk"], geo)),
            P.Instr(Op.ATTN_DV_TILED, flags, 0, (t["q"], t["k"], t["v"], t["do"]), (t["stats"], t["dv"], geo)),
        ]
    arena, ro = a.build()
    return t, prog, arena, ro, td


@pytest.mark.parametrize("geom", GEOMS, ids=["B%dS%dH%dd%d" % g for g in GEOMS])
def test_relaxed_tiled_attention_chain(geom):
    Bq, S, H, d = geom
    rng = np.random.default_rng(S * 131 + d)
    t, prog, arena, ro, td = build(rng, Bq, S, H, d)
    cpu, gpu = arena.copy(), arena.copy()
    ref = oracle.OracleExecutor()
    ref.bind(cpu, ro)
    ref.run(prog(0))
    be = B.CudaBackend(0)
    be.bind(gpu, ro)
    be.run(prog(REL))
    c = be.counters()
    be.close()
    assert c.relaxed_executions == 4, "the tensor-core attention path did not take this geometry"
    for name in ("o", "dq", "dk", "dv"):
        got = gpu[t[name]:t[name] + 4 * td].view(np.float32)
        want = cpu[t[name]:t[name] + 4 * td].view(np.float32)
        assert np.isfinite(got).all(), name
        err = np.max(np.abs(got - want)) / np.max(np.abs(want))
        assert err < 1e-2, f"{name}: {err:.3g} of scale"
    n = Bq * H * S
    gs = gpu[t["stats"]:t["stats"] + 16 * n].view(np.float32).reshape(n, 4)
    cs = cpu[t["stats"]:t["stats"] + 16 * n].view(np.float32).reshape(n, 4)
    assert np.allclose(gs[:, 0], cs[:, 0], rtol=1e-4, atol=1e-4)      # score max
    assert np.allclose(gs[:, 1], cs[:, 1], rtol=2e-3)                 # 1 / denominator
    assert np.max(np.abs(gs[:, 2] - cs[:, 2])) < 1e-2 * max(1.0, np.max(np.abs(cs[:, 2])))  # delta
    assert np.array_equal(gs[:, 3], cs[:, 3])                         # start (0: no mask)


def test_permission_withheld_runs_the_exact_family_bit_for_bit_on_exact_ops():
    Bq, S, H, d = 1, 128, 2, 64
    rng = np.random.default_rng(3)
    t, prog, arena, ro, td = build(rng, Bq, S, H, d)
    gpu = arena.copy()
    be = B.CudaBackend(0)
    be.set_relaxed_allowed(False)
    be.bind(gpu, ro)
    be.run(prog(REL))
    assert be.counters().relaxed_executions == 0
    be.close()
    cpu = arena.copy()
    ref = oracle.OracleExecutor()
    ref.bind(cpu, ro)
    ref.run(prog(0))
    for name in ("o", "dq", "dk", "dv"):
        got = gpu[t[name]:t[name] + 4 * td].view(np.float32)
        want = cpu[t[name]:t[name] + 4 * td].view(np.float32)
        assert np.max(np.abs(got - want)) <= 1e-5 * np.max(np.abs(want)) + 1e-7, name


@pytest.mark.parametrize("geom", [(1, 4096, 2, 64), (1, 4096, 1, 128)], ids=["S4096d64", "S4096d128"])
def test_longest_sweep_sequence_against_the_exact_family_on_the_device(geom):
    """S = 4096, the attention sweep's longest sequence, at both head widths.
    The CPU oracle would need minutes here; the device's own exact family (held
    to the oracle at the sizes above, and independent per (batch, head)) is the
    reference instead."""
    Bq, S, H, d = geom
    rng = np.random.default_rng(S + d)
    t, prog, arena, ro, td = build(rng, Bq, S, H, d)
    exact, fast = arena.copy(), arena.copy()
    be = B.CudaBackend(0)
    be.set_relaxed_allowed(False)
    be.bind(exact, ro)
    be.run(prog(REL))
    assert be.counters().relaxed_executions == 0
    be.close()
    be = B.CudaBackend(0)
    be.bind(fast, ro)
    be.run(prog(REL))
    assert be.counters().relaxed_executions == 4
    be.close()
    for name in ("o", "dq", "dk", "dv"):
        got = fast[t[name]:t[name] + 4 * td].view(np.float32)
        want = exact[t[name]:t[name] + 4 * td].view(np.float32)
        assert np.isfinite(got).all(), name
        err = np.max(np.abs(got - want)) / np.max(np.abs(want))
        assert err < 1e-2, f"{name}: {err:.3g} of scale"
