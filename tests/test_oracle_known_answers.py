"""Known-answer tests: the hand-computed values the reference's own kernel
tests hold (reference: test/runtime/executor/kernels_test.cc:31-42, 237-310,
379-418, 532-556, 1055-1067, 1411-1422, 1469-1525), restated as one-instruction
programs and put to every executor we have: the C restatement, the reference
executor built from its sources (when present), and — under the gpu mark — the
CUDA backend through the C ABI.  Same inputs, same expected numbers, same
tolerances as the reference's tests."""

import math

import numpy as np
import pytest

import oracle
from see_ai_b200 import plan as P
from tests.test_oracle_pinned import Arena

Op = P.Op
f = P.f32_bits


def setup_module(_m):
    oracle.build("oracle")


class _Cpu:
    def __init__(self, cls):
        self.cls = cls

    def run(self, prog, arena, ro, sp=None):
        ex = self.cls()
        ex.bind(arena, ro)
        ex.run(prog, sp if sp is not None else oracle.step_params())
        return arena


class _Gpu:
    def run(self, prog, arena, ro, sp=None):
        from see_ai_b200 import backend as B
        be = B.CudaBackend(0)
        be.bind(arena, ro)
        if sp is None:
            be.run(prog)
        else:
            be.run(prog, B.StepParams(sp.lr, sp.beta1, sp.beta2, sp.eps, sp.weight_decay, 0, sp.step))
        be.close()
        return arena


def _executors():
    out = [pytest.param(lambda: _Cpu(oracle.OracleExecutor), id="restatement")]
    out.append(pytest.param(lambda: _Cpu(oracle.RefExecutor) if oracle.have_ref() else None, id="reference"))
    out.append(pytest.param(lambda: _Gpu(), id="cuda", marks=pytest.mark.gpu))
    return out


@pytest.fixture(params=_executors())
def ex(request):
    made = request.param()
    if made is None:
        pytest.skip("oracle/_ref is not built (reference tree absent)")
    return made


def _f32(arena, off, n):
    return arena[off:off + 4 * n].view(np.float32)


def test_gemm_nn_hand_product(ex):
    a = Arena(np.random.default_rng(0))
    A = a.alloc(6, [1, 2, 3, 4, 5, 6]); B = a.alloc(6, [7, 8, 9, 10, 11, 12])
    C = a.alloc(4, [-1, -1, -1, -1])   # pre-poisoned: the product overwrites
    arena, ro = a.build()
    ex.run([P.Instr(Op.GEMM_NN, 0, 0, (A, B, C, P.NULL_REF), (2, 2, 3))], arena, ro)
    assert np.allclose(_f32(arena, C, 4), [58, 64, 139, 154], atol=1e-6)


def test_elementwise_hand_values(ex):
    a = Arena(np.random.default_rng(0))
    x = a.alloc(6, [1, 2, 3, 4, 5, 6]); b = a.alloc(3, [10, 20, 30])
    y3 = a.alloc(3, [10, 20, 30]); x3 = a.alloc(3, [1, 2, 3])
    r_in = a.alloc(5, [-2, -0.5, 0, 0.5, 2]); r_out = a.alloc(5)
    dy = a.alloc(4, [1, 1, 1, 1]); px = a.alloc(4, [-1, 0, 0.5, 3]); dx = a.alloc(4)
    s_in = a.alloc(3, [1, -2, 4]); s_out = a.alloc(3)
    red_in = a.alloc(6, [1, 2, 3, 10, 20, 30]); red_out = a.alloc(3, [-99, -99, -99])
    add_out = a.alloc(3); bias_out = a.alloc(6)
    fill = a.alloc(4); copy = a.alloc(4)
    arena, ro = a.build()
    prog = [
        P.Instr(Op.ADD_EW, 0, 0, (x3, y3, add_out, P.NULL_REF), (3, 0, 0)),
        P.Instr(Op.ADD_BIAS, 0, 0, (x, b, bias_out, P.NULL_REF), (2, 3, 0)),
        P.Instr(Op.RELU_FWD, 0, 0, (r_in, r_out), (5, 0, 0)),
        P.Instr(Op.RELU_BWD, 0, 0, (dy, px, dx, P.NULL_REF), (4, 0, 0)),
        P.Instr(Op.SCALE, 0, 0, (s_in, s_out, f(2.5)), (3, 0, 0)),
        P.Instr(Op.REDUCE_ROWS, 0, 0, (red_in, red_out), (2, 3, 0)),
        P.Instr(Op.FILL, 0, 0, (fill, f(3.5)), (4, 0, 0)),
        P.Instr(Op.COPY, 0, 0, (fill, copy), (4, 0, 0)),
    ]
    ex.run(prog, arena, ro)
    assert np.allclose(_f32(arena, add_out, 3), [11, 22, 33], atol=1e-6)
    assert np.allclose(_f32(arena, bias_out, 6), [11, 22, 33, 14, 25, 36], atol=1e-6)
    assert np.array_equal(_f32(arena, r_out, 5), np.float32([0, 0, 0, 0.5, 2]))
    assert np.array_equal(_f32(arena, dx, 4), np.float32([0, 0, 1, 1]))   # subgradient 0 at the kink
    assert np.allclose(_f32(arena, s_out, 3), [2.5, -5.0, 10.0], atol=1e-6)
    assert np.allclose(_f32(arena, red_out, 3), [11, 22, 33], atol=1e-6)
    assert np.array_equal(_f32(arena, copy, 4), np.float32([3.5] * 4))


def test_softmax_xent_uniform_logits_give_log_c(ex):
    a = Arena(np.random.default_rng(0))
    logits = a.alloc(8); labels = a.alloc(2, [0, 3], np.int32)
    loss = a.alloc(1); probs = a.alloc(8)
    arena, ro = a.build()
    ex.run([P.Instr(Op.XENT_FWD, 0, 0, (logits, labels, loss, probs), (2, 4, 0))], arena, ro)
    assert abs(_f32(arena, loss, 1)[0] - math.log(4.0)) < 1e-6
    assert np.allclose(_f32(arena, probs, 8), 0.25, atol=1e-6)


def test_softmax_xent_single_class_is_exactly_certain(ex):
    a = Arena(np.random.default_rng(0))
    logits = a.alloc(3, [2.0, -5.0, 100.0]); labels = a.alloc(3, [0, 0, 0], np.int32)
    loss = a.alloc(1, [-1.0]); probs = a.alloc(3)
    arena, ro = a.build()
    ex.run([P.Instr(Op.XENT_FWD, 0, 0, (logits, labels, loss, probs), (3, 1, 0))], arena, ro)
    assert _f32(arena, loss, 1)[0] == 0.0
    assert np.array_equal(_f32(arena, probs, 3), np.float32([1, 1, 1]))


def test_softmax_xent_backward_is_scaled_probs_minus_one_hot(ex):
    a = Arena(np.random.default_rng(0))
    probs = a.alloc(6, [0.2, 0.3, 0.5, 0.1, 0.8, 0.1]); labels = a.alloc(2, [2, 1], np.int32)
    seed = a.alloc(1, [2.0]); d = a.alloc(6)
    arena, ro = a.build()
    ex.run([P.Instr(Op.XENT_BWD, 0, 0, (probs, labels, seed, d), (2, 3, 0))], arena, ro)
    g = _f32(arena, d, 6)
    assert abs(g[0] - 0.2) < 1e-6 and abs(g[2] - (0.5 - 1.0)) < 1e-6 and abs(g[4] - (0.8 - 1.0)) < 1e-6
    assert abs(g[:3].sum()) < 1e-6 and abs(g[3:].sum()) < 1e-6


def test_mse_forward_and_backward(ex):
    a = Arena(np.random.default_rng(0))
    pred = a.alloc(2, [1, 2]); target = a.alloc(2); loss = a.alloc(1)
    seed = a.alloc(1, [2.0]); dpred = a.alloc(2)
    arena, ro = a.build()
    ex.run([P.Instr(Op.MSE_FWD, 0, 0, (pred, target, loss, P.NULL_REF), (2, 0, 0)),
            P.Instr(Op.MSE_BWD, 0, 0, (pred, target, seed, dpred), (2, 0, 0))], arena, ro)
    assert abs(_f32(arena, loss, 1)[0] - 2.5) < 1e-6           # (1 + 4) / 2
    assert np.allclose(_f32(arena, dpred, 2), [2.0, 4.0], atol=1e-6)


def test_sgd_step_with_decoupled_weight_decay(ex):
    a = Arena(np.random.default_rng(0))
    p = a.alloc(2, [1.0, -2.0]); g = a.alloc(2, [0.5, 0.5])
    arena, ro = a.build()
    sp = oracle.step_params(lr=0.1, weight_decay=0.2, step=1)
    ex.run([P.Instr(Op.SGD_STEP, 0, 0, (p, g), (2, 0, 0))], arena, ro, sp)
    got = _f32(arena, p, 2)
    assert abs(got[0] - (1.0 - 0.1 * (0.5 + 0.2 * 1.0))) < 1e-6
    assert abs(got[1] - (-2.0 - 0.1 * (0.5 + 0.2 * -2.0))) < 1e-6


def test_adamw_first_step_matches_closed_form(ex):
    lr, b1, b2, eps, wd, g0, p0 = 0.01, 0.9, 0.999, 1e-8, 0.1, 0.4, 2.0
    a = Arena(np.random.default_rng(0))
    p = a.alloc(1, [p0]); g = a.alloc(1, [g0]); m = a.alloc(1); v = a.alloc(1)
    arena, ro = a.build()
    sp = oracle.step_params(lr=lr, beta1=b1, beta2=b2, eps=eps, weight_decay=wd, step=1)
    ex.run([P.Instr(Op.ADAMW_STEP, 0, 0, (p, g, m, v), (1, 0, 0))], arena, ro, sp)
    # Expected values in f32 arithmetic, as the reference's test computes them.
    F = np.float32
    assert abs(_f32(arena, m, 1)[0] - (F(1.0) - F(b1)) * F(g0)) < 1e-7
    assert abs(_f32(arena, v, 1)[0] - (F(1.0) - F(b2)) * F(g0) * F(g0)) < 1e-9
    expected = F(p0) - F(lr) * (F(g0) / (np.sqrt(F(g0) * F(g0)) + F(eps)) + F(wd) * F(p0))
    assert abs(_f32(arena, p, 1)[0] - expected) < 1e-6


def test_layernorm_zero_variance_row_normalizes_to_beta(ex):
    a = Arena(np.random.default_rng(0))
    x = a.alloc(4, [7.25] * 4); gamma = a.alloc(4, [2.0] * 4); beta = a.alloc(4, [0.5, -1.0, 3.0, 0.0])
    y = a.alloc(4); mean = a.alloc(1); rstd = a.alloc(1)
    arena, ro = a.build()
    ex.run([P.Instr(Op.LAYERNORM_FWD, 0, 0, (x, gamma, beta, y), (P.pack2(1, 4), mean, rstd))], arena, ro)
    assert np.array_equal(_f32(arena, y, 4), np.float32([0.5, -1.0, 3.0, 0.0]))   # bit for bit


def test_embed_gathers_table_rows_by_token_id(ex):
    a = Arena(np.random.default_rng(0))
    table = a.ro_alloc(np.float32([0, 1, 2, 10, 11, 12, 20, 21, 22, 30, 31, 32]))
    tokens = a.alloc(4, [2, 0, 3, 0], np.int32); out = a.alloc(12, [-1.0] * 12)
    arena, ro = a.build()
    ex.run([P.Instr(Op.EMBED_FWD, 0, 0, (tokens, table, out), (4, P.pack2(4, 3), 0))], arena, ro)
    assert np.array_equal(_f32(arena, out, 12), np.float32([20, 21, 22, 0, 1, 2, 30, 31, 32, 0, 1, 2]))


def test_rope_golden_values_pin_the_convention(ex):
    rng = np.random.default_rng(72)
    xv = rng.standard_normal(8).astype(np.float32)   # B=1, S=2, H=1, d=4
    a = Arena(rng)
    x = a.alloc(8, xv); y = a.alloc(8)
    arena, ro = a.build()
    ex.run([P.Instr(Op.ROPE_FWD, 0, 0, (x, y, P.NULL_REF), (P.pack2(1, 2), P.pack2(1, 4), f(10000.0)))],
           arena, ro)
    got = _f32(arena, y, 8)
    r1 = 4   # position 1; theta(s, pair p) = s * base^(-2p/d), rotation [[cos,-sin],[sin,cos]]
    for pair, theta in ((0, 1.0), (1, 0.01)):
        x0, x1 = float(xv[r1 + 2 * pair]), float(xv[r1 + 2 * pair + 1])
        assert abs(got[r1 + 2 * pair] - (x0 * math.cos(theta) - x1 * math.sin(theta))) < 1e-5
        assert abs(got[r1 + 2 * pair + 1] - (x0 * math.sin(theta) + x1 * math.cos(theta))) < 1e-5
    assert np.array_equal(got[:4], xv[:4])   # position 0 is not rotated


def test_attention_single_token_sequence_is_identity_over_v(ex):
    rng = np.random.default_rng(130)
    B, S, H, d = 2, 1, 2, 3
    n = B * S * H * d
    a = Arena(rng)
    q = a.alloc(n, "normal"); k = a.alloc(n, "normal"); v = a.alloc(n, "normal")
    o = a.alloc(n); p = a.alloc(B * H * S * S)
    arena, ro = a.build()
    ex.run([P.Instr(Op.ATTN_FWD, 0, 0, (q, k, v, o), (p, P.pack2(B, S), P.pack2(H, d)))], arena, ro)
    assert np.array_equal(_f32(arena, p, B * H), np.float32([1.0] * (B * H)))
    assert np.array_equal(_f32(arena, o, n), _f32(arena, v, n))
