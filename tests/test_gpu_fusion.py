"""Bias-add fusion.  When a relaxed GEMM is followed by the kAddBias that consumes
its output and nothing reads the un-biased product before it is overwritten, the
backend (in lazy coherence, the engine's mode) lets the GEMM's epilogue add the
bias and write the kAddBias output; the kAddBias launches nothing.  The fused
range must give the bits of the same program run one instruction per range
(where nothing can be fused), must launch one kernel less per fused pair, and a
pair whose intermediate IS read later must be left alone."""

import numpy as np
import pytest

from see_ai_b200 import backend as B
from see_ai_b200 import plan as P
from tests.test_oracle_pinned import Arena

pytestmark = pytest.mark.gpu
Op = P.Op
REL = P.FLAG_RELAXED
CS = P.FLAG_Q8_COL_SCALE


def _build(rng, read_intermediate_later: bool):
    M, K, N = 256, 128, 192
    a = Arena(rng)
    x = a.alloc(M * K, "normal")
    w = a.ro_alloc(rng.integers(-127, 128, size=K * N, dtype=np.int8))
    sc = a.ro_alloc((rng.random(N) * 0.01 + 1e-3).astype(np.float32))
    bias = a.ro_alloc(rng.standard_normal(N).astype(np.float32))
    r = a.alloc(M * N); z = a.alloc(M * N); g = a.alloc(M * N); keep = a.alloc(M * N)
    prog = [
        P.Instr(Op.GEMM_NN_Q8, REL | CS, 0, (x, w, r, sc), (M, N, K)),
        P.Instr(Op.ADD_BIAS, 0, 0, (r, bias, z, P.NULL_REF), (M, N, 0)),
        P.Instr(Op.GELU_FWD, 0, 0, (z, g), (M * N, 0, 0)),
    ]
    if read_intermediate_later:
        prog.append(P.Instr(Op.COPY, 0, 0, (r, keep), (M * N, 0, 0)))
    prog.append(P.Instr(Op.FILL, 0, 0, (r, P.f32_bits(0.0)), (M * N, 0, 0)))   # R is overwritten
    arena, ro = a.build()
    return prog, arena, ro, (r, 4 * M * N)


def _run(prog, arena0, ro, one_range: bool, one_walk: bool = False):
    arena = arena0.copy()
    be = B.CudaBackend(0)
    be.set_coherence(B.COHERENCE_LAZY)
    be.set_attention_one_walk(one_walk)   # (its own test below: another rounding of delta, not the same bits)
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


@pytest.mark.parametrize("later_read", [False, True], ids=["dead", "read-later"])
def test_bias_add_rides_the_gemm_epilogue_only_when_the_product_is_dead(later_read):
    prog, arena0, ro, (r_off, r_bytes) = _build(np.random.default_rng(5), later_read)
    fused, c_fused = _run(prog, arena0, ro, one_range=True)
    split, c_split = _run(prog, arena0, ro, one_range=False)
    assert np.isfinite(fused.view(np.float32)).all()
    assert np.array_equal(fused, split)       # R ends as zeros either way (the FILL)
    # One conversion is saved in a single range regardless (GELU -> nothing here), so
    # compare launches directly: fused drops exactly the kAddBias kernel.
    saved = c_split.kernel_launches - c_fused.kernel_launches
    assert saved == (0 if later_read else 1)
    assert c_fused.fused_dispatches == (0 if later_read else 1) and c_split.fused_dispatches == 0


# ---- activation absorbed into the producing GEMM's epilogue ---------------------------
# GEMM (-> kAddBias) -> activation -> GEMM: when the activation's f32 output is
# read by nothing but the relaxed GEMM that takes its bf16 copy, the first GEMM's
# epilogue writes that copy and the activation launches nothing.  Sizes: one that
# runs the one-tile kernel and one that runs the persistent kernel.

ACT_SIZES = [(256, 128, 192), (4864, 64, 2048)]


def _build_act_fwd(rng, M, K, N, read_g_later):
    a = Arena(rng)
    x = a.alloc(M * K, "normal")
    w1 = a.ro_alloc(rng.integers(-127, 128, size=K * N, dtype=np.int8))
    sc1 = a.ro_alloc((rng.random(N) * 0.01 + 1e-3).astype(np.float32))
    bias = a.ro_alloc(rng.standard_normal(N).astype(np.float32))
    N2 = 64
    w2 = a.ro_alloc(rng.integers(-127, 128, size=N * N2, dtype=np.int8))
    sc2 = a.ro_alloc((rng.random(N2) * 0.01 + 1e-3).astype(np.float32))
    r = a.alloc(M * N); z = a.alloc(M * N); g = a.alloc(M * N); keep = a.alloc(M * N)
    h = a.alloc(M * N2)
    prog = [
        P.Instr(Op.GEMM_NN_Q8, REL | CS, 0, (x, w1, r, sc1), (M, N, K)),
        P.Instr(Op.ADD_BIAS, 0, 0, (r, bias, z, P.NULL_REF), (M, N, 0)),
        P.Instr(Op.GELU_FWD, 0, 0, (z, g), (M * N, 0, 0)),
        P.Instr(Op.GEMM_NN_Q8, REL | CS, 0, (g, w2, h, sc2), (M, N2, N)),
    ]
    if read_g_later:
        prog.append(P.Instr(Op.COPY, 0, 0, (g, keep), (M * N, 0, 0)))
    prog.append(P.Instr(Op.FILL, 0, 0, (r, P.f32_bits(0.0)), (M * N, 0, 0)))
    prog.append(P.Instr(Op.FILL, 0, 0, (g, P.f32_bits(0.0)), (M * N, 0, 0)))
    arena, ro = a.build()
    return prog, arena, ro


@pytest.mark.parametrize("size", ACT_SIZES, ids=["one-tile", "persistent"])
@pytest.mark.parametrize("later_read", [False, True], ids=["dead", "read-later"])
def test_forward_activation_rides_the_gemm_epilogue_only_when_its_f32_output_is_dead(size, later_read):
    M, K, N = size
    prog, arena0, ro = _build_act_fwd(np.random.default_rng(17), M, K, N, later_read)
    fused, c_fused = _run(prog, arena0, ro, one_range=True)
    split, c_split = _run(prog, arena0, ro, one_range=False)
    assert np.isfinite(fused.view(np.float32)).all()
    assert np.array_equal(fused, split)
    saved = c_split.kernel_launches - c_fused.kernel_launches
    # kAddBias in the epilogue (1) and the second GEMM's conversion pass (1) are
    # saved either way; the activation kernel itself (1) only when g is dead.
    assert saved == (2 if later_read else 3)
    assert c_fused.fused_dispatches == (1 if later_read else 2)   # the bias add, and the activation


def _build_act_bwd(rng, M, K, N, read_dy_later, read_dx_later):
    a = Arena(rng)
    up = a.alloc(M * K, "normal")
    x = a.alloc(M * N, "normal")
    w1 = a.ro_alloc(rng.integers(-127, 128, size=N * K, dtype=np.int8))      # [N][K]
    sck = a.ro_alloc((2.0 ** rng.integers(-9, -5, size=K)).astype(np.float32))
    N2 = 64
    w2 = a.ro_alloc(rng.integers(-127, 128, size=N2 * N, dtype=np.int8))     # [N2][N]
    sc2 = a.ro_alloc((rng.random(N) * 0.01 + 1e-3).astype(np.float32))       # per-k scale of the consumer
    dy = a.alloc(M * N); dx = a.alloc(M * N); keep = a.alloc(M * N); out = a.alloc(M * N2)
    prog = [
        P.Instr(Op.GEMM_NT_Q8, REL | CS, 0, (up, w1, dy, sck), (M, N, K)),
        P.Instr(Op.GELU_BWD, 0, 0, (dy, x, dx, P.NULL_REF), (M * N, 0, 0)),
        P.Instr(Op.GEMM_NT_Q8, REL | CS, 0, (dx, w2, out, sc2), (M, N2, N)),
    ]
    if read_dy_later:
        prog.append(P.Instr(Op.COPY, 0, 0, (dy, keep), (M * N, 0, 0)))
    if read_dx_later:
        prog.append(P.Instr(Op.COPY, 0, 0, (dx, keep), (M * N, 0, 0)))
    prog.append(P.Instr(Op.FILL, 0, 0, (dy, P.f32_bits(0.0)), (M * N, 0, 0)))
    prog.append(P.Instr(Op.FILL, 0, 0, (dx, P.f32_bits(0.0)), (M * N, 0, 0)))
    arena, ro = a.build()
    return prog, arena, ro


@pytest.mark.parametrize("size", ACT_SIZES, ids=["one-tile", "persistent"])
@pytest.mark.parametrize("case", ["dead", "dy-read-later", "dx-read-later"])
def test_backward_activation_rides_the_gemm_epilogue(size, case):
    M, K, N = size
    prog, arena0, ro = _build_act_bwd(np.random.default_rng(23), M, K, N, case == "dy-read-later",
                                      case == "dx-read-later")
    fused, c_fused = _run(prog, arena0, ro, one_range=True)
    split, c_split = _run(prog, arena0, ro, one_range=False)
    assert np.isfinite(fused.view(np.float32)).all()
    assert np.array_equal(fused, split)
    saved = c_split.kernel_launches - c_fused.kernel_launches
    # The consumer's conversion pass is saved either way (producer-made copy); the
    # activation kernel too unless its f32 output is read later.  A dy that is read
    # later is still written by the epilogue (same launches saved).
    assert saved == (1 if case == "dx-read-later" else 2)
    assert c_fused.fused_dispatches == (0 if case == "dx-read-later" else 1)


# ---- the engine's train program: fusions on a whole decoder step ----------------------
# The engine declares its train program a complete step, so scratch activations
# that nothing reads before the next pass rewrites them (GELU outputs, GELU
# backward outputs) may stay unwritten.  Same adapters, moments and losses, bit for
# bit, as the same engine with epilogue fusion switched off — eager, while the
# graphs are captured, and on replay.

def _engine_run(fusion: bool, steps: int = 4, lora_fold: bool = False, one_walk: bool = False):
    import torch
    from see_ai_b200 import synth
    from see_ai_b200.engine import Engine
    cfg = synth.DecoderConfig(layers=2, d_model=128, heads=2, ffn=512, vocab=512, seq=128, batch_seqs=4,
                              rank=8, alpha=16.0, targets=("q", "k", "v", "o"), quantized=True,
                              attention="tiled", lr=1e-2, steps=100, seed=3)
    blob = synth.build_decoder_plan(cfg)
    rng = np.random.default_rng(9)
    stream = torch.cuda.Stream()
    eng = Engine(0)
    losses = []
    with torch.cuda.stream(stream):
        eng.backend.set_stream(stream.cuda_stream)
        eng.backend.set_epilogue_fusion(fusion)
        eng.backend.set_lora_fold(lora_fold)
        eng.backend.set_attention_one_walk(one_walk)
        eng.load(blob)
        eng.set_horizon(cfg.steps)
        for _ in range(steps):
            rec = rng.integers(0, cfg.vocab, size=(cfg.batch_seqs, cfg.seq + 1), dtype=np.int32)
            eng.stage_batch(np.ascontiguousarray(rec[:, :-1]).reshape(-1),
                            np.ascontiguousarray(rec[:, 1:]).reshape(-1))
            eng.train_forward_backward(True)
            eng.train_optimizer()
            losses.append(eng.read_loss())
        persist = np.array(eng.read_persistent(), copy=True)
        launches = eng.backend.counters().kernel_launches
        fused = eng.backend.counters().fused_dispatches
    eng.close()
    return persist, np.array(losses, dtype=np.float32), launches, fused


def test_engine_step_with_the_low_rank_fold_stays_within_f32_noise_of_the_step_without():
    """The adapter expand products riding the frozen products' reductions change
    the arithmetic of those sums (pieces of the factors on the tensor cores
    instead of f32 multiply-adds): the step must stay within what such a change
    of summation order does — far inside the bf16 rounding of the frozen products
    themselves."""
    p_on, l_on, n_on, f_on = _engine_run(True, lora_fold=True)
    p_off, l_off, n_off, f_off = _engine_run(True, lora_fold=False)
    assert np.isfinite(l_on).all()
    assert np.allclose(l_on, l_off, rtol=2e-4, atol=0)
    a, b = p_on.view(np.float32).astype(np.float64), p_off.view(np.float32).astype(np.float64)
    assert np.sqrt(np.mean((a - b) ** 2)) <= 5e-2 * np.sqrt(np.mean(b ** 2))   # four AdamW steps amplify sign flips
    # Two layers, four adapters each: eight forward and eight backward expand kernels ride a product.
    # (The launch count does not fall: a small kernel cuts each factor into pieces where the expand
    # kernel ran.  What falls is the traffic: the expand read and rewrote the whole [rows, width] sum.)
    assert f_on - f_off >= 16


def test_engine_step_with_one_walk_dq_stays_within_relaxed_noise_of_the_two_walk_step():
    """dQ with delta taken as dO . O from the forward's kept bf16 copy of its output (one walk over the
    keys) against the two-walk kernel that sums P dP: the same quantity in another rounding, on operands
    that are bf16-rounded either way."""
    p_on, l_on, _n, _f = _engine_run(True, one_walk=True)
    p_off, l_off, _n2, _f2 = _engine_run(True, one_walk=False)
    assert np.isfinite(l_on).all()
    assert not np.array_equal(p_on, p_off), "the one-walk kernel gave the two-walk bits: did it run?"
    assert np.allclose(l_on, l_off, rtol=2e-3, atol=0)
    a, b = p_on.view(np.float32).astype(np.float64), p_off.view(np.float32).astype(np.float64)
    assert np.sqrt(np.mean((a - b) ** 2)) <= 5e-2 * np.sqrt(np.mean(b ** 2))   # four AdamW steps amplify sign flips


def test_engine_step_with_fusions_is_the_unfused_step_bit_for_bit():
    p_on, l_on, n_on, f_on = _engine_run(True)
    p_off, l_off, n_off, f_off = _engine_run(False)
    assert np.isfinite(l_on).all()
    assert np.array_equal(l_on, l_off)
    assert np.array_equal(p_on, p_off)
    # Two layers: per eagerly executed pass at least the two GELU forwards and the
    # two GELU backwards stop launching (plus the bias adds).
    assert n_off - n_on >= 4
    # Per eagerly executed pass: two bias adds, two GELU forwards, two GELU backwards
    # and the loss backward (done by the loss forward's row pass) are absorbed.
    assert f_off == 0 and f_on >= 7


# ---- a following elementwise add as the epilogue's addend ------------------------------

def _build_add(rng, M, K, N, with_bias, product_first, read_later):
    a = Arena(rng)
    x = a.alloc(M * K, "normal")
    w = a.ro_alloc(rng.integers(-127, 128, size=K * N, dtype=np.int8))
    sc = a.ro_alloc((rng.random(N) * 0.01 + 1e-3).astype(np.float32))
    bias = a.ro_alloc(rng.standard_normal(N).astype(np.float32))
    res = a.alloc(M * N, "normal")
    r = a.alloc(M * N); z = a.alloc(M * N); out = a.alloc(M * N); keep = a.alloc(M * N)
    prog = [P.Instr(Op.GEMM_NN_Q8, REL | CS, 0, (x, w, r, sc), (M, N, K))]
    src = r
    if with_bias:
        prog.append(P.Instr(Op.ADD_BIAS, 0, 0, (r, bias, z, P.NULL_REF), (M, N, 0)))
        src = z
    ops = (src, res) if product_first else (res, src)
    prog.append(P.Instr(Op.ADD_EW, 0, 0, (ops[0], ops[1], out, P.NULL_REF), (M * N, 0, 0)))
    if read_later:
        prog.append(P.Instr(Op.COPY, 0, 0, (src, keep), (M * N, 0, 0)))
    prog.append(P.Instr(Op.FILL, 0, 0, (r, P.f32_bits(0.0)), (M * N, 0, 0)))
    prog.append(P.Instr(Op.FILL, 0, 0, (z, P.f32_bits(0.0)), (M * N, 0, 0)))
    arena, ro = a.build()
    return prog, arena, ro


@pytest.mark.parametrize("size", ACT_SIZES, ids=["one-tile", "persistent"])
@pytest.mark.parametrize("with_bias", [False, True], ids=["plain", "after-bias"])
@pytest.mark.parametrize("product_first", [False, True], ids=["x+p", "p+x"])
def test_following_add_rides_the_gemm_epilogue(size, with_bias, product_first):
    M, K, N = size
    prog, arena0, ro = _build_add(np.random.default_rng(31), M, K, N, with_bias, product_first, False)
    fused, c_fused = _run(prog, arena0, ro, one_range=True)
    split, c_split = _run(prog, arena0, ro, one_range=False)
    assert np.isfinite(fused.view(np.float32)).all()
    assert np.array_equal(fused, split)
    assert c_split.kernel_launches - c_fused.kernel_launches == (2 if with_bias else 1)
    assert c_fused.fused_dispatches == (2 if with_bias else 1)


def test_following_add_is_left_alone_when_the_product_is_read_later():
    M, K, N = ACT_SIZES[0]
    prog, arena0, ro = _build_add(np.random.default_rng(32), M, K, N, False, True, True)
    fused, c_fused = _run(prog, arena0, ro, one_range=True)
    split, c_split = _run(prog, arena0, ro, one_range=False)
    assert np.array_equal(fused, split)
    assert c_fused.fused_dispatches == 0 and c_split.kernel_launches == c_fused.kernel_launches


@pytest.mark.parametrize("dx_first", [False, True], ids=["x+dx", "dx+x"])
@pytest.mark.parametrize("in_place", [False, True], ids=["new", "over-addend"])
def test_add_after_layernorm_backward_rides_the_kernel(dx_first, in_place):
    M, D = 512, 256
    rng = np.random.default_rng(41)
    a = Arena(rng)
    x = a.alloc(M * D, "normal"); gamma = a.alloc(D, "normal"); beta = a.alloc(D, "normal")
    y = a.alloc(M * D); mean = a.alloc(M); rstd = a.alloc(M)
    dy = a.alloc(M * D, "normal"); res = a.alloc(M * D, "normal")
    dx = a.alloc(M * D); out = res if in_place else a.alloc(M * D)
    ops = (dx, res) if dx_first else (res, dx)
    prog = [
        P.Instr(Op.LAYERNORM_FWD, 0, P.f32_bits(1e-5), (x, gamma, beta, y), (P.pack2(M, D), mean, rstd)),
        P.Instr(Op.LAYERNORM_BWD, 0, 0, (dy, x, gamma, dx), (mean, rstd, P.pack2(M, D))),
        P.Instr(Op.ADD_EW, 0, 0, (ops[0], ops[1], out, P.NULL_REF), (M * D, 0, 0)),
        P.Instr(Op.FILL, 0, 0, (dx, P.f32_bits(0.0)), (M * D, 0, 0)),
    ]
    arena0, ro = a.build()
    fused, c_fused = _run(prog, arena0, ro, one_range=True)
    split, c_split = _run(prog, arena0, ro, one_range=False)
    assert np.isfinite(fused.view(np.float32)).all()
    assert np.array_equal(fused, split)
    assert c_split.kernel_launches - c_fused.kernel_launches == 1 and c_fused.fused_dispatches == 1


@pytest.mark.parametrize("order", ["nn", "nt"])
@pytest.mark.parametrize("over_addend", [False, True], ids=["new", "over-addend"])
def test_add_after_an_adapter_expand_product_rides_the_kernel(order, over_addend):
    M, N, r = 512, 256, 16
    rng = np.random.default_rng(43)
    a = Arena(rng)
    t = a.alloc(M * r, "normal"); w = a.alloc(r * N, "normal")     # [r][N] (nn) or [N][r] (nt)
    y = a.alloc(M * N, "normal"); res = a.alloc(M * N, "normal")
    z = a.alloc(M * N); out = y if over_addend else a.alloc(M * N)
    op = Op.GEMM_NN if order == "nn" else Op.GEMM_NT
    prog = [
        P.Instr(op, P.FLAG_GEMM_ADDEND, P.f32_bits(2.0), (t, w, z, y), (M, N, r)),
        P.Instr(Op.ADD_EW, 0, 0, (res, z, out, P.NULL_REF), (M * N, 0, 0)),
        P.Instr(Op.FILL, 0, 0, (z, P.f32_bits(0.0)), (M * N, 0, 0)),
    ]
    arena0, ro = a.build()
    fused, c_fused = _run(prog, arena0, ro, one_range=True)
    split, c_split = _run(prog, arena0, ro, one_range=False)
    assert np.isfinite(fused.view(np.float32)).all()
    assert np.array_equal(fused, split)
    assert c_split.kernel_launches - c_fused.kernel_launches == 1 and c_fused.fused_dispatches == 1


def test_layernorm_backward_sum_hands_its_copy_to_the_gemm_that_reads_it():
    M, D, N = 512, 256, 128
    rng = np.random.default_rng(47)
    a = Arena(rng)
    x = a.alloc(M * D, "normal"); gamma = a.alloc(D, "normal"); beta = a.alloc(D, "normal")
    y = a.alloc(M * D); mean = a.alloc(M); rstd = a.alloc(M)
    dy = a.alloc(M * D, "normal"); res = a.alloc(M * D, "normal")
    dx = a.alloc(M * D); total = a.alloc(M * D); out = a.alloc(M * N)
    w = a.ro_alloc(rng.integers(-127, 128, size=N * D, dtype=np.int8))
    sck = a.ro_alloc((2.0 ** rng.integers(-9, -5, size=D)).astype(np.float32))
    prog = [
        P.Instr(Op.LAYERNORM_FWD, 0, P.f32_bits(1e-5), (x, gamma, beta, y), (P.pack2(M, D), mean, rstd)),
        P.Instr(Op.LAYERNORM_BWD, 0, 0, (dy, x, gamma, dx), (mean, rstd, P.pack2(M, D))),
        P.Instr(Op.ADD_EW, 0, 0, (res, dx, total, P.NULL_REF), (M * D, 0, 0)),
        P.Instr(Op.GEMM_NT_Q8, REL | CS, 0, (total, w, out, sck), (M, N, D)),
        P.Instr(Op.FILL, 0, 0, (dx, P.f32_bits(0.0)), (M * D, 0, 0)),
    ]
    arena0, ro = a.build()
    fused, c_fused = _run(prog, arena0, ro, one_range=True)
    split, c_split = _run(prog, arena0, ro, one_range=False)
    assert np.array_equal(fused, split)
    # The add kernel and the GEMM's own conversion pass are both gone.
    assert c_split.kernel_launches - c_fused.kernel_launches == 2 and c_fused.fused_dispatches == 1


# ---- random programs: whatever the planner decides to absorb, the arena ends the same --------
# Outside the engine a tensor counts as dead only if the range overwrites it, so a
# fused range must leave EVERY byte as the one-instruction ranges do.  Programs
# are drawn from products, bias adds, activations (forward and backward), adds,
# consumers, copies and fills over a handful of same-size buffers, in-place forms
# included; any refusal by the runtime guard fails the test as well.

def _random_program(rng, M, K, N):
    a = Arena(rng)
    x = a.alloc(M * K, "normal")
    bufs = [a.alloc(M * N, "normal") for _ in range(5)]
    small = a.alloc(M * 64)
    w = a.ro_alloc(rng.integers(-127, 128, size=K * N, dtype=np.int8))
    sc = a.ro_alloc((rng.random(N) * 0.01 + 1e-3).astype(np.float32))
    bias = a.ro_alloc(rng.standard_normal(N).astype(np.float32))
    w2 = a.ro_alloc(rng.integers(-127, 128, size=64 * N, dtype=np.int8))
    sk = a.ro_alloc((2.0 ** rng.integers(-9, -5, size=N)).astype(np.float32))
    pick = lambda: bufs[int(rng.integers(len(bufs)))]
    prog = []
    for _ in range(int(rng.integers(8, 16))):
        kind = int(rng.integers(8))
        i, j, k = pick(), pick(), pick()
        if kind == 0:
            prog.append(P.Instr(Op.GEMM_NN_Q8, REL | CS, 0, (x, w, j, sc), (M, N, K)))
        elif kind == 1:
            prog.append(P.Instr(Op.ADD_BIAS, 0, 0, (i, bias, j, P.NULL_REF), (M, N, 0)))
        elif kind == 2:
            prog.append(P.Instr(Op.GELU_FWD, 0, 0, (i, j), (M * N, 0, 0)))
        elif kind == 3 and k != j and k != i:
            prog.append(P.Instr(Op.GELU_BWD, 0, 0, (i, k, j, P.NULL_REF), (M * N, 0, 0)))
        elif kind == 4:
            prog.append(P.Instr(Op.ADD_EW, 0, 0, (i, k, j, P.NULL_REF), (M * N, 0, 0)))
        elif kind == 5:
            prog.append(P.Instr(Op.GEMM_NT_Q8, REL | CS, 0, (i, w2, small, sk), (M, 64, N)))
        elif kind == 6 and i != j:
            prog.append(P.Instr(Op.COPY, 0, 0, (i, j), (M * N, 0, 0)))
        else:
            prog.append(P.Instr(Op.FILL, 0, 0, (j, P.f32_bits(0.5)), (M * N, 0, 0)))
        # Products are usually followed by something that can ride their epilogue.
        if kind == 0 and rng.random() < 0.8:
            nxt = int(rng.integers(4))
            o = pick()
            if nxt == 0:
                prog.append(P.Instr(Op.ADD_BIAS, 0, 0, (j, bias, o, P.NULL_REF), (M, N, 0)))
                if rng.random() < 0.7:
                    o2 = pick()
                    if rng.random() < 0.5:
                        prog.append(P.Instr(Op.GELU_FWD, 0, 0, (o, o2), (M * N, 0, 0)))
                    elif k != o:
                        prog.append(P.Instr(Op.ADD_EW, 0, 0, (k, o, o2, P.NULL_REF), (M * N, 0, 0)))
                    if rng.random() < 0.7:
                        prog.append(P.Instr(Op.GEMM_NT_Q8, REL | CS, 0, (o2, w2, small, sk), (M, 64, N)))
            elif nxt == 1:
                prog.append(P.Instr(Op.GELU_FWD, 0, 0, (j, o), (M * N, 0, 0)))
                prog.append(P.Instr(Op.GEMM_NT_Q8, REL | CS, 0, (o, w2, small, sk), (M, 64, N)))
            elif nxt == 2 and k != j and k != o:
                prog.append(P.Instr(Op.GELU_BWD, 0, 0, (j, k, o, P.NULL_REF), (M * N, 0, 0)))
                prog.append(P.Instr(Op.GEMM_NT_Q8, REL | CS, 0, (o, w2, small, sk), (M, 64, N)))
            elif k != j:
                prog.append(P.Instr(Op.ADD_EW, 0, 0, (k, j, o, P.NULL_REF), (M * N, 0, 0)))
    for b in bufs:   # most buffers end overwritten, so intermediates can be proven dead
        if rng.random() < 0.7:
            prog.append(P.Instr(Op.FILL, 0, 0, (b, P.f32_bits(0.25)), (M * N, 0, 0)))
    arena, ro = a.build()
    return prog, arena, ro


@pytest.mark.parametrize("seed", range(24))
def test_random_programs_end_with_the_same_arena_fused_or_not(seed):
    rng = np.random.default_rng(1000 + seed)
    M, K, N = (256, 128, 128) if seed % 4 else (4864, 64, 2048)
    prog, arena0, ro = _random_program(rng, M, K, N)
    fused, c_fused = _run(prog, arena0, ro, one_range=True)
    split, c_split = _run(prog, arena0, ro, one_range=False)
    assert np.array_equal(fused, split), [str(i) for i in prog]
    assert c_split.fused_dispatches == 0


def test_the_random_programs_do_exercise_the_fusions():
    total = 0
    for seed in range(8, 16):
        rng = np.random.default_rng(1000 + seed)
        M, K, N = (256, 128, 128) if seed % 4 else (4864, 64, 2048)
        prog, arena0, ro = _random_program(rng, M, K, N)
        _fused, c = _run(prog, arena0, ro, one_range=True)
        total += c.fused_dispatches
    assert total >= 5


def test_attention_dk_and_dv_share_one_walk():
    from tests.test_gpu_umma import bf16_round
    Bq, S, H, d = 2, 384, 2, 64
    rng = np.random.default_rng(53)
    a = Arena(rng)
    td = Bq * S * H * d
    t = {}
    for name in ("q", "k", "v", "do"):
        t[name] = a.alloc(td, bf16_round(rng.standard_normal(td).astype(np.float32) * 0.7))
    for name in ("o", "dq", "dk", "dv"):
        t[name] = a.alloc(td)
    stats = a.alloc(Bq * H * S * 4)
    gk = a.alloc(Bq * S * 64); gv = a.alloc(Bq * S * 64)
    wq = a.ro_alloc(rng.integers(-127, 128, size=64 * H * d, dtype=np.int8))
    sck = a.ro_alloc((2.0 ** rng.integers(-9, -5, size=H * d)).astype(np.float32))
    bs, hd, geo = P.pack2(Bq, S), P.pack2(H, d), P.pack_attn_geometry(Bq, S, H, d)
    prog = [
        P.Instr(Op.ATTN_FWD_TILED, REL, 0, (t["q"], t["k"], t["v"], t["o"]), (stats, bs, hd)),
        P.Instr(Op.ATTN_DQ_TILED, REL, 0, (t["q"], t["k"], t["v"], t["do"]), (stats, t["dq"], geo)),
        P.Instr(Op.ATTN_DK_TILED, REL, 0, (t["q"], t["k"], t["v"], t["do"]), (stats, t["dk"], geo)),
        P.Instr(Op.ATTN_DV_TILED, REL, 0, (t["q"], t["k"], t["v"], t["do"]), (stats, t["dv"], geo)),
        # The projections' backward products read dK and dV through the copies the pair's kernel made.
        P.Instr(Op.GEMM_NT_Q8, REL | CS, 0, (t["dk"], wq, gk, sck), (Bq * S, 64, H * d)),
        P.Instr(Op.GEMM_NT_Q8, REL | CS, 0, (t["dv"], wq, gv, sck), (Bq * S, 64, H * d)),
    ]
    arena0, ro = a.build()
    fused, c_fused = _run(prog, arena0, ro, one_range=True)
    split, c_split = _run(prog, arena0, ro, one_range=False)
    assert np.isfinite(fused.view(np.float32)).all()
    assert np.array_equal(fused, split)
    assert c_fused.fused_dispatches == 1 and c_split.fused_dispatches == 0
    assert c_fused.relaxed_executions == c_split.relaxed_executions == 6
    dv = fused[t["dv"]:t["dv"] + 4 * td].view(np.float32)
    assert np.abs(dv).max() > 0
    # dQ in one walk (delta = dO . O from the forward's kept bf16 copy of O) against the two-walk kernel
    # (delta = sum P dP): delta itself, dQ, and dK, which reads delta from the stats row.
    from tests.util import compare
    walk1, _c = _run(prog, arena0, ro, one_range=True, one_walk=True)
    assert not np.array_equal(walk1, fused), "the one-walk kernel gave the two-walk bits: did it run?"
    st1 = walk1[stats:stats + 16 * Bq * H * S].view(np.float32).reshape(-1, 4)
    st2 = fused[stats:stats + 16 * Bq * H * S].view(np.float32).reshape(-1, 4)
    assert np.array_equal(st1[:, :2], st2[:, :2])
    ok, ratio = compare(st1[:, 2].tobytes(), st2[:, 2].tobytes(), 1e-2, 1e-6)
    assert ok, ("delta", ratio)
    for name in ("dq", "dk", "dv"):
        ok, ratio = compare(walk1[t[name]:t[name] + 4 * td], fused[t[name]:t[name] + 4 * td], 1e-2, 1e-6)
        assert ok, (name, ratio)
