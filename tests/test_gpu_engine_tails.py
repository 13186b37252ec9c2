"""The engine's host-facing tails on the device, each against the reference's
host-side definition:

  * evaluation: the accuracy tally (first maximum wins, a NaN never wins, rows
    labelled -1 neither judged nor counted) and the real-row loss of a ragged or
    masked batch — integer tallies EQUAL to a host scan written from the
    reference (reference: runtime/dispatcher/update_engine.cc:535-564, 977-1026;
    runtime/executor/loss.cc:78-105);
  * merge: the deltas and the finiteness scan (update_engine.cc:1028-1063);
  * the learning-rate schedule (update_engine.cc:370-391), bit for bit with the
    host's cosf;
  * CUDA-graph replay without any host synchronisation between steps, with the
    schedule on: the same bits as eager steps;
  * data parallelism with standalone clip instructions: the clip reaches the
    update (two ranks emulated on one GPU);
  * a second source model bound at the same offsets is really used;
  * the per-column int8 quantiser: the compiler's levels and scales, bit for bit
    (reference: compiler/backend/allocation/arena_binder.cc:129-190).
"""

import ctypes

import numpy as np
import pytest

import oracle
from see_ai_b200 import backend as B
from see_ai_b200 import dp
from see_ai_b200 import plan as P
from see_ai_b200 import synth
from see_ai_b200.engine import Engine
from tests import runloop as R
from tests.util import Case, compare

pytestmark = pytest.mark.gpu
Op = P.Op


def setup_module(_m):
    if not oracle.have_oracle():
        oracle.build("oracle")


def _tail_plan(rows: int, classes: int, masked: bool) -> bytes:
    """A plan whose eval program leaves CRAFTED probabilities where the engine's
    tail looks for them: the loss forward over the input slot, then a copy of
    the input slot (the crafted values) over the probabilities it wrote."""
    b = synth.PlanBuilder(3)
    x = b.t("x", rows * classes, "io")
    labels = b.t("labels", rows, "io")
    loss = b.t("loss", 1, "io")
    op = Op.XENT_MASKED_FWD if masked else Op.XENT_FWD
    for section in ("train", "eval"):
        b.cur = section
        probs = b.t("probs." + section, rows * classes)
        b.emit(op, (x, labels, loss, probs), (rows, classes))
        if section == "eval":
            b.emit(Op.COPY, (x, probs), (rows * classes,))
    header = dict(input_ref=x, input_floats=rows * classes, label_ref=labels, label_bytes=4 * rows, label_kind=1,
                  loss_ref=loss, lr=1e-3, batch=rows, default_steps=1, input_kind=0, grad_accum_steps=1, seq_len=0)
    return b.assemble(header)


@pytest.mark.parametrize("masked", [False, True], ids=["plain", "masked"])
def test_eval_tail_tallies_equal_the_host_scan(masked):
    rows, classes = 96, 130
    rng = np.random.default_rng(17)
    probs = rng.random((rows, classes)).astype(np.float32)
    probs /= probs.sum(axis=1, keepdims=True)
    labels = rng.integers(0, classes, size=rows).astype(np.int32)
    # duplicated maxima: the FIRST must win (label on the first -> hit, on the second -> miss)
    probs[0, :] = 0.001; probs[0, 7] = 0.4; probs[0, 90] = 0.4; labels[0] = 7
    probs[1, :] = 0.001; probs[1, 7] = 0.4; probs[1, 90] = 0.4; labels[1] = 90
    # (the NaN rows sit past row 80, so that real_rows <= 80 also checks a finite real-row loss)
    # a NaN in column 0 is never displaced: argmax = 0
    probs[90, 0] = np.nan; labels[90] = 0
    probs[91, 0] = np.nan; labels[91] = 5
    # a NaN elsewhere never wins, even over smaller values
    probs[92, :] = 0.002; probs[92, 33] = np.nan; probs[92, 60] = 0.5; labels[92] = 60
    probs[93, :] = 0.002; probs[93, 33] = np.nan; labels[93] = 33       # all equal otherwise: column 0 wins
    probs[6, :] = 0.002; labels[6] = 0
    # the maximum in the last column, and in a column only the last lane of a warp reads
    probs[7, :] = 0.001; probs[7, classes - 1] = 0.9; labels[7] = classes - 1
    probs[8, :] = 0.001; probs[8, 31] = 0.9; labels[8] = 31
    # a probability below the clamp, an exact zero, and a NaN at the label: the loss terms
    probs[9, int(labels[9])] = 1e-20
    probs[10, int(labels[10])] = 0.0
    if masked:
        labels[12:40:3] = -1
    blob = _tail_plan(rows, classes, masked)
    plan = P.Plan(blob)
    eng = Engine(0)
    eng.load(blob)
    gpu = R.GpuStepper(eng)
    cpu = R.CpuStepper(plan, oracle.OracleExecutor())
    for real in (rows, 80, 50, 13, 0):
        eg = gpu.evaluate(probs.reshape(-1), labels, real)
        ec = cpu.evaluate(probs.reshape(-1), labels, real)
        assert eg.has_accuracy
        assert (eg.rows, eg.correct, eg.loss_rows) == (ec.rows, ec.correct, ec.loss_rows), (real, eg, ec)
        if np.isnan(ec.real_row_loss):
            assert np.isnan(eg.real_row_loss)
        else:
            assert abs(eg.real_row_loss - ec.real_row_loss) <= 1e-12 * max(1.0, abs(ec.real_row_loss)), (real, eg, ec)
    # the plain entry point judges the whole batch
    loss, n_rows, n_correct = eng.evaluate(probs.reshape(-1), labels)
    full = cpu.evaluate(probs.reshape(-1), labels, rows)
    assert (n_rows, n_correct) == (full.rows, full.correct)
    eng.close()


def test_set_evaluation_with_a_wrapping_last_batch():
    """A validation set that is not a whole number of batches: the set's loss is
    the real-row loss over each sample once, the accuracy over real rows only."""
    cfg = synth.MlpConfig(dims=(32, 48, 10), batch=16, rank=4, lr=1e-2)
    blob = synth.build_mlp_plan(cfg)
    plan = P.Plan(blob)
    rng = np.random.default_rng(23)
    x = rng.standard_normal((41, 32)).astype(np.float32)    # 41 = 2 * 16 + 9: the third batch wraps
    y = rng.integers(0, 10, size=41).astype(np.int32)
    eng = Engine(0)
    eng.load(blob)
    mg = R.evaluate_set(R.GpuStepper(eng), R.Dataset(x, y), plan.header)
    mc = R.evaluate_set(R.CpuStepper(plan, oracle.OracleExecutor()), R.Dataset(x, y), plan.header)
    assert (mg.correct, mg.counted) == (mc.correct, mc.counted) and mc.counted == 41
    assert abs(mg.loss - mc.loss) <= 1e-6 * abs(mc.loss)
    eng.close()


def test_merge_deltas_and_the_finiteness_scan():
    cfg = synth.MlpConfig(dims=(64, 96, 16), batch=32, rank=8, lr=1e-2)
    blob = synth.build_mlp_plan(cfg)
    plan = P.Plan(blob)
    rng = np.random.default_rng(5)
    eng = Engine(0)
    eng.load(blob)
    cpu = R.CpuStepper(plan, oracle.OracleExecutor())
    for _ in range(3):   # B leaves zero, so the deltas are not trivially zero
        xb = rng.standard_normal((32, 64)).astype(np.float32)
        yb = rng.integers(0, 16, size=32).astype(np.int32)
        eng.train_step(xb, yb)
    cpu.restore(eng.read_persistent())   # the same adapters on both sides: the merge alone is compared
    assert eng.run_merge() is True
    cpu.ex.run(plan.section("merge"), oracle.step_params())
    assert len(plan.emit) == 2
    for e in plan.emit:
        got = eng.read_arena(e.arena_offset, e.byte_size)
        want = cpu.read(e.arena_offset, e.byte_size)
        ok, ratio = compare(got.tobytes(), want.tobytes(), 1e-5, 1e-7)
        assert ok, ratio
        assert np.abs(want.view(np.float32)).max() > 0
    # One infinity planted in an adapter through a host-side write: the merge product spreads it into a
    # delta (as Inf or NaN) and the scan must see it.
    adam = [i for i in plan.section("train") if i.opcode == Op.ADAMW_STEP]
    b_tensor = adam[1]   # the first adapter's B
    poisoned = eng.read_arena(b_tensor.ins[0], 4 * b_tensor.out[0]).view(np.float32).copy()
    poisoned[3] = np.inf
    eng.write_arena(b_tensor.ins[0], poisoned)
    assert eng.run_merge() is False
    poisoned[3] = 0.0
    eng.write_arena(b_tensor.ins[0], poisoned)
    assert eng.run_merge() is True
    eng.close()


def test_learning_rate_schedule_bits():
    libm = ctypes.CDLL("libm.so.6")
    libm.cosf.restype = ctypes.c_float
    libm.cosf.argtypes = [ctypes.c_float]
    f = np.float32

    def want(step, base, warm, horizon, min_factor):
        base = f(base)
        if warm > 0 and step <= warm:
            return f(f(base * f(step)) / f(warm))
        span = horizon - warm if horizon > warm else 0
        floor = f(base * f(min_factor))
        if span == 0 or step - warm >= span:
            return floor
        t = f(f(step - warm) / f(span))
        c = f(libm.cosf(f(f(3.14159265358979323846) * t)))
        return f(floor + f(f(f(base - floor) * f(0.5)) * f(f(1.0) + c)))

    cfg = synth.MlpConfig(dims=(32, 48, 10), batch=16, rank=4, lr=3e-3, lr_schedule=1, warmup_steps=7,
                          min_lr_factor=0.1)
    eng = Engine(0)
    eng.load(synth.build_mlp_plan(cfg))
    for horizon in (100, 1000, 5, 7):
        eng.set_horizon(horizon)
        for step in (1, 3, 7, 8, 9, 50, 53, 99, 100, 101, 500, 999, 1000, 5000):
            eng.set_step(step)
            got = f(eng.effective_lr())
            assert got.tobytes() == want(step, 3e-3, 7, horizon, 0.1).tobytes(), (horizon, step, got)
    flat = Engine(0)
    flat.load(synth.build_mlp_plan(synth.MlpConfig(dims=(32, 48, 10), batch=16, rank=4, lr=3e-3)))
    flat.set_step(77)
    assert f(flat.effective_lr()).tobytes() == f(3e-3).tobytes()
    eng.close()
    flat.close()


def test_graph_replay_without_host_sync_equals_eager_steps():
    """K steps replayed as CUDA graphs with no host synchronisation between them
    (the host runs far ahead of the device) and a learning rate that changes
    every step: adapters and moments must be the bits K eager steps leave."""
    cfg = synth.MlpConfig(dims=(256, 1024, 64), batch=32, rank=8, lr=2e-3, lr_schedule=1, warmup_steps=5,
                          min_lr_factor=0.05)
    blob = synth.build_mlp_plan(cfg)
    rng = np.random.default_rng(31)
    K = 80   # more steps than the backend has pinned scalar slots
    batches = [(rng.standard_normal((32, 256)).astype(np.float32), rng.integers(0, 64, size=32).astype(np.int32))
               for _ in range(K)]

    def run(graphs: bool, sync_every_step: bool):
        eng = Engine(0)
        eng.load(blob)
        eng.set_horizon(K)
        eng.set_use_graphs(graphs)
        for (xb, yb) in batches:
            eng.stage_batch(xb, yb)
            eng.train_forward_backward(True)
            eng.train_optimizer()
            if sync_every_step:
                eng.read_loss()
        loss = eng.read_loss()
        state = eng.read_persistent()
        eng.close()
        return loss, state

    loss_e, state_e = run(False, True)
    loss_g, state_g = run(True, False)
    assert np.float32(loss_e).tobytes() == np.float32(loss_g).tobytes()
    assert np.array_equal(state_e, state_g)


@pytest.mark.parametrize("case_name", ["mlp_unfused_clip", "mlp_global_clip"])
def test_data_parallel_standalone_clip_reaches_the_update(case_name):
    """Two ranks emulated on one GPU (two engines, the gather buffer filled by
    hand): plans whose clip is its own instruction must clip the MEAN gradient
    and feed the clipped values to the optimizer, as a host-side exchange does."""
    import torch
    case = Case(case_name)
    plan = case.plan
    blob = case.z["plan"].tobytes()
    h = plan.header
    rows, dim = h["batch"], h["input_floats"] // h["batch"]
    rng = np.random.default_rng(77)
    g_off, g_bytes = dp.gradient_block(plan)
    train = plan.section("train")
    _bwd, opt = dp.scan_phases(train)
    assert any(i.opcode in (Op.CLIP_NORM, Op.SQNORM_ACCUM, Op.CLIP_GLOBAL) for i in train[opt:])
    classes = max(i.out[1] for i in train if i.opcode == Op.XENT_FWD)

    engines = [Engine(0) for _ in range(2)]
    gathered = torch.zeros(2 * g_bytes, dtype=torch.uint8, device="cuda")
    for e in engines:
        e.load(blob)
        e.backend.set_gradient_gather(2, gathered.data_ptr(), g_off, g_bytes)
    # the CPU twin: two arenas, the host-side exchange (mean written back in place), the optimizer range
    ro = np.frombuffer(bytes(plan.rodata) + b"\0" * 64, dtype=np.uint8).copy()
    arenas, execs = [], []
    for _ in range(2):
        a = plan.stage_arena()
        ex = oracle.OracleExecutor()
        ex.bind(a, ro)
        arenas.append(a)
        execs.append(ex)
    for step in range(1, 4):
        shards = [(rng.standard_normal((rows, dim)).astype(np.float32) * 3.0,   # large inputs: the clip must bite
                   rng.integers(0, classes, size=rows).astype(np.int32)) for _ in range(2)]
        sp = oracle.StepParams(case.lr, h["beta1"], h["beta2"], h["eps"], h["weight_decay"], 0, step)
        for r in range(2):
            # Lockstep: every step starts from the engine's own state on both sides, so that one
            # step's arithmetic is compared and not the drift AdamW makes of earlier differences.
            arenas[r][:h["persistent_size"]] = engines[r].read_persistent()
            xb, yb = shards[r]
            engines[r].stage_batch(xb, yb)
            engines[r].train_forward_backward(True)
            xb8, yb8 = xb.view(np.uint8).reshape(-1), yb.view(np.uint8).reshape(-1)
            arenas[r][h["input_ref"]:h["input_ref"] + xb8.size] = xb8
            arenas[r][h["label_ref"]:h["label_ref"] + yb8.size] = yb8
            execs[r].run(train, sp, 0, opt)
        blocks = [engines[r].read_arena(g_off, g_bytes) for r in range(2)]
        gathered.copy_(torch.from_numpy(np.concatenate(blocks)).cuda())
        torch.cuda.synchronize()
        mean = dp.fixed_order_mean([a[g_off:g_off + g_bytes].view(np.float32) for a in arenas])
        for r in range(2):
            engines[r].train_optimizer()
            arenas[r][g_off:g_off + g_bytes] = mean.view(np.uint8)
            execs[r].run(train, sp, opt, len(train))
        # What the optimizer range leaves in the gradient block is the CLIPPED MEAN on both sides.
        got_block = engines[0].read_arena(g_off, g_bytes)
        ok, ratio = compare(got_block.tobytes(), arenas[0][g_off:g_off + g_bytes].tobytes(), 1e-5, 1e-9)
        assert ok, (step, ratio)
        clipped = np.abs(arenas[0][g_off:g_off + g_bytes].view(np.float32)).max()
        assert clipped < 0.9 * np.abs(mean).max(), "the clip did not bite: the test would prove nothing"
        states = [e.read_persistent() for e in engines]
        assert np.array_equal(states[0], states[1])
        want = arenas[0][:h["persistent_size"]]
        # Per optimizer tensor, against that tensor's own scale: AdamW turns a 1e-6 difference in a
        # gradient element far below the block's maximum into a visible fraction of the learning
        # rate, so element-wise relative bounds are meaningless here.  An update that ignored the
        # clip would leave second moments larger by the square of the clip factor (several times).
        for ins in (i for i in train[opt:] if i.opcode == Op.ADAMW_STEP):
            for ref in (ins.ins[0], ins.ins[2], ins.ins[3]):
                ok, ratio = compare(states[0][ref:ref + 4 * ins.out[0]].tobytes(),
                                    want[ref:ref + 4 * ins.out[0]].tobytes(), 2e-2, 1e-12)
                assert ok, (step, hex(ref), ratio)
    for e in engines:
        e.close()


def test_second_source_model_replaces_the_first():
    """A relaxed GEMM whose frozen weight lies in the source model: after a second
    model is bound at the same offsets the product must use the new weights."""
    M, N, K = 128, 64, 128
    rng = np.random.default_rng(3)
    a = np.zeros(4 * (M * K + M * N) + 128, dtype=np.uint8)
    x = rng.standard_normal((M, K)).astype(np.float32)
    a[:4 * M * K] = x.view(np.uint8).reshape(-1)
    out_off = 4 * M * K
    prog = [P.Instr(Op.GEMM_NN, P.FLAG_RELAXED, 0, (0, P.SOURCE_BIT | 0, out_off, P.NULL_REF), (M, N, K))]
    be = B.CudaBackend(0)
    gpu = a.copy()
    be.bind(gpu, None)
    for seed in (1, 2):
        w = np.random.default_rng(seed).standard_normal((K, N)).astype(np.float32)
        src = w.view(np.uint8).reshape(-1).copy()
        be.bind_source(src)
        be.run(prog)
        got = gpu[out_off:out_off + 4 * M * N].view(np.float32).reshape(M, N)
        want = x.astype(np.float64) @ w.astype(np.float64)
        assert np.abs(got - want).max() <= 2e-2 * np.abs(want).max(), seed
    be.close()


def test_device_quantiser_is_the_compilers_bit_for_bit():
    import torch
    K, N = 300, 260
    rng = np.random.default_rng(9)
    w = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
    w[:, 5] = 0.0                                   # an all-zero column: scale 1
    w[:, 6] = np.float32(1e-41)                     # max / 127 subnormal: scale FLT_MIN
    w[:, 7] = w[:, 7].max() * np.sign(w[:, 7])      # every level +-127
    col = np.abs(w[:, 8]).max()
    w[0, 8], w[1, 8], w[2, 8] = col, np.float32(col * 0.5 / 127.0), np.float32(-col * 2.5 / 127.0)   # ties
    w[3, 9] = np.nan                                # a NaN never becomes the maximum
    want_q, want_s = synth.quantize_columns(np.where(np.isnan(w), np.float32(0), w))
    amax = np.fmax.reduce(np.abs(w), axis=0)
    assert np.array_equal(amax, np.abs(np.where(np.isnan(w), np.float32(0), w)).max(axis=0))
    d_w = torch.from_numpy(w).cuda()
    d_q = torch.zeros((K, N), dtype=torch.int8, device="cuda")
    d_s = torch.zeros(N, dtype=torch.float32, device="cuda")
    be = B.CudaBackend(0)
    be.set_stream(torch.cuda.current_stream().cuda_stream)
    be.quantize_columns(d_w.data_ptr(), K, N, d_q.data_ptr(), d_s.data_ptr())
    torch.cuda.synchronize()
    got_q, got_s = d_q.cpu().numpy(), d_s.cpu().numpy()
    be.close()
    assert got_s.tobytes() == want_s.tobytes()
    assert got_s[5] == 1.0 and got_s[6] == np.finfo(np.float32).tiny
    keep = ~np.isnan(w)
    assert np.array_equal(got_q[keep], want_q[keep])
