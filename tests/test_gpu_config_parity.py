"""The path the benchmark times — the C++ engine with lazy coherence, whole-step
liveness, epilogue fusions, CUDA-graph replay and the tensor-core kernels —
against the reference CPU executor, at the benchmark configurations' stated
shapes, free-running over the same batches.

What each comparison uses:
  * losses: the reference's own rule for its GPU backend, |gpu - cpu| <=
    1e-4 + 2e-3 |cpu| per step (reference: test/runtime/executor/
    metal_backend_test.cc:211-230) for the f32 plans, 2e-2 relative for the
    plan whose frozen-weight GEMMs carry the relaxed (bf16) permission;
  * the gradient block of step 1 (identical state on both sides, so pure
    kernel error): per tensor, |a - b| <= atol + rtol * max|b| (reference:
    tool/frontier_exec.py:49-55) with rtol 1e-5 (f32) — and for the relaxed
    plan the relative RMS error per tensor <= 2e-2;
  * after N steps: the persistent prefix (adapters and moments) per optimizer
    tensor, reported, and held to a drift bound (AdamW's first steps turn a
    1e-7 difference in a near-zero gradient into a difference of the order of
    the learning rate, so no element-wise 1e-5 can hold after a step);
  * the accept / reject verdict of the gate: equal.

Every measured figure is also written to gpurun_out/config_parity.json when
that folder exists.
"""

import json
import os

import numpy as np
import pytest

import oracle
from see_ai_b200 import plan as P
from see_ai_b200 import synth
from see_ai_b200.engine import Engine
from tests import runloop as R
from tests.util import compare

pytestmark = pytest.mark.gpu
Op = P.Op
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_METRICS = {}


def _record(name, **kv):
    _METRICS.setdefault(name, {}).update({k: (float(v) if isinstance(v, (np.floating, float)) else v)
                                          for k, v in kv.items()})
    out = os.path.join(ROOT, "gpurun_out")
    if os.path.isdir(out):
        with open(os.path.join(out, "config_parity.json"), "w") as f:
            json.dump(_METRICS, f, indent=1)


def _cpu_executor():
    """The reference's own CPU executor when its build travelled here, else our
    C restatement of it (pinned to the reference bit for bit by the CPU tests)."""
    if oracle.have_ref():
        ex = oracle.RefExecutor()
        ex.set_threads(os.cpu_count() or 1)
        return ex
    if not oracle.have_oracle():
        oracle.build("oracle")
    return oracle.OracleExecutor()


def _optimizer_tensors(plan: P.Plan):
    """(name, offset, floats) of every parameter and moment the optimizer writes."""
    out = []
    for n, ins in enumerate(i for i in plan.section("train") if i.opcode in (Op.ADAMW_STEP, Op.SGD_STEP)):
        out.append((f"p{n}", ins.ins[0], ins.out[0]))
        if ins.opcode == Op.ADAMW_STEP:
            out.append((f"m{n}", ins.ins[2], ins.out[0]))
            out.append((f"v{n}", ins.ins[3], ins.out[0]))
    return out


def _gradient_tensors(plan: P.Plan):
    return [(f"g{n}", ins.ins[1], ins.out[0])
            for n, ins in enumerate(i for i in plan.section("train") if i.opcode in (Op.ADAMW_STEP, Op.SGD_STEP))]


def _worst(tensors, gpu, cpu, rtol, atol):
    """Largest error / bound over the tensors under the per-tensor-scale rule,
    and the largest relative RMS error."""
    worst, worst_rms, name = 0.0, 0.0, ""
    for (nm, off, n) in tensors:
        a = gpu.read(off, 4 * n)
        b = cpu.read(off, 4 * n)
        _ok, ratio = compare(a.tobytes(), b.tobytes(), rtol, atol)
        fa, fb = a.view(np.float32).astype(np.float64), b.view(np.float32).astype(np.float64)
        den = np.sqrt(np.mean(fb * fb))
        rms = float(np.sqrt(np.mean((fa - fb) ** 2)) / den) if den > 0 else float(np.abs(fa).max())
        if ratio > worst:
            worst, name = ratio, nm
        worst_rms = max(worst_rms, rms)
    return worst, worst_rms, name


def _loss_curve_ok(gpu, cpu, rel, floor):
    gpu, cpu = np.asarray(gpu, np.float64), np.asarray(cpu, np.float64)
    err = np.abs(gpu - cpu)
    tol = floor + rel * np.abs(cpu)
    return bool((err <= tol).all()), float((err / tol).max())


# ---- the feed-forward plan: 256 -> 1024 -> 64, batch 32, LoRA r8, 1000 steps, val-frac 0.1, seed 7 ----

def test_mlp_plan_1000_steps_and_the_gate_verdict():
    cfg = synth.MlpConfig(dims=(256, 1024, 64), batch=32, rank=8, alpha=16.0, lr=1e-3, steps=1000, seed=7)
    blob = synth.build_mlp_plan(cfg)
    plan = P.Plan(blob)
    h = plan.header
    rng = np.random.default_rng(7)
    x = rng.standard_normal((4096, 256)).astype(np.float32)
    y = rng.integers(0, 64, size=4096).astype(np.int32)

    def datasets():
        train = R.Dataset(x.copy(), y.copy())
        val = train.split_validation(0.1)
        train.enable_shuffle(7)
        return train, val

    eng = Engine(0)
    eng.load(blob)
    eng.set_horizon(1000)
    eng.set_use_graphs(True)
    gpu = R.GpuStepper(eng)
    cpu = R.CpuStepper(plan, _cpu_executor())

    tr_g, va_g = datasets()
    tr_c, va_c = datasets()
    rep_g = R.train_run(gpu, tr_g, va_g, h, 1000)
    rep_c = R.train_run(cpu, tr_c, va_c, h, 1000)

    # (Random labels: the held-out loss only rises with training, apart from the first periodic
    # evaluation, which the reference CPU executor scores 1.4e-3 below the source model here — far
    # above any difference between the two executors — so both keep the state of step 100.)
    assert rep_g.verdict == rep_c.verdict, (rep_g, rep_c)
    assert rep_g.best_step == rep_c.best_step
    assert abs(rep_g.val_initial - rep_c.val_initial) <= 1e-5 * abs(rep_c.val_initial)
    assert rep_g.val_initial_accuracy == rep_c.val_initial_accuracy
    figures = {}
    # 2e-3 is what the reference asks of its own GPU backend after 8 steps; beyond a hundred steps of
    # AdamW its release gate prices the drift at 1 % (the comment at metal_backend_test.cc:214-217).
    for n, rel in ((1, 2e-3), (10, 2e-3), (100, 2e-3), (1000, 1e-2)):
        ok, ratio = _loss_curve_ok(rep_g.loss_curve[:n], rep_c.loss_curve[:n], rel, 1e-4)
        figures[f"loss_curve_err_over_bound_{n}"] = ratio
        assert ok, (n, ratio)
    assert abs(rep_g.loss_curve[0] - rep_c.loss_curve[0]) <= 1e-5 * abs(rep_c.loss_curve[0])
    for (sg, lg), (sc, lc) in zip(rep_g.eval_trace, rep_c.eval_trace):
        assert sg == sc and abs(lg - lc) <= 1e-4 + (2e-3 if sg <= 100 else 1e-2) * abs(lc)
    # Both restored the best state they kept: the same step's adapters and moments.
    ratio, rms, name = _worst(_optimizer_tensors(plan), gpu, cpu, 5e-3, 1e-6)
    figures["restored_state_err_over_bound"] = ratio
    assert ratio <= 1.0, (name, ratio)
    _record("mlp_256_1024_64_b32", verdict=rep_g.verdict, best_step=rep_g.best_step,
            val_initial_gpu=rep_g.val_initial, val_initial_cpu=rep_c.val_initial,
            val_last_gpu=rep_g.val_last, val_last_cpu=rep_c.val_last,
            final_train_loss_gpu=rep_g.loss_curve[-1], final_train_loss_cpu=rep_c.loss_curve[-1], **figures)
    eng.close()


def test_mlp_plan_state_after_n_steps():
    """The same plan without the gate's restore: adapters and moments after
    N = 1, 10, 100 steps against the reference CPU executor."""
    cfg = synth.MlpConfig(dims=(256, 1024, 64), batch=32, rank=8, alpha=16.0, lr=1e-3, steps=1000, seed=7)
    blob = synth.build_mlp_plan(cfg)
    plan = P.Plan(blob)
    h = plan.header
    rng = np.random.default_rng(7)
    data = R.Dataset(rng.standard_normal((4096, 256)).astype(np.float32),
                     rng.integers(0, 64, size=4096).astype(np.int32))
    data.enable_shuffle(7)
    eng = Engine(0)
    eng.load(blob)
    eng.set_use_graphs(True)
    gpu, cpu = R.GpuStepper(eng), R.CpuStepper(plan, _cpu_executor())
    tensors, grads = _optimizer_tensors(plan), _gradient_tensors(plan)
    figures = {}
    for step in range(1, 101):
        xb, yb = data.fill_batch(h["batch"])
        lg, lc = gpu.train_step(xb, yb), cpu.train_step(xb, yb)
        assert abs(lg - lc) <= 1e-4 + 2e-3 * abs(lc), (step, lg, lc)
        if step == 1:
            ratio, rms, name = _worst(grads, gpu, cpu, 1e-5, 1e-7)
            figures["grad_step1_err_over_bound"] = ratio
            assert ratio <= 1.0, (name, ratio)
        if step in (1, 10, 100):
            ratio, rms, name = _worst(tensors, gpu, cpu, 5e-3, 1e-6)
            figures[f"state_err_over_bound_{step}"] = ratio
            figures[f"state_rel_rms_{step}"] = rms
            assert ratio <= 1.0, (step, name, ratio)
    _record("mlp_256_1024_64_b32_state", **figures)
    eng.close()


# ---- the small f32 decoder: 4 layers, d256, 4 heads, FFN 1024, vocab 4096, seq 128, 32 sequences ----

def test_f32_decoder_at_its_stated_size_ten_steps():
    cfg = synth.DecoderConfig(layers=4, d_model=256, heads=4, ffn=1024, vocab=4096, seq=128, batch_seqs=32,
                              rank=8, alpha=16.0, targets=("q", "v"), quantized=False, attention="cached",
                              lr=1e-3, steps=500, seed=7)
    blob = synth.build_decoder_plan(cfg)
    plan = P.Plan(blob)
    h = plan.header
    rng = np.random.default_rng(7)
    data = R.Dataset(None, None, rng.integers(0, 4096, size=(96, 129)).astype(np.int32))
    data.enable_shuffle(7)
    eng = Engine(0)
    eng.load(blob)
    eng.set_use_graphs(True)
    gpu, cpu = R.GpuStepper(eng), R.CpuStepper(plan, _cpu_executor())
    tensors, grads = _optimizer_tensors(plan), _gradient_tensors(plan)
    figures = {}
    lg_curve, lc_curve = [], []
    for step in range(1, 11):
        xb, yb = data.fill_batch(h["batch"])
        lg_curve.append(gpu.train_step(xb, yb))
        lc_curve.append(cpu.train_step(xb, yb))
        if step == 1:
            assert abs(lg_curve[0] - lc_curve[0]) <= 1e-5 * abs(lc_curve[0]), (lg_curve, lc_curve)
            ratio, rms, name = _worst(grads, gpu, cpu, 1e-5, 1e-7)
            figures["grad_step1_err_over_bound"] = ratio
            figures["grad_step1_rel_rms"] = rms
            assert ratio <= 1.0, (name, ratio)
        if step in (1, 10):
            ratio, rms, name = _worst(tensors, gpu, cpu, 5e-3, 1e-6)
            figures[f"state_err_over_bound_{step}"] = ratio
            figures[f"state_rel_rms_{step}"] = rms
    ok, ratio = _loss_curve_ok(lg_curve, lc_curve, 2e-3, 1e-4)
    figures["loss_curve_err_over_bound_10"] = ratio
    _record("decoder_f32_L4_d256_S128_B32", loss_gpu=lg_curve, loss_cpu=lc_curve, **figures)
    assert ok, ratio
    # The reference claims 5e-3 relative (+1e-6) for its own GPU backend after 8 steps.
    assert figures["state_err_over_bound_10"] <= 1.0, figures
    # One evaluation batch: integer tallies equal the host scan's, the loss the reference's.
    xb, yb = data.fill_batch(h["batch"])
    eg, ec = gpu.evaluate(xb, yb, h["batch"]), cpu.evaluate(xb, yb, h["batch"])
    assert (eg.rows, eg.loss_rows) == (ec.rows, ec.loss_rows)
    assert abs(eg.correct - ec.correct) <= 2   # the states differ by the drift above; ties in argmax may move
    assert abs(eg.loss - ec.loss) <= 1e-4 + 2e-3 * abs(ec.loss)
    eng.close()


# ---- the int8-weight decoder of the benchmark, one sequence per step, the engine exactly as bench.py drives it ----

def test_int8_relaxed_decoder_one_sequence_ten_steps():
    cfg = synth.DecoderConfig(layers=12, d_model=768, heads=12, ffn=3072, vocab=32000, seq=512, batch_seqs=1,
                              rank=16, alpha=32.0, targets=("q", "k", "v", "o"), quantized=True,
                              attention="tiled", lr=1e-3, steps=1000, seed=7)
    blob = synth.build_decoder_plan(cfg)
    plan = P.Plan(blob)
    h = plan.header
    rng = np.random.default_rng(11)
    eng = Engine(0)
    eng.load(blob)
    eng.set_horizon(cfg.steps)
    eng.set_use_graphs(True)
    gpu, cpu = R.GpuStepper(eng), R.CpuStepper(plan, _cpu_executor())
    tensors, grads = _optimizer_tensors(plan), _gradient_tensors(plan)
    figures = {}
    lg_curve, lc_curve = [], []
    for step in range(1, 11):
        rec = rng.integers(0, cfg.vocab, size=(1, 513)).astype(np.int32)
        xb, yb = np.ascontiguousarray(rec[:, :-1]).reshape(-1), np.ascontiguousarray(rec[:, 1:]).reshape(-1)
        lg_curve.append(gpu.train_step(xb, yb))
        lc_curve.append(cpu.train_step(xb, yb))
        if step == 1:
            ratio, rms, name = _worst(grads, gpu, cpu, 2e-2, 1e-7)
            figures["grad_step1_err_over_bound"] = ratio
            figures["grad_step1_rel_rms"] = rms
            assert rms <= 2e-2, (name, rms)
        if step in (1, 10):
            ratio, rms, name = _worst(tensors, gpu, cpu, 2e-2, 1e-6)
            figures[f"state_err_over_bound_{step}"] = ratio
            figures[f"state_rel_rms_{step}"] = rms
    ok, ratio = _loss_curve_ok(lg_curve, lc_curve, 2e-2, 1e-4)
    figures["loss_curve_err_over_bound_10"] = ratio
    c = eng.backend.counters()
    _record("decoder_int8_relaxed_L12_d768_S512_B1", loss_gpu=lg_curve, loss_cpu=lc_curve,
            relaxed_executions=int(c.relaxed_executions), fused_dispatches=int(c.fused_dispatches), **figures)
    assert c.relaxed_executions > 0, "the tensor-core path did not run"
    assert ok, ratio
    assert figures["state_rel_rms_10"] <= 0.25, figures   # adapters after 10 AdamW steps under bf16 gradient noise
    eng.close()
