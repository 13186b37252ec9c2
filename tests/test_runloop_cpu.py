"""The restated run loop (sample sequence, set evaluation, gate) on the CPU
oracle: the harness the GPU parity tests drive both executors with."""

import numpy as np

import oracle
from see_ai_b200 import plan as P
from see_ai_b200 import synth
from tests import runloop as R


def setup_module(_m):
    if not oracle.have_oracle():
        oracle.build("oracle")


def test_splitmix64_stream_and_permutation_are_deterministic():
    # First outputs of splitmix64 from state 0 (the published reference sequence of the generator).
    st, a = R.splitmix64_next(0)
    st, b = R.splitmix64_next(st)
    assert (a, b) == (0xE220A8397B1DCDAF, 0x6E789E6AA1B965F4)
    d1 = R.Dataset(np.zeros((10, 2), np.float32), np.arange(10, dtype=np.int32))
    d2 = R.Dataset(np.zeros((10, 2), np.float32), np.arange(10, dtype=np.int32))
    d1.enable_shuffle(7); d2.enable_shuffle(7)
    assert sorted(d1.order.tolist()) == list(range(10)) and d1.order.tolist() == d2.order.tolist()
    # serving wraps into a fresh permutation; a saved position replays it
    pos = d1.save_pos()
    first = [d1.fill_batch(4)[1].tolist() for _ in range(6)]
    d1.restore_pos(pos)
    again = [d1.fill_batch(4)[1].tolist() for _ in range(6)]
    assert first == again
    flat = sum(first, [])
    assert sorted(flat[:10]) == list(range(10)) and sorted(flat[10:20]) == list(range(10))


def test_validation_split_takes_the_tail_before_shuffling():
    x = np.arange(40, dtype=np.float32).reshape(20, 2)
    d = R.Dataset(x, np.arange(20, dtype=np.int32))
    v = d.split_validation(0.1)
    assert d.n == 18 and v.n == 2 and v.labels.tolist() == [18, 19]
    t = R.Dataset(None, None, np.arange(5 * 9, dtype=np.int32).reshape(5, 9))
    tv = t.split_validation(0.5)
    assert t.n == 3 and tv.n == 2
    xb, yb = tv.fill_batch(16)
    assert xb.tolist() == list(range(27, 35)) + list(range(36, 44)) and yb[0] == 28


def test_run_loop_gate_on_the_cpu_oracle():
    cfg = synth.MlpConfig(dims=(16, 24, 4), batch=8, rank=4, lr=5e-2)
    plan = P.Plan(synth.build_mlp_plan(cfg))
    rng = np.random.default_rng(1)
    x = rng.standard_normal((100, 16)).astype(np.float32)
    y = (x[:, 0] > 0).astype(np.int32) + 2 * (x[:, 1] > 0).astype(np.int32)   # learnable labels
    train = R.Dataset(x, y)
    val = train.split_validation(0.13)    # 13 samples: the second validation batch wraps
    train.enable_shuffle(3)
    cpu = R.CpuStepper(plan, oracle.OracleExecutor())
    rep = R.train_run(cpu, train, val, plan.header, 60)
    assert rep.verdict == "accepted" and rep.val_final < rep.val_initial
    assert rep.evaluations == 9 and len(rep.loss_curve) == 60
    assert rep.val_final <= min(l for _s, l in rep.eval_trace) + 1e-12
    m = R.evaluate_set(cpu, val, plan.header)
    assert m.counted == 13 and abs(m.loss - rep.val_final) < 1e-6   # the best state was left in the arena
