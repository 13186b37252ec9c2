"""Checkpoint / gate snapshots taken while training continues, and resume from
one.  Training is deterministic, so: a snapshot begun after step 2 and collected
after step 4 must hold exactly the persistent prefix of a run that stopped at
step 2; restoring it (with the timestep) and training two more steps must land
on exactly the state of the uninterrupted four-step run."""

import numpy as np
import pytest

from see_ai_b200 import synth
from see_ai_b200.engine import Engine

pytestmark = pytest.mark.gpu


def _batches(rows, dim, classes, count):
    rng = np.random.default_rng(21)
    return [(rng.standard_normal((rows, dim)).astype(np.float32),
             rng.integers(0, classes, size=rows).astype(np.int32)) for _ in range(count)]


@pytest.mark.parametrize("graphs", [False, True], ids=["eager", "graphs"])
def test_snapshot_while_training_and_resume(graphs):
    cfg = synth.MlpConfig(dims=(64, 96, 12), batch=32, rank=4, lr=1e-2)
    blob = synth.build_mlp_plan(cfg)
    data = _batches(32, 64, 12, 4)

    def fresh():
        eng = Engine(0)
        eng.load(blob)
        eng.set_horizon(100)
        eng.set_use_graphs(graphs)
        return eng

    def steps(eng, lo, hi):
        for x, y in data[lo:hi]:
            eng.train_step(x, y)

    a = fresh()
    steps(a, 0, 2)
    after_two = a.read_persistent()
    a.close()

    b = fresh()
    steps(b, 0, 2)
    b.snapshot_begin()
    steps(b, 2, 4)                       # training goes on while the copy drains
    snap = b.snapshot_wait()
    after_four = b.read_persistent()
    assert b.step == 4
    b.close()
    assert np.array_equal(snap, after_two)
    assert not np.array_equal(snap, after_four)

    c = fresh()
    c.restore(snap, 2)
    assert c.step == 2
    steps(c, 2, 4)
    resumed = c.read_persistent()
    c.close()
    assert np.array_equal(resumed, after_four)
