"""TEST INFRASTRUCTURE: the reference engine's host-side run loop, restated so
that one loop can drive either executor — the CUDA engine or the reference CPU
executor — over the same sample sequence, evaluations and gate.

What is restated, with the reference lines it follows:
  * the sample sequence: validation split = the last floor(n * frac) samples
    (at least 1, at most n - 1) taken before shuffling; EnableShuffle(seed);
    one Fisher-Yates permutation per epoch from a splitmix64 stream; token
    records give inputs tokens[0..S) and labels tokens[1..S]
    (reference: runtime/pipeline/dataset.cc:422-491, 501-553, 555-610;
    source/contract/split.h:35-40);
  * set evaluation: whole batches, the last one wrapping, accuracy over real
    rows only, the set's loss the mean of batch losses or — ragged set or masked
    loss — the real-row loss (reference: runtime/dispatcher/update_engine.cc:432-580,
    977-1026);
  * the gate: best state by strictly lower validation loss, periodic evaluation
    every max(1, horizon / 10) steps except the last, bracketing evaluations,
    verdict "accepted" iff the final validation loss is below the initial one
    (reference: runtime/gating/gate.cc; update_engine.cc:704-768, 886-955;
    runtime/host/update_main.cc:794-809).
"""

from __future__ import annotations

import dataclasses
from typing import List, Optional

import numpy as np

from see_ai_b200 import plan as P

MASK64 = (1 << 64) - 1


def splitmix64_next(state: int):
    state = (state + 0x9E3779B97F4A7C15) & MASK64
    z = state
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK64
    return state, z ^ (z >> 31)


class Dataset:
    """Feature rows (inputs [n, dim] f32, labels [n] i32) or token records
    ([n, S + 1] i32) served in the reference's order."""

    def __init__(self, inputs: Optional[np.ndarray], labels: Optional[np.ndarray],
                 tokens: Optional[np.ndarray] = None):
        self.inputs, self.labels, self.tokens = inputs, labels, tokens
        self.n = len(tokens) if tokens is not None else len(inputs)
        self.order: Optional[np.ndarray] = None
        self.state = 0
        self.origin = 0
        self.cursor = 0
        self.epoch = 0

    def split_validation(self, fraction: float) -> "Dataset":
        assert self.order is None, "split before enabling shuffle"
        val_n = int(float(self.n) * fraction)
        val_n = max(1, min(val_n, self.n - 1))
        train_n = self.n - val_n
        if self.tokens is not None:
            val = Dataset(None, None, self.tokens[train_n:].copy())
            self.tokens = self.tokens[:train_n]
        else:
            val = Dataset(self.inputs[train_n:].copy(), self.labels[train_n:].copy())
            self.inputs, self.labels = self.inputs[:train_n], self.labels[:train_n]
        self.n = train_n
        self.cursor = 0
        return val

    def _reshuffle(self):
        order = list(range(self.n))
        st = self.state
        for i in range(self.n - 1, 0, -1):
            st, r = splitmix64_next(st)
            j = r % (i + 1)
            order[i], order[j] = order[j], order[i]
        self.state = st
        self.order = np.array(order, dtype=np.int64)

    def enable_shuffle(self, seed: int):
        st, r = splitmix64_next(seed & MASK64)
        self.state = r | 1
        self.origin = self.state
        self.epoch = 0
        self._reshuffle()
        self.cursor = 0

    def save_pos(self):
        return (self.cursor, self.epoch)

    def restore_pos(self, pos):
        self.cursor = pos[0]
        if self.order is None or self.epoch == pos[1]:
            return
        self.state = self.origin
        self.epoch = 0
        self._reshuffle()
        while self.epoch < pos[1]:
            self._reshuffle()
            self.epoch += 1

    def rewind(self):
        self.cursor = 0

    def fill_batch(self, rows: int):
        """-> (x, y) for one compiled batch of `rows` rows."""
        if self.tokens is not None:
            S = self.tokens.shape[1] - 1
            recs = rows // S
            idx = np.empty(recs, dtype=np.int64)
        else:
            recs = rows
            idx = np.empty(rows, dtype=np.int64)
        for r in range(recs):
            idx[r] = self.cursor if self.order is None else self.order[self.cursor]
            self.cursor += 1
            if self.cursor == self.n:
                self.cursor = 0
                if self.order is not None:
                    self._reshuffle()
                    self.epoch += 1
        if self.tokens is not None:
            rec = self.tokens[idx]
            return (np.ascontiguousarray(rec[:, :-1]).reshape(-1), np.ascontiguousarray(rec[:, 1:]).reshape(-1))
        return np.ascontiguousarray(self.inputs[idx]), np.ascontiguousarray(self.labels[idx])


@dataclasses.dataclass
class BatchEval:
    loss: float            # the eval program's loss slot
    rows: int              # rows judged for accuracy
    correct: int
    real_row_loss: float   # double
    loss_rows: int
    has_accuracy: bool


def host_scan(probs: np.ndarray, labels: np.ndarray, real: int, loss_slot: float, masked: bool) -> BatchEval:
    """The reference's host scan of one evaluated batch: argmax by a sequential
    scan from column 0 that moves only on a strictly greater value (so the first
    maximum wins, a NaN never wins and a NaN in column 0 is never displaced),
    rows with a negative label neither judged nor counted; the real-row loss as
    the row-order double sum of -log(max(p[label], 1e-12)) (a NaN p kept)."""
    rows = correct = 0
    total = 0.0
    loss_rows = 0
    for r in range(real):
        lab = int(labels[r])
        if lab < 0:
            continue
        row = probs[r]
        arg = 0
        best = row[0]
        if not np.isnan(best):
            # vectorised form of the scan: the first index holding the maximum of the non-NaN values
            vals = np.where(np.isnan(row), -np.inf, row)
            m = vals.max()
            arg = int(np.argmax(vals == m)) if m > best else 0
        rows += 1
        correct += int(arg == lab)
        p = np.float32(row[lab])
        safe = float(p) if np.isnan(p) else float(np.maximum(p, np.float32(1e-12)))
        total -= float(np.log(np.float64(safe)))
        loss_rows += 1
    return BatchEval(loss_slot, rows, correct, total, loss_rows, True)


class CpuStepper:
    """The reference CPU executor (or the oracle restatement) over a plan."""

    def __init__(self, plan: P.Plan, executor, lr: Optional[float] = None):
        self.plan, self.h = plan, plan.header
        self.arena = plan.stage_arena()
        self.ex = executor
        self.ro = np.frombuffer(bytes(plan.rodata) + b"\0" * 64, dtype=np.uint8).copy()
        self.ex.bind(self.arena, self.ro)
        self.train, self.eval_prog = plan.section("train"), plan.section("eval")
        self.step = 0
        self.lr = lr if lr is not None else self.h["lr"]
        self.lr_of_step = None   # optional schedule: step -> lr
        self.masked = any(i.opcode == P.Op.XENT_MASKED_FWD for i in self.eval_prog)
        self.eval_probs = None
        for i in self.eval_prog:
            if i.opcode in (P.Op.XENT_FWD, P.Op.XENT_MASKED_FWD):
                self.eval_probs = (i.ins[3], i.out[0], i.out[1])

    def _stage(self, x, y):
        h = self.h
        xb = np.ascontiguousarray(x).view(np.uint8).reshape(-1)
        yb = np.ascontiguousarray(y).view(np.uint8).reshape(-1)
        self.arena[h["input_ref"]:h["input_ref"] + xb.size] = xb
        self.arena[h["label_ref"]:h["label_ref"] + yb.size] = yb

    def _params(self):
        import oracle
        h = self.h
        lr = self.lr_of_step(self.step) if self.lr_of_step else self.lr
        return oracle.StepParams(lr, h["beta1"], h["beta2"], h["eps"], h["weight_decay"], 0, max(self.step, 1))

    def loss(self) -> float:
        o = self.h["loss_ref"]
        return float(self.arena[o:o + 4].view(np.float32)[0])

    def train_step(self, x, y) -> float:
        self._stage(x, y)
        self.step += 1
        self.ex.run(self.train, self._params())
        return self.loss()

    def evaluate(self, x, y, real: int) -> BatchEval:
        self._stage(x, y)
        self.ex.run(self.eval_prog, self._params())
        off, n, c = self.eval_probs
        probs = self.arena[off:off + 4 * n * c].view(np.float32).reshape(n, c)
        return host_scan(probs, np.asarray(y).reshape(-1), real, self.loss(), self.masked)

    def persistent(self) -> np.ndarray:
        return self.arena[:self.h["persistent_size"]].copy()

    def restore(self, state: np.ndarray):
        self.arena[:state.size] = state

    def read(self, off: int, nbytes: int) -> np.ndarray:
        return self.arena[off:off + nbytes].copy()


class GpuStepper:
    """The CUDA engine through the C ABI (see_engine_*)."""

    def __init__(self, engine):
        self.eng = engine
        self.h = engine.header

    @property
    def step(self):
        return self.eng.step

    def train_step(self, x, y) -> float:
        return self.eng.train_step(x, y)

    def evaluate(self, x, y, real: int) -> BatchEval:
        r = self.eng.evaluate_rows(x, y, real)
        return BatchEval(float(np.float32(r.loss)), int(r.rows), int(r.correct), float(r.real_row_loss),
                         int(r.loss_rows), bool(r.has_accuracy))

    def persistent(self) -> np.ndarray:
        return self.eng.read_persistent()

    def restore(self, state: np.ndarray):
        self.eng.write_arena(0, state)

    def read(self, off: int, nbytes: int) -> np.ndarray:
        return self.eng.read_arena(off, nbytes)


@dataclasses.dataclass
class SetMetrics:
    loss: float
    accuracy: float
    has_accuracy: bool
    correct: int = 0
    counted: int = 0


def evaluate_set(stepper, data: Dataset, header: dict, masked: bool = False) -> SetMetrics:
    pos = data.save_pos()
    data.rewind()
    rows_per_sample = header["seq_len"] if header["input_kind"] == 1 else 1
    per_step = header["batch"] // rows_per_sample
    batches = max(1, (data.n + per_step - 1) // per_step)
    ragged = data.n % per_step != 0
    per_row = ragged or masked
    total = 0.0
    real_loss, real_rows = 0.0, 0
    correct = counted = 0
    has_acc = False
    for b in range(batches):
        x, y = data.fill_batch(header["batch"])
        served = b * per_step
        real = min(per_step, data.n - served if data.n > served else 0) * rows_per_sample
        e = stepper.evaluate(x, y, real)
        total += float(np.float32(e.loss))
        if per_row:
            real_loss += e.real_row_loss
            real_rows += e.loss_rows
        has_acc = e.has_accuracy
        correct += e.correct
        counted += e.rows
    data.restore_pos(pos)
    loss = np.float32((real_loss / real_rows if real_rows else 0.0) if per_row else total / batches)
    acc = np.float32(correct / counted) if has_acc and counted else np.float32(0)
    return SetMetrics(float(loss), float(acc), has_acc and counted > 0, correct, counted)


@dataclasses.dataclass
class Report:
    loss_curve: List[float]
    val_initial: float
    val_last: float
    val_final: float
    best_step: int
    evaluations: int
    verdict: str
    val_initial_accuracy: float = 0.0
    val_final_accuracy: float = 0.0
    eval_trace: List[tuple] = dataclasses.field(default_factory=list)


def train_run(stepper, train: Dataset, val: Dataset, header: dict, steps: int, masked: bool = False) -> Report:
    """A fresh run of `steps` optimizer steps with the default gate: periodic
    evaluation every max(1, steps / 10) steps, best state kept and restored."""
    eval_every = max(1, steps // 10)
    v0 = evaluate_set(stepper, val, header, masked)
    best_loss, best_step, best_acc = v0.loss, stepper.step, v0.accuracy
    best_state = stepper.persistent()
    curve, trace = [], [(stepper.step, v0.loss)]
    evaluations = 0
    for s in range(steps):
        x, y = train.fill_batch(header["batch"])
        curve.append(stepper.train_step(x, y))
        if stepper.step % eval_every == 0 and s + 1 < steps:
            v = evaluate_set(stepper, val, header, masked)
            evaluations += 1
            trace.append((stepper.step, v.loss))
            if np.float32(v.loss) < np.float32(best_loss):
                best_loss, best_step, best_acc = v.loss, stepper.step, v.accuracy
                best_state = stepper.persistent()
    v = evaluate_set(stepper, val, header, masked)
    trace.append((stepper.step, v.loss))
    if np.float32(v.loss) < np.float32(best_loss):
        best_loss, best_step, best_acc = v.loss, stepper.step, v.accuracy
        best_state = stepper.persistent()
    if best_step != stepper.step:
        stepper.restore(best_state)
    improved = np.float32(best_loss) < np.float32(v0.loss)
    return Report(curve, v0.loss, v.loss, best_loss, best_step, evaluations,
                  "accepted" if improved else "rejected", v0.accuracy, best_acc, trace)
