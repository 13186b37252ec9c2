"""Single-node data parallelism for update plans: one process per GPU, the
batch's sequences sharded across ranks, ONE exchange per optimizer step.

The reference has no distributed path at all (its only parallelism is threads
inside one process).  What shards naturally: every opcode is per-row or
per-sequence, and the only cross-row reductions are the loss mean and the
trainable-parameter gradients, which the compiler binds back to back in the
arena (reference: compiler/backend/allocation/arena_binder.cc:56-77).  So each
rank runs the plan compiled for global_rows / N rows, and between the backward
sweep and the first optimizer instruction (the phase boundary of reference
runtime/profiler/step_timings.h:37-59) the ranks all-gather that one gradient
block over NCCL into their own HBM.  The AdamW kernel then sums the N copies in
rank order 0..N-1 and multiplies by the exact power of two 1/N — the same bits
on every rank and on every run, which a ring all-reduce does not promise.
Adapters and moments therefore stay replicated bit for bit.

No peer memory is read by any kernel here: remote gradients arrive through the
collective into local memory first.
"""

from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import numpy as np


def shard_rows(global_rows: int, seq_len: int, world: int, rank: int) -> Tuple[int, int]:
    """Rows [begin, end) of each global batch that `rank` trains on.  Token
    plans shard whole sequences (reference: runtime/loader/plan_loader.cc:226-228:
    batch % seq_len == 0); feature plans shard rows."""
    unit = seq_len if seq_len else 1
    units = global_rows // unit
    if global_rows % unit or units % world:
        raise ValueError(f"{global_rows} rows of {unit}-row units do not split over {world} ranks")
    per = units // world * unit
    return rank * per, (rank + 1) * per


def scan_phases(train) -> Tuple[int, int]:
    """(bwd_begin, opt_begin) of a train section: the instruction after the loss
    forward, and the first clip / optimizer instruction (the engine's phase
    scan, mirrored for hosts that drive the backend seam themselves; reference:
    runtime/profiler/step_timings.h:37-59)."""
    from . import plan as P
    Op = P.Op
    n = len(train)
    bwd, opt = n, n
    for i, ins in enumerate(train):
        if ins.opcode in (Op.XENT_FWD, Op.XENT_MASKED_FWD, Op.MSE_FWD, Op.KL_FWD):
            bwd = i + 1
        if ins.opcode in (Op.CLIP_NORM, Op.SQNORM_ACCUM, Op.CLIP_GLOBAL, Op.SGD_STEP,
                          Op.ADAMW_STEP) and opt == n:
            opt = i
    return bwd, max(opt, bwd)


def gradient_block(plan) -> Tuple[int, int]:
    """(arena offset, bytes) of the block spanning every optimizer instruction's
    gradient operand: what the ranks exchange once per step."""
    from . import plan as P
    prog = plan.section("step") or plan.section("train")
    lo, hi = None, 0
    for ins in prog:
        if ins.opcode in (P.Op.ADAMW_STEP, P.Op.SGD_STEP):
            off = ins.ins[1] & ~(P.RODATA_BIT | P.SOURCE_BIT)
            lo = off if lo is None else min(lo, off)
            hi = max(hi, off + ins.out[0] * 4)
    return (0, 0) if lo is None else (lo, hi - lo)


def host_exchange(arena: np.ndarray, off: int, nbytes: int, group=None) -> None:
    """The exchange on host memory over any torch.distributed backend (gloo on
    CPU): all-gather the block, fold the copies in rank order, write the mean
    back in place.  The device path does the same with the gather landing in HBM
    and the fold inside the optimizer kernel; this form serves hosts that keep
    the arena in their own memory, and the CPU tests."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    if world == 1 or nbytes == 0:
        return
    mine = torch.from_numpy(arena[off:off + nbytes].copy())
    copies = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(copies, mine, group=group)
    mean = fixed_order_mean([c.numpy().view(np.float32) for c in copies])
    arena[off:off + nbytes] = mean.view(np.uint8)


def fixed_order_mean(copies: Sequence[np.ndarray]) -> np.ndarray:
    """The reduction the optimizer kernel applies to gathered gradients: a
    left-to-right f32 sum in rank order, then one multiply by 1/N."""
    acc = copies[0].astype(np.float32).copy()
    for c in copies[1:]:
        acc = (acc + c.astype(np.float32)).astype(np.float32)
    return (acc * np.float32(1.0 / len(copies))).astype(np.float32)


class GradientExchange:
    """The per-step exchange of a data-parallel run.  The collective itself lives in the
    library (see_engine_attach_exchange: an NCCL all-gather on the engine's stream between
    the backward and the optimizer range, the fold in rank order inside the optimizer
    kernels); torch.distributed only carries the 128-byte communicator id from rank 0 to
    the others, and the shard losses for reporting."""

    def __init__(self, engine, group=None):
        import torch
        import torch.distributed as dist
        from . import engine as E
        self.dist = dist
        self.group = group
        self.engine = engine
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.off, self.nbytes = engine.gradient_block()
        if self.world > 1:
            # (refused by the library too; said here before any rank blocks in the collective join)
            if getattr(engine, "has_masked_loss", False):
                raise ValueError("data parallel: plans with a masked cross-entropy are not supported "
                                 "(shards would need a target-count-weighted mean)")
            box = [E.make_exchange_id() if self.rank == 0 else None]
            dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group is not None else 0,
                                       group=group)
            engine.attach_exchange(self.world, self.rank, box[0])

    def exchange(self):
        """Enqueues the step's all-gather on the engine's stream now; without this call the
        engine does it at the start of its optimizer range."""
        if self.world > 1:
            self.engine.exchange()

    def mean_loss(self, local_loss: float) -> float:
        """Mean of the shard losses in rank order (each shard's loss is already a
        mean over its own rows, and shards are equal-sized; plans with a masked
        loss, whose per-shard means are over unequal target counts, are refused
        by the constructor)."""
        import torch
        if self.world == 1:
            return local_loss
        mine = torch.tensor([local_loss], dtype=torch.float32, device="cuda")
        allv = torch.empty(self.world, dtype=torch.float32, device="cuda")
        self.dist.all_gather_into_tensor(allv, mine, group=self.group)
        return float(fixed_order_mean([allv[i:i + 1].cpu().numpy() for i in range(self.world)])[0])
