"""Data-parallel host logic on CPU: two `gloo` ranks, each running the plan
compiled for half the batch through the CPU oracle, exchanging the gradient
block once per step exactly as the device path does (all-gather, fold in rank
order, times 1/N).  Checks: the shards tile the batch; both ranks hold
bit-identical adapters and moments after every step; the exchanged gradient and
the mean loss agree with a single process that trains the whole batch."""

import multiprocessing as mp
import os
import socket
import tempfile

import numpy as np
import pytest

import oracle
from see_ai_b200 import dp, synth
from see_ai_b200 import plan as P

GLOBAL_ROWS, DIMS, RANK, STEPS = 16, (32, 48, 10), 4, 3


def _batches():
    rng = np.random.default_rng(99)
    return [(rng.standard_normal((GLOBAL_ROWS, DIMS[0])).astype(np.float32),
             rng.integers(0, DIMS[-1], size=GLOBAL_ROWS).astype(np.int32)) for _ in range(STEPS)]


def _plan(rows: int) -> P.Plan:
    return P.Plan(synth.build_mlp_plan(synth.MlpConfig(dims=DIMS, batch=rows, rank=RANK, lr=1e-2)))


def _train(plan: P.Plan, rows, exchange, lr=1e-2):
    """Runs STEPS optimizer steps on `rows` (a slice of each global batch).
    Returns per-step (loss, gradient block after the exchange) and the final
    persistent region."""
    h = plan.header
    arena = plan.stage_arena()
    ro = np.frombuffer(bytes(plan.rodata) + b"\0" * 64, dtype=np.uint8).copy()
    ex = oracle.OracleExecutor()
    ex.bind(arena, ro)
    train = plan.section("train")
    _bwd, opt = dp.scan_phases(train)
    g_off, g_bytes = dp.gradient_block(plan)
    log = []
    for step, (x, y) in enumerate(_batches()):
        xb = np.ascontiguousarray(x[rows]).view(np.uint8).reshape(-1)
        yb = np.ascontiguousarray(y[rows]).view(np.uint8).reshape(-1)
        arena[h["input_ref"]:h["input_ref"] + xb.size] = xb
        arena[h["label_ref"]:h["label_ref"] + yb.size] = yb
        sp = oracle.step_params(lr=lr, step=step + 1)
        ex.run(train, sp, 0, opt)
        exchange(arena, g_off, g_bytes)
        loss = float(arena[h["loss_ref"]:h["loss_ref"] + 4].view(np.float32)[0])
        log.append((loss, arena[g_off:g_off + g_bytes].view(np.float32).copy()))
        ex.run(train, sp, opt, len(train))
    return log, arena[:h["persist_init_size"]].copy()


def _train_lockstep(plan: P.Plan, world: int, lr=1e-2):
    """`world` ranks emulated in one process: every rank's forward/backward, the
    rank-ordered fold of their gradient blocks, every rank's optimizer.  Returns
    rank 0's persistent region and the per-step mean losses."""
    h = plan.header
    ro = np.frombuffer(bytes(plan.rodata) + b"\0" * 64, dtype=np.uint8).copy()
    train = plan.section("train")
    _bwd, opt = dp.scan_phases(train)
    g_off, g_bytes = dp.gradient_block(plan)
    arenas, execs = [], []
    for _ in range(world):
        arena = plan.stage_arena()
        ex = oracle.OracleExecutor()
        ex.bind(arena, ro)
        arenas.append(arena)
        execs.append(ex)
    losses = []
    for step, (x, y) in enumerate(_batches()):
        sp = oracle.step_params(lr=lr, step=step + 1)
        for rank in range(world):
            begin, end = dp.shard_rows(GLOBAL_ROWS, 0, world, rank)
            xb = np.ascontiguousarray(x[begin:end]).view(np.uint8).reshape(-1)
            yb = np.ascontiguousarray(y[begin:end]).view(np.uint8).reshape(-1)
            arenas[rank][h["input_ref"]:h["input_ref"] + xb.size] = xb
            arenas[rank][h["label_ref"]:h["label_ref"] + yb.size] = yb
            execs[rank].run(train, sp, 0, opt)
        mean = dp.fixed_order_mean([a[g_off:g_off + g_bytes].view(np.float32) for a in arenas])
        losses.append(dp.fixed_order_mean(
            [a[h["loss_ref"]:h["loss_ref"] + 4].view(np.float32) for a in arenas])[0])
        for rank in range(world):
            arenas[rank][g_off:g_off + g_bytes] = mean.view(np.uint8)
            execs[rank].run(train, sp, opt, len(train))
    return arenas[0][:h["persist_init_size"]].copy(), np.array(losses, dtype=np.float32)


def _worker(rank: int, world: int, port: int, out_dir: str):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        oracle.build("oracle")
        begin, end = dp.shard_rows(GLOBAL_ROWS, 0, world, rank)
        log, persist = _train(_plan(GLOBAL_ROWS // world), slice(begin, end), dp.host_exchange)
        np.savez(os.path.join(out_dir, f"rank{rank}.npz"), persist=persist,
                 losses=np.array([l for l, _ in log], dtype=np.float32),
                 grads=np.stack([g for _, g in log]))
    finally:
        dist.destroy_process_group()


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_shards_tile_the_batch():
    for world in (1, 2, 4, 8):
        spans = [dp.shard_rows(64 * 512, 512, world, r) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == 64 * 512
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert all((e - b) % 512 == 0 for b, e in spans)
    with pytest.raises(ValueError):
        dp.shard_rows(64 * 512, 512, 3, 0)
    with pytest.raises(ValueError):
        dp.shard_rows(1000, 512, 1, 0)


def test_fixed_order_mean_is_left_to_right_then_one_multiply():
    rng = np.random.default_rng(5)
    copies = [rng.standard_normal(1000).astype(np.float32) for _ in range(4)]
    want = ((((copies[0] + copies[1]) + copies[2]) + copies[3]) * np.float32(0.25)).astype(np.float32)
    assert np.array_equal(dp.fixed_order_mean(copies), want)


def test_phase_scan_and_gradient_block_of_a_synthesized_plan():
    plan = _plan(8)
    train = plan.section("train")
    bwd, opt = dp.scan_phases(train)
    assert train[bwd - 1].opcode == P.Op.XENT_FWD
    assert train[opt].opcode in (P.Op.ADAMW_STEP, P.Op.CLIP_NORM, P.Op.SQNORM_ACCUM, P.Op.CLIP_GLOBAL)
    assert all(i.opcode != P.Op.ADAMW_STEP for i in train[:opt])
    off, nbytes = dp.gradient_block(plan)
    grads = sum(i.out[0] * 4 for i in train if i.opcode == P.Op.ADAMW_STEP)
    assert nbytes >= grads and nbytes - grads < 64 * len(train)   # one block, alignment padding only
    assert off + nbytes <= plan.header["arena_size"]


def test_two_gloo_ranks_stay_bit_identical_and_match_the_whole_batch():
    oracle.build("oracle")
    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    with tempfile.TemporaryDirectory() as out_dir:
        procs = [ctx.Process(target=_worker, args=(r, world, port, out_dir)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout=240)
        for p in procs:
            if p.is_alive():
                p.kill()
                pytest.fail("a gloo rank did not finish")
            assert p.exitcode == 0
        r0 = np.load(os.path.join(out_dir, "rank0.npz"))
        r1 = np.load(os.path.join(out_dir, "rank1.npz"))
        # Replicated state: adapters and moments, bit for bit, after three steps.
        assert np.array_equal(r0["persist"], r1["persist"])
        assert np.array_equal(r0["grads"], r1["grads"])
        # The exchange over gloo is the rank-ordered fold, nothing else.
        persist_emulated, losses_emulated = _train_lockstep(_plan(GLOBAL_ROWS // world), world)
        assert np.array_equal(r0["persist"], persist_emulated)
        assert np.array_equal(dp.fixed_order_mean([r0["losses"], r1["losses"]]), losses_emulated)
        # Against one process training the whole batch: same gradient and loss up
        # to f32 summation order (the shards' means are averaged instead of one
        # mean over all rows).
        whole, _ = _train(_plan(GLOBAL_ROWS), slice(0, GLOBAL_ROWS), lambda *a: None)
        g_whole = whole[0][1]
        g_dp = r0["grads"][0]
        assert np.allclose(g_dp, g_whole, rtol=1e-4, atol=1e-7)
        mean_loss = dp.fixed_order_mean([r0["losses"][:1], r1["losses"][:1]])[0]
        assert abs(mean_loss - whole[0][0]) < 1e-5
