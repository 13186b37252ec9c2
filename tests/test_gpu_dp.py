"""Data parallelism on two GPUs: each rank trains half of every batch through
the CUDA engine, the gradient block is all-gathered over NCCL into local HBM and
the optimizer kernel folds the copies in rank order.  Checks: both ranks hold
bit-identical adapters and moments after every step (eager and graph replay),
and they agree with the two-rank CPU run of the same plans (oracle + gloo-style
fold) to f32 tolerance.  Skipped on a box with fewer than two GPUs."""

import multiprocessing as mp
import os
import tempfile

import numpy as np
import pytest

import oracle
from see_ai_b200 import dp
from tests.test_dp_gloo import GLOBAL_ROWS, _batches, _free_port, _plan, _train_lockstep

pytestmark = pytest.mark.gpu


def _gpu_worker(rank: int, world: int, port: int, out_dir: str, graphs: bool, explicit: bool = True):
    import torch
    import torch.distributed as dist
    from see_ai_b200 import synth
    from see_ai_b200.engine import Engine
    from tests.test_dp_gloo import DIMS, RANK
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        blob = synth.build_mlp_plan(synth.MlpConfig(dims=DIMS, batch=GLOBAL_ROWS // world, rank=RANK, lr=1e-2))
        stream = torch.cuda.Stream()
        eng = Engine(rank)
        with torch.cuda.stream(stream):
            eng.backend.set_stream(stream.cuda_stream)
            eng.load(blob)
            eng.set_horizon(1000)
            eng.set_use_graphs(graphs)
            exchange = dp.GradientExchange(eng)
            begin, end = dp.shard_rows(GLOBAL_ROWS, 0, world, rank)
            losses = []
            for x, y in _batches():
                eng.stage_batch(x[begin:end], y[begin:end])
                eng.train_forward_backward(True)
                if explicit:            # otherwise the optimizer call enqueues the all-gather itself
                    exchange.exchange()
                eng.train_optimizer()
                losses.append(exchange.mean_loss(eng.read_loss()))
            persist = eng.read_persistent()
        np.savez(os.path.join(out_dir, f"gpu{rank}.npz"), persist=persist,
                 losses=np.array(losses, dtype=np.float32))
        eng.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("graphs,explicit", [(False, True), (True, True), (True, False)],
                         ids=["eager", "graphs", "graphs-exchange-inside-the-optimizer-call"])
def test_two_gpu_ranks_replicate_state_and_match_the_cpu_ranks(graphs, explicit):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    oracle.build("oracle")
    world = 2
    ctx = mp.get_context("spawn")
    with tempfile.TemporaryDirectory() as out_dir:
        port = _free_port()
        procs = [ctx.Process(target=_gpu_worker, args=(r, world, port, out_dir, graphs, explicit)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout=300)
        for p in procs:
            if p.is_alive():
                p.kill()
                pytest.fail("a rank did not finish")
            assert p.exitcode == 0
        g0 = np.load(os.path.join(out_dir, "gpu0.npz"))
        g1 = np.load(os.path.join(out_dir, "gpu1.npz"))
    assert np.array_equal(g0["persist"], g1["persist"])
    assert np.array_equal(g0["losses"], g1["losses"])

    # The same two shards on the CPU (oracle), folded the same way.
    persist_cpu, losses_cpu = _train_lockstep(_plan(GLOBAL_ROWS // world), world)
    got = g0["persist"].view(np.float32)
    want = persist_cpu.view(np.float32)
    assert np.allclose(got, want, rtol=1e-4, atol=1e-6)
    assert np.allclose(g0["losses"], losses_cpu, rtol=1e-5, atol=1e-6)


def test_two_handles_in_one_process_each_configure_their_own_device():
    """One process, one backend per GPU (the C ABI's "one handle per GPU"): the kernels that
    need more than the default shared memory are configured per device, so the second handle's
    launches succeed and give the first one's bits."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from see_ai_b200 import backend as B
    from see_ai_b200 import plan as P
    from tests.test_gpu_umma import build_case
    rng = np.random.default_rng(7)
    # 4096 x 768 x 768: the persistent tensor-core kernel; 512 x 768 x 768: the one-tile kernel;
    # exact f32 instructions of the same shapes go to the CUDA-core kernels.
    for (M, N, K) in [(4096, 768, 768), (512, 768, 768)]:
        variants, dims, outs, arena, ro, _mags, _mag_of = build_case(rng, M, N, K)
        progs = [[P.Instr(op, fl | P.FLAG_RELAXED, 0, ins, dims) for (_n, op, fl, ins) in variants],
                 [P.Instr(op, fl, 0, ins, dims) for (_n, op, fl, ins) in variants[:3]]]
        for prog in progs:
            images = []
            for dev in (0, 1):
                img = arena.copy()
                be = B.CudaBackend(dev)
                be.bind(img, ro)
                be.run(prog)
                be.close()
                images.append(img)
            assert np.array_equal(images[0], images[1])
            for off in outs[:3]:
                assert np.isfinite(images[0][off:off + 4 * M * N].view(np.float32)).all()
