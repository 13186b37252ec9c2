"""The probe executable with seeml-plan-probe's command line and trace container
(reference: tool/seeml_plan_probe.cc:534-700, tool/probe_trace.h), over the C
ABI.  Without a GPU: it builds, parses its arguments and fails loudly.  On a
GPU: the first train run of a reference-compiled golden plan through it (files
in, `--trace`, arena image out), its trace compared extent by extent with the
trace the reference's own probe wrote for the same run — every extent the
reference says an instruction writes, in order, free-running from the staged
arena — and its `--time` line."""

import json
import os
import subprocess
import tempfile

import numpy as np
import pytest

from see_ai_b200 import build
from see_ai_b200 import plan as P
from tests.util import BIT_EXACT, Case, compare

PROBE = build.PROBE


def setup_module(_m):
    if not os.path.exists(PROBE):
        build.build()


def _have_gpu():
    import torch
    return torch.cuda.is_available()


def test_probe_builds_and_checks_its_arguments():
    assert os.path.exists(PROBE)
    r = subprocess.run([PROBE, "--version"], capture_output=True, text=True)
    assert r.returncode == 0 and r.stdout.startswith("see-cuda-plan-probe")
    r = subprocess.run([PROBE, "--plan", "nowhere"], capture_output=True, text=True)
    assert r.returncode == 1 and "usage" in r.stderr
    r = subprocess.run([PROBE, "--frobnicate"], capture_output=True, text=True)
    assert r.returncode == 1 and "unknown argument" in r.stderr
    with tempfile.TemporaryDirectory() as d:
        bad = os.path.join(d, "bad.seeu")
        open(bad, "wb").write(b"\0" * 4096)
        r = subprocess.run([PROBE, "--plan", bad, "--arena-in", bad, "--arena-out", os.path.join(d, "o")],
                           capture_output=True, text=True)
        assert r.returncode == 1 and "not a .seeu plan" in r.stderr


def _stage(case: Case, d: str):
    run = case.runs[0]
    arena = case.plan.stage_arena()
    case.stage_batch(arena, run)
    plan_path, in_path = os.path.join(d, "plan.seeu"), os.path.join(d, "arena.in")
    open(plan_path, "wb").write(case.z["plan"].tobytes())
    arena.tofile(in_path)
    lr_bits = "%08x" % P.f32_bits(case.lr)
    return run, plan_path, in_path, lr_bits


def test_probe_refuses_to_run_without_a_gpu():
    if _have_gpu():
        pytest.skip("a GPU is present")
    case = Case("mlp_tiny")
    with tempfile.TemporaryDirectory() as d:
        run, plan_path, in_path, lr_bits = _stage(case, d)
        r = subprocess.run([PROBE, "--plan", plan_path, "--section", run["section"], "--arena-in", in_path,
                            "--arena-out", os.path.join(d, "out"), "--lr-bits", lr_bits, "--step", str(run["step"])],
                           capture_output=True, text=True)
        assert r.returncode == 1 and "no CPU fallback" in r.stderr
        assert not os.path.exists(os.path.join(d, "out"))


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["mlp_tiny", "gpt_tiny_tiled"])
def test_probe_trace_agrees_with_the_reference_probes_trace(name):
    case = Case(name)
    with tempfile.TemporaryDirectory() as d:
        run, plan_path, in_path, lr_bits = _stage(case, d)
        out_path, trace_path = os.path.join(d, "arena.out"), os.path.join(d, "trace.sept")
        common = [PROBE, "--plan", plan_path, "--backend", "cpu", "--section", run["section"], "--arena-in", in_path,
                  "--lr-bits", lr_bits, "--step", str(run["step"]), "--threads", "4"]
        r = subprocess.run(common + ["--arena-out", out_path, "--trace", trace_path], capture_output=True, text=True)
        assert r.returncode == 0, r.stderr
        got = P.read_trace(open(trace_path, "rb").read())
        want = run["trace"]
        assert [(i, op, len(ext)) for (i, op, _r, ext) in got] == [(i, op, len(ext)) for (i, op, _r, ext) in want]
        lr = float(np.array([int(lr_bits, 16)], dtype=np.uint32).view(np.float32)[0])
        worst = 0.0
        for (idx, op, _rel, g_ext), (_i, _o, _r2, w_ext) in zip(got, want):
            for (g_off, g_bytes), (w_off, w_bytes) in zip(g_ext, w_ext):
                assert g_off == w_off and len(g_bytes) == len(w_bytes)
                # free-running: earlier 1e-7 differences (libm on the device) carry forward, so even the
                # bit-exact opcodes are held to the differ's default tolerance here (rtol 1e-5, atol 1e-7;
                # reference: tool/frontier_exec.py:2922-2923)
                # An optimizer step moves an element by lr * m / (sqrt(v) + eps); where a gradient is near eps that
                # quotient magnifies a 1e-7 difference of the gradient, so those extents are allowed 1e-3 of one
                # update's size (lr) on top of the looser relative bound.
                if "ADAMW" in P.OP_NAMES[op] or "SGD" in P.OP_NAMES[op]:
                    ok, ratio = compare(g_bytes, w_bytes, 1e-4, 1e-3 * lr)
                else:
                    ok, ratio = compare(g_bytes, w_bytes, 1e-5 if op in BIT_EXACT else 1e-4, 1e-7)
                worst = max(worst, ratio)
                assert ok, (idx, P.OP_NAMES[op], ratio)
        image = np.fromfile(out_path, dtype=np.uint8)
        assert image.size == case.header["arena_size"]
        # --time: one JSON line with the reference probe's keys
        r = subprocess.run(common + ["--arena-out", out_path, "--time", "3"], capture_output=True, text=True)
        assert r.returncode == 0, r.stderr
        line = json.loads(r.stdout.strip().splitlines()[-1])
        assert {"backend", "section", "executions", "ms_median", "ms_min", "ms_max", "relaxed_executions"} <= set(line)
        assert line["backend"] == "cuda" and line["executions"] == 3
