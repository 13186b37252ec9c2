#!/usr/bin/env python3
"""Generates the golden fixtures in this directory from the reference itself.

Run in the authoring container only (it needs the reference tree and the tools
built by build_ref_tools.sh); tests never run it:

    sh tests/golden/build_ref_tools.sh
    python tests/golden/make_golden.py [case ...]

For each case it exports a small model with the reference's own exporter
(tool/export_model.py), compiles it with the reference's `seeml-update-compile`,
stages an arena exactly as the reference's differ does (zeros, the persist_init
image at offset 0, a seeded batch in the I/O slots; tool/frontier_exec.py
`Executor.stage`), and runs the plan's sections through the reference CPU
executor with `seeml-plan-probe --trace`.  What is stored per case, in one
compressed .npz: the sealed plan, the staged batches, and the probe's write
trace of every instruction (the bytes the reference executor wrote).
"""

from __future__ import annotations

import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))
REF = os.environ.get("SEE_REFERENCE_ROOT", "/root/reference")
TOOLS = os.environ.get("SEE_REF_TOOLS", "/tmp/see_ref_tools")
sys.path.insert(0, REPO)
sys.path.insert(0, os.path.join(REF, "tool"))

from see_ai_b200 import plan as P  # noqa: E402


def run(cmd, cwd=None):
    r = subprocess.run(cmd, cwd=cwd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"{' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    return r.stdout


def compile_plan(smf, out_dir, flags):
    run([os.path.join(TOOLS, "seeml-update-compile"), "--source", smf, "--out", out_dir,
         "--no-embed"] + flags, cwd=REF)
    return os.path.join(out_dir, "update_plan.seeu")


def probe(plan_path, section, arena, lr, step, workdir, source=None):
    ain = os.path.join(workdir, "arena_in.bin")
    aout = os.path.join(workdir, "arena_out.bin")
    trace = os.path.join(workdir, "trace.bin")
    arena.tofile(ain)
    for p in (aout, trace):
        if os.path.exists(p):
            os.remove(p)
    cmd = [os.path.join(TOOLS, "seeml-plan-probe"), "--plan", plan_path, "--section", section,
           "--arena-in", ain, "--arena-out", aout, "--trace", trace,
           "--lr-bits", hex(P.f32_bits(lr)), "--step", str(step), "--backend", "cpu",
           "--threads", "3"]
    if source:
        cmd += ["--source", source]
    run(cmd)
    return np.fromfile(aout, dtype=np.uint8), np.fromfile(trace, dtype=np.uint8)


def mlp_smf(path, dims, act="relu", seed=7):
    import torch
    import torch.nn as nn
    import export_model as E
    torch.manual_seed(seed)
    layers = []
    for i in range(len(dims) - 1):
        lin = nn.Linear(dims[i], dims[i + 1])
        nn.init.normal_(lin.weight, 0.0, 0.02)
        nn.init.normal_(lin.bias, 0.0, 0.02)
        layers.append(lin)
        if i + 2 < len(dims):
            layers.append({"relu": nn.ReLU(), "gelu": nn.GELU(approximate="tanh"),
                           "silu": nn.SiLU()}[act])
    E.export_smf(nn.Sequential(*layers), path)


def gpt_smf(path, L, D, H, F, V, S, seed=7):
    """Pre-norm GELU / LayerNorm decoder with a learned token embedding, built
    op by op with the reference exporter's container writer."""
    import export_model as E
    rng = np.random.default_rng(seed)
    b = E._SmfBuilder("x", D, seq_len=S, token_input=True)

    def w(name, *shape, std=0.02):
        a = (rng.standard_normal(shape) * std).astype("<f4")
        b.add_tensor(name, list(shape), np.ascontiguousarray(a))
        return name

    def const(name, n, value):
        b.add_tensor(name, [n], np.full(n, value, dtype="<f4"))
        return name

    w("emb", V, D)
    b.add_op(E.OP_EMBEDDING, "embed", ["x", "emb"], "e")
    prev = "e"
    for i in range(L):
        p = f"l{i}."
        const(p + "ln1_g", D, 1.0); const(p + "ln1_b", D, 0.0)
        b.add_op(E.OP_LAYERNORM, p + "ln1", [prev, p + "ln1_g", p + "ln1_b"], p + "n1")
        for nm in ("wq", "wk", "wv"):
            w(p + nm, D, D)
            b.add_op(E.OP_MATMUL, p + "mm_" + nm, [p + "n1", p + nm], p + nm[1])
        b.add_op(E.OP_ATTENTION, p + "attn", [p + "q", p + "k", p + "v"], p + "a", attr0=H)
        w(p + "wo", D, D)
        b.add_op(E.OP_MATMUL, p + "mm_wo", [p + "a", p + "wo"], p + "o")
        b.add_op(E.OP_ADD, p + "res1", [prev, p + "o"], p + "x1")
        const(p + "ln2_g", D, 1.0); const(p + "ln2_b", D, 0.0)
        b.add_op(E.OP_LAYERNORM, p + "ln2", [p + "x1", p + "ln2_g", p + "ln2_b"], p + "n2")
        w(p + "w1", D, F); w(p + "b1", F)
        b.add_op(E.OP_MATMUL, p + "mm_w1", [p + "n2", p + "w1"], p + "f1")
        b.add_op(E.OP_ADDBIAS, p + "ab1", [p + "f1", p + "b1"], p + "f1b")
        b.add_op(E.OP_GELU, p + "gelu", [p + "f1b"], p + "g")
        w(p + "w2", F, D); w(p + "b2", D)
        b.add_op(E.OP_MATMUL, p + "mm_w2", [p + "g", p + "w2"], p + "f2")
        b.add_op(E.OP_ADDBIAS, p + "ab2", [p + "f2", p + "b2"], p + "f2b")
        b.add_op(E.OP_ADD, p + "res2", [p + "x1", p + "f2b"], p + "x2")
        prev = p + "x2"
    const("lnf_g", D, 1.0); const("lnf_b", D, 0.0)
    b.add_op(E.OP_LAYERNORM, "lnf", [prev, "lnf_g", "lnf_b"], "nf")
    w("w_head", D, V)
    b.add_op(E.OP_MATMUL, "mm_head", ["nf", "w_head"], "logits")
    with open(path, "wb") as f:
        b.write(f)


def llama_smf(path, L, D, H, F, V, S, seed=7):
    import export_model as E
    rng = np.random.default_rng(seed)

    def m(*shape):
        return (rng.standard_normal(shape) * 0.05).astype("<f4")

    blocks = [dict(ln1_g=np.ones(D, "<f4"), wq=m(D, D), wk=m(D, D), wv=m(D, D), wo=m(D, D),
                   ln2_g=np.ones(D, "<f4"), w_gate=m(D, F), w_up=m(D, F), w_down=m(F, D))
              for _ in range(L)]
    head = dict(lnf_g=np.ones(D, "<f4"), w_head=m(D, V))
    E.export_token_decoder_smf(m(V, D), blocks, head, path, seq_len=S, num_heads=H)


COMMON = ["--loss", "xent", "--lr", "1e-3", "--steps", "20"]

CASES = {
    # name: (model builder, kind, compile flags)
    "mlp_tiny": (lambda p: mlp_smf(p, [16, 32, 8]), "class",
                 ["--data-batch", "8", "--lora-rank", "4", "--lora-alpha", "8"]),
    "mlp_unfused_clip": (lambda p: mlp_smf(p, [16, 32, 8], act="silu"), "class",
                         ["--data-batch", "8", "--lora-rank", "4", "--lora-alpha", "8",
                          "--no-fuse-epilogue", "--no-fuse-addend", "--no-fuse-elementwise",
                          "--no-fuse-clip", "--clip-norm", "0.05"]),
    "mlp_global_clip": (lambda p: mlp_smf(p, [16, 32, 8], act="gelu"), "class",
                        ["--data-batch", "8", "--lora-rank", "4", "--lora-alpha", "6",
                         "--clip-norm", "0.05", "--clip-mode", "global"]),
    "mlp_sgd_accum": (lambda p: mlp_smf(p, [16, 32, 8]), "class",
                      ["--data-batch", "8", "--lora-rank", "4", "--lora-alpha", "8",
                       "--optimizer", "sgd", "--grad-accum", "2", "--clip-norm", "0.05"]),
    "gpt_tiny_cached": (lambda p: gpt_smf(p, 2, 32, 2, 64, 64, 8), "token",
                        ["--data-batch", "16", "--lora-rank", "4", "--lora-alpha", "8",
                         "--targets", "wq,wv", "--attention", "cached"]),
    "gpt_tiny_tiled": (lambda p: gpt_smf(p, 2, 32, 2, 64, 64, 8), "token",
                       ["--data-batch", "16", "--lora-rank", "4", "--lora-alpha", "8",
                        "--targets", "wq,wv", "--attention", "tiled"]),
    "gpt_tiny_q8_relaxed": (lambda p: gpt_smf(p, 2, 32, 2, 64, 64, 8), "token",
                            ["--data-batch", "16", "--lora-rank", "4", "--lora-alpha", "8",
                             "--targets", "wq,wk,wv,wo", "--attention", "tiled",
                             "--quantize-base", "--precision", "certified-bf16"]),
    "llama_tiny_bf16": (lambda p: llama_smf(p, 1, 32, 2, 48, 64, 8), "token",
                        ["--data-batch", "16", "--lora-rank", "4", "--lora-alpha", "8",
                         "--bf16-base", "--attention", "cached"]),
}


def make_case(name, out_path):
    builder, kind, flags = CASES[name]
    rng = np.random.default_rng(1234)
    with tempfile.TemporaryDirectory() as tmp:
        smf = os.path.join(tmp, "model.smf")
        builder(smf)
        plan_path = compile_plan(smf, os.path.join(tmp, "pkg"), COMMON + flags)
        with open(plan_path, "rb") as f:
            blob = f.read()
        plan = P.Plan(blob)
        assert plan.verify_seal(), "python seal disagrees with the compiler's"
        h = plan.header
        store = {"plan": np.frombuffer(blob, dtype=np.uint8)}
        needs_source = any(r != P.NULL_REF and (r >> 62) == 1
                           for ins in plan.eval for r in ins.ins)
        if needs_source:
            with open(smf, "rb") as f:
                store["source_model"] = np.frombuffer(f.read(), dtype=np.uint8)

        def batch():
            rows = h["batch"]
            if kind == "token":
                vocab = 64
                S = h["seq_len"]
                rec = rng.integers(0, vocab, size=(rows // S, S + 1), dtype=np.int32)
                return rec[:, :-1].reshape(-1).copy(), rec[:, 1:].reshape(-1).copy()
            x = rng.standard_normal((rows, h["input_floats"] // rows)).astype(np.float32)
            y = rng.integers(0, 8, size=rows, dtype=np.int32)
            return x, y

        def stage(arena, x, y):
            xb = np.ascontiguousarray(x).view(np.uint8).reshape(-1)
            yb = np.ascontiguousarray(y).view(np.uint8).reshape(-1)
            arena[h["input_ref"]:h["input_ref"] + xb.size] = xb
            arena[h["label_ref"]:h["label_ref"] + yb.size] = yb

        arena = plan.stage_arena()
        runs = []
        lr = 1e-3
        accum = max(1, h["grad_accum_steps"])
        step_no = 0
        for _ in range(2):
            step_no += 1
            for _micro in range(accum):
                x, y = batch()
                stage(arena, x, y)
                runs.append(("train", step_no, x, y))
            if accum > 1:
                runs.append(("step", step_no, None, None))
        x, y = batch()
        runs.append(("eval", step_no, x, y))
        runs.append(("merge", step_no, None, None))

        arena = plan.stage_arena()
        store["n_runs"] = np.array(len(runs))
        for i, (section, step, x, y) in enumerate(runs):
            if x is not None:
                stage(arena, x, y)
                store[f"run{i}_x"] = np.asarray(x)
                store[f"run{i}_y"] = np.asarray(y)
            arena, trace = probe(plan_path, section, arena, lr, step, tmp,
                                 source=smf if (needs_source and section == "eval") else None)
            store[f"run{i}_section"] = np.array(section)
            store[f"run{i}_step"] = np.array(step)
            store[f"run{i}_trace"] = trace
        store["lr"] = np.array(lr, dtype=np.float32)
        store["final_arena"] = arena
        np.savez_compressed(out_path, **store)
    ops = sorted({i.opcode for sec in ("train", "eval", "merge", "step") for i in plan.section(sec)})
    print(f"{name}: {os.path.getsize(out_path)} bytes; arena {h['arena_size']}; "
          f"train/eval/merge/step = {len(plan.train)}/{len(plan.eval)}/{len(plan.merge)}/"
          f"{len(plan.step)}; opcodes {[P.OP_NAMES[o] for o in ops]}")


if __name__ == "__main__":
    names = sys.argv[1:] or list(CASES)
    for n in names:
        make_case(n, os.path.join(HERE, n + ".npz"))
