"""The plan synthesizer against the reference compiler: for the same tiny
models, the synthesized instruction streams (opcode, flags, immediate, shape
words) equal the streams `seeml-update-compile` emitted (the golden plans) —
forward, loss and backward in order; the optimizer steps as a multiset (their
order follows the reference's tensor numbering, which carries no arithmetic).
Operand offsets are layout, not arithmetic, and are compared only for validity:
the synthesized plan must execute on the CPU oracle and train."""

import collections

import numpy as np
import pytest

import oracle
from see_ai_b200 import plan as P
from see_ai_b200 import synth
from tests.util import Case

Op = P.Op

# Which `out` words of an opcode are shape words (the rest are operand refs).
SHAPE_WORDS = {
    Op.LAYERNORM_FWD: (0,), Op.LAYERNORM_BWD: (2,), Op.ATTN_FWD: (1, 2), Op.ATTN_FWD_TILED: (1, 2),
    Op.ATTN_DQ_TILED: (2,), Op.ATTN_DK_TILED: (2,), Op.ATTN_DV_TILED: (2,),
}


def signature(ins: P.Instr):
    words = SHAPE_WORDS.get(ins.opcode, (0, 1, 2))
    extra = ()
    if ins.opcode == Op.FILL:
        extra = (ins.ins[1],)
    if ins.opcode == Op.GEMM_ACC_NN:
        extra = (ins.ins[3],)
    return (P.OP_NAMES[ins.opcode], ins.flags, ins.imm, tuple(ins.out[w] for w in words), extra)


def split_optimizer(prog):
    opt = [i for i, ins in enumerate(prog) if ins.opcode in (Op.ADAMW_STEP, Op.SGD_STEP)]
    cut = opt[0] if opt else len(prog)
    return prog[:cut], prog[cut:]


GPT = dict(layers=2, d_model=32, heads=2, ffn=64, vocab=64, seq=8, batch_seqs=2, rank=4, alpha=8.0,
           steps=20)
CASES = {
    "gpt_tiny_cached": synth.DecoderConfig(**GPT, targets=("q", "v"), attention="cached"),
    "gpt_tiny_tiled": synth.DecoderConfig(**GPT, targets=("q", "v"), attention="tiled"),
    "gpt_tiny_q8_relaxed": synth.DecoderConfig(**GPT, targets=("q", "k", "v", "o"), attention="tiled",
                                               quantized=True),
}


@pytest.mark.parametrize("name", list(CASES))
def test_decoder_streams_match_reference_compiler(name):
    ref = Case(name).plan
    ours = P.Plan(synth.build_decoder_plan(CASES[name]))
    assert ours.verify_seal()
    body_r, opt_r = split_optimizer(ref.train)
    body_o, opt_o = split_optimizer(ours.train)
    sig_r, sig_o = [signature(i) for i in body_r], [signature(i) for i in body_o]
    for k, (a, b) in enumerate(zip(sig_r, sig_o)):
        assert a == b, f"train[{k}]: reference {a} != synthesized {b}"
    assert len(sig_r) == len(sig_o)
    assert collections.Counter(map(signature, opt_r)) == collections.Counter(map(signature, opt_o))
    assert collections.Counter(map(signature, ref.merge)) == collections.Counter(map(signature, ours.merge))
    # eval: the reference reads the shipped f32 file through source refs for a
    # quantized plan; the shapes and the op sequence still agree for f32 plans.
    if not CASES[name].quantized:
        assert [signature(i) for i in ref.eval] == [signature(i) for i in ours.eval]
    assert ours.header["persistent_size"] == ref.header["persistent_size"]
    assert ours.header["batch"] == ref.header["batch"] and ours.header["seq_len"] == ref.header["seq_len"]


def test_mlp_stream_matches_reference_compiler():
    ref = Case("mlp_tiny").plan
    ours = P.Plan(synth.build_mlp_plan(synth.MlpConfig(dims=(16, 32, 8), batch=8, rank=4, alpha=8.0,
                                                       steps=20)))
    body_r, opt_r = split_optimizer(ref.train)
    body_o, opt_o = split_optimizer(ours.train)
    assert [signature(i) for i in body_r] == [signature(i) for i in body_o]
    assert collections.Counter(map(signature, opt_r)) == collections.Counter(map(signature, opt_o))
    assert [signature(i) for i in ref.eval] == [signature(i) for i in ours.eval]
    assert ours.header["persistent_size"] == ref.header["persistent_size"]


@pytest.mark.parametrize("name", list(CASES))
def test_synthesized_plan_trains_on_the_oracle(name):
    """No operand aliasing, no use of an unwritten transient: the loss falls over
    a few steps on a repeated batch, and a poisoned arena changes nothing."""
    oracle.build("oracle")
    plan = P.Plan(synth.build_decoder_plan(CASES[name]))
    h = plan.header
    rng = np.random.default_rng(0)
    rec = rng.integers(0, 64, size=(h["batch"] // h["seq_len"], h["seq_len"] + 1), dtype=np.int32)
    x, y = rec[:, :-1].reshape(-1).copy(), rec[:, 1:].reshape(-1).copy()
    losses = {}
    for poison in (False, True):
        arena = plan.stage_arena()
        if poison:  # transients start as NaN: every read of an unwritten slot would surface
            arena[h["persistent_size"]:].view(np.float32)[:] = np.nan
        arena[h["input_ref"]:h["input_ref"] + x.nbytes] = x.view(np.uint8)
        arena[h["label_ref"]:h["label_ref"] + y.nbytes] = y.view(np.uint8)
        ex = oracle.OracleExecutor()
        ex.bind(arena, np.frombuffer(plan.rodata, dtype=np.uint8).copy())
        out = []
        for step in range(1, 6):
            ex.run(plan.train, oracle.step_params(lr=1e-2, weight_decay=0.0, step=step))
            out.append(float(arena[h["loss_ref"]:h["loss_ref"] + 4].view(np.float32)[0]))
        losses[poison] = out
    assert losses[False] == losses[True]
    assert all(np.isfinite(losses[False]))
    assert losses[False][-1] < losses[False][0]
