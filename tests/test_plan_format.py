"""The plan container: read the reference compiler's plans, verify the seal,
round-trip our writer."""

import numpy as np
import pytest

from see_ai_b200 import plan as P
from tests.util import CASES, Case


@pytest.mark.parametrize("name", CASES)
def test_reads_reference_plans_and_verifies_seal(name):
    c = Case(name)
    h = c.header
    assert h["magic"] == P.SEEU_MAGIC and h["version"] == 26
    assert c.plan.verify_seal()
    assert len(c.plan.train) == h["train_instr_count"] > 0
    assert h["persist_init_size"] == h["persistent_size"]
    # Every run's trace names instructions of the section it ran.
    for run in c.runs:
        prog = c.plan.section(run["section"])
        assert len(run["trace"]) == len(prog)
        for (idx, op, _rel, _ext) in run["trace"]:
            assert prog[idx].opcode == op


def test_seal_detects_corruption():
    c = Case("mlp_tiny")
    blob = bytearray(c.plan.blob)
    blob[c.header["rodata_offset"] + 5] ^= 1
    assert not P.Plan(bytes(blob)).verify_seal()


def test_writer_round_trip():
    c = Case("gpt_tiny_tiled")
    h = dict(c.header)
    blob = P.write_plan(h, c.plan.train, c.plan.eval, c.plan.merge, c.plan.step,
                        bytes(c.plan.rodata), bytes(c.plan.persist_init), c.plan.emit)
    p2 = P.Plan(blob)
    assert p2.verify_seal()
    assert [i.pack() for i in p2.train] == [i.pack() for i in c.plan.train]
    assert [i.pack() for i in p2.eval] == [i.pack() for i in c.plan.eval]
    assert bytes(p2.rodata) == bytes(c.plan.rodata)
    assert bytes(p2.persist_init) == bytes(c.plan.persist_init)
    assert p2.header["arena_size"] == h["arena_size"]
    assert p2.header["rodata_offset"] % 16384 == 0


def test_instruction_word_layout():
    i = P.Instr(P.Op.GEMM_NN, P.FLAG_GEMM_ADDEND, P.f32_bits(2.0), (1, 2, 3, 4), (5, 6, 7))
    raw = i.pack()
    assert len(raw) == 64
    assert P.Instr.unpack(raw) == i
    assert P.bits_f32(P.f32_bits(0.25)) == 0.25
