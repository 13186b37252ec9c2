"""The benchmark workloads and the work they are credited with.

Five configurations: the feed-forward plan (1), the isolated GEMM training-step
sweep (2), the small f32 decoder (3), the int8-weight decoder (4) and the
attention sweep (5).  Plans come from `synth`; the two sweeps are hand-built
instruction programs in the pattern the reference's kernel benchmarks use
(reference: tool/seeml_bench.cc:210-336).  `algorithmic_work` is the credit a
roofline figure is computed from — never a kernel's actual traffic: 2 M N K per
GEMM, 4 / 8 B H S^2 d per attention forward / backward with the causal mask not
discounted (reference: source/statistics/plan_work.h:34-62), and for the
bandwidth-bound opcodes the bytes an ideal kernel moves per element.
"""

from __future__ import annotations

import dataclasses
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from . import plan as P
from . import synth

Op = P.Op


# ---- configurations built from plans ------------------------------------------------------

def mlp_config(batch: int = 32) -> synth.MlpConfig:
    return synth.MlpConfig(dims=(256, 1024, 64), batch=batch, rank=8, alpha=16.0, lr=1e-3, steps=1000, seed=7)


def small_decoder_config(batch_seqs: int = 32) -> synth.DecoderConfig:
    return synth.DecoderConfig(layers=4, d_model=256, heads=4, ffn=1024, vocab=4096, seq=128,
                               batch_seqs=batch_seqs, rank=8, alpha=16.0, targets=("q", "v"), quantized=False,
                               attention="cached", lr=1e-3, steps=500, seed=7)


def int8_decoder_config(batch_seqs: int = 64) -> synth.DecoderConfig:
    return synth.DecoderConfig(layers=12, d_model=768, heads=12, ffn=3072, vocab=32000, seq=512,
                               batch_seqs=batch_seqs, rank=16, alpha=32.0, targets=("q", "k", "v", "o"),
                               quantized=True, attention="tiled", lr=1e-3, steps=1000, seed=7)


@dataclasses.dataclass
class PlanWorkload:
    key: str
    description: str
    unit: str                  # what a "token" is: tokens or samples
    global_units: int          # loss-target rows per optimizer step, all ranks together
    seq: int                   # rows per sequence (1: feature rows)
    dtype: str
    vocab: int = 0
    input_dim: int = 0
    classes: int = 0

    def build(self, world: int) -> bytes:
        raise NotImplementedError

    def batches(self, rows: int, count: int, seed: int):
        rng = np.random.default_rng(seed)
        out = []
        for _ in range(count):
            if self.seq > 1:
                rec = rng.integers(0, self.vocab, size=(rows // self.seq, self.seq + 1), dtype=np.int32)
                out.append((np.ascontiguousarray(rec[:, :-1]).reshape(-1), np.ascontiguousarray(rec[:, 1:]).reshape(-1)))
            else:
                out.append((rng.standard_normal((rows, self.input_dim)).astype(np.float32),
                            rng.integers(0, self.classes, size=rows).astype(np.int32)))
        return out


class MlpWorkload(PlanWorkload):
    def __init__(self):
        super().__init__("mlp", "feed-forward LoRA update: 256 -> 1024 (ReLU) -> 64 classes, batch 32, f32, LoRA r8 "
                         "alpha 16 on both products, AdamW lr 1e-3", "samples", 32, 1, "f32", input_dim=256, classes=64)

    def build(self, world: int) -> bytes:
        return synth.build_mlp_plan(mlp_config(32 // world))


class SmallDecoderWorkload(PlanWorkload):
    def __init__(self):
        super().__init__("decoder_f32", "f32 decoder LoRA update: 4 layers, d_model 256, 4 heads, FFN 1024 GELU, "
                         "vocab 4096, seq 128, batch 32 sequences, LoRA r8 alpha 16 on Q/V, cached attention, AdamW",
                         "tokens", 32 * 128, 128, "f32", vocab=4096)

    def build(self, world: int) -> bytes:
        return synth.build_decoder_plan(small_decoder_config(32 // world))


class Int8DecoderWorkload(PlanWorkload):
    def __init__(self, layers: int = 12, batch_seqs: int = 64):
        self.layers, self.batch_seqs = layers, batch_seqs
        super().__init__("decoder_int8", f"int8-weight decoder LoRA update: {layers} layers, d_model 768, 12 heads, "
                         f"FFN 3072, vocab 32000, seq 512, global batch {batch_seqs} sequences, LoRA r16 alpha 32 on "
                         "Q/K/V/O, relaxed bf16 GEMMs, AdamW", "tokens", batch_seqs * 512, 512, "bf16", vocab=32000)

    def build(self, world: int) -> bytes:
        cfg = int8_decoder_config(self.batch_seqs // world)
        cfg.layers = self.layers
        return synth.build_decoder_plan(cfg)


def plan_workload(config: int) -> PlanWorkload:
    return {1: MlpWorkload, 3: SmallDecoderWorkload, 4: Int8DecoderWorkload}[config]()


# ---- hand-built sweep programs --------------------------------------------------------------

def _al(n: int, a: int = 64) -> int:
    return (n + a - 1) // a * a


def bf16_representable(x: np.ndarray) -> np.ndarray:
    b = x.astype(np.float32).view(np.uint32).astype(np.uint64)
    b = (b + 0x7FFF + ((b >> 16) & 1)) & 0xFFFF0000
    return b.astype(np.uint32).view(np.float32)


@dataclasses.dataclass
class Program:
    instrs: List[P.Instr]
    arena: np.ndarray
    rodata: np.ndarray
    refs: Dict[str, int]
    flops: float


def gemm_step_program(S: int, relaxed: bool, rank: int = 8, seed: int = 0) -> Program:
    """One training step around a square frozen weight W [S, S]: C = A W, dA = dC W^T,
    dW-shaped product A^T dC, and the six rank-r products of a LoRA adapter on W
    (t = A La, C += s t Lb, dT = s dC Lb^T, dLb = s t^T dC, dA += dT La^T, dLa = A^T dT).
    f32: exact opcodes.  bf16: the two frozen-weight products carry the relaxed
    permission and every operand is bf16-representable, so both precisions see
    identical inputs."""
    rng = np.random.default_rng(seed + S)
    r = rank
    refs, size = {}, 0
    for name, n in (("A", S * S), ("dC", S * S), ("C0", S * S), ("C", S * S), ("dA0", S * S), ("dA", S * S),
                    ("dW", S * S), ("La", S * r), ("Lb", r * S), ("t", S * r), ("dT", S * r), ("dLa", S * r),
                    ("dLb", r * S)):
        refs[name] = size
        size = _al(size + 4 * n)
    arena = np.zeros(size, dtype=np.uint8)

    def put(name, arr):
        arena[refs[name]:refs[name] + arr.nbytes] = arr.view(np.uint8).reshape(-1)

    conv = bf16_representable if relaxed else (lambda v: v)
    put("A", conv(rng.standard_normal((S, S)).astype(np.float32)))
    put("dC", conv(rng.standard_normal((S, S)).astype(np.float32)))
    put("La", (rng.standard_normal((S, r)) / np.sqrt(S)).astype(np.float32))
    put("Lb", (rng.standard_normal((r, S)) * 0.02).astype(np.float32))
    W = conv((rng.standard_normal((S, S)) * 0.02).astype(np.float32))
    rodata = W.view(np.uint8).reshape(-1).copy()
    w_ref = P.RODATA_BIT
    rel = P.FLAG_RELAXED if relaxed else 0
    s_bits = P.f32_bits(2.0)
    o = refs
    instrs = [
        P.Instr(Op.GEMM_NN, rel, 0, (o["A"], w_ref, o["C0"], P.NULL_REF), (S, S, S)),
        P.Instr(Op.GEMM_NN, 0, 0, (o["A"], o["La"], o["t"], P.NULL_REF), (S, r, S)),
        P.Instr(Op.GEMM_NN, P.FLAG_GEMM_ADDEND, s_bits, (o["t"], o["Lb"], o["C"], o["C0"]), (S, S, r)),
        P.Instr(Op.GEMM_NT, 0, s_bits, (o["dC"], o["Lb"], o["dT"], P.NULL_REF), (S, r, S)),
        P.Instr(Op.GEMM_TN, 0, s_bits, (o["t"], o["dC"], o["dLb"], P.NULL_REF), (r, S, S)),
        P.Instr(Op.GEMM_TN, 0, 0, (o["A"], o["dT"], o["dLa"], P.NULL_REF), (S, r, S)),
        P.Instr(Op.GEMM_NT, rel, 0, (o["dC"], w_ref, o["dA0"], P.NULL_REF), (S, S, S)),
        P.Instr(Op.GEMM_NT, P.FLAG_GEMM_ADDEND, 0, (o["dT"], o["La"], o["dA"], o["dA0"]), (S, S, r)),
        P.Instr(Op.GEMM_TN, 0, 0, (o["A"], o["dC"], o["dW"], P.NULL_REF), (S, S, S)),
        # The two un-adapted products are scratch: cleared before the step ends, as a plan's
        # next pass would overwrite them (this is what lets a backend prove them dead).
        P.Instr(Op.FILL, 0, 0, (o["C0"], 0), (S * S, 0, 0)),
        P.Instr(Op.FILL, 0, 0, (o["dA0"], 0), (S * S, 0, 0)),
    ]
    flops = sum(2.0 * i.out[0] * i.out[1] * i.out[2] for i in instrs if i.opcode in (Op.GEMM_NN, Op.GEMM_NT, Op.GEMM_TN))
    return Program(instrs, arena, rodata, refs, flops)


def attention_chain_program(Bq: int, S: int, H: int, d: int, relaxed: bool = True, seed: int = 0) -> Program:
    """The tiled causal attention chain a plan carries: forward, dQ (writes delta),
    dK (reads it), dV; Q, K, V, dO ~ N(0, 1) rounded to bf16-representable f32."""
    rng = np.random.default_rng(seed + S + d)
    td = Bq * S * H * d
    refs, size = {}, 0
    for name in ("q", "k", "v", "do", "o", "dq", "dk", "dv"):
        refs[name] = size
        size = _al(size + 4 * td)
    refs["stats"] = size
    size = _al(size + 16 * Bq * H * S)
    arena = np.zeros(size, dtype=np.uint8)
    for name in ("q", "k", "v", "do"):
        arena[refs[name]:refs[name] + 4 * td] = bf16_representable(
            rng.standard_normal(td, dtype=np.float32)).view(np.uint8)
    o = refs
    bs, hd, geo = P.pack2(Bq, S), P.pack2(H, d), P.pack_attn_geometry(Bq, S, H, d)
    fl = P.FLAG_RELAXED if relaxed else 0
    instrs = [
        P.Instr(Op.ATTN_FWD_TILED, fl, 0, (o["q"], o["k"], o["v"], o["o"]), (o["stats"], bs, hd)),
        P.Instr(Op.ATTN_DQ_TILED, fl, 0, (o["q"], o["k"], o["v"], o["do"]), (o["stats"], o["dq"], geo)),
        P.Instr(Op.ATTN_DK_TILED, fl, 0, (o["q"], o["k"], o["v"], o["do"]), (o["stats"], o["dk"], geo)),
        P.Instr(Op.ATTN_DV_TILED, fl, 0, (o["q"], o["k"], o["v"], o["do"]), (o["stats"], o["dv"], geo)),
    ]
    flops = 12.0 * Bq * H * S * S * d
    return Program(instrs, arena, np.zeros(64, dtype=np.uint8), refs, flops)


# ---- algorithmic work per instruction -------------------------------------------------------

_BYTES_PER_ELEM = {
    Op.ADD_EW: 12, Op.MUL_EW: 12, Op.ACCUMULATE: 12, Op.RELU_BWD: 12, Op.GELU_BWD: 12, Op.SILU_BWD: 12,
    Op.ADD_BIAS: 8, Op.RELU_FWD: 8, Op.GELU_FWD: 8, Op.SILU_FWD: 8, Op.SCALE: 8, Op.COPY: 8, Op.FILL: 4,
    Op.ADAMW_STEP: 28, Op.SGD_STEP: 12,
}


def algorithmic_work(ins: P.Instr) -> Tuple[float, float]:
    """-> (flops, bytes) an instruction is credited with.  GEMMs and attention:
    flops (bytes 0: they are tensor-bound); everything else: bytes."""
    op = ins.opcode
    if op in (Op.GEMM_NN, Op.GEMM_NT, Op.GEMM_TN, Op.GEMM_ACC_NN, Op.GEMM_NN_Q8, Op.GEMM_NT_Q8,
              Op.GEMM_NN_BF16, Op.GEMM_NT_BF16):
        return 2.0 * ins.out[0] * ins.out[1] * ins.out[2], 0.0
    if op in (Op.ATTN_FWD, Op.ATTN_FWD_TILED):
        Bq, S, H, d = ins.out[1] >> 32, ins.out[1] & 0xFFFFFFFF, ins.out[2] >> 32, ins.out[2] & 0xFFFFFFFF
        return 4.0 * Bq * H * S * S * d, 0.0
    if op in (Op.ATTN_DQ_TILED, Op.ATTN_DK_TILED, Op.ATTN_DV_TILED):
        g = ins.out[2]
        Bq, S, H, d = g >> 48, (g >> 32) & 0xFFFF, (g >> 16) & 0xFFFF, g & 0xFFFF
        return 8.0 * Bq * H * S * S * d / 3.0, 0.0     # the backward's 8 B H S^2 d over its three opcodes
    if op in _BYTES_PER_ELEM:
        n = ins.out[0] * ins.out[1] if op == Op.ADD_BIAS else ins.out[0]
        return 0.0, float(_BYTES_PER_ELEM[op] * n)
    if op in (Op.LAYERNORM_FWD, Op.RMSNORM_FWD):
        rows, cols = ins.out[0] >> 32, ins.out[0] & 0xFFFFFFFF
        return 0.0, float(8 * rows * cols + 8 * rows)
    if op == Op.LAYERNORM_BWD:
        rows, cols = ins.out[2] >> 32, ins.out[2] & 0xFFFFFFFF
        return 0.0, float(12 * rows * cols)
    if op == Op.RMSNORM_BWD:
        rows, cols = ins.out[1] >> 32, ins.out[1] & 0xFFFFFFFF
        return 0.0, float(12 * rows * cols)
    if op in (Op.XENT_FWD, Op.XENT_MASKED_FWD, Op.XENT_BWD, Op.XENT_MASKED_BWD):
        return 0.0, float(8 * ins.out[0] * ins.out[1])
    if op == Op.EMBED_FWD:
        rows, dim = ins.out[0], ins.out[1] & 0xFFFFFFFF
        return 0.0, float(8 * rows * dim + 4 * rows)
    return 0.0, 0.0
