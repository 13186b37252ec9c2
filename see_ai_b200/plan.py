"""The `.seeu` update-plan container: reader, writer and instruction words.

This is a fresh statement of the wire format the reference compiler emits
(reference: source/plan/schema.h:298-397 for the 320-byte header and the emit
entry, source/plan/instruction.h:44-232 for the opcodes, :311-384 for the
flags, :438-449 for the 64-byte instruction word; source/identity/hash.h:80-161
for the seal).  A plan written by `seeml-update-compile` is read unchanged;
plans written here (the synthetic benchmark programs) use the same container so
the C++ loader has exactly one format to parse.
"""

from __future__ import annotations

import dataclasses
import struct
from typing import List, Optional, Sequence

import numpy as np

SEEU_MAGIC = 0x55454553  # "SEEU", little-endian
SEEU_VERSION = 26
HEADER_BYTES = 320
INSTR_BYTES = 64
PLAN_HASH_OFFSET = 216
RODATA_ALIGNMENT = 16384

RODATA_BIT = 1 << 63
SOURCE_BIT = 1 << 62
NULL_REF = (1 << 64) - 1


class Op:
    """Opcode numbers (reference: source/plan/instruction.h:44-232)."""

    NOP = 0
    GEMM_NN = 1
    GEMM_NT = 2
    GEMM_TN = 3
    GEMM_ACC_NN = 4
    ADD_EW = 5
    ADD_BIAS = 6
    RELU_FWD = 7
    RELU_BWD = 8
    SCALE = 9
    REDUCE_ROWS = 10
    XENT_FWD = 11
    XENT_BWD = 12
    MSE_FWD = 13
    MSE_BWD = 14
    KL_FWD = 15
    KL_BWD = 16
    SGD_STEP = 17
    ADAMW_STEP = 18
    FILL = 19
    COPY = 20
    MUL_EW = 21
    GELU_FWD = 22
    GELU_BWD = 23
    SILU_FWD = 24
    SILU_BWD = 25
    LAYERNORM_FWD = 26
    LAYERNORM_BWD = 27
    CLIP_NORM = 28
    GEMM_NN_Q8 = 29
    GEMM_NT_Q8 = 30
    RMSNORM_FWD = 31
    RMSNORM_BWD = 32
    ROPE_FWD = 33
    ROPE_BWD = 34
    ATTN_FWD = 35
    ATTN_DP = 36
    ATTN_DV = 37
    SOFTMAX_ROWS_BWD = 38
    ATTN_DQ = 39
    ATTN_DK = 40
    EMBED_FWD = 41
    ACCUMULATE = 42
    GEMM_NN_BF16 = 43
    GEMM_NT_BF16 = 44
    ROPE_TABLE = 45
    FUSED_MAP = 46
    ATTN_FWD_TILED = 47
    ATTN_DQ_TILED = 48
    ATTN_DK_TILED = 49
    ATTN_DV_TILED = 50
    XENT_MASKED_FWD = 51
    XENT_MASKED_BWD = 52
    SQNORM_ACCUM = 53
    CLIP_GLOBAL = 54
    SEGMENT_STARTS = 55
    ATTN_FWD_SEG = 56
    ATTN_FWD_TILED_SEG = 57


OP_NAMES = {v: k for k, v in vars(Op).items() if k.isupper()}

# Instruction flags (reference: source/plan/instruction.h:311-384).
FLAG_EPILOGUE_BIAS = 1 << 0
FLAG_ACT_SHIFT = 1
FLAG_ACT_MASK = 3 << 1
FLAG_GEMM_ADDEND = 1 << 3
FLAG_Q8_COL_SCALE = 1 << 4
FLAG_RELAXED = 1 << 5
ACT_NONE, ACT_RELU, ACT_GELU, ACT_SILU = 0, 1, 2, 3

_INSTR = struct.Struct("<HHI4Q3Q")
assert _INSTR.size == INSTR_BYTES

_HEADER_FIELDS = [
    ("magic", "I"), ("version", "I"),
    ("arena_size", "Q"), ("persistent_size", "Q"),
    ("input_ref", "Q"), ("input_floats", "Q"),
    ("label_ref", "Q"), ("label_bytes", "Q"),
    ("label_kind", "I"), ("optimizer_kind", "I"),
    ("loss_ref", "Q"),
    ("train_instr_offset", "Q"), ("train_instr_count", "Q"),
    ("merge_instr_offset", "Q"), ("merge_instr_count", "Q"),
    ("rodata_offset", "Q"), ("rodata_size", "Q"),
    ("persist_init_offset", "Q"), ("persist_init_size", "Q"),
    ("emit_table_offset", "Q"), ("emit_count", "Q"),
    ("lr", "f"), ("beta1", "f"), ("beta2", "f"), ("eps", "f"),
    ("weight_decay", "f"), ("gemm_tile_k", "I"),
    ("batch", "Q"), ("default_steps", "Q"),
    ("eval_instr_offset", "Q"), ("eval_instr_count", "Q"),
    ("source_model_hash", "Q"), ("plan_hash", "Q"),
    ("lr_schedule", "I"), ("gemm_tile_n", "I"),
    ("warmup_steps", "Q"), ("min_lr_factor", "f"), ("clip_norm", "f"),
    ("input_kind", "I"), ("grad_accum_steps", "I"),
    ("seq_len", "Q"),
    ("step_instr_offset", "Q"), ("step_instr_count", "Q"),
    ("tokenizer_hash", "Q"), ("corpus_hash", "Q"),
    ("split_seed", "Q"), ("val_split_hash", "Q"),
    ("val_frac_bits", "I"), ("data_flags", "I"),
]
_HEADER = struct.Struct("<" + "".join(f for _, f in _HEADER_FIELDS))
assert _HEADER.size == HEADER_BYTES


def f32_bits(x: float) -> int:
    return struct.unpack("<I", struct.pack("<f", x))[0]


def bits_f32(b: int) -> float:
    return struct.unpack("<f", struct.pack("<I", b & 0xFFFFFFFF))[0]


def pack2(hi: int, lo: int) -> int:
    return (hi << 32) | lo


def pack_attn_geometry(B: int, S: int, H: int, d: int) -> int:
    return (B << 48) | (S << 32) | (H << 16) | d


def rodata_ref(off: int) -> int:
    return off | RODATA_BIT


@dataclasses.dataclass
class Instr:
    opcode: int
    flags: int = 0
    imm: int = 0
    ins: Sequence[int] = (NULL_REF, NULL_REF, NULL_REF, NULL_REF)
    out: Sequence[int] = (0, 0, 0)

    def pack(self) -> bytes:
        ins = list(self.ins) + [NULL_REF] * (4 - len(self.ins))
        out = list(self.out) + [0] * (3 - len(self.out))
        return _INSTR.pack(self.opcode, self.flags, self.imm, *ins, *out)

    @staticmethod
    def unpack(raw: bytes) -> "Instr":
        v = _INSTR.unpack(raw)
        return Instr(v[0], v[1], v[2], tuple(v[3:7]), tuple(v[7:10]))

    def __str__(self) -> str:
        name = OP_NAMES.get(self.opcode, str(self.opcode))
        ins = ",".join("-" if r == NULL_REF else hex(r) for r in self.ins)
        out = ",".join(hex(o) for o in self.out)
        return f"{name:<18} f={self.flags:#x} imm={self.imm:#x} in[{ins}] out[{out}]"


def pack_program(instrs: Sequence[Instr]) -> bytes:
    return b"".join(i.pack() for i in instrs)


def unpack_program(raw: bytes) -> List[Instr]:
    return [Instr.unpack(raw[i:i + INSTR_BYTES])
            for i in range(0, len(raw), INSTR_BYTES)]


# --- the seal (reference: source/identity/hash.h:36-161) ----------------------

_FNV_OFFSET = 0xCBF29CE484222325
_FNV_PRIME = 0x100000001B3
_M64 = (1 << 64) - 1
_HASH_CHUNK = 1 << 20
_MAX_CHUNKS = 256


def _mix_word(state: int, word: int) -> int:
    for b in range(8):
        state ^= (word >> (8 * b)) & 0xFF
        state = (state * _FNV_PRIME) & _M64
    return state


def _striped_fnv(data: np.ndarray) -> int:
    """Eight interleaved FNV-1a lanes, byte i feeding lane i mod 8."""
    n = int(data.size)
    lanes = np.array([_FNV_OFFSET ^ ((0x9E3779B97F4A7C15 * (l + 1)) & _M64)
                      for l in range(8)], dtype=np.uint64)
    prime = np.uint64(_FNV_PRIME)
    full = n // 8
    if full:
        body = data[:full * 8].reshape(full, 8).astype(np.uint64)
        with np.errstate(over="ignore"):
            for row in body:
                lanes = (lanes ^ row) * prime
    tail = data[full * 8:]
    with np.errstate(over="ignore"):
        for l, byte in enumerate(tail):
            lanes[l] = (lanes[l] ^ np.uint64(byte)) * prime
    h = _FNV_OFFSET
    for l in range(8):
        h = _mix_word(h, int(lanes[l]))
    return _mix_word(h, n)


def _chunk_grain(n: int, grain: int) -> int:
    cap = (n + _MAX_CHUNKS - 1) // _MAX_CHUNKS
    return max(grain, cap, 1)


def _striped_fnv_many(chunks: np.ndarray) -> List[int]:
    """_striped_fnv over every row of `chunks` [n_chunks, chunk_bytes] at once
    (chunk_bytes a multiple of 8): the lanes' recurrence is sequential along a
    chunk but independent across chunks, so the steps are vectorised over chunks."""
    n_chunks, size = chunks.shape
    lanes = np.tile(np.array([_FNV_OFFSET ^ ((0x9E3779B97F4A7C15 * (l + 1)) & _M64)
                              for l in range(8)], dtype=np.uint64), (n_chunks, 1))
    prime = np.uint64(_FNV_PRIME)
    body = chunks.reshape(n_chunks, size // 8, 8)
    with np.errstate(over="ignore"):
        for step in range(size // 8):
            lanes = (lanes ^ body[:, step, :].astype(np.uint64)) * prime
    out = []
    for c in range(n_chunks):
        h = _FNV_OFFSET
        for l in range(8):
            h = _mix_word(h, int(lanes[c, l]))
        out.append(_mix_word(h, size))
    return out


def plan_self_hash(blob: bytes) -> int:
    """Chunked striped fold over the blob with the hash field read as zero."""
    data = np.frombuffer(blob, dtype=np.uint8).copy()
    data[PLAN_HASH_OFFSET:PLAN_HASH_OFFSET + 8] = 0
    n = int(data.size)
    grain = _chunk_grain(n, _HASH_CHUNK)
    full = n // grain if grain % 8 == 0 else 0
    partials: List[int] = []
    if full > 1:
        partials = _striped_fnv_many(data[:full * grain].reshape(full, grain))
        rest = range(full * grain, n, grain)
    else:
        rest = range(0, n, grain)
    partials += [_striped_fnv(data[b:min(b + grain, n)]) for b in rest]
    if not partials:
        partials = [_striped_fnv(data)]
    h = _FNV_OFFSET
    for p in partials:
        h = _mix_word(h, p)
    return _mix_word(h, n)


# --- the container -------------------------------------------------------------

@dataclasses.dataclass
class EmitEntry:
    smf_data_offset: int
    byte_size: int
    arena_offset: int


class Plan:
    """A decoded plan.  `header` is a dict over the 320-byte header's fields."""

    def __init__(self, blob: bytes):
        if len(blob) < HEADER_BYTES:
            raise ValueError("plan: truncated header")
        self.blob = blob
        vals = _HEADER.unpack_from(blob, 0)
        self.header = {n: v for (n, _), v in zip(_HEADER_FIELDS, vals)}
        h = self.header
        if h["magic"] != SEEU_MAGIC:
            raise ValueError("plan: not a .seeu plan")
        if not (4 <= h["version"] <= SEEU_VERSION):
            raise ValueError(f"plan: unsupported version {h['version']}")

        def section(off, count):
            end = off + count * INSTR_BYTES
            if end > len(blob):
                raise ValueError("plan: a program section lies outside the file")
            return unpack_program(blob[off:end])

        self.train = section(h["train_instr_offset"], h["train_instr_count"])
        self.eval = section(h["eval_instr_offset"], h["eval_instr_count"])
        self.merge = section(h["merge_instr_offset"], h["merge_instr_count"])
        self.step = section(h["step_instr_offset"], h["step_instr_count"])
        if h["rodata_offset"] + h["rodata_size"] > len(blob):
            raise ValueError("plan: rodata lies outside the file")
        if h["persist_init_offset"] + h["persist_init_size"] > len(blob):
            raise ValueError("plan: persist_init lies outside the file")
        self.emit = []
        for i in range(h["emit_count"]):
            self.emit.append(EmitEntry(*struct.unpack_from(
                "<3Q", blob, h["emit_table_offset"] + 24 * i)))

    @staticmethod
    def load(path: str) -> "Plan":
        with open(path, "rb") as f:
            return Plan(f.read())

    def verify_seal(self) -> bool:
        return plan_self_hash(self.blob) == self.header["plan_hash"]

    @property
    def rodata(self) -> memoryview:
        h = self.header
        return memoryview(self.blob)[h["rodata_offset"]:h["rodata_offset"] + h["rodata_size"]]

    @property
    def persist_init(self) -> memoryview:
        h = self.header
        return memoryview(self.blob)[h["persist_init_offset"]:
                                     h["persist_init_offset"] + h["persist_init_size"]]

    def section(self, name: str) -> List[Instr]:
        return {"train": self.train, "eval": self.eval,
                "merge": self.merge, "step": self.step}[name]

    def arena_bytes(self) -> int:
        """The allocation the runtime makes: arena_size rounded up to 16 KiB
        (reference: runtime/loader/plan_loader.cc:251-288)."""
        a = 16384
        return (self.header["arena_size"] + a - 1) // a * a

    def stage_arena(self) -> np.ndarray:
        arena = np.zeros(self.header["arena_size"], dtype=np.uint8)
        pi = np.frombuffer(self.persist_init, dtype=np.uint8)
        arena[:pi.size] = pi
        return arena


def _align(n: int, a: int) -> int:
    return (n + a - 1) // a * a


def write_plan(header: dict, train: Sequence[Instr], eval_: Sequence[Instr],
               merge: Sequence[Instr], step: Sequence[Instr],
               rodata: bytes, persist_init: bytes,
               emit: Sequence[EmitEntry] = (), seal: bool = True) -> bytes:
    """Assembles a plan blob: header, programs, persist_init, emit table, then
    rodata on a 16 KiB boundary with the blob padded to a 16 KiB multiple."""
    h = {n: 0 for n, _ in _HEADER_FIELDS}
    h.update(magic=SEEU_MAGIC, version=SEEU_VERSION, input_ref=NULL_REF,
             label_ref=NULL_REF, loss_ref=NULL_REF, optimizer_kind=1,
             lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01)
    h.update(header)
    cur = _align(HEADER_BYTES, 64)
    parts = []

    def place(raw: bytes, align: int = 64) -> int:
        nonlocal cur
        cur = _align(cur, align)
        off = cur
        parts.append((off, raw))
        cur += len(raw)
        return off

    h["train_instr_offset"] = place(pack_program(train)); h["train_instr_count"] = len(train)
    h["eval_instr_offset"] = place(pack_program(eval_)); h["eval_instr_count"] = len(eval_)
    h["merge_instr_offset"] = place(pack_program(merge)); h["merge_instr_count"] = len(merge)
    h["step_instr_offset"] = place(pack_program(step)); h["step_instr_count"] = len(step)
    h["persist_init_offset"] = place(persist_init); h["persist_init_size"] = len(persist_init)
    emit_raw = b"".join(struct.pack("<3Q", e.smf_data_offset, e.byte_size, e.arena_offset)
                        for e in emit)
    h["emit_table_offset"] = place(emit_raw); h["emit_count"] = len(emit)
    h["rodata_offset"] = place(rodata, RODATA_ALIGNMENT); h["rodata_size"] = len(rodata)
    total = _align(cur, RODATA_ALIGNMENT)
    blob = bytearray(total)
    h["plan_hash"] = 0
    blob[:HEADER_BYTES] = _HEADER.pack(*[h[n] for n, _ in _HEADER_FIELDS])
    for off, raw in parts:
        blob[off:off + len(raw)] = raw
    if seal:
        struct.pack_into("<Q", blob, PLAN_HASH_OFFSET, plan_self_hash(bytes(blob)))
    return bytes(blob)


# --- the probe's write trace (reference: tool/probe_trace.h) -----------------

TRACE_MAGIC = 0x54504553  # "SEPT"


def read_trace(raw: bytes):
    """-> list of (index, opcode, relaxed, [(arena_offset, bytes)])."""
    magic, version, count = struct.unpack_from("<IIQ", raw, 0)
    if magic != TRACE_MAGIC or version != 2:
        raise ValueError("trace: bad magic or version")
    pos = 16
    out = []
    for _ in range(count):
        index, opcode, n_ext, relaxed = struct.unpack_from("<IHHI", raw, pos)
        pos += 12
        ext = []
        for _ in range(n_ext):
            off, nbytes = struct.unpack_from("<QQ", raw, pos)
            pos += 16
            ext.append((off, bytes(raw[pos:pos + nbytes])))
            pos += nbytes
        out.append((index, opcode, relaxed, ext))
    return out
