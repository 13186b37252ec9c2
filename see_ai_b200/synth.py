"""Synthetic update plans of the shapes the reference compiler emits.

The benchmark configurations need plans far larger than any fixture can carry
(the int8 decoder's frozen weights alone are ~200 MB), and the reference
compiler is not available where the benchmark runs.  This module writes such
plans directly: the same instruction patterns `seeml-update-compile` lowers a
LoRA site, a pre-norm decoder block and the loss to (reference:
compiler/analysis/algebra/lora_grafter.cc:170-206, compiler/analysis/calculus/
autodiff.cc:74-97, compiler/backend/selection/instruction_lowering.cc:96-209),
the arena laid out as the reference binder lays it out — persistent prefix,
I/O slots, pinned gradients and deltas back to back, then transients reused by
liveness (reference: compiler/backend/allocation/arena_binder.cc:28-121, 224-316)
— in the same sealed `.seeu` container.  tests/test_synth_matches_reference.py
holds the instruction streams to those of plans the reference compiler itself
produced for the same tiny models.
"""

from __future__ import annotations

import dataclasses
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from . import plan as P

Op = P.Op
ALIGN = 64


def _al(n: int, a: int = ALIGN) -> int:
    return (n + a - 1) // a * a


@dataclasses.dataclass(eq=False)
class T:
    """A symbolic tensor: `kind` decides which arena region (or rodata) holds it."""
    name: str
    nbytes: int
    kind: str  # persistent | io | pinned | transient | rodata
    off: int = -1
    data: Optional[np.ndarray] = None  # initial bytes (rodata, persistent)

    @property
    def ref(self) -> int:
        assert self.off >= 0, self.name
        return (self.off | P.RODATA_BIT) if self.kind == "rodata" else self.off


class PlanBuilder:
    def __init__(self, seed: int = 7):
        self.rng = np.random.default_rng(seed)
        self.persistent: List[T] = []
        self.io: List[T] = []
        self.pinned: List[T] = []
        self.rodata: List[T] = []
        self.programs: Dict[str, List[tuple]] = {"train": [], "eval": [], "merge": [], "step": []}
        self.cur = "train"
        self.emits: List[Tuple[T, int]] = []   # (delta tensor, byte offset of its weight in the model file)

    # ---- tensors ----
    def t(self, name, n_floats, kind="transient", data=None, elem=4) -> T:
        x = T(name, int(n_floats) * elem, kind, data=data)
        {"persistent": self.persistent, "io": self.io, "pinned": self.pinned,
         "rodata": self.rodata, "transient": []}[kind].append(x)
        return x

    def ro(self, name, array: np.ndarray) -> T:
        a = np.ascontiguousarray(array)
        return self.t(name, a.nbytes, "rodata", data=a.view(np.uint8).reshape(-1), elem=1)

    # ---- instructions ----
    def emit(self, opcode, ins=(), out=(), flags=0, imm=0):
        self.programs[self.cur].append((opcode, flags, imm, tuple(ins), tuple(out)))

    # ---- layout + assembly ----
    def assemble(self, header: dict) -> bytes:
        off = 0
        for x in self.persistent:
            x.off = off
            off = _al(off + x.nbytes)
        persistent_size = off
        for x in self.io + self.pinned:
            x.off = off
            off = _al(off + x.nbytes)
        transient_base = off
        arena_size = transient_base
        # Transients: per program, linear scan over first/last use with a free list.
        for prog in self.programs.values():
            first, last = {}, {}
            for i, (_op, _f, _imm, ins, out) in enumerate(prog):
                for v in list(ins) + list(out):
                    if isinstance(v, T) and v.kind == "transient":
                        first.setdefault(id(v), (i, v))
                        last[id(v)] = i
            expiring: Dict[int, List[T]] = {}
            for key, i in last.items():
                expiring.setdefault(i, []).append(first[key][1])
            births: Dict[int, List[T]] = {}
            for key, (i, v) in first.items():
                births.setdefault(i, []).append(v)
            free: List[Tuple[int, int]] = []  # (offset, bytes), disjoint
            top = transient_base
            for i in range(len(prog)):
                for v in births.get(i, []):
                    need = _al(v.nbytes)
                    best = None
                    for j, (o, n) in enumerate(free):
                        if n >= need and (best is None or n < free[best][1]):
                            best = j
                    if best is not None:
                        o, n = free.pop(best)
                        v.off = o
                        if n > need:
                            free.append((o + need, n - need))
                    else:
                        v.off = top
                        top += need
                # A result never shares its slot with an operand of the same
                # instruction: slots are released only after the instruction.
                for v in expiring.get(i, []):
                    free.append((v.off, _al(v.nbytes)))
                    free.sort()
                    merged: List[Tuple[int, int]] = []
                    for o, n in free:
                        if merged and merged[-1][0] + merged[-1][1] == o:
                            merged[-1] = (merged[-1][0], merged[-1][1] + n)
                        else:
                            merged.append((o, n))
                    free = merged
            arena_size = max(arena_size, top)
        ro_off = 0
        ro_parts = []
        for x in self.rodata:
            x.off = ro_off
            ro_parts.append((ro_off, x.data))
            ro_off = _al(ro_off + x.nbytes)
        rodata = np.zeros(ro_off, dtype=np.uint8)
        for o, d in ro_parts:
            rodata[o:o + d.size] = d
        persist = np.zeros(persistent_size, dtype=np.uint8)
        for x in self.persistent:
            if x.data is not None:
                persist[x.off:x.off + x.data.size] = x.data

        def lower(prog):
            out = []
            for (op, flags, imm, ins, outs) in prog:
                ins = [v.ref if isinstance(v, T) else v for v in ins]
                outs = [v.ref if isinstance(v, T) else v for v in outs]
                out.append(P.Instr(op, flags, imm, tuple(ins + [P.NULL_REF] * (4 - len(ins))),
                                   tuple(outs + [0] * (3 - len(outs)))))
            return out

        h = {k: (v.ref if isinstance(v, T) else v) for k, v in header.items()}
        h.update(arena_size=arena_size, persistent_size=persistent_size)
        emit = [P.EmitEntry(smf_off, t.nbytes, t.off) for (t, smf_off) in self.emits]
        return P.write_plan(h, lower(self.programs["train"]), lower(self.programs["eval"]),
                            lower(self.programs["merge"]), lower(self.programs["step"]),
                            rodata.tobytes(), persist.tobytes(), emit=emit)


# ---- LoRA site helpers -----------------------------------------------------------

@dataclasses.dataclass
class Adapter:
    name: str
    k_in: int
    n_out: int
    A: T
    B: T
    mA: T
    vA: T
    mB: T
    vB: T
    gA: Optional[T] = None
    gB: Optional[T] = None
    delta: Optional[T] = None


def make_adapter(b: PlanBuilder, name: str, k_in: int, n_out: int, rank: int) -> Adapter:
    a_init = (b.rng.standard_normal((k_in, rank)) / np.sqrt(k_in)).astype(np.float32)
    A = b.t(name + ".A", k_in * rank, "persistent", data=a_init.view(np.uint8).reshape(-1))
    B = b.t(name + ".B", rank * n_out, "persistent")
    return Adapter(name, k_in, n_out, A, B, None, None, None, None)


def add_moments(b: PlanBuilder, ad: Adapter, rank: int):
    ad.mA = b.t(ad.name + ".mA", ad.k_in * rank, "persistent")
    ad.vA = b.t(ad.name + ".vA", ad.k_in * rank, "persistent")
    ad.mB = b.t(ad.name + ".mB", rank * ad.n_out, "persistent")
    ad.vB = b.t(ad.name + ".vB", rank * ad.n_out, "persistent")


def quantize_columns(w: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    """Symmetric per-column int8: scale = max|col| / 127, round half away from
    zero, clamp to +-127 (reference: compiler/backend/allocation/arena_binder.cc:129-190)."""
    amax = np.max(np.abs(w), axis=0)
    scale = np.where(amax > 0, amax / 127.0, 1.0).astype(np.float32)
    scale = np.maximum(scale, np.finfo(np.float32).tiny)
    q = (w / scale).astype(np.float32).astype(np.float64)   # the f32 quotient; + 0.5 is then exact
    q = np.clip(np.where(q >= 0, np.floor(q + 0.5), np.ceil(q - 0.5)), -127, 127).astype(np.int8)
    return q, scale


class Weight:
    """A frozen [K, N] weight in rodata: f32, or int8 + per-column scales."""

    def __init__(self, b: PlanBuilder, name: str, k: int, n: int, quant: bool, std: float = 0.02):
        w = (b.rng.standard_normal((k, n), dtype=np.float32) * np.float32(std))
        self.k, self.n, self.quant = k, n, quant
        if quant:
            q, s = quantize_columns(w)
            self.w = b.ro(name, q)
            self.s = b.ro(name + ".scale", s)
        else:
            self.w = b.ro(name, w)
            self.s = None


def gemm_fwd(b: PlanBuilder, x: T, w: Weight, out: T, M: int, relaxed: bool, flags: int = 0,
             in3=None):
    """out[M, n] = x[M, k] @ W  (+ fused epilogue flags on the f32 form)."""
    if w.quant:
        b.emit(Op.GEMM_NN_Q8, (x, w.w, out, w.s), (M, w.n, w.k),
               flags=P.FLAG_Q8_COL_SCALE | (P.FLAG_RELAXED if relaxed else 0) | flags)
    else:
        ins = (x, w.w, out) + ((in3,) if in3 is not None else ())
        b.emit(Op.GEMM_NN, ins, (M, w.n, w.k), flags=flags | (P.FLAG_RELAXED if relaxed else 0))


def gemm_dx(b: PlanBuilder, dy: T, w: Weight, out: T, M: int, relaxed: bool, addend: Optional[T] = None):
    """out[M, k] = dy[M, n] @ W^T   (W read as [N' = k, K' = n])."""
    if w.quant:
        assert addend is None
        b.emit(Op.GEMM_NT_Q8, (dy, w.w, out, w.s), (M, w.k, w.n),
               flags=P.FLAG_Q8_COL_SCALE | (P.FLAG_RELAXED if relaxed else 0))
    else:
        fl = (P.FLAG_RELAXED if relaxed else 0) | (P.FLAG_GEMM_ADDEND if addend is not None else 0)
        ins = (dy, w.w, out) + ((addend,) if addend is not None else ())
        b.emit(Op.GEMM_NT, ins, (M, w.k, w.n), flags=fl)


def lora_fwd(b: PlanBuilder, x: T, ad: Adapter, base: T, out: T, M: int, rank: int, alpha_bits: int) -> T:
    t = b.t(ad.name + ".t", M * rank)
    b.emit(Op.GEMM_NN, (x, ad.A, t), (M, rank, ad.k_in))
    b.emit(Op.GEMM_NN, (t, ad.B, out, base), (M, ad.n_out, rank), flags=P.FLAG_GEMM_ADDEND,
           imm=alpha_bits)
    return t


# ---- the decoder ---------------------------------------------------------------------

@dataclasses.dataclass
class DecoderConfig:
    layers: int
    d_model: int
    heads: int
    ffn: int
    vocab: int
    seq: int
    batch_seqs: int            # sequences per step on this rank
    rank: int = 8
    alpha: float = 16.0
    targets: Sequence[str] = ("q", "v")
    quantized: bool = False    # int8 base + per-column scales + relaxed frozen GEMMs
    attention: str = "cached"  # cached | tiled
    lr: float = 1e-3
    steps: int = 500
    seed: int = 7

    @property
    def rows(self) -> int:
        return self.batch_seqs * self.seq


def build_decoder_plan(cfg: DecoderConfig) -> bytes:
    b = PlanBuilder(cfg.seed)
    M, D, H, F, V, S, L, r = cfg.rows, cfg.d_model, cfg.heads, cfg.ffn, cfg.vocab, cfg.seq, cfg.layers, cfg.rank
    d = D // H
    Bq = cfg.batch_seqs
    quant = cfg.quantized
    relaxed = quant
    tiled = cfg.attention == "tiled"
    alpha_bits = P.f32_bits(cfg.alpha / r)
    bs, hd = P.pack2(Bq, S), P.pack2(H, d)
    geom = P.pack_attn_geometry(Bq, S, H, d)
    rows_cols = P.pack2(M, D)

    # ---- frozen weights ----
    emb = b.ro("emb", (b.rng.standard_normal((V, D), dtype=np.float32) * np.float32(0.02)))
    ones, zeros = np.ones(D, np.float32), np.zeros(D, np.float32)
    layers = []
    for l in range(L):
        p = f"l{l}."
        lw = dict(ln1_g=b.ro(p + "ln1_g", ones), ln1_b=b.ro(p + "ln1_b", zeros))
        for nm in ("q", "k", "v"):
            lw["w" + nm] = Weight(b, p + "w" + nm, D, D, quant)
        lw["wo"] = Weight(b, p + "wo", D, D, quant)
        lw["ln2_g"] = b.ro(p + "ln2_g", ones); lw["ln2_b"] = b.ro(p + "ln2_b", zeros)
        lw["w1"] = Weight(b, p + "w1", D, F, quant)
        lw["b1"] = b.ro(p + "b1", (b.rng.standard_normal(F, dtype=np.float32) * np.float32(0.02)))
        lw["w2"] = Weight(b, p + "w2", F, D, quant)
        lw["b2"] = b.ro(p + "b2", (b.rng.standard_normal(D, dtype=np.float32) * np.float32(0.02)))
        layers.append(lw)
    lnf_g, lnf_b = b.ro("lnf_g", ones), b.ro("lnf_b", zeros)
    w_head = Weight(b, "w_head", D, V, quant)

    # ---- persistent: adapters, then moments ----
    adapters: List[Dict[str, Adapter]] = []
    for l in range(L):
        adapters.append({nm: make_adapter(b, f"l{l}.w{nm}", D, D, r) for nm in ("q", "k", "v", "o")
                         if nm in cfg.targets})
    for l in range(L):
        for ad in adapters[l].values():
            add_moments(b, ad, r)
    # ---- I/O, then pinned gradients and deltas ----
    tokens = b.t("tokens", M, "io")
    labels = b.t("labels", M, "io")
    loss = b.t("loss", 1, "io")
    for l in range(L):
        for ad in adapters[l].values():
            ad.gB = b.t(ad.name + ".gB", r * D, "pinned")
            ad.gA = b.t(ad.name + ".gA", D * r, "pinned")
    for l in range(L):
        for ad in adapters[l].values():
            ad.delta = b.t(ad.name + ".delta", D * D, "pinned")

    def forward(train: bool):
        saved = []
        x = b.t("e", M * D)
        b.emit(Op.EMBED_FWD, (tokens, emb, x), (M, P.pack2(V, D)))
        rel = relaxed and train
        for l in range(L):
            lw, ads = layers[l], adapters[l]
            s = dict(x_in=x)
            n1 = b.t(f"l{l}.n1", M * D)
            s["mean1"], s["rstd1"] = b.t(f"l{l}.mean1", M), b.t(f"l{l}.rstd1", M)
            b.emit(Op.LAYERNORM_FWD, (x, lw["ln1_g"], lw["ln1_b"], n1), (rows_cols, s["mean1"], s["rstd1"]))
            s["n1"] = n1
            proj = {}
            for nm in ("q", "k", "v"):
                if nm in ads:
                    base = b.t(f"l{l}.{nm}_base", M * D)
                    gemm_fwd(b, n1, lw["w" + nm], base, M, rel)
                    out = b.t(f"l{l}.{nm}", M * D)
                    s["t" + nm] = lora_fwd(b, n1, ads[nm], base, out, M, r, alpha_bits)
                    proj[nm] = out
                else:
                    out = b.t(f"l{l}.{nm}", M * D)
                    gemm_fwd(b, n1, lw["w" + nm], out, M, rel)
                    proj[nm] = out
            s.update(q=proj["q"], k=proj["k"], v=proj["v"])
            a = b.t(f"l{l}.a", M * D)
            if tiled:
                s["stats"] = b.t(f"l{l}.stats", Bq * H * S * 4)
                b.emit(Op.ATTN_FWD_TILED, (proj["q"], proj["k"], proj["v"], a), (s["stats"], bs, hd),
                       flags=P.FLAG_RELAXED if rel else 0)
            else:
                s["P"] = b.t(f"l{l}.P", Bq * H * S * S)
                b.emit(Op.ATTN_FWD, (proj["q"], proj["k"], proj["v"], a), (s["P"], bs, hd))
            s["a"] = a
            x1 = b.t(f"l{l}.x1", M * D)
            if "o" in ads or quant:
                o = b.t(f"l{l}.o", M * D)
                if "o" in ads:
                    base = b.t(f"l{l}.o_base", M * D)
                    gemm_fwd(b, a, lw["wo"], base, M, rel)
                    s["to"] = lora_fwd(b, a, ads["o"], base, o, M, r, alpha_bits)
                else:
                    gemm_fwd(b, a, lw["wo"], o, M, rel)
                b.emit(Op.ADD_EW, (x, o, x1), (M * D,))
            else:
                gemm_fwd(b, a, lw["wo"], x1, M, rel, flags=P.FLAG_GEMM_ADDEND, in3=x)
            s["x1"] = x1
            n2 = b.t(f"l{l}.n2", M * D)
            s["mean2"], s["rstd2"] = b.t(f"l{l}.mean2", M), b.t(f"l{l}.rstd2", M)
            b.emit(Op.LAYERNORM_FWD, (x1, lw["ln2_g"], lw["ln2_b"], n2), (rows_cols, s["mean2"], s["rstd2"]))
            f1b = b.t(f"l{l}.f1b", M * F)
            if quant:
                f1 = b.t(f"l{l}.f1", M * F)
                gemm_fwd(b, n2, lw["w1"], f1, M, rel)
                b.emit(Op.ADD_BIAS, (f1, lw["b1"], f1b), (M, F))
            else:
                gemm_fwd(b, n2, lw["w1"], f1b, M, rel, flags=P.FLAG_EPILOGUE_BIAS, in3=lw["b1"])
            s["f1b"] = f1b
            g = b.t(f"l{l}.g", M * F)
            b.emit(Op.GELU_FWD, (f1b, g), (M * F,))
            f2b = b.t(f"l{l}.f2b", M * D)
            if quant:
                f2 = b.t(f"l{l}.f2", M * D)
                gemm_fwd(b, g, lw["w2"], f2, M, rel)
                b.emit(Op.ADD_BIAS, (f2, lw["b2"], f2b), (M, D))
            else:
                gemm_fwd(b, g, lw["w2"], f2b, M, rel, flags=P.FLAG_EPILOGUE_BIAS, in3=lw["b2"])
            x2 = b.t(f"l{l}.x2", M * D)
            b.emit(Op.ADD_EW, (x1, f2b, x2), (M * D,))
            x = x2
            saved.append(s)
        nf = b.t("nf", M * D)
        meanf, rstdf = b.t("meanf", M), b.t("rstdf", M)
        b.emit(Op.LAYERNORM_FWD, (x, lnf_g, lnf_b, nf), (rows_cols, meanf, rstdf))
        logits = b.t("logits", M * V)
        gemm_fwd(b, nf, w_head, logits, M, rel)
        probs = b.t("probs", M * V)
        b.emit(Op.XENT_FWD, (logits, labels, loss, probs), (M, V))
        return saved, x, meanf, rstdf, logits, probs

    # ---- train program ----
    b.cur = "train"
    saved, x_last, meanf, rstdf, logits, probs = forward(True)
    seed = b.t("seed", 1)
    b.emit(Op.FILL, (seed, P.f32_bits(1.0)), (1,))
    dlogits = b.t("dlogits", M * V)
    b.emit(Op.XENT_BWD, (probs, labels, seed, dlogits), (M, V))
    d_nf = b.t("d_nf", M * D)
    gemm_dx(b, dlogits, w_head, d_nf, M, relaxed)
    d_x = b.t("d_x", M * D)
    b.emit(Op.LAYERNORM_BWD, (d_nf, x_last, lnf_g, d_x), (meanf, rstdf, rows_cols))

    def site_backward(l, nm, dy, x_in, t, acc, need_dx, w):
        """One LoRA site's backward; returns the running input gradient."""
        ad = adapters[l].get(nm)
        p = f"l{l}.{nm}"
        if ad is None:
            if not need_dx:
                return acc
            if acc is None:
                out = b.t(p + ".dx", M * D)
                gemm_dx(b, dy, w, out, M, relaxed)
                return out
            out = b.t(p + ".dx", M * D)
            if w.quant:
                gemm_dx(b, dy, w, out, M, relaxed)
                s2 = b.t(p + ".dxs", M * D)
                b.emit(Op.ADD_EW, (acc, out, s2), (M * D,))
                return s2
            gemm_dx(b, dy, w, out, M, relaxed, addend=acc)
            return out
        dt = b.t(p + ".dt", M * r)
        b.emit(Op.GEMM_NT, (dy, ad.B, dt), (M, r, D), imm=alpha_bits)
        b.emit(Op.GEMM_TN, (t, dy, ad.gB), (r, D, M), imm=alpha_bits)
        if not need_dx:
            b.emit(Op.GEMM_TN, (x_in, dt, ad.gA), (D, r, M))
            return acc
        if acc is None:   # the first contribution to this input's gradient
            b.emit(Op.GEMM_TN, (x_in, dt, ad.gA), (D, r, M))
            base = b.t(p + ".dx0", M * D)
            gemm_dx(b, dy, w, base, M, relaxed)
            out = b.t(p + ".dx", M * D)
            b.emit(Op.GEMM_NT, (dt, ad.A, out, base), (M, D, r), flags=P.FLAG_GEMM_ADDEND)
            return out
        part = b.t(p + ".dxl", M * D)
        b.emit(Op.GEMM_NT, (dt, ad.A, part, acc), (M, D, r), flags=P.FLAG_GEMM_ADDEND)
        b.emit(Op.GEMM_TN, (x_in, dt, ad.gA), (D, r, M))
        out = b.t(p + ".dx", M * D)
        if w.quant:
            gemm_dx(b, dy, w, out, M, relaxed)
            s2 = b.t(p + ".dxs", M * D)
            b.emit(Op.ADD_EW, (part, out, s2), (M * D,))
            return s2
        gemm_dx(b, dy, w, out, M, relaxed, addend=part)
        return out

    for l in reversed(range(L)):
        lw, s = layers[l], saved[l]
        d_g = b.t(f"l{l}.d_g", M * F)
        gemm_dx(b, d_x, lw["w2"], d_g, M, relaxed)
        d_f1b = b.t(f"l{l}.d_f1b", M * F)
        b.emit(Op.GELU_BWD, (d_g, s["f1b"], d_f1b), (M * F,))
        d_n2 = b.t(f"l{l}.d_n2", M * D)
        gemm_dx(b, d_f1b, lw["w1"], d_n2, M, relaxed)
        d_ln2 = b.t(f"l{l}.d_ln2", M * D)
        b.emit(Op.LAYERNORM_BWD, (d_n2, s["x1"], lw["ln2_g"], d_ln2), (s["mean2"], s["rstd2"], rows_cols))
        d_x1 = b.t(f"l{l}.d_x1", M * D)
        b.emit(Op.ADD_EW, (d_x, d_ln2, d_x1), (M * D,))
        d_a = site_backward(l, "o", d_x1, s["a"], s.get("to"), None, True, lw["wo"])
        need = l > 0   # the embedding is frozen: layer 0 needs no input gradient
        # A projection's gradient is dead when nothing consumes it: no adapter on
        # the projection and no input gradient wanted (the reference's DCE drops it).
        live = {nm: need or nm in adapters[l] for nm in "qkv"}
        dq, dk, dv = (b.t(f"l{l}.d{n}", M * D) for n in "qkv")
        if tiled:
            fl = P.FLAG_RELAXED if relaxed else 0
            for nm, op, res in (("q", Op.ATTN_DQ_TILED, dq), ("k", Op.ATTN_DK_TILED, dk),
                                ("v", Op.ATTN_DV_TILED, dv)):
                # dK reads the delta the dQ pass leaves in the stats row, so dQ stays
                # whenever dK is wanted.
                if live[nm] or (nm == "q" and live["k"]):
                    b.emit(op, (s["q"], s["k"], s["v"], d_a), (s["stats"], res, geom), flags=fl)
        else:
            dP, dS = b.t(f"l{l}.dP", Bq * H * S * S), b.t(f"l{l}.dS", Bq * H * S * S)
            if live["v"]:
                b.emit(Op.ATTN_DV, (s["P"], d_a, dv), (bs, hd))
            if live["q"] or live["k"]:
                b.emit(Op.ATTN_DP, (d_a, s["v"], dP), (bs, hd))
                b.emit(Op.SOFTMAX_ROWS_BWD, (s["P"], dP, dS), (P.pack2(Bq * H * S, S),))
            if live["q"]:
                b.emit(Op.ATTN_DQ, (dS, s["k"], dq), (bs, hd))
            if live["k"]:
                b.emit(Op.ATTN_DK, (dS, s["q"], dk), (bs, hd))
        acc = None
        for nm, dy in (("v", dv), ("k", dk), ("q", dq)):
            acc = site_backward(l, nm, dy, s["n1"], s.get("t" + nm), acc, need, lw["w" + nm])
        if need:
            d_ln1 = b.t(f"l{l}.d_ln1", M * D)
            b.emit(Op.LAYERNORM_BWD, (acc, s["x_in"], lw["ln1_g"], d_ln1), (s["mean1"], s["rstd1"], rows_cols))
            d_xin = b.t(f"l{l}.d_xin", M * D)
            b.emit(Op.ADD_EW, (d_x1, d_ln1, d_xin), (M * D,))
            d_x = d_xin
    for l in range(L):
        for ad in adapters[l].values():
            b.emit(Op.ADAMW_STEP, (ad.A, ad.gA, ad.mA, ad.vA), (D * r, 0))
            b.emit(Op.ADAMW_STEP, (ad.B, ad.gB, ad.mB, ad.vB), (r * D, 0))

    # ---- eval program: the forward and the loss, exact arithmetic ----
    b.cur = "eval"
    forward(False)
    # ---- merge program: each adapter's delta = (alpha / r) * A @ B ----
    b.cur = "merge"
    smf_off = 0
    for l in range(L):
        for ad in adapters[l].values():
            b.emit(Op.FILL, (ad.delta, 0), (D * D,))
            b.emit(Op.GEMM_ACC_NN, (ad.A, ad.B, ad.delta, alpha_bits), (D, D, r))
            b.emits.append((ad.delta, smf_off))
            smf_off += D * D * 4

    header = dict(input_ref=tokens, input_floats=M, label_ref=labels, label_bytes=4 * M, label_kind=1,
                  loss_ref=loss, lr=cfg.lr, batch=M, default_steps=cfg.steps, lr_schedule=0,
                  input_kind=1, grad_accum_steps=1, seq_len=S, weight_decay=0.01)
    return _finish(b, header)


def _finish(b: PlanBuilder, header: dict) -> bytes:
    return b.assemble(header)   # header values that are tensors resolve after layout


# ---- the feed-forward plan (the CPU-runnable reference case) ------------------------

@dataclasses.dataclass
class MlpConfig:
    dims: Sequence[int] = (256, 1024, 64)
    batch: int = 32
    rank: int = 8
    alpha: float = 16.0
    lr: float = 1e-3
    steps: int = 1000
    seed: int = 7
    lr_schedule: int = 0        # 1: linear warm-up, then a cosine down to lr * min_lr_factor
    warmup_steps: int = 0
    min_lr_factor: float = 0.0


def build_mlp_plan(cfg: MlpConfig) -> bytes:
    b = PlanBuilder(cfg.seed)
    M, r = cfg.batch, cfg.rank
    alpha_bits = P.f32_bits(cfg.alpha / r)
    dims = list(cfg.dims)
    n_layers = len(dims) - 1
    ws, biases = [], []
    for i in range(n_layers):
        ws.append(Weight(b, f"w{i}", dims[i], dims[i + 1], False))
        biases.append(b.ro(f"b{i}", b.rng.standard_normal(dims[i + 1], dtype=np.float32) * np.float32(0.02)))
    ads = []
    for i in range(n_layers):
        a_init = (b.rng.standard_normal((dims[i], r)) / np.sqrt(dims[i])).astype(np.float32)
        A = b.t(f"w{i}.A", dims[i] * r, "persistent", data=a_init.view(np.uint8).reshape(-1))
        B = b.t(f"w{i}.B", r * dims[i + 1], "persistent")
        ads.append(Adapter(f"w{i}", dims[i], dims[i + 1], A, B, None, None, None, None))
    for ad in ads:
        ad.mA = b.t(ad.name + ".mA", ad.k_in * r, "persistent"); ad.vA = b.t(ad.name + ".vA", ad.k_in * r, "persistent")
        ad.mB = b.t(ad.name + ".mB", r * ad.n_out, "persistent"); ad.vB = b.t(ad.name + ".vB", r * ad.n_out, "persistent")
    x0 = b.t("x", M * dims[0], "io")
    labels = b.t("labels", M, "io")
    loss = b.t("loss", 1, "io")
    for ad in reversed(ads):
        ad.gB = b.t(ad.name + ".gB", r * ad.n_out, "pinned")
        ad.gA = b.t(ad.name + ".gA", ad.k_in * r, "pinned")
    for ad in ads:
        ad.delta = b.t(ad.name + ".delta", ad.k_in * ad.n_out, "pinned")

    def forward():
        x = x0
        saved = []
        for i in range(n_layers):
            base = b.t(f"z{i}", M * dims[i + 1])
            gemm_fwd(b, x, ws[i], base, M, False)
            zl = b.t(f"zl{i}", M * dims[i + 1])
            t = lora_fwd(b, x, ads[i], base, zl, M, r, alpha_bits)
            zb = b.t(f"zb{i}", M * dims[i + 1])
            b.emit(Op.ADD_BIAS, (zl, biases[i], zb), (M, dims[i + 1]))
            s = dict(x=x, t=t, zb=zb)
            if i + 1 < n_layers:
                h = b.t(f"h{i}", M * dims[i + 1])
                b.emit(Op.RELU_FWD, (zb, h), (M * dims[i + 1],))
                x = h
            else:
                x = zb
            saved.append(s)
        probs = b.t("probs", M * dims[-1])
        b.emit(Op.XENT_FWD, (x, labels, loss, probs), (M, dims[-1]))
        return saved, probs

    b.cur = "train"
    saved, probs = forward()
    seed = b.t("seed", 1)
    b.emit(Op.FILL, (seed, P.f32_bits(1.0)), (1,))
    dy = b.t("dlogits", M * dims[-1])
    b.emit(Op.XENT_BWD, (probs, labels, seed, dy), (M, dims[-1]))
    for i in reversed(range(n_layers)):
        ad, s = ads[i], saved[i]
        dt = b.t(f"dt{i}", M * r)
        b.emit(Op.GEMM_NT, (dy, ad.B, dt), (M, r, dims[i + 1]), imm=alpha_bits)
        b.emit(Op.GEMM_TN, (s["t"], dy, ad.gB), (r, dims[i + 1], M), imm=alpha_bits)
        b.emit(Op.GEMM_TN, (s["x"], dt, ad.gA), (dims[i], r, M))
        if i > 0:
            dx0 = b.t(f"dx0_{i}", M * dims[i])
            gemm_dx(b, dy, ws[i], dx0, M, False)
            dx = b.t(f"dx{i}", M * dims[i])
            b.emit(Op.GEMM_NT, (dt, ad.A, dx, dx0), (M, dims[i], r), flags=P.FLAG_GEMM_ADDEND)
            dz = b.t(f"dz{i}", M * dims[i])
            b.emit(Op.RELU_BWD, (dx, saved[i - 1]["zb"], dz), (M * dims[i],))
            dy = dz
    for ad in ads:
        b.emit(Op.ADAMW_STEP, (ad.A, ad.gA, ad.mA, ad.vA), (ad.k_in * r, 0))
        b.emit(Op.ADAMW_STEP, (ad.B, ad.gB, ad.mB, ad.vB), (r * ad.n_out, 0))
    b.cur = "eval"
    forward()
    b.cur = "merge"
    smf_off = 0
    for ad in ads:
        b.emit(Op.FILL, (ad.delta, 0), (ad.k_in * ad.n_out,))
        b.emit(Op.GEMM_ACC_NN, (ad.A, ad.B, ad.delta, alpha_bits), (ad.k_in, ad.n_out, r))
        b.emits.append((ad.delta, smf_off))
        smf_off += ad.k_in * ad.n_out * 4
    header = dict(input_ref=x0, input_floats=M * dims[0], label_ref=labels, label_bytes=4 * M,
                  label_kind=1, loss_ref=loss, lr=cfg.lr, batch=M, default_steps=cfg.steps,
                  lr_schedule=cfg.lr_schedule, warmup_steps=cfg.warmup_steps,
                  min_lr_factor=cfg.min_lr_factor, input_kind=0, grad_accum_steps=1, seq_len=0,
                  weight_decay=0.01)
    return _finish(b, header)
