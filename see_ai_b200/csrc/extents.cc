#include "extents.h"

#include <cmath>

namespace see {

const char* OpName(uint16_t op) {
  static const char* const kNames[kOpCount] = {
      "nop", "gemm.nn", "gemm.nt", "gemm.tn", "gemm.acc.nn", "add.ew", "add.bias",
      "relu.fwd", "relu.bwd", "scale", "reduce.rows", "xent.fwd", "xent.bwd",
      "mse.fwd", "mse.bwd", "kl.fwd", "kl.bwd", "sgd.step", "adamw.step", "fill",
      "copy", "mul.ew", "gelu.fwd", "gelu.bwd", "silu.fwd", "silu.bwd",
      "layernorm.fwd", "layernorm.bwd", "clip.norm", "gemm.nn.q8", "gemm.nt.q8",
      "rmsnorm.fwd", "rmsnorm.bwd", "rope.fwd", "rope.bwd", "attn.fwd", "attn.dp",
      "attn.dv", "softmax.rows.bwd", "attn.dq", "attn.dk", "embed.fwd", "accumulate",
      "gemm.nn.bf16", "gemm.nt.bf16", "rope.table", "fused.map", "attn.fwd.tiled",
      "attn.dq.tiled", "attn.dk.tiled", "attn.dv.tiled", "xent.masked.fwd",
      "xent.masked.bwd", "sqnorm.accum", "clip.global", "segment.starts",
      "attn.fwd.seg", "attn.fwd.tiled.seg"};
  return op < kOpCount ? kNames[op] : "?";
}

namespace {

bool ProductFits(uint64_t a, uint64_t b, uint64_t* out) {
  return !__builtin_mul_overflow(a, b, out);
}

struct Builder {
  const Instruction& ins;
  uint64_t limit[3];
  Extents* out;
  bool ok = true;

  // `count` elements of `elem` bytes at `ref`.
  void Add(uint64_t ref, uint64_t count, bool write, bool read, uint64_t elem = 4) {
    if (!ok) return;
    uint64_t bytes = 0;
    if (ref == kNullRef || !ProductFits(count, elem, &bytes)) { ok = false; return; }
    const Space sp = RefSpace(ref);
    const uint64_t off = RefOffset(ref);
    if (write && sp != kArena) { ok = false; return; }
    if (off % (elem < 4 ? elem : 4) != 0) { ok = false; return; }
    if (off > limit[sp] || bytes > limit[sp] - off) { ok = false; return; }
    if (out->count >= 8) { ok = false; return; }
    Extent& e = out->e[out->count++];
    e.off = off; e.bytes = bytes; e.space = sp; e.write = write; e.read = read;
  }
  void R(uint64_t ref, uint64_t count, uint64_t elem = 4) { Add(ref, count, false, true, elem); }
  void W(uint64_t ref, uint64_t count) { Add(ref, count, true, false); }
  void RW(uint64_t ref, uint64_t count) { Add(ref, count, true, true); }
};

bool FiniteImm(uint64_t word) {
  return (word >> 32) == 0 && std::isfinite(BitsToF32(word));
}

}  // namespace

std::string DescribeInstruction(const Instruction& ins, uint64_t arena_bytes,
                                uint64_t rodata_bytes, uint64_t source_bytes,
                                Extents* out) {
  out->count = 0;
  if (ins.opcode >= kOpCount) return "unknown opcode " + std::to_string(ins.opcode);
  if (ins.flags & ~kKnownFlags) return std::string(OpName(ins.opcode)) + ": unknown flag bits";
  Builder b{ins, {arena_bytes, rodata_bytes, source_bytes}, out};
  const uint64_t dim_a = ins.out[0], dim_b = ins.out[1], dim_c = ins.out[2];
  uint64_t a_elems = 0, b_elems = 0, c_elems = 0, row_elems = 0;
  auto fail = [&](const char* why = "operand out of bounds or malformed dims") {
    return std::string(OpName(ins.opcode)) + ": " + why;
  };
  auto attn = [&](uint64_t B, uint64_t S, uint64_t H, uint64_t d, uint64_t* td, uint64_t* pn) {
    uint64_t bs = 0, hd = 0, bhs = 0;
    if (B == 0 || S == 0 || H == 0 || d == 0) return false;
    return ProductFits(B, S, &bs) && ProductFits(H, d, &hd) && ProductFits(bs, hd, td) &&
           ProductFits(bs, H, &bhs) && ProductFits(bhs, S, pn);
  };

  switch (static_cast<Op>(ins.opcode)) {
    case kNop:
      break;
    case kGemmNN: case kGemmNT: case kGemmTN: case kGemmAccNN:
    case kGemmNNQ8: case kGemmNTQ8: case kGemmNNBF16: case kGemmNTBF16: {
      const bool q8 = ins.opcode == kGemmNNQ8 || ins.opcode == kGemmNTQ8;
      const bool bf = ins.opcode == kGemmNNBF16 || ins.opcode == kGemmNTBF16;
      if (!ProductFits(dim_a, dim_c, &a_elems) || !ProductFits(dim_c, dim_b, &b_elems) || !ProductFits(dim_a, dim_b, &c_elems)) return fail();
      if ((q8 || bf) && RefSpace(ins.in[1]) != kRodata) return fail("narrow weight outside rodata");
      b.R(ins.in[0], a_elems);
      b.R(ins.in[1], b_elems, q8 ? 1 : bf ? 2 : 4);
      if (ins.opcode == kGemmAccNN) b.RW(ins.in[2], c_elems); else b.W(ins.in[2], c_elems);
      const bool f32w = ins.opcode == kGemmNN || ins.opcode == kGemmNT || ins.opcode == kGemmTN;
      if (ins.flags & kFlagEpilogueBias) {
        if (ins.opcode != kGemmNN && ins.opcode != kGemmNNBF16) return fail("bias flag on this opcode");
        if (ins.flags & kFlagGemmAddend) return fail("bias and addend share in[3]");
        b.R(ins.in[3], dim_b);
      }
      if ((ins.flags & kFlagActMask) && ins.opcode != kGemmNN && ins.opcode != kGemmNNBF16 &&
          ins.opcode != kGemmNNQ8)
        return fail("activation flag on this opcode");
      if (ins.flags & kFlagGemmAddend) {
        if (!f32w) return fail("addend flag on this opcode");
        b.R(ins.in[3], c_elems);
      }
      if (ins.flags & kFlagQ8ColScale) {
        if (!q8 || RefSpace(ins.in[3]) != kRodata) return fail("column scales");
        b.R(ins.in[3], ins.opcode == kGemmNTQ8 ? dim_c : dim_b);
      } else if (q8) {
        const float s = BitsToF32(ins.in[3]);
        if ((ins.in[3] >> 32) != 0 || !std::isfinite(s) || !(s > 0.0f))
          return fail("dequant scale must be a finite positive float");
      }
      if (ins.opcode == kGemmAccNN && !FiniteImm(ins.in[3])) return fail("alpha");
      if (ins.imm != 0 && (!f32w || !std::isfinite(BitsToF32(ins.imm)))) return fail("alpha imm");
      break;
    }
    case kAddEW: case kMulEW: case kReluBwd: case kGeluBwd: case kSiluBwd:
      b.R(ins.in[0], dim_a); b.R(ins.in[1], dim_a); b.W(ins.in[2], dim_a);
      break;
    case kAddBias:
      if (!ProductFits(dim_a, dim_b, &c_elems)) return fail();
      b.R(ins.in[0], c_elems); b.R(ins.in[1], dim_b); b.W(ins.in[2], c_elems);
      break;
    case kReluFwd: case kGeluFwd: case kSiluFwd: case kCopy:
      b.R(ins.in[0], dim_a); b.W(ins.in[1], dim_a);
      break;
    case kScale:
      if (!FiniteImm(ins.in[2])) return fail("scale immediate");
      b.R(ins.in[0], dim_a); b.W(ins.in[1], dim_a);
      break;
    case kLayerNormFwd: {
      const uint64_t rows = Hi32(dim_a), cols = Lo32(dim_a);
      if (!ProductFits(rows, cols, &row_elems) || cols == 0) return fail();
      b.R(ins.in[0], row_elems); b.R(ins.in[1], cols); b.R(ins.in[2], cols); b.W(ins.in[3], row_elems);
      b.W(ins.out[1], rows); b.W(ins.out[2], rows);
      break;
    }
    case kLayerNormBwd: {
      const uint64_t rows = Hi32(dim_c), cols = Lo32(dim_c);
      if (!ProductFits(rows, cols, &row_elems) || cols == 0) return fail();
      b.R(ins.in[0], row_elems); b.R(ins.in[1], row_elems); b.R(ins.in[2], cols); b.W(ins.in[3], row_elems);
      b.R(ins.out[0], rows); b.R(ins.out[1], rows);
      break;
    }
    case kRmsNormFwd: {
      const uint64_t rows = Hi32(dim_a), cols = Lo32(dim_a);
      if (!ProductFits(rows, cols, &row_elems) || cols == 0) return fail();
      b.R(ins.in[0], row_elems); b.R(ins.in[1], cols); b.W(ins.in[2], row_elems); b.W(ins.in[3], rows);
      break;
    }
    case kRmsNormBwd: {
      const uint64_t rows = Hi32(dim_b), cols = Lo32(dim_b);
      if (!ProductFits(rows, cols, &row_elems) || cols == 0) return fail();
      b.R(ins.in[0], row_elems); b.R(ins.in[1], row_elems); b.R(ins.in[2], cols); b.W(ins.in[3], row_elems);
      b.R(ins.out[0], rows);
      break;
    }
    case kClipNorm:
      if (!FiniteImm(ins.in[1])) return fail("clip threshold");
      b.RW(ins.in[0], dim_a);
      break;
    case kSqNormAccum:
      b.R(ins.in[0], dim_a); b.RW(ins.in[1], 1);
      break;
    case kClipGlobal:
      if (!FiniteImm(ins.in[2])) return fail("clip threshold");
      b.RW(ins.in[0], dim_a); b.R(ins.in[1], 1);
      break;
    case kReduceRows:
      if (!ProductFits(dim_a, dim_b, &c_elems)) return fail();
      b.R(ins.in[0], c_elems); b.W(ins.in[1], dim_b);
      break;
    case kSoftmaxXEntFwd: case kSoftmaxXEntMaskedFwd:
      if (!ProductFits(dim_a, dim_b, &row_elems) || dim_a == 0 || dim_b == 0) return fail();
      b.R(ins.in[0], row_elems); b.R(ins.in[1], dim_a); b.W(ins.in[2], 1); b.W(ins.in[3], row_elems);
      break;
    case kSoftmaxXEntBwd: case kSoftmaxXEntMaskedBwd:
      if (!ProductFits(dim_a, dim_b, &row_elems) || dim_a == 0 || dim_b == 0) return fail();
      b.R(ins.in[0], row_elems); b.R(ins.in[1], dim_a); b.R(ins.in[2], 1); b.W(ins.in[3], row_elems);
      break;
    case kMseFwd:
      b.R(ins.in[0], dim_a); b.R(ins.in[1], dim_a); b.W(ins.in[2], 1);
      break;
    case kMseBwd:
      b.R(ins.in[0], dim_a); b.R(ins.in[1], dim_a); b.R(ins.in[2], 1); b.W(ins.in[3], dim_a);
      break;
    case kKLDistillFwd:
      if (!ProductFits(Hi32(dim_b), Lo32(dim_b), &row_elems) || row_elems == 0) return fail();
      b.R(ins.in[0], row_elems); b.R(ins.in[1], row_elems); b.W(ins.in[2], 1); b.W(ins.in[3], row_elems);
      b.W(ins.out[0], row_elems);
      break;
    case kKLDistillBwd:
      if (!ProductFits(Hi32(dim_a), Lo32(dim_a), &row_elems) || row_elems == 0) return fail();
      b.R(ins.in[0], row_elems); b.R(ins.in[1], row_elems); b.R(ins.in[2], 1); b.W(ins.in[3], row_elems);
      break;
    case kSgdStep:
      if (!FiniteImm(dim_b)) return fail("clip word");
      b.RW(ins.in[0], dim_a); b.R(ins.in[1], dim_a);
      break;
    case kAccumulate:
      b.RW(ins.in[0], dim_a); b.R(ins.in[1], dim_a);
      break;
    case kAdamWStep:
      if (!FiniteImm(dim_b)) return fail("clip word");
      b.RW(ins.in[0], dim_a); b.R(ins.in[1], dim_a); b.RW(ins.in[2], dim_a); b.RW(ins.in[3], dim_a);
      break;
    case kFill:
      b.W(ins.in[0], dim_a);
      break;
    case kRopeFwd: case kRopeBwd: {
      uint64_t td = 0, pn = 0;
      if (!attn(Hi32(dim_a), Lo32(dim_a), Hi32(dim_b), Lo32(dim_b), &td, &pn) || Lo32(dim_b) % 2) return fail();
      const float base = BitsToF32(dim_c);
      if ((dim_c >> 32) != 0 || !std::isfinite(base) || !(base > 1.0f)) return fail("rope base");
      b.R(ins.in[0], td); b.W(ins.in[1], td);
      if (ins.in[2] != kNullRef) b.R(ins.in[2], Lo32(dim_a) * Lo32(dim_b));
      break;
    }
    case kRopeTable: {
      const uint64_t S = Hi32(dim_a), d = Lo32(dim_a);
      const float base = BitsToF32(dim_b);
      uint64_t table = 0;
      if (S == 0 || d == 0 || d % 2 || (dim_b >> 32) != 0 || !std::isfinite(base) ||
          !(base > 1.0f) || !ProductFits(S, d, &table))
        return fail();
      b.W(ins.in[0], table);
      break;
    }
    case kFusedMap: {
      bool uses[3] = {false, false, false};
      int stages = 0;
      for (; stages < 4; ++stages) {
        const uint8_t st = static_cast<uint8_t>(dim_b >> (8 * stages));
        const uint8_t kind = st & 0x0F, arg = (st >> 4) & 3;
        if (kind == kFEnd) break;
        if (kind > kFSilu) return fail("unknown fused stage");
        if (kind == kFAdd || kind == kFMul) {
          if (arg != 1 && arg != 2) return fail("fused stage operand slot");
          uses[arg] = true;
        } else if (kind == kFScale && arg > 1) {
          return fail("fused stage immediate");
        }
      }
      if (stages == 0) return fail("empty fused program");
      b.R(ins.in[0], dim_a);
      for (int s = 1; s <= 2; ++s) {
        if (uses[s]) b.R(ins.in[s], dim_a);
        else if (ins.in[s] != kNullRef) return fail("unused fused operand present");
      }
      b.W(ins.in[3], dim_a);
      break;
    }
    case kAttnFwd: {
      uint64_t td = 0, pn = 0;
      if (!attn(Hi32(dim_b), Lo32(dim_b), Hi32(dim_c), Lo32(dim_c), &td, &pn)) return fail();
      b.R(ins.in[0], td); b.R(ins.in[1], td); b.R(ins.in[2], td); b.W(ins.in[3], td);
      b.W(ins.out[0], pn);
      break;
    }
    case kSegmentStarts: {
      uint64_t t = 0;
      if (Hi32(dim_a) == 0 || Lo32(dim_a) == 0 || !ProductFits(Hi32(dim_a), Lo32(dim_a), &t) || dim_b > 0x7FFFFFFFu)
        return fail();
      b.R(ins.in[0], t); b.W(ins.in[1], t);
      break;
    }
    case kAttnFwdSeg: {
      const AttnGeom g = UnpackAttnGeom(dim_b);
      uint64_t td = 0, pn = 0;
      if (!attn(g.B, g.S, g.H, g.d, &td, &pn)) return fail();
      b.R(ins.in[0], td); b.R(ins.in[1], td); b.R(ins.in[2], td); b.W(ins.in[3], td);
      b.W(ins.out[0], pn); b.R(dim_c, g.B * g.S);
      break;
    }
    case kAttnDP: {
      uint64_t td = 0, pn = 0;
      if (!attn(Hi32(dim_a), Lo32(dim_a), Hi32(dim_b), Lo32(dim_b), &td, &pn)) return fail();
      b.R(ins.in[0], td); b.R(ins.in[1], td); b.W(ins.in[2], pn);
      break;
    }
    case kAttnDV: case kAttnDQ: case kAttnDK: {
      uint64_t td = 0, pn = 0;
      if (!attn(Hi32(dim_a), Lo32(dim_a), Hi32(dim_b), Lo32(dim_b), &td, &pn)) return fail();
      b.R(ins.in[0], pn); b.R(ins.in[1], td); b.W(ins.in[2], td);
      break;
    }
    case kSoftmaxRowsBwd:
      if (!ProductFits(Hi32(dim_a), Lo32(dim_a), &row_elems) || Lo32(dim_a) == 0) return fail();
      b.R(ins.in[0], row_elems); b.R(ins.in[1], row_elems); b.W(ins.in[2], row_elems);
      break;
    case kAttnFwdTiled: {
      uint64_t td = 0, pn = 0;
      if (!attn(Hi32(dim_b), Lo32(dim_b), Hi32(dim_c), Lo32(dim_c), &td, &pn)) return fail();
      b.R(ins.in[0], td); b.R(ins.in[1], td); b.R(ins.in[2], td); b.W(ins.in[3], td);
      b.W(ins.out[0], Hi32(dim_b) * Lo32(dim_b) * Hi32(dim_c) * kAttnStatsWidth);
      break;
    }
    case kAttnFwdTiledSeg: {
      const AttnGeom g = UnpackAttnGeom(dim_b);
      uint64_t td = 0, pn = 0;
      if (!attn(g.B, g.S, g.H, g.d, &td, &pn)) return fail();
      b.R(ins.in[0], td); b.R(ins.in[1], td); b.R(ins.in[2], td); b.W(ins.in[3], td);
      b.W(ins.out[0], g.B * g.S * g.H * kAttnStatsWidth); b.R(dim_c, g.B * g.S);
      break;
    }
    case kAttnDQTiled: case kAttnDKTiled: case kAttnDVTiled: {
      const AttnGeom g = UnpackAttnGeom(dim_c);
      uint64_t td = 0, pn = 0;
      if (!attn(g.B, g.S, g.H, g.d, &td, &pn)) return fail();
      b.R(ins.in[0], td); b.R(ins.in[1], td); b.R(ins.in[2], td); b.R(ins.in[3], td);
      const uint64_t st = g.B * g.S * g.H * kAttnStatsWidth;
      if (ins.opcode == kAttnDQTiled) b.RW(ins.out[0], st); else b.R(ins.out[0], st);
      b.W(ins.out[1], td);
      break;
    }
    case kEmbedFwd: {
      const uint64_t vocab = Hi32(dim_b), dim = Lo32(dim_b);
      uint64_t vd = 0, td = 0;
      if (!ProductFits(vocab, dim, &vd) || !ProductFits(dim_a, dim, &td) || dim == 0) return fail();
      if (RefSpace(ins.in[1]) == kArena) return fail("embedding table in the arena");
      b.R(ins.in[0], dim_a); b.R(ins.in[1], vd); b.W(ins.in[2], td);
      break;
    }
    case kOpCount:
      return fail();
  }
  if (!b.ok) return fail();
  return {};
}

}  // namespace see
