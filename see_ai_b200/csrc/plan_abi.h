// The update-plan wire format as this backend reads it: the 64-byte
// instruction word, opcode numbers, flag bits, reference decoding and the
// 320-byte plan header.  Written fresh from the format's specification
// (reference: source/plan/instruction.h:44-232 opcodes, :311-384 flags,
// :438-449 the instruction word; source/plan/schema.h:298-397 header + emit
// entry).  Shared by host code and device code, so it stays plain C++17.
#ifndef SEE_CUDA_PLAN_ABI_H_
#define SEE_CUDA_PLAN_ABI_H_

#include <cstdint>
#include <cstring>

namespace see {

constexpr uint64_t kRodataBit = 1ull << 63;
constexpr uint64_t kSourceBit = 1ull << 62;
constexpr uint64_t kNullRef = ~0ull;

enum Space : uint8_t { kArena = 0, kRodata = 1, kSource = 2 };

inline Space RefSpace(uint64_t ref) {
  if (ref & kRodataBit) return kRodata;
  if (ref & kSourceBit) return kSource;
  return kArena;
}
inline uint64_t RefOffset(uint64_t ref) { return ref & ~(kRodataBit | kSourceBit); }

enum Op : uint16_t {
  kNop = 0, kGemmNN = 1, kGemmNT = 2, kGemmTN = 3, kGemmAccNN = 4,
  kAddEW = 5, kAddBias = 6, kReluFwd = 7, kReluBwd = 8, kScale = 9,
  kReduceRows = 10, kSoftmaxXEntFwd = 11, kSoftmaxXEntBwd = 12,
  kMseFwd = 13, kMseBwd = 14, kKLDistillFwd = 15, kKLDistillBwd = 16,
  kSgdStep = 17, kAdamWStep = 18, kFill = 19, kCopy = 20, kMulEW = 21,
  kGeluFwd = 22, kGeluBwd = 23, kSiluFwd = 24, kSiluBwd = 25,
  kLayerNormFwd = 26, kLayerNormBwd = 27, kClipNorm = 28,
  kGemmNNQ8 = 29, kGemmNTQ8 = 30, kRmsNormFwd = 31, kRmsNormBwd = 32,
  kRopeFwd = 33, kRopeBwd = 34, kAttnFwd = 35, kAttnDP = 36, kAttnDV = 37,
  kSoftmaxRowsBwd = 38, kAttnDQ = 39, kAttnDK = 40, kEmbedFwd = 41,
  kAccumulate = 42, kGemmNNBF16 = 43, kGemmNTBF16 = 44, kRopeTable = 45,
  kFusedMap = 46, kAttnFwdTiled = 47, kAttnDQTiled = 48, kAttnDKTiled = 49,
  kAttnDVTiled = 50, kSoftmaxXEntMaskedFwd = 51, kSoftmaxXEntMaskedBwd = 52,
  kSqNormAccum = 53, kClipGlobal = 54, kSegmentStarts = 55, kAttnFwdSeg = 56,
  kAttnFwdTiledSeg = 57,
  kOpCount = 58,
};

const char* OpName(uint16_t op);

constexpr uint16_t kFlagEpilogueBias = 1u << 0;
constexpr uint16_t kFlagActShift = 1;
constexpr uint16_t kFlagActMask = 3u << 1;
constexpr uint16_t kFlagGemmAddend = 1u << 3;
constexpr uint16_t kFlagQ8ColScale = 1u << 4;
constexpr uint16_t kFlagRelaxed = 1u << 5;
constexpr uint16_t kKnownFlags = 0x3F;

enum Act : uint8_t { kActNone = 0, kActRelu = 1, kActGelu = 2, kActSilu = 3 };
inline Act ActOf(uint16_t flags) { return static_cast<Act>((flags & kFlagActMask) >> kFlagActShift); }

// kFusedMap stage bytes (reference: source/plan/instruction.h:261-297).
enum FusedKind : uint8_t { kFEnd = 0, kFAdd = 1, kFMul = 2, kFScale = 3, kFRelu = 4, kFGelu = 5, kFSilu = 6 };

constexpr uint64_t kAttnStatsWidth = 4;

#pragma pack(push, 1)
struct Instruction {
  uint16_t opcode;
  uint16_t flags;
  uint32_t imm;
  uint64_t in[4];
  uint64_t out[3];
};

struct PlanHeader {
  uint32_t magic, version;
  uint64_t arena_size, persistent_size;
  uint64_t input_ref, input_floats, label_ref, label_bytes;
  uint32_t label_kind, optimizer_kind;
  uint64_t loss_ref;
  uint64_t train_instr_offset, train_instr_count;
  uint64_t merge_instr_offset, merge_instr_count;
  uint64_t rodata_offset, rodata_size;
  uint64_t persist_init_offset, persist_init_size;
  uint64_t emit_table_offset, emit_count;
  float lr, beta1, beta2, eps, weight_decay;
  uint32_t gemm_tile_k;
  uint64_t batch, default_steps;
  uint64_t eval_instr_offset, eval_instr_count;
  uint64_t source_model_hash, plan_hash;
  uint32_t lr_schedule, gemm_tile_n;
  uint64_t warmup_steps;
  float min_lr_factor, clip_norm;
  uint32_t input_kind, grad_accum_steps;
  uint64_t seq_len;
  uint64_t step_instr_offset, step_instr_count;
  uint64_t tokenizer_hash, corpus_hash, split_seed, val_split_hash;
  uint32_t val_frac_bits, data_flags;
};

struct EmitEntry {
  uint64_t smf_data_offset, byte_size, arena_offset;
};
#pragma pack(pop)

static_assert(sizeof(Instruction) == 64, "instruction word is one cache line");
static_assert(sizeof(PlanHeader) == 320, "plan header layout");
static_assert(sizeof(EmitEntry) == 24, "emit entry layout");

constexpr uint32_t kSeeuMagic = 0x55454553u;
constexpr uint32_t kSeeuVersion = 26;
constexpr uint32_t kSeeuOldestReadable = 4;
constexpr uint64_t kArenaAlignment = 16384;

inline float BitsToF32(uint64_t bits) {
  const uint32_t b = static_cast<uint32_t>(bits);
  float f;
  std::memcpy(&f, &b, 4);
  return f;
}
inline uint32_t F32Bits(float f) {
  uint32_t b;
  std::memcpy(&b, &f, 4);
  return b;
}
inline float GemmAlphaOf(uint32_t imm) { return imm == 0 ? 1.0f : BitsToF32(imm); }
inline float NormEpsOf(uint32_t imm) { return imm == 0 ? 1e-5f : BitsToF32(imm); }

struct AttnGeom { uint64_t B, S, H, d; };
inline AttnGeom UnpackAttnGeom(uint64_t w) {
  return {w >> 48, (w >> 32) & 0xFFFF, (w >> 16) & 0xFFFF, w & 0xFFFF};
}
inline uint64_t Hi32(uint64_t w) { return w >> 32; }
inline uint64_t Lo32(uint64_t w) { return w & 0xFFFFFFFFull; }

// Per-range scalars the optimizer instructions read (reference:
// runtime/executor/backend.h:56-63).
struct StepParams {
  float lr = 0.0f, beta1 = 0.9f, beta2 = 0.999f, eps = 1e-8f, weight_decay = 0.0f;
  uint32_t pad = 0;
  uint64_t step = 0;
};

}  // namespace see

#endif  // SEE_CUDA_PLAN_ABI_H_
