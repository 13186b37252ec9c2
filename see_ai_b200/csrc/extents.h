// Operand extents of one instruction: which byte ranges of which address
// space it reads and writes.  The backend uses them to bounds-check every
// operand before a kernel is launched, to copy written ranges back to the
// host arena in strict-coherence mode, and to track which cached operand
// conversions a write invalidates.  Same per-opcode table as the reference
// validator proves at load (reference: runtime/verifier/plan_validator.cc:367-748).
#ifndef SEE_CUDA_EXTENTS_H_
#define SEE_CUDA_EXTENTS_H_

#include <cstddef>
#include <cstdint>
#include <string>

#include "plan_abi.h"

namespace see {

struct Extent {
  uint64_t off = 0;
  uint64_t bytes = 0;
  Space space = kArena;
  bool write = false;
  bool read = true;  // a written extent that is also read (in-place operands)
};

struct Extents {
  Extent e[8];
  size_t count = 0;
};

// Fills `out`; returns an empty string, or why the instruction is malformed
// (unknown opcode or flag, overflowing dims, an operand outside its space).
// `source_bytes` == 0 means no source model is bound.
std::string DescribeInstruction(const Instruction& ins, uint64_t arena_bytes,
                                uint64_t rodata_bytes, uint64_t source_bytes,
                                Extents* out);

}  // namespace see

#endif  // SEE_CUDA_EXTENTS_H_
