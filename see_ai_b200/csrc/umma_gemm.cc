#include "umma_gemm.h"
namespace see::umma {
struct Impl {};
std::string Init(Context*, int) { return {}; }
void Destroy(Context*) {}
void InvalidateAll(Context*) {}
void InvalidateRange(Context*, uint64_t, uint64_t) {}
void PlanRange(Context*, const Instruction*, size_t, size_t) {}
std::string TryGemm(Context*, const k::GemmArgs&, int, uint64_t, uint64_t, uint64_t, cudaStream_t,
                    int* launches) { *launches = 0; return {}; }
}  // namespace see::umma
