// Interface between the tcgen05 adapter-backward kernel (k_lora_umma.cu) and the
// host code that encodes its tensor maps (umma_gemm.cc).
#ifndef SEE_CUDA_LORA_UMMA_H_
#define SEE_CUDA_LORA_UMMA_H_

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstddef>

#include "kernels.h"

namespace see::k {

// r = 16, N and K multiples of 128 whose accumulators fit tensor memory, at least one 64-row tile.
bool LoraBackwardUmmaSupported(size_t M, size_t N, size_t K, size_t r);
// Blocks the kernel runs for M rows on a device with `sms` multiprocessors (one set of partial sums each).
int LoraBackwardUmmaBlocks(size_t M, int sms);
// map_dy: f32 [M, N] row-major, box {128, 64}, no swizzle; map_x: f32 [M, K] likewise;
// map_b: f32 [16, N], box {128, 16}.  Writes a.dt (and a.dt_pieces) and `blocks` sets of partial
// sums into a.partials (dB [16][N] then dA [K][16] each); LoraFoldPartials makes dB and dA of them.
cudaError_t LoraBackwardUmmaLaunch(const CUtensorMap& map_dy, const CUtensorMap& map_x, const CUtensorMap& map_b,
                                   const LoraBackwardArgs& a, int blocks, DeviceStatus* status, cudaStream_t s);
// Process-wide switch (on by default): off sends every site to the kernel of k_lora_mma.cu.
void LoraBackwardUmmaSet(bool on);
bool LoraBackwardUmmaEnabled();
// dB = alpha_db * sum of the blocks' partial sums, dA likewise, added in block order (k_lora_mma.cu).
void LoraFoldPartials(const LoraBackwardArgs& a, int blocks, cudaStream_t s);

}  // namespace see::k

#endif  // SEE_CUDA_LORA_UMMA_H_
