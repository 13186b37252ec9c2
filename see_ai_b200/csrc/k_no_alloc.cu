// see_cuda_xent_forward_static: softmax cross-entropy forward for callers that
// are not allowed to allocate device memory.
//
// Who that is: code running inside someone else's memory budget — a plugin
// loaded into a host process that has already handed every byte of device
// memory to its own pool, a real-time or safety-reviewed loop where a
// cudaMalloc (which can synchronize the device and can fail) is not permitted
// after start-up, or a region being recorded into a CUDA graph by the caller,
// where allocation calls are illegal.  The regular path (the backend's
// kSoftmaxXEntFwd instruction) sizes a per-row scratch buffer with cudaMalloc
// the first time it meets a batch; this entry point never does.
//
// Instead the scratch lives in this file as a fixed device array: one double
// per row for up to kNoAllocMaxRows rows (512 KiB) plus one counter.  Every
// GPU that loads the library carries that array until the process exits.  The
// caller passes the inputs and outputs as device pointers, exactly as the
// kernel sees them.
//
// Things a caller must know:
//  * The first call on each device looks up the array's device address
//    (cudaGetSymbolAddress, with that device current).  Make that first call
//    before starting any stream capture.  Rows of 4096 to 32768 classes take a
//    different kernel whose first launch on a device raises its shared-memory
//    limit: make a first call of THAT width class before capture too.
//  * All calls share the one array.  Two calls whose kernels can overlap on
//    the GPU (different streams, no ordering between them) race on it.
//  * Nothing in the array has to start at zero: each call overwrites the
//    entries it reads (rows 0..N-1 and the counter) before reading them, so
//    the previous call's leftovers are harmless.
//  * N above kNoAllocMaxRows is refused with SEE_ERROR and a message; nothing
//    is launched.
#include <cuda_runtime.h>

#include <atomic>
#include <cstdio>

#include "../../include/see_cuda.h"
#include "kernels.h"

namespace {

constexpr unsigned long long kNoAllocMaxRows = 65536;
constexpr int kMaxDevices = 64;

struct alignas(256) NoAllocScratch {
  double rows[kNoAllocMaxRows];
  unsigned long long count;
};

// In host code this name is only a handle for the runtime's symbol table — not
// a device address.  Kernels get the address cudaGetSymbolAddress returns.
static __device__ __align__(256) NoAllocScratch g_no_alloc_scratch;

// Written once per device; atomic because nothing stops two host threads from
// making the first call on a device at the same moment (both then look the same
// address up and store the same value).
std::atomic<NoAllocScratch*> g_scratch_on_device[kMaxDevices] = {};
thread_local char g_no_alloc_error[256] = "";

int Fail(const char* what, cudaError_t e) {
  if (e == cudaSuccess)
    std::snprintf(g_no_alloc_error, sizeof(g_no_alloc_error), "cuda: xent_forward_static: %s", what);
  else
    std::snprintf(g_no_alloc_error, sizeof(g_no_alloc_error), "cuda: xent_forward_static: %s: %s",
                  what, cudaGetErrorString(e));
  return SEE_ERROR;
}

}  // namespace

extern "C" {

const char* see_cuda_static_last_error(void) { return g_no_alloc_error; }

uint64_t see_cuda_static_max_rows(void) { return kNoAllocMaxRows; }

int see_cuda_xent_forward_static(const float* logits, const int32_t* labels, float* loss,
                                 float* probs, uint64_t rows, uint64_t classes, int masked,
                                 void* cuda_stream) {
  if (!logits || !labels || !loss || !probs) return Fail("null operand", cudaSuccess);
  if (rows == 0 || classes == 0) return Fail("empty batch", cudaSuccess);
  if (rows > kNoAllocMaxRows) {
    std::snprintf(g_no_alloc_error, sizeof(g_no_alloc_error),
                  "cuda: xent_forward_static: %llu rows exceed the fixed scratch of %llu rows; "
                  "use the backend's kSoftmaxXEntFwd instruction for larger batches",
                  static_cast<unsigned long long>(rows), kNoAllocMaxRows);
    return SEE_ERROR;
  }
  int device = -1;
  if (cudaError_t e = cudaGetDevice(&device); e != cudaSuccess) return Fail("cudaGetDevice", e);
  if (device < 0 || device >= kMaxDevices) return Fail("device ordinal out of range", cudaSuccess);
  if (!g_scratch_on_device[device].load(std::memory_order_acquire)) {
    // Set-up, once per device, with that device current.
    NoAllocScratch* ptr = nullptr;
    if (cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_no_alloc_scratch);
        e != cudaSuccess)
      return Fail("cudaGetSymbolAddress", e);
    if (!ptr) return Fail("the scratch symbol has no device address", cudaSuccess);
    g_scratch_on_device[device].store(ptr, std::memory_order_release);
  }
  NoAllocScratch* scratch = g_scratch_on_device[device].load(std::memory_order_acquire);
  see::k::SoftmaxXEntFwd(masked != 0, logits, labels, loss, probs, rows, classes, scratch->rows,
                         &scratch->count, static_cast<cudaStream_t>(cuda_stream));
  if (cudaError_t e = cudaGetLastError(); e != cudaSuccess) return Fail("launch", e);
  g_no_alloc_error[0] = '\0';
  return SEE_OK;
}

}  // extern "C"
