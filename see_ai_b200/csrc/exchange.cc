#include "exchange.h"

#include <dlfcn.h>

#include <cstring>
#include <mutex>

namespace see {

namespace {

// The few NCCL entry points this file uses, with the library's public C types
// (an opaque communicator pointer, a 128-byte id passed by value, enum values as
// ints: ncclSuccess 0, ncclUint8 1).
struct NcclId { char bytes[kExchangeIdBytes]; };
using GetUniqueIdFn = int (*)(NcclId*);
using CommInitRankFn = int (*)(void**, int, NcclId, int);
using AllGatherFn = int (*)(const void*, void*, size_t, int, void*, cudaStream_t);
using CommDestroyFn = int (*)(void*);
using GetErrorStringFn = const char* (*)(int);
constexpr int kNcclUint8 = 1;

struct Nccl {
  void* lib = nullptr;
  GetUniqueIdFn get_unique_id = nullptr;
  CommInitRankFn comm_init_rank = nullptr;
  AllGatherFn all_gather = nullptr;
  CommDestroyFn comm_destroy = nullptr;
  GetErrorStringFn get_error_string = nullptr;
  std::string error;
};

const Nccl& Library() {
  static Nccl n;
  static std::once_flag once;
  std::call_once(once, [] {
    // A copy already mapped into the process (a host framework's) is reused.
    for (const char* name : {"libnccl.so.2", "libnccl.so"}) {
      n.lib = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
      if (n.lib) break;
    }
    if (!n.lib) {
      n.error = "exchange: libnccl.so.2 is not loadable in this process";
      return;
    }
    n.get_unique_id = reinterpret_cast<GetUniqueIdFn>(dlsym(n.lib, "ncclGetUniqueId"));
    n.comm_init_rank = reinterpret_cast<CommInitRankFn>(dlsym(n.lib, "ncclCommInitRank"));
    n.all_gather = reinterpret_cast<AllGatherFn>(dlsym(n.lib, "ncclAllGather"));
    n.comm_destroy = reinterpret_cast<CommDestroyFn>(dlsym(n.lib, "ncclCommDestroy"));
    n.get_error_string = reinterpret_cast<GetErrorStringFn>(dlsym(n.lib, "ncclGetErrorString"));
    if (!n.get_unique_id || !n.comm_init_rank || !n.all_gather || !n.comm_destroy || !n.get_error_string)
      n.error = "exchange: the NCCL library lacks an entry point this backend needs";
  });
  return n;
}

std::string Why(const Nccl& n, const char* what, int rc) {
  return std::string("exchange: ") + what + ": " + n.get_error_string(rc);
}

}  // namespace

std::expected<void, std::string> MakeExchangeId(uint8_t out[kExchangeIdBytes]) {
  const Nccl& n = Library();
  if (!n.error.empty()) return std::unexpected(n.error);
  NcclId id;
  if (int rc = n.get_unique_id(&id); rc != 0) return std::unexpected(Why(n, "ncclGetUniqueId", rc));
  std::memcpy(out, id.bytes, kExchangeIdBytes);
  return {};
}

std::expected<std::unique_ptr<GradientExchange>, std::string> GradientExchange::Join(
    int world, int rank, const uint8_t id[kExchangeIdBytes], uint64_t bytes) {
  if (world < 2 || rank < 0 || rank >= world) return std::unexpected(std::string("exchange: bad world / rank"));
  if (bytes == 0) return std::unexpected(std::string("exchange: the plan has no gradient block to exchange"));
  const Nccl& n = Library();
  if (!n.error.empty()) return std::unexpected(n.error);
  std::unique_ptr<GradientExchange> x(new GradientExchange());
  x->world_ = world;
  x->rank_ = rank;
  x->bytes_ = bytes;
  if (cudaMalloc(&x->gathered_, bytes * static_cast<uint64_t>(world)) != cudaSuccess) {
    cudaGetLastError();
    return std::unexpected(std::string("exchange: gather buffer allocation failed"));
  }
  NcclId nid;
  std::memcpy(nid.bytes, id, kExchangeIdBytes);
  if (int rc = n.comm_init_rank(&x->comm_, world, nid, rank); rc != 0)
    return std::unexpected(Why(n, "ncclCommInitRank", rc));
  return x;
}

GradientExchange::~GradientExchange() {
  if (comm_) Library().comm_destroy(comm_);
  if (gathered_) cudaFree(gathered_);
}

std::expected<void, std::string> GradientExchange::AllGather(const void* local, cudaStream_t s) {
  const Nccl& n = Library();
  if (int rc = n.all_gather(local, gathered_, bytes_, kNcclUint8, comm_, s); rc != 0)
    return std::unexpected(Why(n, "ncclAllGather", rc));
  return {};
}

}  // namespace see
