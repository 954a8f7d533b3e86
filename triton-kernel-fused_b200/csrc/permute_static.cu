// b200moe_permute_build_static: the expert permutation for callers that cannot allocate device memory.
//
// b200moe_permute_build needs a scratch buffer (the per-chunk histograms) that its caller must
// allocate.  Some callers have no way to do that at the point where they route tokens: a plugin that
// runs inside a host framework which has already handed all free device memory to its own arena, a
// serving loop under a latency budget in which cudaMalloc (a device-wide synchronisation) is banned,
// or code running while someone else's stream capture forbids allocation calls.  For them the scratch
// lives in a fixed array that is part of this library's device image.
#include <mutex>

#include "common.cuh"

namespace b200moe {

// 1 MiB of histogram scratch: ceil(T*k/512) * E int32 entries must fit.  Every GPU on which this
// library's module is loaded carries the array until the process exits.
constexpr size_t kStaticScratchBytes = 1u << 20;
static __device__ __align__(256) unsigned char g_permute_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;

// The array's name is only a host-side handle for the symbol: the address kernels can use has to be
// asked for, once per device and with that device current.  The address is cached per device ordinal for
// the life of the process; a cudaDeviceReset() destroys the context the address belongs to, so a process
// that resets a device must not call this entry point on it afterwards.
static int static_scratch(void** out) {
  static std::mutex mu;
  static void* ptrs[kMaxDevices] = {nullptr};
  int dev = 0;
  B200_CUDA(cudaGetDevice(&dev));
  B200_CHECK_ARG(dev >= 0 && dev < kMaxDevices, B200MOE_E_UNSUPPORTED, "device ordinal %d not supported", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (ptrs[dev] == nullptr) {
    void* p = nullptr;
    B200_CUDA(cudaGetSymbolAddress(&p, g_permute_scratch));
    ptrs[dev] = p;
  }
  *out = ptrs[dev];
  return 0;
}

}  // namespace b200moe

using namespace b200moe;

extern "C" int b200moe_permute_build_static(const int64_t* idx, int64_t T, int k, int E, int32_t* counts,
                                            int32_t* offs, int32_t* poffs, int32_t* slot_row, int32_t* row_slot,
                                            int32_t* tile_expert, int32_t* order, int32_t* slot_pos,
                                            int32_t* status, b200moe_stream_t stream) {
  // the ranges are checked before T * k is formed, so the product below cannot overflow
  B200_CHECK_ARG(T >= 0 && T < (1LL << 31) && k >= 1 && k <= B200MOE_MAX_TOPK && E >= 1 && E <= B200MOE_MAX_EXPERTS,
                 B200MOE_E_BAD_SHAPE, "permute_build_static: T = %lld, k = %d (1..%d), E = %d (1..%d)", (long long)T, k,
                 B200MOE_MAX_TOPK, E, B200MOE_MAX_EXPERTS);
  const size_t need = b200moe_permute_ws_bytes(T * k, E);
  B200_CHECK_ARG(need <= kStaticScratchBytes, B200MOE_E_WS_TOO_SMALL,
                 "permute_build_static: T*k = %lld slots over E = %d experts need %zu bytes of scratch, the built-in "
                 "array holds %zu; use b200moe_permute_build with a caller-allocated workspace",
                 (long long)(T * k), E, need, kStaticScratchBytes);
  void* ws = nullptr;
  int rc = static_scratch(&ws);
  if (rc) return rc;
  // The histogram kernel overwrites every entry it later reads, so nothing in the shared array has
  // to be cleared between calls.
  return b200moe_permute_build(idx, T, k, E, counts, offs, poffs, slot_row, row_slot, tile_expert, order, slot_pos,
                               ws, kStaticScratchBytes, status, stream);
}
