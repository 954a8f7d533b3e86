// Host-side helpers shared by the translation units of libb200moe: error reporting and checks.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/b200moe.h"

namespace b200moe {

// codes written by kernels into the caller's `status` word
enum : int {
  ST_OK = 0,
  ST_WAIT_PRODUCER = 1,   // TMA producer: a shared-memory stage never became free
  ST_WAIT_MMA_FULL = 2,   // MMA issuer: a stage never filled
  ST_WAIT_MMA_TMEM = 3,   // MMA issuer: the accumulator was never drained
  ST_WAIT_EPILOGUE = 4,   // epilogue: the accumulator never completed
  ST_BAD_EXPERT_INDEX = 5,// permute: an expert index outside [0, E)
  ST_SELFTEST_TIMEOUT = 6,// self-test: a wait that nothing completes ran out, as intended
  ST_WAIT_PEER = 7,       // cross-rank barrier: a peer's arrival never showed up within the limit
  ST_EP_CAPACITY = 8      // expert parallel with fixed buffers: a rank would receive more rows than its buffers hold
};

void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);
int num_sms();
int gemm_cta_budget();   // CTAs a persistent GEMM may occupy (num_sms() minus the reserved SMs)
int exchange_sm_budget();   // SMs (= fat CTAs) the home-side pull kernel of the expert-parallel exchange may occupy

#define B200_CHECK_ARG(cond, code, ...)  \
  do {                                   \
    if (!(cond)) {                       \
      ::b200moe::set_error(__VA_ARGS__); \
      return (code);                     \
    }                                    \
  } while (0)

#define B200_CUDA(call)                                                   \
  do {                                                                    \
    cudaError_t e__ = (call);                                             \
    if (e__ != cudaSuccess) return ::b200moe::cuda_fail(e__, #call);      \
  } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace b200moe
