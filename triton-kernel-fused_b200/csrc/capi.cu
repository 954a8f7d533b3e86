// Library-wide host helpers: version, thread-local error text, status decoding, device properties.
#include <stdarg.h>

#include <atomic>
#include <mutex>

#include "common.cuh"
#include "ptx.cuh"

namespace b200moe {

static thread_local char g_err[512] = "no error";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int cuda_fail(cudaError_t e, const char* what) {
  set_error("CUDA error %d (%s) at %s", static_cast<int>(e), cudaGetErrorString(e), what);
  return B200MOE_E_CUDA;
}

int num_sms() {
  static int n = 0;
  static std::once_flag once;
  std::call_once(once, [] {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
  });
  return n;
}

// One CTA waits on an mbarrier that nothing ever completes, with a limit of `limit_cycles` SM clocks:
// the wait gives up, the status word receives ST_SELFTEST_TIMEOUT and the kernel returns normally.
__global__ void selftest_bounded_wait_kernel(int* status, long long limit_cycles) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();
  const bool done = mbar_wait(smem_u32(&bar), 0, &abort_flag, ST_SELFTEST_TIMEOUT, limit_cycles);
  __syncthreads();
  if (threadIdx.x == 0 && !done && abort_flag != 0) atomicCAS(status, 0, abort_flag);
}

static std::atomic<int> g_reserved_sms{0};

int gemm_cta_budget() {
  int n = num_sms() - g_reserved_sms.load(std::memory_order_relaxed);
  n &= ~1;                      // pair kernels launch clusters of two
  return n < 2 ? 2 : n;
}

static std::atomic<int> g_exchange_sms{0};

int exchange_sm_budget() {
  const int n = g_exchange_sms.load(std::memory_order_relaxed);
  return n > 0 ? n : num_sms();
}

}  // namespace b200moe

extern "C" {

int b200moe_selftest_bounded_wait(int32_t* status, int64_t limit_cycles, b200moe_stream_t stream) {
  if (status == nullptr || limit_cycles < 1000 || limit_cycles > 2000000000LL) {
    b200moe::set_error("selftest_bounded_wait: status must be non-null and 1e3 <= limit_cycles <= 2e9");
    return B200MOE_E_BAD_SHAPE;
  }
  b200moe::selftest_bounded_wait_kernel<<<1, 64, 0, (cudaStream_t)stream>>>(status, limit_cycles);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return b200moe::cuda_fail(e, "selftest_bounded_wait launch");
  return 0;
}

int b200moe_set_reserved_sms(int n) {
  if (n < 0 || n >= b200moe::num_sms()) {
    b200moe::set_error("set_reserved_sms: %d is outside [0, %d)", n, b200moe::num_sms());
    return B200MOE_E_BAD_SHAPE;
  }
  b200moe::g_reserved_sms.store(n, std::memory_order_relaxed);
  return 0;
}

int b200moe_set_exchange_sms(int n) {
  if (n < 0 || n > b200moe::num_sms()) {
    b200moe::set_error("set_exchange_sms: %d is outside [0, %d]", n, b200moe::num_sms());
    return B200MOE_E_BAD_SHAPE;
  }
  b200moe::g_exchange_sms.store(n, std::memory_order_relaxed);
  return 0;
}

const char* b200moe_version(void) { return "b200moe 0.1 (sm_100a)"; }

const char* b200moe_last_error_string(void) { return b200moe::g_err; }

const char* b200moe_status_string(int s) {
  switch (s) {
    case b200moe::ST_OK: return "ok";
    case b200moe::ST_WAIT_PRODUCER: return "GEMM: TMA producer gave up waiting for a free shared-memory stage";
    case b200moe::ST_WAIT_MMA_FULL: return "GEMM: MMA issuer gave up waiting for a filled stage";
    case b200moe::ST_WAIT_MMA_TMEM: return "GEMM: MMA issuer gave up waiting for a drained accumulator";
    case b200moe::ST_WAIT_EPILOGUE: return "GEMM: epilogue gave up waiting for a finished accumulator";
    case b200moe::ST_BAD_EXPERT_INDEX: return "permute: expert index outside [0, E)";
    case b200moe::ST_SELFTEST_TIMEOUT: return "self-test: the bounded wait ran out (expected)";
    case b200moe::ST_WAIT_PEER: return "expert-parallel barrier: a peer rank did not arrive within the limit";
    case b200moe::ST_EP_CAPACITY: return "expert parallel: more rows routed to one rank than the fixed-capacity buffers hold; nothing was computed";
    default: return "unknown status";
  }
}

}  // extern "C"
