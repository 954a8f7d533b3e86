// Library-wide host helpers: version, thread-local error text, status decoding, device properties.
#include <stdarg.h>

#include <atomic>
#include <mutex>

#include "common.cuh"

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

static std::atomic<int> g_reserved_sms{0};

int gemm_cta_budget() {
  int n = num_sms() - g_reserved_sms.load(std::memory_order_relaxed);
  n &= ~1;                      // pair kernels launch clusters of two
  return n < 2 ? 2 : n;
}

}  // namespace b200moe

extern "C" {

int b200moe_set_reserved_sms(int n) {
  if (n < 0 || n >= b200moe::num_sms()) {
    b200moe::set_error("set_reserved_sms: %d is outside [0, %d)", n, b200moe::num_sms());
    return B200MOE_E_BAD_SHAPE;
  }
  b200moe::g_reserved_sms.store(n, std::memory_order_relaxed);
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
    default: return "unknown status";
  }
}

}  // extern "C"
