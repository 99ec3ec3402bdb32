// ABI-level helpers of liblitedsa_b200.so: version, error strings.
#include "common.cuh"

#include <atomic>

namespace lt {
static std::atomic<int> g_epoch{0};
static std::atomic<unsigned long long> g_wait_limit_ns{kWaitLimitNs};
int next_launch_epoch() {
  int e = g_epoch.fetch_add(1, std::memory_order_relaxed) + 1;
  e &= 0x7fffffff;
  return e == 0 ? next_launch_epoch() : e;
}
unsigned long long wait_limit_ns() { return g_wait_limit_ns.load(std::memory_order_relaxed); }
}  // namespace lt

extern "C" int litedsa_abi_version(void) { return 4; }

// Limit of a single device-side wait for all later launches of this process (0 = the
// default of 2 s).  Returns the previous value through *previous_ns when given.
extern "C" int litedsa_set_wait_limit_ns(uint64_t limit_ns, uint64_t* previous_ns) {
  const unsigned long long v = limit_ns ? (unsigned long long)limit_ns : lt::kWaitLimitNs;
  const unsigned long long old = lt::g_wait_limit_ns.exchange(v, std::memory_order_relaxed);
  if (previous_ns) *previous_ns = old;
  return LITEDSA_OK;
}

extern "C" const char* litedsa_error_string(int code) {
  switch (code) {
    case LITEDSA_OK: return "ok";
    case LITEDSA_ERR_ARG: return "bad argument (null pointer or inconsistent optional arguments)";
    case LITEDSA_ERR_SHAPE: return "shape rule of the operator violated";
    case LITEDSA_ERR_UNSUPPORTED: return "configuration not supported by this build";
    case LITEDSA_ERR_CUDA: return "CUDA runtime or driver call failed";
    case LITEDSA_ERR_TIMEOUT: return "device-side bounded wait expired";
    default: return "unknown litedsa error code";
  }
}
