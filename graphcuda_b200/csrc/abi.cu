// Library-level entry points: version, status text, thread-local error text.
#include "common.cuh"

#include <atomic>
#include <cstring>

namespace {
thread_local char g_last_error[512] = {0};
}

namespace {
std::atomic<long long> g_launches{0};
}

namespace gc {
void count_launches(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
  return code;
}
}  // namespace gc

extern "C" {

int gc_abi_version(void) { return 3; }

long long gc_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

const char* gc_last_error(void) { return g_last_error; }

const char* gc_status_string(int status) {
  switch (status) {
    case GC_OK: return "ok";
    case GC_ERR_INVALID: return "invalid argument";
    case GC_ERR_UNSUPPORTED: return "unsupported configuration";
    case GC_ERR_CUDA: return "CUDA error";
    case GC_ERR_WORKSPACE: return "workspace missing or too small";
    case GC_ERR_DEVICE_FLAG: return "a device-side bounded wait ran out";
    default: return "unknown status";
  }
}

}  // extern "C"
