// Error reporting and device queries shared by every entry point.
#include <atomic>

#include "common.cuh"

namespace lm {

namespace {
thread_local char g_error[512] = "";
std::atomic<unsigned long long> g_launches{0};
}

void note_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

int set_error(int code, const char* fmt, ...) {
  va_list args;
  va_start(args, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, args);
  va_end(args);
  return code;
}

int sm_count() {
  static int cached[64] = {0};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 0;
  if (cached[device] == 0) {
    int value = 0;
    if (cudaDeviceGetAttribute(&value, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return 0;
    cached[device] = value;
  }
  return cached[device];
}

}  // namespace lm

extern "C" int lm_version(void) { return 1; }

extern "C" const char* lm_last_error_string(void) { return lm::g_error; }

extern "C" int lm_sm_count(int* out) {
  LM_REQUIRE(out, "sm_count: null pointer");
  *out = lm::sm_count();
  if (*out <= 0) return lm::set_error(LM_ERR_CUDA, "no CUDA device");
  return LM_OK;
}

extern "C" unsigned long long lm_launch_count(void) { return lm::g_launches.load(std::memory_order_relaxed); }
