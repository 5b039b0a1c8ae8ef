// Error bookkeeping of the C ABI: last-error message per thread, launch counter, version.
#include "errors.h"
#include "../../include/eisen_b200.h"

#include <atomic>
#include <cstdio>
#include <cstring>

namespace eisen {

static thread_local char g_err[512] = "";
static std::atomic<long long> g_launches{0};
static std::atomic<int> g_deterministic{0};

bool deterministic() { return g_deterministic.load(std::memory_order_relaxed) != 0; }

void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

void set_error(const char* msg) {
  std::snprintf(g_err, sizeof(g_err), "%s", msg ? msg : "");
}
int fail(int code, const char* msg) {
  set_error(msg);
  return code;
}
int check_launch(const char* what) {
  count_launch();
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) return 0;
  char buf[400];
  std::snprintf(buf, sizeof(buf), "%s: %s", what, cudaGetErrorString(e));
  set_error(buf);
  return EISEN_ERR_CUDA;
}

}  // namespace eisen

extern "C" {

const char* eisen_last_error(void) { return eisen::g_err; }
const char* eisen_version(void) { return "eisen_b200 0.1 (sm_100a)"; }
long long eisen_launch_count(void) { return eisen::g_launches.load(); }
int eisen_set_deterministic(int on) {
  eisen::g_deterministic.store(on ? 1 : 0);
  return 0;
}
int eisen_get_deterministic(void) { return eisen::g_deterministic.load(); }
}  // extern "C"
