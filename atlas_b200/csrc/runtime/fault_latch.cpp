// One-shot, process-wide fault latch: the first fatal condition (lost CUDA context, dead control plane) sticks; the
// HTTP layer turns it into 503 and a supervisor restarts the process.
// Reference behaviour: crates/avarok-core/src/fault.rs:1-60.
#include <atomic>
#include <cstring>
#include <mutex>
#include <string>

#include "runtime_api.h"

namespace {
std::atomic<int> g_tripped{0};
std::mutex g_mu;
std::string g_reason;
}  // namespace

extern "C" {

int atlas_fault_trip(const char* reason) {
  std::lock_guard<std::mutex> g(g_mu);
  if (g_tripped.load()) return 0;
  g_reason = reason ? reason : "";
  g_tripped.store(1);
  return 1;
}

int atlas_fault_tripped(void) { return g_tripped.load(); }

int atlas_fault_reason(char* out, int cap) {
  std::lock_guard<std::mutex> g(g_mu);
  if (!g_tripped.load()) {
    if (cap > 0) out[0] = 0;
    return 0;
  }
  if (cap > 0) {
    std::strncpy(out, g_reason.c_str(), cap - 1);
    out[cap - 1] = 0;
  }
  return (int)g_reason.size();
}

void atlas_fault_reset_for_tests(void) {
  std::lock_guard<std::mutex> g(g_mu);
  g_tripped.store(0);
  g_reason.clear();
}

}  // extern "C"
