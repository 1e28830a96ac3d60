// Library-level entry points: version and the optional per-kernel event timing registry.
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <utility>
#include <vector>

#include "fla_b200_internal.h"
#include "kernel_timer.h"

namespace fla {
namespace {
struct Record {
  std::vector<std::pair<cudaEvent_t, cudaEvent_t>> events;
  cudaEvent_t pending = nullptr;
};
std::mutex g_mu;
bool g_enabled = false;
std::map<std::string, Record> g_records;
}  // namespace

bool kernel_timing_enabled() { return g_enabled; }

void kernel_timing_begin(const char* name, cudaStream_t s) {
  std::lock_guard<std::mutex> lk(g_mu);
  Record& r = g_records[name];
  cudaEvent_t e;
  if (cudaEventCreate(&e) != cudaSuccess) return;
  cudaEventRecord(e, s);
  r.pending = e;
}

void kernel_timing_end(const char* name, cudaStream_t s) {
  std::lock_guard<std::mutex> lk(g_mu);
  Record& r = g_records[name];
  if (!r.pending) return;
  cudaEvent_t e;
  if (cudaEventCreate(&e) != cudaSuccess) return;
  cudaEventRecord(e, s);
  r.events.emplace_back(r.pending, e);
  r.pending = nullptr;
}
}  // namespace fla

extern "C" FLA_API int fla_b200_version(void) { return 100; }

extern "C" FLA_API int fla_b200_kernel_timing_enable(int enable) {
  std::lock_guard<std::mutex> lk(fla::g_mu);
  fla::g_enabled = enable != 0;
  for (auto& kv : fla::g_records) {
    for (auto& ev : kv.second.events) {
      cudaEventDestroy(ev.first);
      cudaEventDestroy(ev.second);
    }
    if (kv.second.pending) cudaEventDestroy(kv.second.pending);
  }
  fla::g_records.clear();
  return FLA_OK;
}

extern "C" FLA_API int fla_b200_kernel_timing_read(const char* kernel_name, float* total_ms, int* launches) {
  if (!kernel_name || !total_ms || !launches) return FLA_ERR_NULL;
  std::lock_guard<std::mutex> lk(fla::g_mu);
  *total_ms = 0.f;
  *launches = 0;
  auto it = fla::g_records.find(kernel_name);
  if (it == fla::g_records.end()) return FLA_OK;
  for (auto& ev : it->second.events) {
    if (cudaEventSynchronize(ev.second) != cudaSuccess) return FLA_ERR_CUDA;
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, ev.first, ev.second) != cudaSuccess) return FLA_ERR_CUDA;
    *total_ms += ms;
    *launches += 1;
  }
  return FLA_OK;
}
