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

// The operators whose kernels wait on barriers keep a status word at the head of their workspace (cleared at launch,
// set to FLA_ERR_TIMEOUT by a wait that ran out).  This reads it back: it waits for `stream`, so call it only where a
// synchronisation is acceptable (a debug mode, the end of a step, a failing test).
extern "C" FLA_API int fla_b200_read_status_word(const void* workspace, void* stream, int32_t* status_out) {
  if (!workspace || !status_out) return FLA_ERR_NULL;
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  int32_t word = 0;
  if (cudaMemcpyAsync(&word, workspace, sizeof(word), cudaMemcpyDeviceToHost, cs) != cudaSuccess) return FLA_ERR_CUDA;
  if (cudaStreamSynchronize(cs) != cudaSuccess) return FLA_ERR_CUDA;
  *status_out = word;
  return FLA_OK;
}
