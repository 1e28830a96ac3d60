// Optional per-kernel CUDA-event timing, off by default.  When enabled through
// fla_b200_kernel_timing_enable(1) every kernel launch made by the library is bracketed by two events
// on the launching stream; fla_b200_kernel_timing_read() synchronises those events and returns the
// accumulated device time and launch count for one kernel name.  Used by the benchmark to report the
// duration of the dominant kernel without a profiler attached.
#pragma once
#include <cuda_runtime.h>

namespace fla {

bool kernel_timing_enabled();
void kernel_timing_begin(const char* name, cudaStream_t s);
void kernel_timing_end(const char* name, cudaStream_t s);

struct KernelTimer {
  const char* name;
  cudaStream_t s;
  bool on;
  KernelTimer(const char* n, cudaStream_t st) : name(n), s(st), on(kernel_timing_enabled()) {
    if (on) kernel_timing_begin(name, s);
  }
  ~KernelTimer() {
    if (on) kernel_timing_end(name, s);
  }
};

}  // namespace fla
