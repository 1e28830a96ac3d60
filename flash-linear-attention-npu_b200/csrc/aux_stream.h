// A cached second stream per (device, caller stream) with fork / join events, for entry points that launch their work as
// two halves: the chunk-parallel kernel of the first half then fills the SMs that the second half's scan (one CTA per SM,
// more chains than SMs) leaves idle.  Streams and events are created on first use and never destroyed.
#pragma once
#include <cuda_runtime.h>
#include <mutex>

namespace fla {

struct AuxStream {
  cudaStream_t user = nullptr, s = nullptr;   // s: high priority, non-blocking
  cudaEvent_t fork = nullptr, join = nullptr;
  std::mutex mu;                              // held while a caller records / waits on the two events
};

int sm_count(int dev);
// nullptr when `user` is being captured, when eight caller streams of the device already have one, or when creation failed
AuxStream* aux_stream_for(int dev, cudaStream_t user);

}  // namespace fla
