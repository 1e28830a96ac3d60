#include "aux_stream.h"

namespace fla {
namespace {
constexpr int kAuxPerDevice = 8;
std::mutex g_aux_mu;
AuxStream g_aux[64][kAuxPerDevice];
int g_aux_used[64] = {};
int g_sm_count[64] = {};
}  // namespace

int sm_count(int dev) {
  std::lock_guard<std::mutex> lk(g_aux_mu);
  if (!g_sm_count[dev] && cudaDeviceGetAttribute(&g_sm_count[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) g_sm_count[dev] = 1 << 30;
  return g_sm_count[dev];
}

AuxStream* aux_stream_for(int dev, cudaStream_t user) {
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(user, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) return nullptr;
  std::lock_guard<std::mutex> lk(g_aux_mu);
  for (int i = 0; i < g_aux_used[dev]; ++i)
    if (g_aux[dev][i].user == user) return g_aux[dev][i].s ? &g_aux[dev][i] : nullptr;
  if (g_aux_used[dev] == kAuxPerDevice) return nullptr;
  AuxStream& a = g_aux[dev][g_aux_used[dev]++];
  a.user = user;
  int lo = 0, hi = 0;
  cudaDeviceGetStreamPriorityRange(&lo, &hi);
  if (cudaStreamCreateWithPriority(&a.s, cudaStreamNonBlocking, hi) != cudaSuccess ||
      cudaEventCreateWithFlags(&a.fork, cudaEventDisableTiming) != cudaSuccess ||
      cudaEventCreateWithFlags(&a.join, cudaEventDisableTiming) != cudaSuccess) {
    a.s = nullptr;   // remembered as unavailable: the single-stream path is used
    return nullptr;
  }
  return &a;
}

}  // namespace fla
