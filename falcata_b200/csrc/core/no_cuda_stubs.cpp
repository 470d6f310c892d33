// Host-only builds (sanitizer runs of the CPU tests): the entry points of the CUDA module, answering "no device".
// Compiled to nothing unless FB_NO_CUDA is defined.
#ifdef FB_NO_CUDA
#include "fb/gbdt.h"

namespace fb {
void FreeDeviceDataset(DeviceDataset*) {}
DeviceEngine* CreateDeviceEngine(const Config&, const Dataset*, const ObjectiveFunction*, int) { Log::Fatal("This build has no CUDA module"); return nullptr; }
bool CudaAvailable() { return false; }
void DeviceBinDataset(Dataset*, const void*, int, int32_t, int32_t, bool, bool) { Log::Fatal("This build has no CUDA module"); }
void DeviceGatherRows(const void*, int, int32_t, int32_t, bool, const int32_t*, int32_t, std::vector<char>*) { Log::Fatal("This build has no CUDA module"); }
void DeviceBinDatasetChunk(Dataset*, const void*, int, int32_t, int32_t, bool, bool, int32_t, int32_t) { Log::Fatal("This build has no CUDA module"); }
void DevicePredict(const GBDT*, const void*, int, int32_t, int32_t, bool, int, int, int, float*) { Log::Fatal("This build has no CUDA module"); }
}  // namespace fb

extern "C" int FB_OpBernoulliRowsHost(int n, long long global_offset, unsigned int seed, double fraction, int* out_idx, int* out_count) {
  int c = 0;
  for (int i = 0; i < n; ++i) {
    const float u = fb::U01From24(fb::Philox4x32_10(static_cast<uint32_t>(static_cast<unsigned long long>(global_offset) + static_cast<unsigned long long>(i)), 0x5A3Du, 0xBA660000u, 0u, seed, 0x9876u).v[0]);
    if (static_cast<double>(u) < fraction) out_idx[c++] = i;
  }
  *out_count = c;
  return 0;
}
#endif
