#include "fb/gbdt.h"
namespace fb {
void FreeDeviceDataset(DeviceDataset*) {}
DeviceEngine* CreateDeviceEngine(const Config&, const Dataset*, const ObjectiveFunction*, int) { Log::Fatal("no cuda"); }
bool CudaAvailable() { return false; }
void DeviceBinDataset(Dataset*, const void*, int, int32_t, int32_t, bool, bool) { Log::Fatal("no cuda"); }
void DevicePredict(const GBDT*, const void*, int, int32_t, int32_t, bool, int, int, int, float*) { Log::Fatal("no cuda"); }
}
