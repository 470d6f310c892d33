// Symmetric heap implementation: allocation, IPC handle exchange, small in-kernel all-reduce.
#include "fabric.h"

#include "fb/c_api.h"

namespace fb {

namespace {
constexpr size_t kFlagRegion = 64 * 1024;     // flag slots (128 B each) at the start of the heap
constexpr size_t kArSlot = 1024;              // bytes one rank contributes to a small all-reduce

__global__ void FabricAllReduceKernel(FabricView v, int op, const void* src, void* dst, int count, size_t data_off, size_t flag_off, unsigned int epoch) {
  const int esz = op == kFabricMaxF32 ? 4 : 8;
  const int words = count * esz / 4;
  const int buf = epoch & 1u;
  const unsigned int* s32 = static_cast<const unsigned int*>(src);
  for (int r = 0; r < v.world; ++r) {
    unsigned int* d = reinterpret_cast<unsigned int*>(v.base[r] + data_off + (static_cast<size_t>(buf) * v.world + v.rank) * kArSlot);
    for (int i = threadIdx.x; i < words; i += blockDim.x) d[i] = s32[i];
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    for (int r = 0; r < v.world; ++r) StoreFlagAfterFence(reinterpret_cast<unsigned int*>(v.base[r] + flag_off) + v.rank, epoch);
  }
  FabricWait w; w.world = v.world; w.flags = reinterpret_cast<const unsigned int*>(v.base[v.rank] + flag_off); w.epoch = epoch; w.max_spins = v.max_spins; w.status = v.status;
  FabricWaitAll(w);
  const char* local = v.base[v.rank] + data_off + static_cast<size_t>(buf) * v.world * kArSlot;
  for (int i = threadIdx.x; i < count; i += blockDim.x) {
    if (op == kFabricMaxF32) {
      float m = 0.f; for (int r = 0; r < v.world; ++r) m = fmaxf(m, reinterpret_cast<const volatile float*>(local + r * kArSlot)[i]);
      static_cast<float*>(dst)[i] = m;
    } else if (op == kFabricSumI64) {
      long long a = 0; for (int r = 0; r < v.world; ++r) a += reinterpret_cast<const volatile long long*>(local + r * kArSlot)[i];
      static_cast<long long*>(dst)[i] = a;
    } else {
      double a = 0; for (int r = 0; r < v.world; ++r) a += reinterpret_cast<const volatile double*>(local + r * kArSlot)[i];   // fixed rank order
      static_cast<double*>(dst)[i] = a;
    }
  }
}
}  // namespace

Fabric& Fabric::Get() { static Fabric f; return f; }

void Fabric::Create(int rank, int world, size_t bytes, char out_handle[64]) {
  if (world < 1 || world > kMaxRanks) Log::Fatal("The symmetric heap supports 1..%d ranks (got %d)", kMaxRanks, world);
  Destroy();
  rank_ = rank; world_ = world; guards_.clear(); fixed_guards_ = 0;
  bytes_ = ((bytes + kFlagRegion + 2 * kMaxRanks * kArSlot + 4095) / 4096) * 4096 + (1 << 20);
  void* p = nullptr;
  FB_CUDA(cudaMalloc(&p, bytes_));
  FB_CUDA(cudaMemset(p, 0, bytes_));
  base_[rank] = static_cast<char*>(p);
  FB_CUDA(cudaMalloc(&counters_, 16 * sizeof(unsigned int)));
  FB_CUDA(cudaMemset(counters_, 0, 16 * sizeof(unsigned int)));
  status_ = counters_ + 15;
  flag_bytes_ = kFlagRegion;
  cudaIpcMemHandle_t h;
  FB_CUDA(cudaIpcGetMemHandle(&h, p));
  static_assert(sizeof(h) == 64, "IPC handle size");
  memcpy(out_handle, &h, 64);
  FB_CUDA(cudaDeviceSynchronize());
}

void Fabric::Connect(const char* handles) {
  for (int r = 0; r < world_; ++r) {
    if (r == rank_) continue;
    cudaIpcMemHandle_t h; memcpy(&h, handles + 64 * r, 64);
    void* p = nullptr;
    FB_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    base_[r] = static_cast<char*>(p);
  }
  connected_ = true;
  flag_cursor_ = 0; cursor_ = flag_bytes_;
  // the small all-reduce owns one flag slot and a double-buffered data area for the heap's lifetime
  ar_flag_off_ = NewFlagSlot();
  ar_data_off_ = Alloc(2 * kMaxRanks * kArSlot);
  flag_bytes_ = cursor_;   // Reset() keeps the all-reduce area
  fixed_flag_cursor_ = flag_cursor_;
  fixed_guards_ = guards_.size();
}

void Fabric::Destroy() {
  if (base_[rank_] == nullptr) return;
  cudaDeviceSynchronize();
  for (int r = 0; r < world_; ++r) { if (r != rank_ && base_[r] != nullptr) cudaIpcCloseMemHandle(base_[r]); }
  cudaFree(base_[rank_]);
  if (counters_) cudaFree(counters_);
  for (int r = 0; r < kMaxRanks; ++r) base_[r] = nullptr;
  counters_ = nullptr; status_ = nullptr; connected_ = false; world_ = 1; rank_ = 0; bytes_ = 0;
}

size_t Fabric::Alloc(size_t bytes, size_t align) {
  cursor_ = (cursor_ + align - 1) / align * align;
  const size_t off = cursor_;
  cursor_ += bytes;
  const bool guard = DebugFlags::Get().canary;
  if (guard) { cursor_ = (cursor_ + 15) / 16 * 16; guards_.push_back(cursor_); cursor_ += kGuardBytes; }
  if (cursor_ > bytes_) Log::Fatal("Symmetric heap exhausted: need %zu bytes, have %zu (create the fabric with a larger heap)", cursor_, bytes_);
  if (guard) FB_CUDA(cudaMemset(base_[rank_] + guards_.back(), 0xC5, kGuardBytes));
  return off;
}

int Fabric::CheckCanaries(cudaStream_t s) const {
  if (guards_.empty()) return -1;
  FB_CUDA(cudaStreamSynchronize(s));
  std::vector<unsigned char> h(kGuardBytes);
  for (size_t g = 0; g < guards_.size(); ++g) {
    FB_CUDA(cudaMemcpy(h.data(), base_[rank_] + guards_[g], kGuardBytes, cudaMemcpyDeviceToHost));
    for (size_t i = 0; i < kGuardBytes; ++i) if (h[i] != 0xC5) return static_cast<int>(g);
  }
  return -1;
}

size_t Fabric::NewFlagSlot() {
  const size_t off = flag_cursor_;
  flag_cursor_ += 128;
  if (flag_cursor_ > kFlagRegion) Log::Fatal("Out of flag slots in the symmetric heap");
  return off;
}

FabricView Fabric::View() const {
  FabricView v; v.rank = rank_; v.world = world_; v.max_spins = max_spins_; v.status = status_;
  for (int r = 0; r < kMaxRanks; ++r) v.base[r] = base_[r];
  return v;
}

int Fabric::CheckStatus(cudaStream_t s) {
  unsigned int h = 0;
  FB_CUDA(cudaMemcpyAsync(&h, status_, sizeof(h), cudaMemcpyDeviceToHost, s));
  FB_CUDA(cudaStreamSynchronize(s));
  if (h != 0) FB_CUDA(cudaMemsetAsync(status_, 0, sizeof(unsigned int), s));
  return static_cast<int>(h);
}

void Fabric::AllReduce(FabricOp op, const void* src, void* dst, int count, cudaStream_t s) {
  const int esz = op == kFabricMaxF32 ? 4 : 8;
  if (static_cast<size_t>(count) * esz > kArSlot) Log::Fatal("Small all-reduce payload too large (%d elements)", count);
  FabricAllReduceKernel<<<1, 128, 0, s>>>(View(), static_cast<int>(op), src, dst, count, ar_data_off_, ar_flag_off_, NextEpoch());
  FB_LAUNCHED(); FB_KERNEL_CHECK();
}

}  // namespace fb

using namespace fb;

namespace { thread_local std::string g_fabric_error; }

extern "C" {

const char* FB_FabricLastError() { return g_fabric_error.c_str(); }

// Allocate this rank's symmetric heap on the current device; `out_handle` receives 64 bytes to all-gather.
int FB_FabricCreate(int rank, int world, int64_t heap_bytes, char* out_handle) {
  try { Fabric::Get().Create(rank, world, static_cast<size_t>(heap_bytes), out_handle); } catch (std::exception& e) { g_fabric_error = e.what(); return -1; }
  return 0;
}
// Map every peer's heap; `handles` is world x 64 bytes ordered by rank.
int FB_FabricConnect(const char* handles) {
  try { Fabric::Get().Connect(handles); } catch (std::exception& e) { g_fabric_error = e.what(); return -1; }
  return 0;
}
int FB_FabricDestroy() {
  try { Fabric::Get().Destroy(); } catch (std::exception& e) { g_fabric_error = e.what(); return -1; }
  return 0;
}
// Test hooks of the debug guards: carve a region, overwrite heap bytes from the host, check the guards.
int FB_FabricDebugAlloc(int64_t bytes, int64_t* out_offset) {
  try { *out_offset = static_cast<int64_t>(Fabric::Get().Alloc(static_cast<size_t>(bytes))); } catch (std::exception& e) { g_fabric_error = e.what(); return -1; }
  return 0;
}
int FB_FabricDebugFill(int64_t offset, int64_t bytes, int value) {
  try { FB_CUDA(cudaMemset(Fabric::Get().Local<char>(static_cast<size_t>(offset)), value, static_cast<size_t>(bytes))); FB_CUDA(cudaDeviceSynchronize()); }
  catch (std::exception& e) { g_fabric_error = e.what(); return -1; }
  return 0;
}
int FB_FabricCheckCanaries(int* out_broken_region) {
  try { *out_broken_region = Fabric::Get().CheckCanaries(0); } catch (std::exception& e) { g_fabric_error = e.what(); return -1; }
  return 0;
}
int FB_FabricSetMaxSpins(int64_t spins) { Fabric::Get().set_max_spins(static_cast<unsigned long long>(spins)); return 0; }
// Test hook: all-reduce `count` elements of a device vector (op: 0 max f32, 1 sum i64, 2 sum f64); returns the status word.
int FB_FabricAllReduce(int op, const void* src, void* dst, int count, int* out_status) {
  try {
    Fabric::Get().AllReduce(static_cast<FabricOp>(op), src, dst, count, 0);
    *out_status = Fabric::Get().CheckStatus(0);
  } catch (std::exception& e) { g_fabric_error = e.what(); return -1; }
  return 0;
}

}  // extern "C"
