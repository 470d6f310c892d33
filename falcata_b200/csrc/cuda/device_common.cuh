// Common device-side plumbing: error checks that raise (never abort), owned device buffers,
// a launch counter, bounded cross-rank waits and the descriptor structs shared by the kernels.
//
// Parity: include/Falcata/cuda/cuda_utils.hu (CUDASUCCESS_OR_FATAL L62-68, CUDAVector L181-333,
// allocation with sizes in the out-of-memory message L85-105).
#pragma once
#include <cuda_runtime.h>

#include <atomic>
#include <cstdint>
#include <string>
#include <vector>

#include "fb/common.h"
#include "fb/dataset.h"
#include "fb/kinds.h"
#include "fb/split_math.h"

namespace fb {

#define FB_CUDA(call)                                                                                          \
  do {                                                                                                         \
    cudaError_t _e = (call);                                                                                   \
    if (_e != cudaSuccess) ::fb::Log::Fatal("CUDA error %s (%s) at %s:%d", cudaGetErrorName(_e), cudaGetErrorString(_e), __FILE__, __LINE__); \
  } while (0)

// Number of kernels launched by this library in this process (reported by bench.py).
inline std::atomic<int64_t>& LaunchCounter() { static std::atomic<int64_t> c{0}; return c; }
#define FB_LAUNCHED() (::fb::LaunchCounter().fetch_add(1, std::memory_order_relaxed))
// FALCATA_DEBUG_SYNC=1 (or FALCATA_DEBUG=sync) serialises the device work: every launcher waits for its kernel and reports an error at the
// launch site (file:line of the launcher) instead of at the next synchronisation point of the training loop.
inline bool DebugSyncLaunches() { static const bool v = getenv("FALCATA_DEBUG_SYNC") != nullptr || DebugFlags::Get().sync; return v; }
#define FB_KERNEL_CHECK() do { FB_CUDA(cudaGetLastError()); if (::fb::DebugSyncLaunches()) FB_CUDA(cudaDeviceSynchronize()); } while (0)

template <typename T>
class DevBuf {
 public:
  DevBuf() {}
  ~DevBuf() { Free(); }
  DevBuf(const DevBuf&) = delete;
  DevBuf& operator=(const DevBuf&) = delete;
  DevBuf(DevBuf&& o) noexcept : p_(o.p_), n_(o.n_), cap_(o.cap_) { o.p_ = nullptr; o.n_ = o.cap_ = 0; }
  DevBuf& operator=(DevBuf&& o) noexcept { if (this != &o) { Free(); p_ = o.p_; n_ = o.n_; cap_ = o.cap_; o.p_ = nullptr; o.n_ = o.cap_ = 0; } return *this; }
  void Alloc(size_t n) {
    if (n <= cap_) { n_ = n; return; }
    Free();
    cudaError_t e = cudaMalloc(&p_, std::max<size_t>(n, 1) * sizeof(T));
    if (e != cudaSuccess) {
      size_t fr = 0, tot = 0; cudaMemGetInfo(&fr, &tot);
      Log::Fatal("Out of device memory: tried to allocate %.2f MB (free %.2f MB of %.2f MB): %s", n * sizeof(T) / 1048576.0, fr / 1048576.0, tot / 1048576.0, cudaGetErrorString(e));
    }
    n_ = cap_ = n;
  }
  void Free() { if (p_ != nullptr) { cudaFree(p_); p_ = nullptr; } n_ = cap_ = 0; }
  void Zero(cudaStream_t s) { if (n_) FB_CUDA(cudaMemsetAsync(p_, 0, n_ * sizeof(T), s)); }
  void Upload(const T* h, size_t n, cudaStream_t s) { Alloc(n); if (n) FB_CUDA(cudaMemcpyAsync(p_, h, n * sizeof(T), cudaMemcpyHostToDevice, s)); }
  void Upload(const std::vector<T>& v, cudaStream_t s) { Upload(v.data(), v.size(), s); }
  void Download(T* h, size_t n, cudaStream_t s) const { if (n) FB_CUDA(cudaMemcpyAsync(h, p_, n * sizeof(T), cudaMemcpyDeviceToHost, s)); }
  T* get() const { return p_; }
  size_t size() const { return n_; }
 private:
  T* p_ = nullptr; size_t n_ = 0, cap_ = 0;
};

template <typename T>
class PinnedBuf {
 public:
  ~PinnedBuf() { if (p_) cudaFreeHost(p_); }
  void Alloc(size_t n) { if (n <= cap_) { n_ = n; return; } if (p_) cudaFreeHost(p_); FB_CUDA(cudaMallocHost(&p_, std::max<size_t>(n, 1) * sizeof(T))); n_ = cap_ = n; }
  T* get() const { return p_; }
  size_t size() const { return n_; }
  T& operator[](size_t i) { return p_[i]; }
 private:
  T* p_ = nullptr; size_t n_ = 0, cap_ = 0;
};

// --------------------------------------------------------------- layouts ----
// Binned rows on the device: row-major bytes, one byte per feature group, `row_stride` bytes per
// row (a multiple of 16). When `gh_in_row` the last 4 bytes of each row hold the packed quantized
// gradient word of the current tree, so one 32-byte sector fetch serves bins and gradients.
struct DeviceDataset {
  int device = 0;
  data_size_t num_data = 0;
  int num_groups = 0;
  int row_stride = 0;
  int gh_offset = -1;
  DevBuf<uint8_t> rows;
  DevBuf<uint8_t> cols;        // optional column-major copy [num_groups x num_data]: the row partition reads ONE column
  DevBuf<float> label, weight;
  DevBuf<int> query_boundaries;
  int num_queries = 0;
  DevBuf<FeatureMeta> feature_meta;
  DevBuf<int> group_bin_start;
};

// One histogram bin of the pool. Quantized: packed (int32 grad << 32) + uint32 hess in one 64-bit
// word so that one `red.add.u64` (local, peer or multimem) updates both. Full precision: double2.
typedef unsigned long long hist_q_t;
FB_HD inline long long HistQGrad(hist_q_t v) { return static_cast<long long>(v) >> 32; }   // hess part is non-negative: floor division recovers grad
FB_HD inline long long HistQHess(hist_q_t v) { return static_cast<long long>(v & 0xFFFFFFFFull); }
FB_HD inline hist_q_t HistQPack(long long g, long long h) { return (static_cast<unsigned long long>(g) << 32) + static_cast<unsigned long long>(h); }

// A feature partition of the construct kernel: the groups whose bins share one shared-memory tile.
struct HistPartition { int group_begin, group_end, bin_begin, bin_count; };

// One construct task of a level: build the histogram of rows idx[begin, begin+count) into pool slot `slot`.
struct HistTask { int slot; int begin; int count; int buffer; int block_begin; int num_blocks; int pad0, pad1; };

// One split of a level as the partition kernels need it.
struct PartSplit {
  int leaf;            // leaf being split (left child keeps the id)
  int right_leaf;      // id of the new leaf
  int begin, count;    // window of the parent
  int buffer;          // index buffer (0/1) the window currently lives in
  int group;           // byte column of the split feature
  int bundled, group_offset, num_bin, most_freq_bin;
  int threshold, default_left, missing_type, default_bin;
  int is_categorical;
  uint32_t cat_bitset[8];
  int chunk_begin;     // first partition chunk of this split in the flat chunk grid
  int num_chunks;
  int owner;           // feature-parallel: rank that owns the split feature and broadcasts the bitmap
  int pad_[2];         // keeps sizeof a multiple of 16: arrays of different record types share one upload blob
};
static_assert(sizeof(PartSplit) % 16 == 0, "level blob records must keep 16-byte alignment");

// Per-leaf device record (windows + totals) that the level kernels read and update.
struct LeafInfo {
  int begin, count, buffer, depth;
  int hist_slot;
  int num_data_global;         // exact rows of the leaf over all ranks
  double sum_g, sum_h;         // real-valued totals
  long long sum_gi, sum_hi;    // integer totals (quantized)
  double output;
  double min_c, max_c;         // monotone range of the output (-inf, +inf when unconstrained)
  double pkey[4];              // leaf-wise growth: the parent's order key (see LeafwiseChildKey), +inf padded
};

// Bounded spin on a flag written by a peer rank. Returns false when the budget ran out; callers
// then record kStatusWaitTimeout and skip their work — the kernel always terminates.
__device__ inline bool WaitFlagGE(const volatile unsigned int* flag, unsigned int expected, unsigned long long max_spins) {
  for (unsigned long long i = 0; i < max_spins; ++i) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (static_cast<int>(v - expected) >= 0) return true;
    __nanosleep(64);
  }
  return false;
}

// Flag store that follows an explicit system-scope fence: the fence orders the data, so the stores to the
// individual peers need no ordering among themselves and go out back to back (a release store per peer would
// wait for the previous one's round trip).
__device__ inline void StoreFlagAfterFence(unsigned int* flag, unsigned int value) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(value) : "memory");
}

__device__ inline void StoreFlagRelease(unsigned int* flag, unsigned int value) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(value) : "memory");
}

}  // namespace fb
