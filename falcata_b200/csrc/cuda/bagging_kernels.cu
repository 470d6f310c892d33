// K11: bagging on the device. Flags (Philox keyed on the global row id) -> per-chunk counts ->
// exclusive scan -> stable scatter of the in-bag row ids. The draw is the one the host learner makes
// (GBDT::Bagging), so a bagged model does not depend on where it is trained or on the rank count.
// Parity: src/boosting/cuda/cuda_bagging.cu:L43-114 (flags + scan + scatter), src/boosting/bagging.hpp.
#include "kernels.cuh"

#include <cub/device/device_radix_sort.cuh>

namespace fb {

namespace {

constexpr int kBagChunk = 1024;

__device__ inline bool BagDraw(const BagArgs& a, int i) {
  double frac = a.fraction;
  uint32_t c0, c3;
  if (a.by_query) {
    // the query that holds row i: last boundary <= i
    int lo = 0, hi = a.num_queries - 1;
    while (lo < hi) { const int m = (lo + hi + 1) >> 1; if (a.query_boundaries[m] <= i) lo = m; else hi = m - 1; }
    c0 = static_cast<uint32_t>(a.global_query_offset + static_cast<unsigned long long>(lo)); c3 = 1u;
  } else {
    c0 = static_cast<uint32_t>(a.global_row_offset + static_cast<unsigned long long>(i)); c3 = 0u;
    if (a.balanced) frac = a.label[i] > 0.f ? a.pos_fraction : a.neg_fraction;
  }
  const float u = U01From24(Philox4x32_10(c0, a.round, 0xBA660000u, c3, a.seed, 0x9876u).v[0]);
  return static_cast<double>(u) < frac;
}

__global__ void __launch_bounds__(kBagChunk) BagFlagsKernel(BagArgs a) {
  const int i = blockIdx.x * kBagChunk + threadIdx.x;
  const int in = (i < a.n && BagDraw(a, i)) ? 1 : 0;
  if (i < a.n) a.mask[i] = static_cast<uint8_t>(in);
  const int cnt = __syncthreads_count(in);
  if (threadIdx.x == 0) a.chunk_count[blockIdx.x] = cnt;
}

// One block: chunk counts -> exclusive offsets (in place), total -> bag_count.
__global__ void __launch_bounds__(1024) BagScanKernel(int* chunk_count, int num_chunks, int* bag_count) {
  __shared__ int warp_sum[32];
  __shared__ int carry;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  for (int base = 0; base < num_chunks; base += 1024) {
    const int k = base + threadIdx.x;
    const int v = k < num_chunks ? chunk_count[k] : 0;
    int x = v;
    for (int o = 1; o < 32; o <<= 1) { const int y = __shfl_up_sync(0xffffffffu, x, o); if (lane >= o) x += y; }
    if (lane == 31) warp_sum[w] = x;
    __syncthreads();
    if (w == 0) {
      int s = warp_sum[lane];
      for (int o = 1; o < 32; o <<= 1) { const int y = __shfl_up_sync(0xffffffffu, s, o); if (lane >= o) s += y; }
      warp_sum[lane] = s;
    }
    __syncthreads();
    const int before = carry + (w > 0 ? warp_sum[w - 1] : 0) + x - v;
    if (k < num_chunks) chunk_count[k] = before;
    __syncthreads();
    if (threadIdx.x == 1023) carry = before + v;
    __syncthreads();
  }
  if (threadIdx.x == 0) *bag_count = carry;
}

__global__ void __launch_bounds__(kBagChunk) BagScatterKernel(BagArgs a) {
  __shared__ int warp_cnt[32];
  const int i = blockIdx.x * kBagChunk + threadIdx.x;
  const int in = (i < a.n && a.mask[i] != 0) ? 1 : 0;
  const unsigned int b = __ballot_sync(0xffffffffu, in);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  if (lane == 0) warp_cnt[w] = __popc(b);
  __syncthreads();
  if (w == 0) {
    const int c = warp_cnt[lane];
    int s = c;
    for (int o = 1; o < 32; o <<= 1) { const int y = __shfl_up_sync(0xffffffffu, s, o); if (lane >= o) s += y; }
    warp_cnt[lane] = s - c;   // exclusive
  }
  __syncthreads();
  if (in) a.bag_idx[a.chunk_count[blockIdx.x] + warp_cnt[w] + __popc(b & ((1u << lane) - 1u))] = i;
}

__global__ void GossMagnitudeKernel(GossArgs a) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= a.n) return;
  float m = 0.f;
  for (int k = 0; k < a.num_class; ++k) m += fabsf(a.grad[static_cast<size_t>(k) * a.n + i] * a.hess[static_cast<size_t>(k) * a.n + i]);
  a.mag[i] = m;
}

__global__ void __launch_bounds__(kBagChunk) GossFlagsKernel(GossArgs a) {
  const int i = blockIdx.x * kBagChunk + threadIdx.x;
  int in = 0;
  if (i < a.n) {
    const float thr = a.sorted[a.top_k - 1];   // the top_k-th largest magnitude
    if (a.mag[i] >= thr) in = 1;
    else {
      const float u = U01From24(Philox4x32_10(static_cast<uint32_t>(a.global_row_offset + static_cast<unsigned long long>(i)), a.iter, 0x60550000u, 0u, a.seed, 0x1234u).v[0]);
      if (static_cast<double>(u) < a.prob) {
        in = 1;
        for (int k = 0; k < a.num_class; ++k) { a.grad[static_cast<size_t>(k) * a.n + i] *= a.multiply; a.hess[static_cast<size_t>(k) * a.n + i] *= a.multiply; }
      }
    }
    a.mask[i] = static_cast<uint8_t>(in);
  }
  const int cnt = __syncthreads_count(in);
  if (threadIdx.x == 0) a.chunk_count[blockIdx.x] = cnt;
}

}  // namespace

size_t GossSortTempBytes(int n) {
  size_t bytes = 0;
  cub::DeviceRadixSort::SortKeysDescending(nullptr, bytes, static_cast<const float*>(nullptr), static_cast<float*>(nullptr), n);
  return bytes;
}

void LaunchGoss(const GossArgs& a, cudaStream_t s) {
  if (a.n <= 0) { FB_CUDA(cudaMemsetAsync(a.bag_count, 0, sizeof(int), s)); return; }
  GossMagnitudeKernel<<<(a.n + 255) / 256, 256, 0, s>>>(a); FB_LAUNCHED(); FB_KERNEL_CHECK();
  size_t bytes = a.sort_temp_bytes;
  FB_CUDA(cub::DeviceRadixSort::SortKeysDescending(a.sort_temp, bytes, a.mag, a.sorted, a.n, 0, 32, s)); FB_LAUNCHED();
  const int chunks = (a.n + kBagChunk - 1) / kBagChunk;
  GossFlagsKernel<<<chunks, kBagChunk, 0, s>>>(a); FB_LAUNCHED(); FB_KERNEL_CHECK();
  BagScanKernel<<<1, 1024, 0, s>>>(a.chunk_count, chunks, a.bag_count); FB_LAUNCHED(); FB_KERNEL_CHECK();
  BagArgs b = BagArgs(); b.n = a.n; b.mask = a.mask; b.bag_idx = a.bag_idx; b.chunk_count = a.chunk_count; b.bag_count = a.bag_count;
  BagScatterKernel<<<chunks, kBagChunk, 0, s>>>(b); FB_LAUNCHED(); FB_KERNEL_CHECK();
}

void LaunchBagging(const BagArgs& a, cudaStream_t s) {
  if (a.n <= 0) { FB_CUDA(cudaMemsetAsync(a.bag_count, 0, sizeof(int), s)); return; }
  const int chunks = (a.n + kBagChunk - 1) / kBagChunk;
  BagFlagsKernel<<<chunks, kBagChunk, 0, s>>>(a); FB_LAUNCHED(); FB_KERNEL_CHECK();
  BagScanKernel<<<1, 1024, 0, s>>>(a.chunk_count, chunks, a.bag_count); FB_LAUNCHED(); FB_KERNEL_CHECK();
  BagScatterKernel<<<chunks, kBagChunk, 0, s>>>(a); FB_LAUNCHED(); FB_KERNEL_CHECK();
}

}  // namespace fb
