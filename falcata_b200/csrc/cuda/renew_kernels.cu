// Leaf renewal by a percentile of the residuals (L1: the median; quantile: alpha), on the device: the residuals
// label - score of every leaf's rows are written leaf by leaf (the final partition keeps a leaf's rows in one window
// of an index buffer), sorted per leaf with a segmented sort, and a small kernel reads the order statistics.
// Unweighted data only; weighted percentiles stay on the host.
// Parity: src/objective/cuda/cuda_regression_objective.cu:L183, L402 (leaf renewal of L1 / quantile on the device),
// src/objective/regression_objective.hpp (PercentileFun: linear interpolation between order statistics).
#include <cub/device/device_segmented_sort.cuh>

#include "engine.h"

namespace fb {

namespace {

__global__ void LeafResidualKernel(const LeafInfo* __restrict__ leaves, const int* __restrict__ out_begin, const int* __restrict__ idx0, const int* __restrict__ idx1,
                                   const float* __restrict__ score, const float* __restrict__ label, double* __restrict__ residual) {
  const int l = blockIdx.y;
  const int cnt = leaves[l].count;
  const int* window = (leaves[l].buffer ? idx1 : idx0) + leaves[l].begin;
  const int base = out_begin[l];
  for (int k = blockIdx.x * blockDim.x + threadIdx.x; k < cnt; k += gridDim.x * blockDim.x) {
    const int row = window[k];
    residual[base + k] = static_cast<double>(label[row]) - static_cast<double>(score[row]);
  }
}

__global__ void LeafPercentileKernel(const double* __restrict__ sorted, const int* __restrict__ out_begin, int num_leaves, double alpha, double* __restrict__ out) {
  const int l = blockIdx.x * blockDim.x + threadIdx.x;
  if (l >= num_leaves) return;
  const int b = out_begin[l], cnt = out_begin[l + 1] - b;
  if (cnt <= 0) { out[l] = 0.0; return; }
  if (cnt == 1) { out[l] = sorted[b]; return; }
  const double pos = alpha * (cnt - 1);
  const int lo = static_cast<int>(floor(pos)); const int hi = min(cnt - 1, lo + 1);
  const double frac = pos - lo;
  out[l] = sorted[b + lo] * (1.0 - frac) + sorted[b + hi] * frac;
}

}  // namespace

// out_host[l] = the alpha-percentile of (label - score) over leaf l's rows (0 for an empty leaf). `leaves_host` is the
// downloaded copy of `leaves_dev`. Scratch buffers grow on demand and are kept by the caller.
void DeviceRenewPercentile(const LeafInfo* leaves_dev, const LeafInfo* leaves_host, int num_leaves, const int* idx0, const int* idx1, const float* score,
                           const float* label, int n, double alpha, DevBuf<double>* keys_in, DevBuf<double>* keys_out, DevBuf<int>* offsets, DevBuf<double>* out_dev,
                           DevBuf<char>* temp, double* out_host, cudaStream_t s) {
  std::vector<int> begin(num_leaves + 1, 0);
  int max_count = 0;
  for (int l = 0; l < num_leaves; ++l) { const int c = std::max(0, leaves_host[l].count); begin[l + 1] = begin[l] + c; max_count = std::max(max_count, c); }
  const int total = begin[num_leaves];
  if (total > n) Log::Fatal("Leaf windows cover %d rows of %d", total, n);
  if (keys_in->size() < static_cast<size_t>(std::max(1, total))) { keys_in->Alloc(std::max(1, n)); keys_out->Alloc(std::max(1, n)); }
  if (offsets->size() < static_cast<size_t>(num_leaves + 1)) offsets->Alloc(num_leaves + 1);
  if (out_dev->size() < static_cast<size_t>(num_leaves)) out_dev->Alloc(num_leaves);
  FB_CUDA(cudaMemcpyAsync(offsets->get(), begin.data(), sizeof(int) * (num_leaves + 1), cudaMemcpyHostToDevice, s));
  if (total > 0) {
    const int threads = 256;
    const int bx = std::max(1, std::min(64, (max_count + threads * 4 - 1) / (threads * 4)));
    LeafResidualKernel<<<dim3(bx, num_leaves), threads, 0, s>>>(leaves_dev, offsets->get(), idx0, idx1, score, label, keys_in->get());
    FB_LAUNCHED(); FB_KERNEL_CHECK();
    size_t bytes = 0;
    FB_CUDA(cub::DeviceSegmentedSort::SortKeys(nullptr, bytes, keys_in->get(), keys_out->get(), total, num_leaves, offsets->get(), offsets->get() + 1, s));
    if (temp->size() < bytes + 16) temp->Alloc(bytes + 16);
    FB_CUDA(cub::DeviceSegmentedSort::SortKeys(temp->get(), bytes, keys_in->get(), keys_out->get(), total, num_leaves, offsets->get(), offsets->get() + 1, s));
    FB_LAUNCHED();
  }
  LeafPercentileKernel<<<(num_leaves + 127) / 128, 128, 0, s>>>(keys_out->get(), offsets->get(), num_leaves, alpha, out_dev->get());
  FB_LAUNCHED(); FB_KERNEL_CHECK();
  FB_CUDA(cudaMemcpyAsync(out_host, out_dev->get(), sizeof(double) * num_leaves, cudaMemcpyDeviceToHost, s));
  FB_CUDA(cudaStreamSynchronize(s));   // `begin` and `out_host` are host memory of this call
}

}  // namespace fb
