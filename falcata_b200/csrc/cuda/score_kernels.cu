// K6 / K7 / K10: score update through the final partition, tree traversal on binned rows
// (validation sets, rollback), packed-forest traversal on raw feature rows (Booster.predict),
// output transforms and pointwise metrics.
// Parity: src/treelearner/cuda/cuda_data_partition.cu:L2112-2177 (leaf map + train score update),
// src/io/cuda/cuda_tree.cu:L455-566 (binned traversal), src/boosting/cuda/cuda_score_updater.cu:L13-29,
// src/metric/cuda/cuda_pointwise_metric.cu:L21; the raw-feature kernel replaces the cuML FIL route
// of python-package/falcata/basic.py:L5067-5163.
#include "kernels.cuh"

#include <cuda_fp16.h>

namespace fb {

namespace {

// grid (leaf, slice): every leaf's window is walked by gridDim.y blocks
__global__ void AddLeafOutputsKernel(const LeafInfo* __restrict__ leaves, const double* __restrict__ leaf_value, const int* __restrict__ idx0,
                                     const int* __restrict__ idx1, float* __restrict__ score) {
  const LeafInfo L = leaves[blockIdx.x];
  const float v = static_cast<float>(leaf_value[blockIdx.x]);
  const int* idx = (L.buffer ? idx1 : idx0) + L.begin;
  for (int p = blockIdx.y * blockDim.x + threadIdx.x; p < L.count; p += gridDim.y * blockDim.x) score[idx[p]] += v;
}

// Leaf-wise growth: bring every leaf's rows into index buffer 0 at the leaf's own positions. The leaves tile the row
// range by position, so afterwards the rows of ANY node of the tree are the contiguous range of buffer 0 that its
// leaves cover - which is what a pruned subtree needs to become one leaf again.
// Parity: src/treelearner/cuda/part.cu:L1846 (CollapseLeafWindowsKernel).
__global__ void CollapseLeafWindowsKernel(const LeafInfo* __restrict__ leaves, int* __restrict__ idx0, const int* __restrict__ idx1) {
  const LeafInfo L = leaves[blockIdx.x];
  if (L.buffer == 0) return;
  for (int p = blockIdx.y * blockDim.x + threadIdx.x; p < L.count; p += gridDim.y * blockDim.x) idx0[L.begin + p] = idx1[L.begin + p];
}

// The same update straight from the device's leaf records, enqueued behind the last level without waiting for the
// host: leaf value = record output x shrinkage (what the host tree holds after Shrink). It applies itself only when
// the controller reports the tree complete and split at least once; otherwise it does nothing and the host-side
// update runs after the read-back.
__global__ void AddLeafOutputsFromRecordsKernel(const LeafInfo* __restrict__ leaves, const LevelCtrl* __restrict__ ctrl, double shrinkage, int max_leaves,
                                                const int* __restrict__ idx0, const int* __restrict__ idx1, float* __restrict__ score, int decided_ahead) {
  const LevelCtrl c = *ctrl;
  // decided_ahead: the record was written by the tail of the last level's search and may already count splits that no
  // partition has applied yet (their leaf records do not exist): the tree is complete only when none are pending
  const bool complete = (c.done || c.num_leaves >= max_leaves || c.frontier_count == 0) && (!decided_ahead || c.num_splits == 0);
  if (!complete || c.num_leaves <= 1 || static_cast<int>(blockIdx.x) >= c.num_leaves) return;
  const LeafInfo L = leaves[blockIdx.x];
  const float v = static_cast<float>(L.output * shrinkage);
  const int* idx = (L.buffer ? idx1 : idx0) + L.begin;
  for (int p = blockIdx.y * blockDim.x + threadIdx.x; p < L.count; p += gridDim.y * blockDim.x) score[idx[p]] += v;
}

// K6r: per-leaf sums of the TRUE (unquantized) gradients over the final partition, for leaf renewal.
// grid (leaf, kRenewSlices): every slice walks a strided part of the leaf's window and reduces in a fixed
// order; the host adds the slices (and the ranks) in a fixed order too.
constexpr int kRenewSlices = 32;
__global__ void __launch_bounds__(256) LeafGradSumsKernel(const LeafInfo* __restrict__ leaves, const int* __restrict__ idx0, const int* __restrict__ idx1,
                                                          const float* __restrict__ grad, const float* __restrict__ hess, double* __restrict__ partial) {
  const LeafInfo L = leaves[blockIdx.x];
  const int* idx = (L.buffer ? idx1 : idx0) + L.begin;
  double g = 0, h = 0;
  for (int p = blockIdx.y * blockDim.x + threadIdx.x; p < L.count; p += gridDim.y * blockDim.x) { const int r = idx[p]; g += grad[r]; h += hess[r]; }
  __shared__ double sg[256], sh[256];
  sg[threadIdx.x] = g; sh[threadIdx.x] = h;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) { if (threadIdx.x < o) { sg[threadIdx.x] += sg[threadIdx.x + o]; sh[threadIdx.x] += sh[threadIdx.x + o]; } __syncthreads(); }
  if (threadIdx.x == 0) { partial[2 * (blockIdx.x * gridDim.y + blockIdx.y)] = sg[0]; partial[2 * (blockIdx.x * gridDim.y + blockIdx.y) + 1] = sh[0]; }
}

__global__ void AddConstantKernel(float* score, int n, float v) { const int i = blockIdx.x * blockDim.x + threadIdx.x; if (i < n) score[i] += v; }

__global__ void AddTreeBinnedKernel(DevTree t, const uint8_t* __restrict__ rows, int row_stride, int n, float scale, float* __restrict__ score) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  if (t.num_leaves <= 1) { score[i] += scale * t.leaf_value[0]; return; }
  const uint8_t* rp = rows + static_cast<size_t>(i) * row_stride;
  int node = 0;
  while (node >= 0) {
    int fb = rp[t.split_group[node]];
    if (t.bundled[node]) {
      const int rel = fb - t.group_offset[node];
      fb = (rel < 0 || rel >= t.num_bin[node] - 1) ? t.most_freq_bin[node] : (rel >= t.most_freq_bin[node] ? rel + 1 : rel);
    }
    const int dt = t.decision[node], mt = (dt >> 2) & 3;
    bool left;
    if (dt & 1) left = (t.cat_bits[node * 8 + ((fb >> 5) & 7)] >> (fb & 31)) & 1;   // categorical: set of bins
    else if ((mt == 1 && fb == t.default_bin[node]) || (mt == 2 && fb == t.nan_bin[node])) left = (dt & 2) != 0;
    else left = fb <= t.threshold_bin[node];
    node = left ? t.left[node] : t.right[node];
  }
  score[i] += scale * t.leaf_value[~node];
}

template <typename T> __device__ inline float LoadF(const T* p, size_t i) { return static_cast<float>(p[i]); }
template <> __device__ inline float LoadF<__half>(const __half* p, size_t i) { return __half2float(p[i]); }

// One thread per row; the packed forest is read through L1/L2 (all rows walk the same trees, so the
// nodes stay cache-resident) and the row's features are re-read from its own cache lines.
template <typename T>
__global__ void PredictRawKernel(const ForestNode* __restrict__ nodes, const unsigned int* __restrict__ cat_words, const int* __restrict__ tree_root, int num_trees, int num_class,
                                 const T* __restrict__ data, int nrow, int ncol, bool row_major, float* __restrict__ out, float inv_avg) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= nrow) return;
  for (int c = 0; c < num_class; ++c) {
    float acc = 0.f;
    for (int t = c; t < num_trees; t += num_class) {
      int n = tree_root[t];
      ForestNode nd = nodes[n];
      while (!(nd.flags & 8)) {
        float v = LoadF<T>(data, row_major ? static_cast<size_t>(i) * ncol + nd.feature : static_cast<size_t>(nd.feature) * nrow + i);
        const int mt = (nd.flags >> 1) & 3;
        bool left;
        if (nd.flags & 16) {
          // categorical: left iff the (integer) category is in the node's set; NaN and negatives go right
          left = false;
          if (!isnan(v)) {
            const int iv = static_cast<int>(v);
            const int off = __float_as_int(nd.threshold), nw = nd.flags >> 8;
            if (iv >= 0 && (iv >> 5) < nw) left = (cat_words[off + (iv >> 5)] >> (iv & 31)) & 1;
          }
          n = left ? nd.left : nd.right;
          nd = nodes[n];
          continue;
        }
        if (isnan(v) && mt != 2) v = 0.f;
        if ((mt == 1 && fabsf(v) <= 1e-35f) || (mt == 2 && isnan(v))) left = nd.flags & 1;
        else left = v <= nd.threshold;
        n = left ? nd.left : nd.right;
        nd = nodes[n];
      }
      acc += nd.threshold;
    }
    out[static_cast<size_t>(c) * nrow + i] = acc * inv_avg;
  }
}

__global__ void ConvertOutputKernel(int obj_kind, float sigmoid, float* out, int nrow, int num_class) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= nrow) return;
  switch (obj_kind) {
    case kObjBinary: case kObjXent: out[i] = 1.f / (1.f + expf(-sigmoid * out[i])); break;
    case kObjMulticlassOVA: for (int c = 0; c < num_class; ++c) out[static_cast<size_t>(c) * nrow + i] = 1.f / (1.f + expf(-sigmoid * out[static_cast<size_t>(c) * nrow + i])); break;
    case kObjMulticlass: {
      float mx = out[i]; for (int c = 1; c < num_class; ++c) mx = fmaxf(mx, out[static_cast<size_t>(c) * nrow + i]);
      float sum = 0.f; for (int c = 0; c < num_class; ++c) sum += expf(out[static_cast<size_t>(c) * nrow + i] - mx);
      for (int c = 0; c < num_class; ++c) out[static_cast<size_t>(c) * nrow + i] = expf(out[static_cast<size_t>(c) * nrow + i] - mx) / sum;
      break;
    }
    case kObjPoisson: case kObjGamma: case kObjTweedie: out[i] = expf(out[i]); break;
    case kObjXentLambda: out[i] = log1pf(expf(out[i])); break;
    default: break;
  }
}

// Pointwise metric partial sums: (sum of weighted loss, sum of weights) per block, summed in a fixed order.
__global__ void PointwiseMetricKernel(int metric_kind, int obj_kind, float sigmoid, const float* __restrict__ score, const float* __restrict__ label,
                                      const float* __restrict__ weight, int n, int num_class, double* __restrict__ partial) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  double loss = 0, wsum = 0;
  if (i < n) {
    const float w = weight ? weight[i] : 1.f, y = label[i];
    float v = 0.f;
    if (metric_kind == kMetMultiLogloss || metric_kind == kMetMultiError) {
      float mx = score[i]; for (int c = 1; c < num_class; ++c) mx = fmaxf(mx, score[static_cast<size_t>(c) * n + i]);
      float sum = 0.f; for (int c = 0; c < num_class; ++c) sum += expf(score[static_cast<size_t>(c) * n + i] - mx);
      const int yi = static_cast<int>(y); const float sy = score[static_cast<size_t>(yi) * n + i];
      if (metric_kind == kMetMultiLogloss) {
        float p = obj_kind == kObjMulticlassOVA ? 1.f / (1.f + expf(-sigmoid * sy)) : expf(sy - mx) / sum;
        v = p > 1e-15f ? -logf(p) : -logf(1e-15f);
      } else { int larger = 0; for (int c = 0; c < num_class; ++c) larger += score[static_cast<size_t>(c) * n + i] >= sy; v = larger > 1 ? 1.f : 0.f; }
    } else {
      float s = score[i];
      if (metric_kind == kMetBinaryLogloss || metric_kind == kMetBinaryError) {
        const float p = 1.f / (1.f + expf(-sigmoid * s));
        if (metric_kind == kMetBinaryLogloss) { const float q = y > 0.f ? p : 1.f - p; v = q > 1e-15f ? -logf(q) : -logf(1e-15f); }
        else v = (p <= 0.5f) == (y > 0.f) ? 1.f : 0.f;
      } else {
        if (obj_kind == kObjPoisson || obj_kind == kObjGamma || obj_kind == kObjTweedie) s = expf(s);
        const float d = s - y;
        v = metric_kind == kMetL1 ? fabsf(d) : d * d;
      }
    }
    loss = static_cast<double>(v) * w; wsum = w;
  }
  for (int o = 16; o > 0; o >>= 1) { loss += __shfl_xor_sync(0xffffffffu, loss, o); wsum += __shfl_xor_sync(0xffffffffu, wsum, o); }
  __shared__ double s1[32], s2[32];
  const int wq = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) { s1[wq] = loss; s2[wq] = wsum; }
  __syncthreads();
  if (threadIdx.x == 0) {
    double a = 0, b = 0; for (int k = 0; k < (blockDim.x + 31) / 32; ++k) { a += s1[k]; b += s2[k]; }
    partial[2 * blockIdx.x] = a; partial[2 * blockIdx.x + 1] = b;
  }
}

__global__ void __launch_bounds__(1024) SumPartials2Kernel(const double* __restrict__ partial, int nblocks, double* __restrict__ out2) {
  // one block, fixed order: thread t takes blocks t, t+1024, ...; then a fixed shared-memory tree (the same sum on every run)
  __shared__ double sa[1024], sb[1024];
  double a = 0, b = 0;
  for (int k = threadIdx.x; k < nblocks; k += 1024) { a += partial[2 * k]; b += partial[2 * k + 1]; }
  sa[threadIdx.x] = a; sb[threadIdx.x] = b;
  __syncthreads();
  for (int o = 512; o > 0; o >>= 1) { if (threadIdx.x < o) { sa[threadIdx.x] += sa[threadIdx.x + o]; sb[threadIdx.x] += sb[threadIdx.x + o]; } __syncthreads(); }
  if (threadIdx.x == 0) { out2[0] = sa[0]; out2[1] = sb[0]; }
}

}  // namespace

void LaunchAddLeafOutputs(const LeafInfo* leaves, const double* leaf_value, int num_leaves, const int* idx0, const int* idx1, float* score, cudaStream_t s) {
  if (num_leaves <= 0) return;
  AddLeafOutputsKernel<<<dim3(num_leaves, 64), 256, 0, s>>>(leaves, leaf_value, idx0, idx1, score);
  FB_LAUNCHED(); FB_KERNEL_CHECK();
}
void LaunchAddLeafOutputsFromRecords(const LeafInfo* leaves, const LevelCtrl* ctrl, double shrinkage, int max_leaves, const int* idx0, const int* idx1, float* score,
                                     cudaStream_t s, bool decided_ahead) {
  if (max_leaves <= 0) return;
  AddLeafOutputsFromRecordsKernel<<<dim3(max_leaves, 64), 256, 0, s>>>(leaves, ctrl, shrinkage, max_leaves, idx0, idx1, score, decided_ahead ? 1 : 0);
  FB_LAUNCHED(); FB_KERNEL_CHECK();
}
void LaunchCollapseLeafWindows(const LeafInfo* leaves, int num_leaves, int* idx0, const int* idx1, cudaStream_t s) {
  if (num_leaves <= 0) return;
  CollapseLeafWindowsKernel<<<dim3(num_leaves, 64), 256, 0, s>>>(leaves, idx0, idx1);
  FB_LAUNCHED(); FB_KERNEL_CHECK();
}
int LeafGradSumSlices() { return kRenewSlices; }
void LaunchLeafGradSums(const LeafInfo* leaves, int num_leaves, const int* idx0, const int* idx1, const float* grad, const float* hess, double* partial, cudaStream_t s) {
  if (num_leaves <= 0) return;
  LeafGradSumsKernel<<<dim3(num_leaves, kRenewSlices), 256, 0, s>>>(leaves, idx0, idx1, grad, hess, partial);
  FB_LAUNCHED(); FB_KERNEL_CHECK();
}
__global__ void ScaleAddKernel(float* score, int n, float a, float b) { const int i = blockIdx.x * blockDim.x + threadIdx.x; if (i < n) score[i] = a * score[i] + b; }
void LaunchScaleAdd(float* score, int n, float a, float b, cudaStream_t s) {
  if (n <= 0) return;
  ScaleAddKernel<<<(n + 255) / 256, 256, 0, s>>>(score, n, a, b);
  FB_LAUNCHED(); FB_KERNEL_CHECK();
}
__global__ void AddVectorKernel(float* score, const float* __restrict__ values, int n) { const int i = blockIdx.x * blockDim.x + threadIdx.x; if (i < n) score[i] += values[i]; }
void LaunchAddVector(float* score, const float* values, int n, cudaStream_t s) {
  if (n <= 0) return;
  AddVectorKernel<<<(n + 255) / 256, 256, 0, s>>>(score, values, n);
  FB_LAUNCHED(); FB_KERNEL_CHECK();
}
void LaunchAddConstant(float* score, int n, float v, cudaStream_t s) {
  if (n <= 0) return;
  AddConstantKernel<<<(n + 255) / 256, 256, 0, s>>>(score, n, v);
  FB_LAUNCHED(); FB_KERNEL_CHECK();
}
void LaunchAddTreeBinned(const DevTree& t, const uint8_t* rows, int row_stride, int n, float scale, float* score, cudaStream_t s) {
  if (n <= 0) return;
  AddTreeBinnedKernel<<<(n + 255) / 256, 256, 0, s>>>(t, rows, row_stride, n, scale, score);
  FB_LAUNCHED(); FB_KERNEL_CHECK();
}
template <typename T>
void LaunchPredictRaw(const ForestNode* nodes, const unsigned int* cat_words, const int* tree_root, int num_trees, int num_class, const T* data, int nrow, int ncol, bool row_major,
                      float* out, bool average, cudaStream_t s) {
  if (nrow <= 0) return;
  const int iters = num_trees / std::max(1, num_class);
  const float inv = (average && iters > 0) ? 1.f / iters : 1.f;
  PredictRawKernel<T><<<(nrow + 127) / 128, 128, 0, s>>>(nodes, cat_words, tree_root, num_trees, num_class, data, nrow, ncol, row_major, out, inv);
  FB_LAUNCHED(); FB_KERNEL_CHECK();
}
template void LaunchPredictRaw<float>(const ForestNode*, const unsigned int*, const int*, int, int, const float*, int, int, bool, float*, bool, cudaStream_t);
template void LaunchPredictRaw<double>(const ForestNode*, const unsigned int*, const int*, int, int, const double*, int, int, bool, float*, bool, cudaStream_t);
template void LaunchPredictRaw<__half>(const ForestNode*, const unsigned int*, const int*, int, int, const __half*, int, int, bool, float*, bool, cudaStream_t);

void LaunchConvertOutput(int obj_kind, double sigmoid, float* out, int nrow, int num_class, cudaStream_t s) {
  if (nrow <= 0) return;
  ConvertOutputKernel<<<(nrow + 255) / 256, 256, 0, s>>>(obj_kind, static_cast<float>(sigmoid), out, nrow, num_class);
  FB_LAUNCHED(); FB_KERNEL_CHECK();
}

void LaunchPointwiseMetric(int metric_kind, int obj_kind, double sigmoid, const float* score, const float* label, const float* weight, int n, int num_class,
                           double* partial, int partial_capacity, double* out2, cudaStream_t s) {
  const int blocks = std::max(1, (n + 255) / 256);
  if (blocks > partial_capacity) Log::Fatal("partial-sum buffer too small");
  PointwiseMetricKernel<<<blocks, 256, 0, s>>>(metric_kind, obj_kind, static_cast<float>(sigmoid), score, label, weight, n, num_class, partial);
  FB_LAUNCHED(); FB_KERNEL_CHECK();
  SumPartials2Kernel<<<1, 1024, 0, s>>>(partial, blocks, out2);
  FB_LAUNCHED(); FB_KERNEL_CHECK();
}

}  // namespace fb
