// K10 (rank-type metrics): AUC by a device radix sort and tie-group reduction, NDCG@k by one block per query.
// The pointwise metrics live in score_kernels.cu (PointwiseMetricKernel).
// Parity: src/metric/cuda/cuda_binary_metric.cu / cuda_rank_metric (sorted sweep with tie groups, DCG with
// label gains and log2 discounts), src/metric/dcg_calculator.cpp:L34-174.
#include "kernels.cuh"

#include <cub/device/device_radix_sort.cuh>
#include <cub/device/device_reduce.cuh>
#include <cub/device/device_scan.cuh>

namespace fb {

namespace {

struct AucWork {
  DevBuf<float> keys_out; DevBuf<int> idx_in, idx_out, num_groups;
  DevBuf<double> pos, neg, gpos, gneg, pos_before, contrib, sums;
  DevBuf<float> gkeys; DevBuf<char> temp;
  size_t cap = 0;
  void Ensure(size_t n, size_t temp_bytes) {
    if (n > cap) {
      keys_out.Alloc(n); idx_in.Alloc(n); idx_out.Alloc(n); pos.Alloc(n); neg.Alloc(n); gpos.Alloc(n); gneg.Alloc(n); pos_before.Alloc(n); contrib.Alloc(n); gkeys.Alloc(n);
      num_groups.Alloc(1); sums.Alloc(3); cap = n;
    }
    if (temp.size() < temp_bytes) temp.Alloc(temp_bytes);
  }
};

AucWork& Work() { static thread_local AucWork w; return w; }

__global__ void IotaKernel(int* p, int n) { const int i = blockIdx.x * blockDim.x + threadIdx.x; if (i < n) p[i] = i; }

__global__ void AucWeightsKernel(const int* __restrict__ order, const float* __restrict__ label, const float* __restrict__ weight, int n,
                                 double* __restrict__ pos, double* __restrict__ neg) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int r = order[i];
  const double w = weight != nullptr ? static_cast<double>(weight[r]) : 1.0;
  const bool p = label[r] > 0.f;
  pos[i] = p ? w : 0.0; neg[i] = p ? 0.0 : w;
}

// a negative of tie group g is beaten by the positives of higher score and ties with those of its own group
__global__ void AucContribKernel(const double* __restrict__ gpos, const double* __restrict__ gneg, const double* __restrict__ pos_before, const int* __restrict__ num_groups,
                                 int n, double* __restrict__ contrib) {
  const int g = blockIdx.x * blockDim.x + threadIdx.x;
  if (g >= n) return;
  contrib[g] = g < *num_groups ? gneg[g] * (pos_before[g] + 0.5 * gpos[g]) : 0.0;
}

constexpr int kNdcgMaxDocs = 4096;
constexpr int kNdcgMaxK = 8;
struct NdcgKs { int k[kNdcgMaxK]; int count; };

// One block per query. A document's position in the score order (ties keep document order, like a stable sort)
// and in the ideal order (by label) is found by counting; DCG and ideal DCG at every k are block sums.
__global__ void __launch_bounds__(256) NdcgKernel(const float* __restrict__ score, const float* __restrict__ label, const int* __restrict__ qb, int num_queries,
                                                  const double* __restrict__ gains, int num_gains, NdcgKs ks, double* __restrict__ out /* [query][count] */) {
  __shared__ float s_score[kNdcgMaxDocs]; __shared__ float s_label[kNdcgMaxDocs];
  __shared__ double s_red[256];
  const int q = blockIdx.x;
  if (q >= num_queries) return;
  const int begin = qb[q], cnt = min(qb[q + 1] - qb[q], kNdcgMaxDocs);
  for (int i = threadIdx.x; i < cnt; i += blockDim.x) { s_score[i] = score[begin + i]; s_label[i] = label[begin + i]; }
  __syncthreads();
  double dcg[kNdcgMaxK], idcg[kNdcgMaxK];
  for (int j = 0; j < kNdcgMaxK; ++j) dcg[j] = idcg[j] = 0.0;
  for (int i = threadIdx.x; i < cnt; i += blockDim.x) {
    const float si = s_score[i], li = s_label[i];
    int rs = 0, rl = 0;
    for (int j = 0; j < cnt; ++j) {
      const float sj = s_score[j], lj = s_label[j];
      rs += (sj > si || (sj == si && j < i)) ? 1 : 0;
      rl += (lj > li || (lj == li && j < i)) ? 1 : 0;
    }
    const int lab = min(max(static_cast<int>(li), 0), num_gains - 1);
    const double g = gains[lab];
    const double ds = g / log2(2.0 + rs), dl = g / log2(2.0 + rl);
    for (int j = 0; j < ks.count; ++j) { if (rs < ks.k[j]) dcg[j] += ds; if (rl < ks.k[j]) idcg[j] += dl; }
  }
  for (int j = 0; j < ks.count; ++j) {
    double both[2] = {dcg[j], idcg[j]};
    double res[2];
    for (int t = 0; t < 2; ++t) {
      s_red[threadIdx.x] = both[t];
      __syncthreads();
      for (int o = 128; o > 0; o >>= 1) { if (threadIdx.x < o) s_red[threadIdx.x] += s_red[threadIdx.x + o]; __syncthreads(); }
      res[t] = s_red[0];
      __syncthreads();
    }
    if (threadIdx.x == 0) out[static_cast<size_t>(q) * ks.count + j] = res[1] > 0.0 ? res[0] / res[1] : 1.0;   // no relevant document: counts as 1
  }
}

// fixed-order sum of the per-query values: one thread per k
__global__ void NdcgSumKernel(const double* __restrict__ per_query, int num_queries, int count, double* __restrict__ out) {
  const int j = threadIdx.x;
  if (j >= count) return;
  double s = 0; for (int q = 0; q < num_queries; ++q) s += per_query[static_cast<size_t>(q) * count + j];
  out[j] = s;
}

}  // namespace

// AUC of (score, label, weight) on the device. Returns false when there are no positive or no negative rows
// (out[0] = 1 as the host metric reports). out: [auc, sum of positive weights, sum of negative weights].
void DeviceAuc(const float* score, const float* label, const float* weight, int n, double out[3], cudaStream_t s) {
  AucWork& w = Work();
  size_t t1 = 0, t2 = 0, t3 = 0, t4 = 0;
  cub::DeviceRadixSort::SortPairsDescending(nullptr, t1, static_cast<const float*>(nullptr), static_cast<float*>(nullptr), static_cast<const int*>(nullptr), static_cast<int*>(nullptr), n);
  cub::DeviceReduce::ReduceByKey(nullptr, t2, static_cast<const float*>(nullptr), static_cast<float*>(nullptr), static_cast<const double*>(nullptr), static_cast<double*>(nullptr),
                                 static_cast<int*>(nullptr), cub::Sum(), n);
  cub::DeviceScan::ExclusiveSum(nullptr, t3, static_cast<const double*>(nullptr), static_cast<double*>(nullptr), n);
  cub::DeviceReduce::Sum(nullptr, t4, static_cast<const double*>(nullptr), static_cast<double*>(nullptr), n);
  size_t tb = std::max(std::max(t1, t2), std::max(t3, t4)) + 256;
  w.Ensure(static_cast<size_t>(std::max(1, n)), tb);
  const int blocks = (n + 255) / 256;
  IotaKernel<<<blocks, 256, 0, s>>>(w.idx_in.get(), n); FB_LAUNCHED();
  size_t tbytes = w.temp.size();
  FB_CUDA(cub::DeviceRadixSort::SortPairsDescending(w.temp.get(), tbytes, score, w.keys_out.get(), w.idx_in.get(), w.idx_out.get(), n, 0, 32, s)); FB_LAUNCHED();
  AucWeightsKernel<<<blocks, 256, 0, s>>>(w.idx_out.get(), label, weight, n, w.pos.get(), w.neg.get()); FB_LAUNCHED();
  tbytes = w.temp.size();
  FB_CUDA(cub::DeviceReduce::ReduceByKey(w.temp.get(), tbytes, w.keys_out.get(), w.gkeys.get(), w.pos.get(), w.gpos.get(), w.num_groups.get(), cub::Sum(), n, s)); FB_LAUNCHED();
  tbytes = w.temp.size();
  FB_CUDA(cub::DeviceReduce::ReduceByKey(w.temp.get(), tbytes, w.keys_out.get(), w.gkeys.get(), w.neg.get(), w.gneg.get(), w.num_groups.get(), cub::Sum(), n, s)); FB_LAUNCHED();
  // entries past num_groups of gpos are stale, but they come after every valid prefix and AucContrib ignores them
  tbytes = w.temp.size();
  FB_CUDA(cub::DeviceScan::ExclusiveSum(w.temp.get(), tbytes, w.gpos.get(), w.pos_before.get(), n, s)); FB_LAUNCHED();
  AucContribKernel<<<blocks, 256, 0, s>>>(w.gpos.get(), w.gneg.get(), w.pos_before.get(), w.num_groups.get(), n, w.contrib.get()); FB_LAUNCHED();
  tbytes = w.temp.size(); FB_CUDA(cub::DeviceReduce::Sum(w.temp.get(), tbytes, w.contrib.get(), w.sums.get(), n, s));
  tbytes = w.temp.size(); FB_CUDA(cub::DeviceReduce::Sum(w.temp.get(), tbytes, w.pos.get(), w.sums.get() + 1, n, s));
  tbytes = w.temp.size(); FB_CUDA(cub::DeviceReduce::Sum(w.temp.get(), tbytes, w.neg.get(), w.sums.get() + 2, n, s)); FB_LAUNCHED();
  double h[3];
  FB_CUDA(cudaMemcpyAsync(h, w.sums.get(), sizeof(h), cudaMemcpyDeviceToHost, s));
  FB_CUDA(cudaStreamSynchronize(s));
  out[1] = h[1]; out[2] = h[2];
  out[0] = (h[1] > 0 && h[2] > 0) ? h[0] / (h[1] * h[2]) : 1.0;
}

// NDCG@k summed over the queries: out[j] = sum over queries of ndcg@ks[j]. Returns false when a query is too long for the kernel.
bool DeviceNdcgSums(const float* score, const float* label, const int* query_boundaries, int num_queries, int max_docs, const double* gains, int num_gains,
                    const std::vector<int>& ks, double* out, cudaStream_t s) {
  if (max_docs > kNdcgMaxDocs || static_cast<int>(ks.size()) > kNdcgMaxK || ks.empty() || num_queries <= 0) return false;
  NdcgKs k; k.count = static_cast<int>(ks.size()); for (int j = 0; j < kNdcgMaxK; ++j) k.k[j] = j < k.count ? ks[j] : 0;
  static thread_local DevBuf<double> per_query, sums;
  if (per_query.size() < static_cast<size_t>(num_queries) * k.count) per_query.Alloc(static_cast<size_t>(num_queries) * k.count);
  if (sums.size() < kNdcgMaxK) sums.Alloc(kNdcgMaxK);
  NdcgKernel<<<num_queries, 256, 0, s>>>(score, label, query_boundaries, num_queries, gains, num_gains, k, per_query.get()); FB_LAUNCHED(); FB_KERNEL_CHECK();
  NdcgSumKernel<<<1, 32, 0, s>>>(per_query.get(), num_queries, k.count, sums.get()); FB_LAUNCHED(); FB_KERNEL_CHECK();
  FB_CUDA(cudaMemcpyAsync(out, sums.get(), sizeof(double) * k.count, cudaMemcpyDeviceToHost, s));
  FB_CUDA(cudaStreamSynchronize(s));
  return true;
}

}  // namespace fb
