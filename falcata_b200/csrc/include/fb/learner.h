// Tree learner interface, the host (CPU) histogram learner, the column sampler and the host
// gradient quantizer. The CPU learner is both `device_type=cpu` and the oracle that every device
// kernel and the multi-rank paths are checked against.
//
// Parity: include/Falcata/tree_learner.h (interface), src/treelearner/serial_tree_learner.cpp
// (Train L189-262, ConstructHistograms L425, FindBestSplitsFromHistograms L494, SplitInner L783),
// src/treelearner/data_partition.hpp, leaf_splits.hpp, col_sampler.hpp,
// gradient_discretizer.cpp; parallel modes: data_parallel_tree_learner.cpp:L125-451,
// feature_parallel_tree_learner.cpp:L38-79, voting_parallel_tree_learner.cpp:L152-481.
#pragma once
#include <functional>
#include <memory>
#include <vector>
#include "fb/config.h"
#include "fb/dataset.h"
#include "fb/split_math.h"
#include "fb/tree.h"

namespace fb {

// Host collectives injected by the embedding process (torch.distributed over gloo in the tests,
// any other transport in production). Parity: FLC_NetworkInitWithFunctions, src/c_api.cpp:L3218.
struct Network {
  typedef void (*AllreduceSumFn)(void* buf, int64_t count, int dtype /*0 f64, 1 i64*/);
  typedef void (*AllgatherFn)(const void* in, int64_t bytes, void* out /* world * bytes */);
  // Optional: sendbuf holds, one after the other, the block of 8-byte elements meant for every rank (counts[r] elements for
  // rank r); recv gets counts[own rank] elements: the element-wise sum over all ranks of their blocks for this rank, added in
  // rank order. A transport without it is served by the all-reduce.
  typedef void (*ReduceScatterFn)(const void* sendbuf, const int64_t* counts, void* recv, int dtype /*0 f64, 1 i64*/);
  static ReduceScatterFn& reduce_scatter() { static ReduceScatterFn f = nullptr; return f; }
  static int& rank() { static int r = 0; return r; }
  static int& world() { static int w = 1; return w; }
  static AllreduceSumFn& allreduce() { static AllreduceSumFn f = nullptr; return f; }
  static AllgatherFn& allgather() { static AllgatherFn f = nullptr; return f; }
  static bool active() { return world() > 1 && allreduce() != nullptr && allgather() != nullptr; }
  static void SumDouble(double* p, int64_t n) { if (active()) allreduce()(p, n, 0); }
  static void SumInt64(int64_t* p, int64_t n) { if (active()) allreduce()(p, n, 1); }
  static double MaxDouble(double v);
  static void Gather(const void* in, int64_t bytes, std::vector<char>* out) {
    out->resize(static_cast<size_t>(bytes) * world());
    if (active()) allgather()(in, bytes, out->data()); else memcpy(out->data(), in, bytes);
  }
};

// TCP mesh between processes (core/socket_network.cpp): the command line's distributed mode and FB_NetworkInit
void SocketNetworkInit(const std::string& machines, int local_listen_port, int timeout_minutes, int num_machines);
void SocketNetworkFree();
bool SocketNetworkActive();
std::string ReadMachineListFile(const std::string& path);
// Helpers for data sets whose rows are spread over the processes of the mesh: this process's first global row number and
// the total (rows are numbered in rank order), and the concatenation in rank order of every process's bin sample
// (row-major doubles, ncol values a row), which all processes then hold alike.
void GatherRowCounts(int64_t local_rows, int64_t* global_offset, int64_t* global_total);
void AllGatherSampleRows(std::vector<double>* sample, int ncol);

// Counter-based per-tree / per-node feature sampling (resumable: depends only on seed and ids).
class ColSampler {
 public:
  void Init(const Config& cfg, const Dataset* ds);
  void ResetByTree(int tree_index);
  const std::vector<int8_t>& used_by_tree() const { return used_; }
  // Features a node may search: the tree's sample, restricted to the interaction sets that contain every feature
  // already used on the node's path (real feature indices), then sampled per node when feature_fraction_bynode < 1.
  std::vector<int8_t> SampleByNode(int tree_index, int node_id, const std::vector<int>* path_real = nullptr) const;
  bool by_node() const { return frac_bynode_ < 1.0 || !interaction_sets_.empty(); }
  double bynode_fraction() const { return frac_bynode_; }
  int seed() const { return seed_; }
  const std::vector<std::vector<int>>& interaction_sets() const { return interaction_sets_; }
  int num_used() const { return num_used_; }
 private:
  double frac_bytree_ = 1.0, frac_bynode_ = 1.0;
  int seed_ = 0, nfeat_ = 0, num_used_ = 0;
  std::vector<int8_t> used_;
  std::vector<std::vector<int>> interaction_sets_;
  std::vector<int> real_index_;   // inner feature -> real feature
};

// Quantization scales of one tree and the packed per-row words.
struct QuantState {
  double g_scale = 1.0, h_scale = 1.0;
  int bins = 4;
  bool stochastic = true;
};
// (int16 grad << 16) | uint16 hess
inline int32_t PackGH(int gi, int hi) { return static_cast<int32_t>((static_cast<uint32_t>(gi) << 16) | (static_cast<uint32_t>(hi) & 0xFFFFu)); }
FB_HD inline int UnpackG(int32_t w) { return w >> 16; }
FB_HD inline int UnpackH(int32_t w) { return static_cast<int>(static_cast<uint32_t>(w) & 0xFFFFu); }

// One row's quantized pair; the same code runs in the device kernel.
FB_HD inline int32_t QuantizeRow(float g, float h, float inv_g_scale, float inv_h_scale, bool stochastic, uint32_t seed,
                                 uint32_t iter_key, uint64_t global_row) {
  int gi, hi;
  if (stochastic) {
    Philox4 r = Philox4x32_10(static_cast<uint32_t>(global_row), iter_key, 0x9E3779B9u ^ static_cast<uint32_t>(global_row >> 32), 0xBB67AE85u,
                              seed, seed ^ 0x85EBCA6Bu);
    const float ug = U01From24(r.v[0]), uh = U01From24(r.v[1]);
#if defined(__CUDA_ARCH__)
    gi = static_cast<int>(__fmaf_rn(g, inv_g_scale, g >= 0.f ? ug : -ug));
    hi = static_cast<int>(__fmaf_rn(h, inv_h_scale, uh));
#else
    gi = static_cast<int>(std::fmaf(g, inv_g_scale, g >= 0.f ? ug : -ug));
    hi = static_cast<int>(std::fmaf(h, inv_h_scale, uh));
#endif
  } else {
#if defined(__CUDA_ARCH__)
    gi = static_cast<int>(__fmaf_rn(g, inv_g_scale, g >= 0.f ? 0.5f : -0.5f));
    hi = static_cast<int>(__fmaf_rn(h, inv_h_scale, 0.5f));
#else
    gi = static_cast<int>(std::fmaf(g, inv_g_scale, g >= 0.f ? 0.5f : -0.5f));
    hi = static_cast<int>(std::fmaf(h, inv_h_scale, 0.5f));
#endif
  }
  return static_cast<int32_t>((static_cast<uint32_t>(gi) << 16) | (static_cast<uint32_t>(hi) & 0xFFFFu));
}

// Fixed-point quantization with error feedback and saturation (the same code runs in the device kernel).
// `residual`: two int8 per row, (hessian, gradient) rounding errors of the previous round in 1/128 of a level; they are
// added before rounding and replaced by this round's errors, which removes the bias of deterministic rounding over the
// rounds. `clamp` > 0: the gradient saturates at +-clamp levels (used with the outlier-robust scale); saturation is not
// fed back, or a saturated row would carry an ever-growing residual.
// Parity: src/treelearner/cuda/cuda_gradient_discretizer.cu:L300-335.
FB_HD inline int32_t QuantizeRowFeedback(float g, float h, float inv_g_scale, float inv_h_scale, int clamp, int8_t* residual) {
  float ge = 0.f, he = 0.f;
  if (residual != nullptr) { he = static_cast<float>(residual[0]) * 0.0078125f; ge = static_cast<float>(residual[1]) * 0.0078125f; }
  // one explicitly fused multiply-add per value: the same single rounding on the host and on the device, whatever the
  // compilers would contract on their own
#if defined(__CUDA_ARCH__)
  const float xg = __fmaf_rn(g, inv_g_scale, ge), xh = __fmaf_rn(h, inv_h_scale, he);
#else
  const float xg = std::fmaf(g, inv_g_scale, ge), xh = std::fmaf(h, inv_h_scale, he);
#endif
  // the double 0.5 keeps the rounding sequence free of fused multiply-adds on every target
  int q = xg > 0.f ? static_cast<int>(static_cast<double>(xg) + 0.5) : static_cast<int>(static_cast<double>(xg) - 0.5);
  int qh = static_cast<int>(static_cast<double>(xh) + 0.5);
  if (residual != nullptr) {
    const double eh = (static_cast<double>(xh) - qh) * 128.0, eg = (static_cast<double>(xg) - q) * 128.0;
    int rh = static_cast<int>(eh >= 0 ? eh + 0.5 : eh - 0.5), rg = static_cast<int>(eg >= 0 ? eg + 0.5 : eg - 0.5);
    rh = rh > 127 ? 127 : (rh < -127 ? -127 : rh); rg = rg > 127 ? 127 : (rg < -127 ? -127 : rg);
    residual[0] = static_cast<int8_t>(rh); residual[1] = static_cast<int8_t>(rg);
  }
  if (clamp > 0) { q = q > clamp ? clamp : (q < -clamp ? -clamp : q); }
  if (qh < 0) qh = 0;
  return static_cast<int32_t>((static_cast<uint32_t>(q) << 16) | (static_cast<uint32_t>(qh) & 0xFFFFu));
}

// Outlier-robust gradient scale of the fixed-point mode. `hist` counts the rows by log-magnitude: bucket b holds
// |g| in (gmax * 2^-((b+1)/128), gmax * 2^-(b/128)], kQuantMagBuckets buckets in all (16 octaves). Walking down from the
// largest magnitudes: if a small set of rows (at most 5 % of `num_rows`) is followed by at least one empty octave and
// then more rows, those first rows are outliers above a gap and the scale is anchored at the upper edge of the first
// bucket below the gap (the outliers saturate); otherwise the scale stays at the maximum. Returns the magnitude that
// maps to the top level. Parity: src/treelearner/cuda/cuda_gradient_discretizer.cu:L88-222.
constexpr int kQuantMagBuckets = 2048;
constexpr int kQuantMagPerOctave = 128;
FB_HD inline int QuantMagBucket(float abs_g, float gmax) {
  // abs_g in (0, gmax]
#if defined(__CUDA_ARCH__)
  int b = static_cast<int>(floorf(-log2f(abs_g / gmax) * static_cast<float>(kQuantMagPerOctave)));
#else
  int b = static_cast<int>(std::floor(-std::log2(abs_g / gmax) * static_cast<float>(kQuantMagPerOctave)));
#endif
  return b < 0 ? 0 : (b >= kQuantMagBuckets ? kQuantMagBuckets - 1 : b);
}
template <typename Count>
FB_HD inline float RobustGradAnchor(const Count* hist, long long num_rows, float gmax) {
  const long long max_outliers = static_cast<long long>(0.05 * static_cast<double>(num_rows));
  long long outliers = 0; bool seen = false; int gap = 0, bulk_top = -1;
  for (int b = 0; b < kQuantMagBuckets; ++b) {
    const long long c = static_cast<long long>(hist[b]);
    if (c == 0) { if (seen) ++gap; continue; }
    if (seen && gap >= kQuantMagPerOctave && outliers <= max_outliers) { bulk_top = b; break; }
    seen = true; gap = 0; outliers += c;
    if (outliers > max_outliers) break;
  }
  if (bulk_top < 0) return gmax;
  // gmax * 2^(-bulk_top / 128) by exact halvings and repeated single-precision products with one constant, so that the
  // host and the device arrive at the same bits
  float anchor = gmax;
  for (int o = 0; o < bulk_top / kQuantMagPerOctave; ++o) anchor *= 0.5f;
  const float step = 0.99459942f;   // 2^(-1/128)
  for (int k = 0; k < bulk_top % kQuantMagPerOctave; ++k) {
#if defined(__CUDA_ARCH__)
    anchor = __fmul_rn(anchor, step);
#else
    anchor = anchor * step;
#endif
  }
  return (anchor > 0.f && anchor <= gmax) ? anchor : gmax;
}

class ObjectiveFunction;

class TreeLearner {
 public:
  virtual ~TreeLearner() {}
  virtual void Init(const Dataset* train, const Config& cfg) = 0;
  virtual void ResetConfig(const Config& cfg) = 0;
  // grad/hess: host pointers for the CPU learner, device pointers for the CUDA learner.
  virtual Tree* Train(const score_t* grad, const score_t* hess, int tree_index) = 0;
  virtual void SetBaggingData(const data_size_t* used_indices, data_size_t num) = 0;
  // score += tree output for the training rows, through the final partition.
  virtual void AddPredictionToScore(const Tree* tree, double* score) const = 0;
  // Re-fit leaf outputs from a per-leaf functional (L1 / quantile / mape objectives).
  virtual void RenewTreeOutput(Tree* tree, const ObjectiveFunction* obj, std::function<double(const label_t*, int)> residual,
                               data_size_t total_num_data, const data_size_t* bag_indices, data_size_t bag_cnt, const double* score) const = 0;
  virtual Tree* FitByExistingTree(const Tree* old_tree, const score_t* grad, const score_t* hess) const = 0;
  virtual const data_size_t* LeafIndices(int leaf, data_size_t* count) const = 0;
  virtual bool on_device() const { return false; }
};

TreeLearner* CreateTreeLearner(const Config& cfg);
TreeLearner* CreateCPUTreeLearner(const Config& cfg);

// One node of a forced-splits file (forcedsplits_filename): split `feature` (index in the data) at `threshold`; left / right
// are indices of the child nodes in the same array or -1. Parity: src/treelearner/serial_tree_learner.cpp (ForceSplits).
struct ForcedSplitNode { int feature = -1; double threshold = 0.0; int left = -1, right = -1; };
std::vector<ForcedSplitNode> LoadForcedSplitsFile(const std::string& filename);
TreeLearner* CreateCUDATreeLearner(const Config& cfg);   // defined in the CUDA module

}  // namespace fb
