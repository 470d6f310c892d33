// K7 driver: pack the host trees into one node array and run the raw-feature traversal kernel.
// Parity: python-package/falcata/basic.py:L5067-5163 (device predict route), include/Falcata/tree.h:L361-439
// (decision semantics). Categorical nodes carry an offset into one word array with all nodes' category sets.
#include "engine.h"

#include <cuda_fp16.h>

namespace fb {

bool DevicePredictTiled(const GBDT* gbdt, const void* device_data, int dtype, int32_t nrow, int32_t ncol, bool row_major, int first_tree, int num_trees, int K,
                        bool leaf_index, float inv_avg, float* out_device, cudaStream_t s);

static void PredictGeneralRaw(const GBDT* gbdt, const void* device_data, int dtype, int32_t nrow, int32_t ncol, bool row_major, int start_iter, int use, int K,
                              float* out_device);

void DevicePredict(const GBDT* gbdt, const void* device_data, int dtype, int32_t nrow, int32_t ncol, bool row_major, int predict_type,
                   int start_iter, int num_iter, float* out_device) {
  if (!CudaAvailable()) Log::Fatal("No CUDA device is available for device prediction");
  if (predict_type != 0 && predict_type != 1 && predict_type != 2) Log::Fatal("Device prediction supports normal scores, raw scores and leaf indices");
  const int K = gbdt->num_tree_per_iteration_;
  const int iters = static_cast<int>(gbdt->models_.size()) / std::max(1, K);
  start_iter = std::max(0, std::min(start_iter, iters));
  const int use = num_iter > 0 ? std::min(num_iter, iters - start_iter) : iters - start_iter;
  if (ncol <= gbdt->max_feature_idx_) Log::Fatal("The number of features in data (%d) is not the same as it was in training data (%d)", ncol, gbdt->max_feature_idx_ + 1);
  // the tiled kernel (rows staged in shared memory, trees streamed through it) covers numerical forests; everything
  // else - categorical splits, very wide or very deep forests - walks the general node array below
  bool tiled = false;
  if (use > 0 && std::getenv("FALCATA_PREDICT_GENERAL") == nullptr) {
    const float inv = (gbdt->average_output_ && use > 0) ? 1.f / use : 1.f;
    tiled = DevicePredictTiled(gbdt, device_data, dtype, nrow, ncol, row_major, start_iter * K, use * K, K, predict_type == 2, inv, out_device, 0);
  }
  if (predict_type == 2) {
    if (!tiled) Log::Fatal("Leaf-index prediction on the device covers numerical forests of at most 4096 leaves per tree; predict on the host");
    return;
  }
  if (tiled) {
    if (DebugFlags::Get().verify) {
      // self-check: the general kernel's raw scores for the same rows and trees
      const size_t cells = static_cast<size_t>(nrow) * K;
      DevBuf<float> ref; ref.Alloc(cells);
      FB_CUDA(cudaStreamSynchronize(0));
      PredictGeneralRaw(gbdt, device_data, dtype, nrow, ncol, row_major, start_iter, use, K, ref.get());
      std::vector<float> a(cells), b(cells);
      FB_CUDA(cudaMemcpy(a.data(), out_device, cells * sizeof(float), cudaMemcpyDeviceToHost));
      FB_CUDA(cudaMemcpy(b.data(), ref.get(), cells * sizeof(float), cudaMemcpyDeviceToHost));
      double worst = 0.0; size_t at = 0;
      for (size_t i = 0; i < cells; ++i) { const double d = std::fabs(static_cast<double>(a[i]) - b[i]) / (1.0 + std::fabs(static_cast<double>(b[i]))); if (d > worst) { worst = d; at = i; } }
      if (worst > 1e-5) Log::Fatal("FALCATA_VERIFY: the tiled predict kernel differs from the general one at cell %lld: %.9g against %.9g", static_cast<long long>(at), a[at], b[at]);
      Log::Info("FALCATA_VERIFY: tiled predict equals the general kernel on %lld scores (largest relative difference %.3g)", static_cast<long long>(cells), worst);
    }
    if (predict_type == 0 && gbdt->objective_ != nullptr) {
      const int kind = gbdt->objective_->DeviceKind();
      const double sig = (kind == kObjBinary || kind == kObjMulticlassOVA) ? gbdt->objective_->DeviceParam(0) : 1.0;
      if (kind >= 0) LaunchConvertOutput(kind, sig, out_device, nrow, K, 0);
    }
    FB_CUDA(cudaStreamSynchronize(0));
    return;
  }
  PredictGeneralRaw(gbdt, device_data, dtype, nrow, ncol, row_major, start_iter, use, K, out_device);
  if (predict_type == 0 && gbdt->objective_ != nullptr) {
    const int kind = gbdt->objective_->DeviceKind();
    const double sig = (kind == kObjBinary || kind == kObjMulticlassOVA) ? gbdt->objective_->DeviceParam(0) : 1.0;
    if (kind >= 0) LaunchConvertOutput(kind, sig, out_device, nrow, K, 0);
  }
  FB_CUDA(cudaStreamSynchronize(0));
}

// The general kernel: raw scores of trees [start_iter * K, (start_iter + use) * K) into out_device ([K][nrow] floats).
static void PredictGeneralRaw(const GBDT* gbdt, const void* device_data, int dtype, int32_t nrow, int32_t ncol, bool row_major, int start_iter, int use, int K,
                              float* out_device) {
  std::vector<ForestNode> nodes; std::vector<int> roots; std::vector<unsigned int> cat_words(1, 0u);
  for (int t = start_iter * K; t < (start_iter + use) * K; ++t) {
    const Tree& T = *gbdt->models_[t];
    if (T.is_linear) Log::Fatal("Device prediction does not cover linear leaves; predict on the host");
    const int base = static_cast<int>(nodes.size());
    roots.push_back(base);
    const int ni = T.num_leaves - 1;
    // internal node s -> base + s ; leaf l -> base + ni + l
    for (int s = 0; s < ni; ++s) {
      ForestNode nd; nd.threshold = static_cast<float>(T.threshold[s]);
      // keep "v <= threshold" exact for float inputs: round the double threshold DOWN to float
      if (static_cast<double>(nd.threshold) > T.threshold[s]) nd.threshold = std::nextafterf(nd.threshold, -std::numeric_limits<float>::infinity());
      nd.feature = T.split_feature[s];
      nd.left = T.left_child[s] >= 0 ? base + T.left_child[s] : base + ni + (~T.left_child[s]);
      nd.right = T.right_child[s] >= 0 ? base + T.right_child[s] : base + ni + (~T.right_child[s]);
      nd.flags = ((T.decision_type[s] & kDefaultLeftMask) ? 1 : 0) | (Tree::MissingTypeOf(T.decision_type[s]) << 1);
      if (T.decision_type[s] & kCategoricalMask) {
        const int ci = static_cast<int>(T.threshold[s]);
        const int lo = T.cat_boundaries[ci], nw = T.cat_boundaries[ci + 1] - lo;
        const int off = static_cast<int>(cat_words.size());
        for (int w = 0; w < nw; ++w) cat_words.push_back(T.cat_threshold[lo + w]);
        memcpy(&nd.threshold, &off, sizeof(int));
        nd.flags |= 16 | (nw << 8);
      }
      nodes.push_back(nd);
    }
    for (int l = 0; l < T.num_leaves; ++l) { ForestNode nd; nd.threshold = static_cast<float>(T.leaf_value[l]); nd.feature = 0; nd.left = nd.right = 0; nd.flags = 8; nodes.push_back(nd); }
    if (ni == 0) roots.back() = base;   // single leaf: the root is the leaf itself
  }
  cudaStream_t s = 0;
  DevBuf<ForestNode> d_nodes; DevBuf<int> d_roots; DevBuf<unsigned int> d_cat;
  d_nodes.Upload(nodes, s); d_roots.Upload(roots, s); d_cat.Upload(cat_words, s);
  const int nt = static_cast<int>(roots.size());
  if (nt == 0) { FB_CUDA(cudaMemsetAsync(out_device, 0, sizeof(float) * static_cast<size_t>(nrow) * K, s)); FB_CUDA(cudaStreamSynchronize(s)); return; }
  switch (dtype) {
    case kF32: LaunchPredictRaw<float>(d_nodes.get(), d_cat.get(), d_roots.get(), nt, K, static_cast<const float*>(device_data), nrow, ncol, row_major, out_device, gbdt->average_output_, s); break;
    case kF64: LaunchPredictRaw<double>(d_nodes.get(), d_cat.get(), d_roots.get(), nt, K, static_cast<const double*>(device_data), nrow, ncol, row_major, out_device, gbdt->average_output_, s); break;
    case kF16: LaunchPredictRaw<__half>(d_nodes.get(), d_cat.get(), d_roots.get(), nt, K, static_cast<const __half*>(device_data), nrow, ncol, row_major, out_device, gbdt->average_output_, s); break;
    default: Log::Fatal("Device prediction takes f32, f64 or f16 input");
  }
  FB_CUDA(cudaStreamSynchronize(s));
}

}  // namespace fb
