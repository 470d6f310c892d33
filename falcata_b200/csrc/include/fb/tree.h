// Host tree model: arrays, split bookkeeping, prediction, text (de)serialisation, JSON,
// if-else code generation and TreeSHAP.
// Parity: include/Falcata/tree.h (array set, decision_type bit layout L29-30, L271-290; decisions
// L361-439), src/io/tree.cpp (Split L66-82, ToString L344-414, ToJSON L416-526, parse L690-871,
// TreeSHAP L873-1036). The text form is the LightGBM v4 tree block and must stay compatible.
#pragma once
#include <string>
#include <vector>
#include "fb/common.h"

namespace fb {

constexpr int8_t kCategoricalMask = 1;
constexpr int8_t kDefaultLeftMask = 2;

class Tree {
 public:
  explicit Tree(int max_leaves = 2, bool track_branch = false, bool is_linear = false);
  // Parse one "Tree=i" block body (lines after the Tree= line up to the blank line).
  Tree(const char* str, size_t* used_len);

  int num_leaves = 1;
  int num_cat = 0;
  int max_leaves = 2;
  double shrinkage = 1.0;
  bool is_linear = false;
  std::vector<int> left_child, right_child;
  std::vector<int> split_feature_inner, split_feature;
  std::vector<uint32_t> threshold_in_bin;
  std::vector<double> threshold;
  std::vector<int8_t> decision_type;
  std::vector<float> split_gain;
  std::vector<int> leaf_parent;
  std::vector<double> leaf_value, leaf_weight;
  std::vector<int> leaf_count;
  std::vector<double> internal_value, internal_weight;
  std::vector<int> internal_count;
  std::vector<int> leaf_depth;
  std::vector<int> cat_boundaries_inner, cat_boundaries;
  std::vector<uint32_t> cat_threshold_inner, cat_threshold;
  // linear leaves
  std::vector<double> leaf_const;
  std::vector<std::vector<double>> leaf_coeff;
  std::vector<std::vector<int>> leaf_features, leaf_features_inner;

  // Numerical split of `leaf`; returns the new (right) leaf index. The left child keeps `leaf`.
  int Split(int leaf, int feature_inner, int real_feature, uint32_t threshold_bin, double threshold_double,
            double left_value, double right_value, int left_cnt, int right_cnt, double left_weight,
            double right_weight, float gain, int missing_type, bool default_left);
  int SplitCategorical(int leaf, int feature_inner, int real_feature, const uint32_t* threshold_bin, int num_threshold_bin,
                       const uint32_t* threshold, int num_threshold, double left_value, double right_value, int left_cnt,
                       int right_cnt, double left_weight, double right_weight, float gain, int missing_type);
  void SetLeafOutput(int leaf, double v) { leaf_value[leaf] = v; }
  void Shrink(double rate);
  void AddBias(double val);
  void AsConstantTree(double val);
  int MaxDepth() const;

  inline static int MissingTypeOf(int8_t dt) { return (dt >> 2) & 3; }
  inline static void SetMissingType(int8_t* dt, int mt) { *dt = static_cast<int8_t>((*dt & 3) | (mt << 2)); }

  inline int Decide(double fval, int node) const {
    const int8_t dt = decision_type[node];
    if (dt & kCategoricalMask) {
      if (std::isnan(fval)) return right_child[node];
      int iv = static_cast<int>(fval);
      if (iv < 0) return right_child[node];
      int ci = static_cast<int>(threshold[node]);
      int lo = cat_boundaries[ci], n = cat_boundaries[ci + 1] - lo;
      if ((iv >> 5) < n && ((cat_threshold[lo + (iv >> 5)] >> (iv & 31)) & 1)) return left_child[node];
      return right_child[node];
    }
    const int mt = MissingTypeOf(dt);
    if (std::isnan(fval) && mt != 2) fval = 0.0;
    if ((mt == 1 && std::fabs(fval) <= kZeroThreshold) || (mt == 2 && std::isnan(fval)))
      return (dt & kDefaultLeftMask) ? left_child[node] : right_child[node];
    return fval <= threshold[node] ? left_child[node] : right_child[node];
  }
  inline int LeafIndex(const double* row) const {
    if (num_leaves <= 1) return 0;
    int node = 0;
    while (node >= 0) node = Decide(row[split_feature[node]], node);
    return ~node;
  }
  inline double Predict(const double* row) const {
    if (num_leaves <= 1) return leaf_value[0];
    int leaf = LeafIndex(row);
    if (!is_linear) return leaf_value[leaf];
    double out = leaf_const[leaf];
    for (size_t k = 0; k < leaf_features[leaf].size(); ++k) {
      double v = row[leaf_features[leaf][k]];
      if (std::isnan(v)) return leaf_value[leaf];
      out += leaf_coeff[leaf][k] * v;
    }
    return out;
  }
  // Decide on a feature bin (training/validation data in binned form).
  inline int DecideBin(int fbin, int node, int default_bin, int nan_bin) const {
    const int8_t dt = decision_type[node];
    if (dt & kCategoricalMask) {
      int ci = static_cast<int>(threshold_in_bin[node]);
      int lo = cat_boundaries_inner[ci], n = cat_boundaries_inner[ci + 1] - lo;
      if ((fbin >> 5) < n && ((cat_threshold_inner[lo + (fbin >> 5)] >> (fbin & 31)) & 1)) return left_child[node];
      return right_child[node];
    }
    const int mt = MissingTypeOf(dt);
    if ((mt == 1 && fbin == default_bin) || (mt == 2 && fbin == nan_bin))
      return (dt & kDefaultLeftMask) ? left_child[node] : right_child[node];
    return static_cast<uint32_t>(fbin) <= threshold_in_bin[node] ? left_child[node] : right_child[node];
  }
  void PredictContrib(const double* row, int num_features, double* out) const;
  double ExpectedValue() const;
  std::string ToString() const;
  std::string ToJSON() const;
  std::string ToIfElse(int index, bool predict_leaf_index) const;
 private:
  std::string NodeToJSON(int index) const;
  std::string NodeToIfElse(int index, bool predict_leaf_index) const;
  void RecomputeMaxDepth();
  void Resize(int n);
  void SplitCommon(int leaf, int feature_inner, int real_feature, double left_value, double right_value, int left_cnt,
                   int right_cnt, double left_weight, double right_weight, float gain);
};

}  // namespace fb
