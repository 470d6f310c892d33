// Host histogram tree learner: serial, plus data-/feature-/voting-parallel over injected
// collectives. See fb/learner.h for the parity notes.
//
// Growth policies:
//   leaf  : best-first. The leaf with the largest gain is split until num_leaves is reached.
//   level : all splittable leaves of a level are split together; when the leaf budget binds, the
//           level's candidates with the largest gains win (ties: lower leaf index). Splits of a
//           level are applied in ascending leaf order, which fixes the leaf numbering.
// The device learner implements exactly the same two policies, so trees can be compared.
#include "fb/learner.h"

#include <omp.h>
#include "fb/objective.h"

#include <fstream>
#include <functional>
#include <numeric>
#include <sstream>
#include <queue>

namespace fb {

// Forced splits: a JSON tree {"feature": f, "threshold": v, "left": {...}, "right": {...}} flattened depth-first; node 0 is the root.
std::vector<ForcedSplitNode> LoadForcedSplitsFile(const std::string& filename) {
  std::vector<ForcedSplitNode> forced_;
  if (filename.empty()) return forced_;
  std::ifstream f(filename);
  if (!f) Log::Fatal("Cannot open forced splits file %s", filename.c_str());
  std::stringstream ss; ss << f.rdbuf();
  const std::string t = ss.str();
  size_t pos = 0;
  auto skip_ws = [&]() { while (pos < t.size() && isspace(static_cast<unsigned char>(t[pos]))) ++pos; };
  std::function<int()> parse_object = [&]() -> int {
    skip_ws();
    if (pos >= t.size() || t[pos] != '{') Log::Fatal("Forced splits file: expected '{' at offset %d", static_cast<int>(pos));
    ++pos;
    const int id = static_cast<int>(forced_.size()); forced_.emplace_back();
    for (;;) {
      skip_ws();
      if (pos < t.size() && t[pos] == '}') { ++pos; break; }
      if (pos < t.size() && t[pos] == ',') { ++pos; continue; }
      if (pos >= t.size() || t[pos] != '"') Log::Fatal("Forced splits file: expected a key at offset %d", static_cast<int>(pos));
      const size_t e = t.find('"', pos + 1);
      if (e == std::string::npos) Log::Fatal("Forced splits file: unterminated key");
      const std::string key = t.substr(pos + 1, e - pos - 1);
      pos = e + 1; skip_ws();
      if (pos >= t.size() || t[pos] != ':') Log::Fatal("Forced splits file: expected ':' after \"%s\"", key.c_str());
      ++pos; skip_ws();
      if (key == "left" || key == "right") { const int c = parse_object(); if (key == "left") forced_[id].left = c; else forced_[id].right = c; }
      else {
        size_t e2 = pos; while (e2 < t.size() && t[e2] != ',' && t[e2] != '}') ++e2;
        const double v = atof(t.substr(pos, e2 - pos).c_str());
        if (key == "feature") forced_[id].feature = static_cast<int>(v); else if (key == "threshold") forced_[id].threshold = v;
        pos = e2;
      }
    }
    return id;
  };
  skip_ws();
  if (pos < t.size()) parse_object();
  if (!forced_.empty() && forced_[0].feature < 0) forced_.clear();   // "{}"
  return forced_;
}


double Network::MaxDouble(double v) {
  if (!active()) return v;
  std::vector<char> all; Gather(&v, sizeof(double), &all);
  double m = v; const double* p = reinterpret_cast<const double*>(all.data());
  for (int i = 0; i < world(); ++i) m = std::max(m, p[i]);
  return m;
}

// ------------------------------------------------------------ ColSampler ----
void ColSampler::Init(const Config& cfg, const Dataset* ds) {
  frac_bytree_ = cfg.feature_fraction; frac_bynode_ = cfg.feature_fraction_bynode; seed_ = cfg.feature_fraction_seed;
  nfeat_ = ds->num_features; used_.assign(nfeat_, 1); num_used_ = nfeat_;
  interaction_sets_.clear();
  real_index_.assign(nfeat_, 0); for (int f = 0; f < nfeat_; ++f) real_index_[f] = ds->feature_meta[f].real_index;
  if (!cfg.interaction_constraints.empty()) {
    // "[0,1,2],[2,3]" over real feature indices
    std::string s = cfg.interaction_constraints; std::vector<int> cur; std::string num; bool in = false;
    for (char c : s) {
      if (c == '[') { in = true; cur.clear(); num.clear(); }
      else if (c == ']') { if (!num.empty()) cur.push_back(atoi(num.c_str())); num.clear(); if (in) interaction_sets_.push_back(cur); in = false; }
      else if (c == ',') { if (in && !num.empty()) { cur.push_back(atoi(num.c_str())); num.clear(); } }
      else if (!isspace(static_cast<unsigned char>(c))) num.push_back(c);
    }
  }
}

// Deterministic subset: rank features by a Philox word keyed on (seed, tree, feature) and keep the
// k smallest. Independent of any generator state, hence identical after a resume and on any rank.
static std::vector<int8_t> SampleFeatures(int n, double frac, uint32_t seed, uint32_t a, uint32_t b, const std::vector<int8_t>* within) {
  std::vector<int8_t> used(n, 0);
  std::vector<int> pool;
  for (int f = 0; f < n; ++f) if (within == nullptr || (*within)[f]) pool.push_back(f);
  int k = std::max(1, static_cast<int>(std::floor(frac * static_cast<double>(pool.size()) + 0.5)));
  k = std::min<int>(k, static_cast<int>(pool.size()));
  std::vector<std::pair<uint32_t, int>> keyed;
  for (int f : pool) keyed.emplace_back(Philox4x32_10(static_cast<uint32_t>(f), a, b, 0x51ED27u, seed, 0xC0FFEEu).v[0], f);
  std::sort(keyed.begin(), keyed.end());
  for (int i = 0; i < k; ++i) used[keyed[i].second] = 1;
  return used;
}

void ColSampler::ResetByTree(int tree_index) {
  if (frac_bytree_ >= 1.0) { used_.assign(nfeat_, 1); num_used_ = nfeat_; return; }
  used_ = SampleFeatures(nfeat_, frac_bytree_, static_cast<uint32_t>(seed_), static_cast<uint32_t>(tree_index), 0u, nullptr);
  num_used_ = 0; for (auto u : used_) num_used_ += u;
}

// Parity: src/treelearner/col_sampler.hpp (GetByNode: a constraint set applies when it holds every feature of the
// branch; the allowed features are the union of the applying sets; the per-node sample is drawn inside them).
std::vector<int8_t> ColSampler::SampleByNode(int tree_index, int node_id, const std::vector<int>* path_real) const {
  std::vector<int8_t> within = used_;
  if (!interaction_sets_.empty()) {
    std::vector<int8_t> allowed_real;
    for (const auto& set : interaction_sets_) {
      bool applies = true;
      if (path_real != nullptr) for (int pf : *path_real) if (std::find(set.begin(), set.end(), pf) == set.end()) { applies = false; break; }
      if (!applies) continue;
      for (int rf : set) { if (rf < 0) continue; if (static_cast<int>(allowed_real.size()) <= rf) allowed_real.resize(rf + 1, 0); allowed_real[rf] = 1; }
    }
    for (int f = 0; f < nfeat_; ++f) { const int rf = real_index_[f]; if (rf >= static_cast<int>(allowed_real.size()) || !allowed_real[rf]) within[f] = 0; }
  }
  if (frac_bynode_ >= 1.0) return within;
  bool any = false; for (auto u : within) any = any || u;
  if (!any) return within;
  return SampleFeatures(nfeat_, frac_bynode_, static_cast<uint32_t>(seed_), static_cast<uint32_t>(tree_index), static_cast<uint32_t>(node_id) + 1u, &within);
}

// ----------------------------------------------------------- CPU learner ----
namespace {

struct LeafState {
  int begin = 0, count = 0;          // window in indices_
  int id = 0;                        // leaf index in the tree
  double sum_g = 0, sum_h = 0;
  int64_t sum_gi = 0, sum_hi = 0;
  int64_t global_count = 0;          // rows of the leaf over all ranks
  double output = 0;
  int depth = 0;
  std::vector<int> path;             // real features split on above this leaf (interaction constraints)
  SplitRecord best;
  std::vector<double> hist;          // 2 * num_total_bin (g, h) real-valued, or
  std::vector<int64_t> hist_i;       // 2 * num_total_bin integer sums when quantized
  bool has_hist = false;
  int64_t hist_stamp = 0;            // when the histogram was last produced or read (least recently used ones are dropped first)
  std::vector<uint16_t> box;         // monotone_constraints_method=intermediate / advanced: per feature the (first, last) bin of the leaf's cell
  // advanced: the leaves whose cells touch this leaf's along a monotone feature, listed when the leaf is about to be
  // searched: output, +1 when this leaf lies below the neighbour (its output is an upper bound), the separating feature
  struct Neighbour { double output; int dir; int sep; const uint16_t* box; };
  std::vector<Neighbour> neighbours;
  double min_constraint = -std::numeric_limits<double>::infinity(), max_constraint = std::numeric_limits<double>::infinity();
};

class CPUTreeLearner : public TreeLearner {
 public:
  explicit CPUTreeLearner(const Config& cfg) : cfg_(cfg) {}
  void Init(const Dataset* train, const Config& cfg) override;
  void ResetConfig(const Config& cfg) override { cfg_ = cfg; SetParams(); col_sampler_.Init(cfg_, ds_); }
  Tree* Train(const score_t* grad, const score_t* hess, int tree_index) override;
  void SetBaggingData(const data_size_t* used, data_size_t num) override {
    if (used == nullptr) { bag_.clear(); use_bag_ = false; } else { bag_.assign(used, used + num); use_bag_ = true; }
  }
  void AddPredictionToScore(const Tree* tree, double* score) const override;
  void RenewTreeOutput(Tree* tree, const ObjectiveFunction* obj, std::function<double(const label_t*, int)> residual,
                       data_size_t total_num_data, const data_size_t* bag_indices, data_size_t bag_cnt, const double* score) const override;
  Tree* FitByExistingTree(const Tree* old_tree, const score_t* grad, const score_t* hess) const override;
  const data_size_t* LeafIndices(int leaf, data_size_t* count) const override { *count = leaves_[leaf].count; return indices_.data() + leaves_[leaf].begin; }

 private:
  void SetParams();
  void Quantize(const score_t* grad, const score_t* hess, int tree_index);
  void ConstructHistogram(LeafState* leaf);
  void SubtractHistogram(LeafState* parent, const LeafState& smaller, LeafState* larger);
  void FindBestSplit(LeafState* leaf, int leaf_id, int tree_index);
  void FindBestSplitMany(const std::vector<int>& ids, int tree_index);
  bool PrepareLeafScan(LeafState* leaf, int leaf_id, int tree_index, LeafScanInfo* L, std::vector<int8_t>* mask);
  void FinishLeafScan(LeafState* leaf, const LeafScanInfo& L, SplitRecord* per);
  void ScanNumerical(const LeafState& leaf, int f, const LeafScanInfo& L, SplitRecord* best) const;
  void ScanCategorical(const LeafState& leaf, int f, const LeafScanInfo& L, SplitRecord* best) const;
  int ApplySplit(Tree* tree, int leaf_id);
  void ReduceHistogramAcrossRanks(LeafState* leaf);
  void SyncBestSplit(SplitRecord* rec) const;
  bool FeatureOwned(int f) const { return !(parallel_data_ || parallel_feature_) || f % Network::world() == Network::rank(); }

  Config cfg_;
  SplitParams sp_;
  const Dataset* ds_ = nullptr;
  ColSampler col_sampler_;
  std::vector<data_size_t> indices_, tmp_;
  std::vector<LeafState> leaves_;
  std::vector<data_size_t> bag_;
  bool use_bag_ = false;
  bool quant_ = false, parallel_data_ = false, parallel_feature_ = false, parallel_voting_ = false;
  QuantState qs_;
  std::vector<int32_t> gh_packed_;
  // reduce-scatter of histograms: per rank the histogram slots of the features it owns, the block sizes in 8-byte elements,
  // and the packed send / receive buffers (8-byte cells holding doubles or 64-bit integers)
  std::vector<std::vector<int>> rs_slots_; std::vector<int64_t> rs_counts_; std::vector<int64_t> rs_send_, rs_recv_;
  std::vector<int8_t> ef_residual_;   // fixed-point error feedback: (hessian, gradient) residuals per row, one slot per class
  const score_t* grad_ = nullptr; const score_t* hess_ = nullptr;
  std::vector<int8_t> node_feature_mask_;
  std::vector<int64_t> voted_hist_i_; std::vector<double> voted_hist_;
  // cost-effective boosting, per-feature penalties (by real column index). Coupled: charged once per feature, until
  // the model first splits on it. Lazy: charged per row of the leaf that has not yet been sent through a split on the
  // feature. Parity: src/treelearner/cost_effective_gradient_boosting.hpp (DeltaGain, UpdateLeafBestSplits simplified:
  // cached candidates of other leaves are not re-scored when a feature becomes free).
  std::vector<double> cegb_coupled_, cegb_lazy_;
  std::vector<char> cegb_feature_used_;
  std::vector<std::vector<bool>> cegb_row_paid_;   // [real feature with a lazy penalty][row]
  double CegbFeaturePenalty(int inner_feature, const LeafState& leaf) const;
  void CegbAfterSplit(int inner_feature, const LeafState& leaf);
  std::vector<int8_t> voted_;      // voting-parallel: features whose histograms are globally reduced for the current leaf
  int cur_tree_index_ = 0, cur_leaf_id_ = 0;
  Random extra_rand_{6};
  // forced splits (forcedsplits_filename): a tree of (feature, threshold) applied from the root before normal growth
  using ForcedNode = ForcedSplitNode;
  std::vector<ForcedNode> forced_;
  // histogram_pool_size (MB): at most this many leaf histograms are kept; the least recently used are dropped and a leaf
  // whose histogram is gone gets both children built from the data when it splits. Parity: src/treelearner/feature_histogram.hpp
  // (HistogramPool: LRU cache of leaf histograms bounded by histogram_pool_size).
  int hist_pool_cap_ = 0;            // leaves with a histogram allowed at once (0: unbounded)
  int64_t hist_clock_ = 0;
  void TouchHistogram(LeafState* leaf) { leaf->hist_stamp = ++hist_clock_; }
  void DropHistogram(LeafState* leaf) { std::vector<double>().swap(leaf->hist); std::vector<int64_t>().swap(leaf->hist_i); leaf->has_hist = false; }
  void EnforceHistogramPool(int num_leaves, int keep_a, int keep_b);
  bool mono_intermediate_ = false;   // monotone bounds from the neighbouring leaves' outputs instead of the split's mid point
  bool mono_advanced_ = false;       // ... and per threshold: a child is bounded only by the neighbours that its own part of the cell touches
  int mono_num_leaves_ = 0;          // leaves of the tree under construction (for the neighbour lists)
  int RelateLeaves(int a, int b, int* sep) const;
  std::vector<int> mono_dirty_;      // leaves whose bounds the last ApplySplit tightened (their best split is stale)
  void TightenMonotoneBounds(const Tree* tree, int left_id, int right_id);
  int forced_feature_ = -1, forced_bin_ = -1;   // non-negative while FindBestSplit evaluates one forced (feature, bin)
  void LoadForcedSplits();
  void ForceSplits(Tree* tree, int tree_index);
};

void CPUTreeLearner::SetParams() {
  sp_.lambda_l1 = cfg_.lambda_l1; sp_.lambda_l2 = cfg_.lambda_l2; sp_.max_delta_step = cfg_.max_delta_step; sp_.path_smooth = cfg_.path_smooth;
  sp_.min_sum_hessian_in_leaf = cfg_.min_sum_hessian_in_leaf; sp_.min_gain_to_split = cfg_.min_gain_to_split;
  sp_.min_data_in_leaf = cfg_.min_data_in_leaf; sp_.max_depth = cfg_.max_depth;
  sp_.max_cat_threshold = cfg_.max_cat_threshold; sp_.max_cat_to_onehot = cfg_.max_cat_to_onehot; sp_.min_data_per_group = cfg_.min_data_per_group;
  sp_.cat_l2 = cfg_.cat_l2; sp_.cat_smooth = cfg_.cat_smooth; sp_.extra_trees = cfg_.extra_trees ? 1 : 0;
  sp_.cegb_split = cfg_.cegb_tradeoff * cfg_.cegb_penalty_split;
  sp_.monotone_penalty = cfg_.monotone_penalty;
  auto parse_penalties = [&](const std::string& text, const char* name, std::vector<double>* out) {
    out->clear();
    if (text.empty()) return;
    for (auto& t : SplitAny(text, ",")) { const std::string s = Trim(t); if (!s.empty()) out->push_back(atof(s.c_str())); }
    if (static_cast<int>(out->size()) != ds_->num_total_features) Log::Fatal("%s should be the same size as feature number.", name);
    bool any = false; for (double v : *out) any = any || v != 0.0;
    if (!any) out->clear();
  };
  parse_penalties(cfg_.cegb_penalty_feature_coupled, "cegb_penalty_feature_coupled", &cegb_coupled_);
  parse_penalties(cfg_.cegb_penalty_feature_lazy, "cegb_penalty_feature_lazy", &cegb_lazy_);
  if (!cegb_coupled_.empty()) cegb_feature_used_.assign(ds_->num_total_features, 0);
  if (!cegb_lazy_.empty()) {
    cegb_row_paid_.assign(ds_->num_total_features, std::vector<bool>());
    for (int j = 0; j < ds_->num_total_features; ++j) if (cegb_lazy_[j] > 0.0) cegb_row_paid_[j].assign(ds_->num_data, false);
  }
  if ((!cegb_coupled_.empty() || !cegb_lazy_.empty()) && Network::active() && cfg_.tree_learner != "serial")
    Log::Fatal("Per-feature CEGB penalties are not available with a parallel tree learner");
  sp_.use_mc = 0; for (const auto& m : ds_->feature_meta) if (m.monotone != 0) sp_.use_mc = 1;
  mono_advanced_ = sp_.use_mc != 0 && cfg_.monotone_constraints_method == "advanced";
  mono_intermediate_ = sp_.use_mc != 0 && (cfg_.monotone_constraints_method == "intermediate" || mono_advanced_);
  hist_pool_cap_ = 0;
  if (cfg_.histogram_pool_size > 0.0 && ds_ != nullptr) {
    const double per_leaf = static_cast<double>(ds_->num_total_bin) * 2.0 * 8.0;   // (g, h) as doubles or 64-bit integers
    hist_pool_cap_ = std::max(2, static_cast<int>(cfg_.histogram_pool_size * 1024.0 * 1024.0 / std::max(1.0, per_leaf)));
  }
  quant_ = cfg_.quant != QuantMode::None;
  qs_.bins = cfg_.quant_bins_resolved; qs_.stochastic = cfg_.quant == QuantMode::Stochastic;
  const bool net = Network::active();
  parallel_data_ = net && cfg_.tree_learner == "data";
  parallel_feature_ = net && cfg_.tree_learner == "feature";
  parallel_voting_ = net && cfg_.tree_learner == "voting";
  extra_rand_ = Random(cfg_.extra_seed);
}

void CPUTreeLearner::Init(const Dataset* train, const Config& cfg) {
  ds_ = train; cfg_ = cfg;
  rs_counts_.clear(); rs_slots_.clear();
  if (!ds_->has_host_bins()) Log::Fatal("The CPU learner needs host-resident bins (dataset was built device-only)");
  SetParams();
  col_sampler_.Init(cfg_, ds_);
  indices_.resize(ds_->num_data); tmp_.resize(ds_->num_data);
  LoadForcedSplits();
}

// forcedsplits_filename: nested JSON objects {"feature": i, "threshold": v, "left": {...}, "right": {...}} over real
// feature indices. Parity: src/treelearner/serial_tree_learner.cpp:L641-781 (ForceSplits: breadth-first from the
// root, a forced split that does not improve the leaf is ignored together with its subtree).
void CPUTreeLearner::LoadForcedSplits() { forced_ = LoadForcedSplitsFile(cfg_.forcedsplits_filename); }

void CPUTreeLearner::ForceSplits(Tree* tree, int tree_index) {
  std::queue<std::pair<int, int>> q;   // (leaf id, forced node)
  q.push({0, 0});
  while (!q.empty() && tree->num_leaves < cfg_.num_leaves) {
    const int leaf = q.front().first; const ForcedNode fn = forced_[q.front().second]; q.pop();
    if (fn.feature < 0 || fn.feature >= ds_->num_total_features) continue;
    const int inner = ds_->used_feature_map[fn.feature];
    if (inner < 0 || ds_->feature_meta[inner].bin_type != static_cast<int>(BinType::Numerical)) {
      Log::Warning("Forced split on feature %d is ignored (constant or categorical feature)", fn.feature);
      continue;
    }
    const int nb = ds_->feature_meta[inner].num_bin;
    forced_feature_ = inner; forced_bin_ = std::min(static_cast<int>(ds_->mappers[fn.feature]->ValueToBin(fn.threshold)), nb - 2);
    const SplitRecord kept = leaves_[leaf].best;
    FindBestSplit(&leaves_[leaf], leaf, tree_index);
    forced_feature_ = forced_bin_ = -1;
    if (leaves_[leaf].best.feature < 0 || !(leaves_[leaf].best.gain > 0.0)) {
      Log::Warning("Forced split on feature %d is ignored: it does not improve the leaf", fn.feature);
      leaves_[leaf].best = kept;
      continue;
    }
    const int right = ApplySplit(tree, leaf);
    FindBestSplit(&leaves_[leaf], leaf, tree_index);
    FindBestSplit(&leaves_[right], right, tree_index);
    if (fn.left >= 0) q.push({leaf, fn.left});
    if (fn.right >= 0) q.push({right, fn.right});
  }
}

void CPUTreeLearner::Quantize(const score_t* grad, const score_t* hess, int tree_index) {
  const data_size_t n = ds_->num_data;
  double mg = 0, mh = 0;
  const data_size_t cnt = use_bag_ ? static_cast<data_size_t>(bag_.size()) : n;
  for (data_size_t k = 0; k < cnt; ++k) {
    data_size_t i = use_bag_ ? bag_[k] : k;
    mg = std::max(mg, static_cast<double>(std::fabs(grad[i]))); mh = std::max(mh, static_cast<double>(std::fabs(hess[i])));
  }
  mg = Network::MaxDouble(mg); mh = Network::MaxDouble(mh);
  // fixed point: the outlier-robust scale (single-target objectives, at most 256 levels) and the error feedback, as in
  // the device engine; both are keyed by the same plan switches
  const Plan plan = Plan::FromString(cfg_.cuda_plan);
  const bool fixed = !qs_.stochastic;
  int clamp = 0;
  float gmax = static_cast<float>(mg);
  if (fixed && plan.robust_scale && qs_.bins <= 256 && cfg_.num_class <= 1 && gmax > 0.f) {
    std::vector<int64_t> hist(kQuantMagBuckets, 0);
    int64_t rows = 0;
    for (data_size_t k = 0; k < cnt; ++k) {
      const data_size_t i = use_bag_ ? bag_[k] : k;
      const float a = std::fabs(grad[i]);
      if (a > 0.f) ++hist[QuantMagBucket(a, gmax)];
      ++rows;
    }
    Network::SumInt64(hist.data(), kQuantMagBuckets); Network::SumInt64(&rows, 1);
    const float anchor = RobustGradAnchor(hist.data(), rows, gmax);
    if (anchor < gmax) { gmax = anchor; clamp = qs_.bins / 2; }
  }
  // scales are computed in fp32 exactly as on the device
  float gs = gmax / static_cast<float>(qs_.bins / 2), hs = static_cast<float>(mh) / static_cast<float>(qs_.bins);
  if (!(gs > 0.f)) gs = 1.f;
  if (!(hs > 0.f)) hs = 1.f;
  qs_.g_scale = gs; qs_.h_scale = hs;
  const float ig = 1.0f / gs, ih = 1.0f / hs;
  gh_packed_.resize(n);
  const uint32_t seed = static_cast<uint32_t>(cfg_.seed);
  const bool feedback = fixed && plan.quant_ef;
  int8_t* residual = nullptr;
  if (feedback) {
    const int slots = std::max(1, cfg_.num_class);
    if (ef_residual_.size() != static_cast<size_t>(slots) * 2 * n) ef_residual_.assign(static_cast<size_t>(slots) * 2 * n, 0);
    residual = ef_residual_.data() + static_cast<size_t>(tree_index % slots) * 2 * n;   // one slot per class tree of a round
  }
  std::vector<char> in_bag;
  if (feedback && use_bag_) { in_bag.assign(n, 0); for (data_size_t i : bag_) in_bag[i] = 1; }
#pragma omp parallel for schedule(static) num_threads(RowThreads(n))
  for (data_size_t i = 0; i < n; ++i) {
    if (fixed && (feedback || clamp > 0)) {
      // out-of-bag residuals do not move: nothing consumes those rows' values this round
      int8_t* r = (residual != nullptr && (in_bag.empty() || in_bag[i])) ? residual + 2 * static_cast<size_t>(i) : nullptr;
      gh_packed_[i] = QuantizeRowFeedback(grad[i], hess[i], ig, ih, clamp, r);
    } else {
      gh_packed_[i] = QuantizeRow(grad[i], hess[i], ig, ih, qs_.stochastic, seed, static_cast<uint32_t>(tree_index), static_cast<uint64_t>(ds_->global_row_offset + i));
    }
  }
}

void CPUTreeLearner::ConstructHistogram(LeafState* leaf) {
  ScopedTimer timer("CPUTreeLearner::ConstructHistogram");
  const int nb = ds_->num_total_bin, ng = ds_->num_groups;
  const data_size_t* idx = indices_.data() + leaf->begin;
  // large leaves: row blocks on worker threads with private histograms, merged in thread order (integer bins:
  // exact for any thread count; real-valued bins: the summation order follows the thread count)
  // large leaves: row blocks with private histograms, merged in block order (integer bins: exact for any block count;
  // real-valued bins: the summation order follows the block count, which follows the thread limit)
  const int team = omp_get_max_threads();
  const int nblocks = leaf->count >= 8192 ? std::max(1, std::min(team, leaf->count / 4096)) : 1;
  // medium leaves: the feature groups are dealt to the worker threads, each walking all the leaf's rows for its groups. A
  // bin still receives its rows in row order, so the sums are those of the serial loop whatever the thread count.
  const int gchunks = nblocks > 1 ? 1 : std::max(1, std::min(std::min(team, ng / 2), static_cast<int>(static_cast<int64_t>(leaf->count) * ng / 8192)));
  const int* start = ds_->group_bin_start.data();
  if (quant_) leaf->hist_i.assign(2 * static_cast<size_t>(nb), 0); else leaf->hist.assign(2 * static_cast<size_t>(nb), 0.0);
  // rows [lo, hi) of the leaf, groups [g0, g1), into H
  auto accumulate_i = [&](int lo, int hi, int g0, int g1, int64_t* H) {
    for (int k = lo; k < hi; ++k) {
      const data_size_t i = idx[k];
      const int32_t w = gh_packed_[i];
      const int64_t g = UnpackG(w), h = UnpackH(w);
      for (int gidx = g0; gidx < g1; ++gidx) { const int s = start[gidx] + ds_->GroupBin(i, gidx); H[2 * s] += g; H[2 * s + 1] += h; }
    }
  };
  auto accumulate_d = [&](int lo, int hi, int g0, int g1, double* H) {
    for (int k = lo; k < hi; ++k) {
      const data_size_t i = idx[k];
      const double g = grad_[i], h = hess_[i];
      for (int gidx = g0; gidx < g1; ++gidx) { const int s = start[gidx] + ds_->GroupBin(i, gidx); H[2 * s] += g; H[2 * s + 1] += h; }
    }
  };
  const int count = leaf->count;
  if (nblocks > 1) {
    std::vector<std::vector<int64_t>> priv_i(quant_ ? nblocks : 0); std::vector<std::vector<double>> priv_d(quant_ ? 0 : nblocks);
#pragma omp parallel for schedule(static, 1) num_threads(team)
    for (int b = 0; b < nblocks; ++b) {
      const int lo = static_cast<int>(static_cast<int64_t>(count) * b / nblocks), hi = static_cast<int>(static_cast<int64_t>(count) * (b + 1) / nblocks);
      if (quant_) { priv_i[b].assign(2 * static_cast<size_t>(nb), 0); accumulate_i(lo, hi, 0, ng, priv_i[b].data()); }
      else { priv_d[b].assign(2 * static_cast<size_t>(nb), 0.0); accumulate_d(lo, hi, 0, ng, priv_d[b].data()); }
    }
    // merge: bins dealt to the threads, every bin adds its blocks in block order
    const int64_t cells = 2 * static_cast<int64_t>(nb);
#pragma omp parallel for schedule(static) num_threads(team)
    for (int64_t c = 0; c < cells; ++c) {
      if (quant_) { int64_t s = 0; for (int b = 0; b < nblocks; ++b) s += priv_i[b][c]; leaf->hist_i[c] = s; }
      else { double s = 0.0; for (int b = 0; b < nblocks; ++b) s += priv_d[b][c]; leaf->hist[c] = s; }
    }
  } else if (gchunks > 1) {
#pragma omp parallel for schedule(static, 1) num_threads(team)
    for (int c = 0; c < gchunks; ++c) {
      const int g0 = ng * c / gchunks, g1 = ng * (c + 1) / gchunks;
      if (quant_) accumulate_i(0, count, g0, g1, leaf->hist_i.data()); else accumulate_d(0, count, g0, g1, leaf->hist.data());
    }
  } else {
    if (quant_) accumulate_i(0, count, 0, ng, leaf->hist_i.data()); else accumulate_d(0, count, 0, ng, leaf->hist.data());
  }
  leaf->has_hist = true;
  ReduceHistogramAcrossRanks(leaf);
}

void CPUTreeLearner::ReduceHistogramAcrossRanks(LeafState* leaf) {
  if (!(parallel_data_ || parallel_voting_)) return;
  // Data-parallel: sum every rank's local histogram. (The device path reduce-scatters into
  // owners; on the host a full sum followed by owned-feature search is equivalent.)
  if (parallel_voting_) return;   // voting reduces only voted features, inside FindBestSplit
  if (Network::reduce_scatter() != nullptr && Network::world() > 1) {
    // Reduce-scatter: every rank needs the global bins of the features it searches only. The (g, h) pairs of the features
    // owned by rank r are packed one after the other, in feature order, into r's block; what comes back is the sum over
    // the ranks of this rank's block. Bins of the other features keep this rank's local sums: nothing reads them but the
    // subtraction, whose result for those features is local again.
    const int W = Network::world(), R = Network::rank();
    if (rs_counts_.empty()) {
      rs_counts_.assign(W, 0); rs_slots_.assign(W, {});
      for (int f = 0; f < ds_->num_features; ++f) {
        const FeatureMeta& m = ds_->feature_meta[f]; const int n = m.bundled ? m.num_bin - 1 : m.num_bin;
        for (int b = 0; b < n; ++b) rs_slots_[f % W].push_back(m.hist_offset + b);
      }
      for (int r = 0; r < W; ++r) rs_counts_[r] = 2 * static_cast<int64_t>(rs_slots_[r].size());
    }
    int64_t total = 0; for (int r = 0; r < W; ++r) total += rs_counts_[r];
    rs_send_.resize(static_cast<size_t>(total)); rs_recv_.resize(static_cast<size_t>(rs_counts_[R]));
    size_t o = 0;
    for (int r = 0; r < W; ++r) for (int s : rs_slots_[r]) {
      if (quant_) { memcpy(&rs_send_[o], &leaf->hist_i[2 * static_cast<size_t>(s)], 16); } else { memcpy(&rs_send_[o], &leaf->hist[2 * static_cast<size_t>(s)], 16); }
      o += 2;
    }
    Network::reduce_scatter()(rs_send_.data(), rs_counts_.data(), rs_recv_.data(), quant_ ? 1 : 0);
    o = 0;
    for (int s : rs_slots_[R]) {
      if (quant_) memcpy(&leaf->hist_i[2 * static_cast<size_t>(s)], &rs_recv_[o], 16); else memcpy(&leaf->hist[2 * static_cast<size_t>(s)], &rs_recv_[o], 16);
      o += 2;
    }
    return;
  }
  if (quant_) Network::SumInt64(leaf->hist_i.data(), static_cast<int64_t>(leaf->hist_i.size()));
  else Network::SumDouble(leaf->hist.data(), static_cast<int64_t>(leaf->hist.size()));
}

// larger = parent - smaller, in the parent's own buffer (the parent is a leaf no more)
void CPUTreeLearner::SubtractHistogram(LeafState* parent, const LeafState& smaller, LeafState* larger) {
  if (quant_) {
    larger->hist_i = std::move(parent->hist_i);
    int64_t* d = larger->hist_i.data(); const int64_t* s = smaller.hist_i.data();
    for (size_t i = 0, n = larger->hist_i.size(); i < n; ++i) d[i] -= s[i];
  } else {
    larger->hist = std::move(parent->hist);
    double* d = larger->hist.data(); const double* s = smaller.hist.data();
    for (size_t i = 0, n = larger->hist.size(); i < n; ++i) d[i] -= s[i];
  }
  larger->has_hist = true;
}

// Gains of every threshold of one feature from its prefix sums, for the plain regularisation (no L1, no output cap,
// no smoothing, no monotone range): out[t] = gain above `shift`, or -inf where a child is too small or the gain does
// not clear the shift. No iteration depends on another, so the compiler vectorises the loop; every operation is a
// correctly rounded IEEE add / multiply / divide in the order EvalCandidate uses, so the values equal the scalar scan's
// bit for bit whatever the vector width.
#if defined(__x86_64__) && defined(__GNUC__) && !defined(__clang__)
__attribute__((target_clones("default", "avx2", "avx512f")))
#endif
static void PlainGainPass(int n, const double* pg, const double* ph, const double* pc, double sum_g, double sum_h, double num_data, double min_data,
                          double min_h, double l2, double shift, double* out) {
  const double ninf = -std::numeric_limits<double>::infinity();
  for (int t = 0; t < n; ++t) {
    const double lg = pg[t], lh = ph[t], lc = pc[t];
    const double rg = sum_g - lg, rh = sum_h - lh, rc = num_data - lc;
    const double gain = (lg * lg) / ((lh + kEpsilon) + l2) + (rg * rg) / ((rh + kEpsilon) + l2);
    const bool ok = (lc >= min_data) & (rc >= min_data) & (lh >= min_h) & (rh >= min_h) & (gain > shift);
    out[t] = ok ? gain - shift : ninf;
  }
}

// EvalCandidate with separate output ranges for the two children (monotone_constraints_method=advanced): the outputs
// are clamped to their own ranges, a split on a monotone feature must order them, and the gain is taken at the clamped
// outputs. Same primitives and the same order of operations as SplitGain's constrained branch.
static double EvalCandidateBounded(double lg, double lh, int lcnt, const LeafScanInfo& L, const SplitParams& p, int monotone, double lmin, double lmax,
                                   double rmin, double rmax, double* lout, double* rout) {
  const double ninf = -std::numeric_limits<double>::infinity();
  const int rcnt = L.num_data - lcnt;
  const double rg = FB_SUB(L.sum_g, lg), rh = FB_SUB(L.sum_h, lh);
  if (lcnt < p.min_data_in_leaf || rcnt < p.min_data_in_leaf) return ninf;
  if (lh < p.min_sum_hessian_in_leaf || rh < p.min_sum_hessian_in_leaf) return ninf;
  if (lmin > lmax || rmin > rmax) return ninf;   // nothing fits between the neighbours
  const double lhe = FB_ADD(lh, kEpsilon), rhe = FB_ADD(rh, kEpsilon);
  *lout = ClampOutput(LeafOutput(lg, lhe, p, lcnt, L.parent_output), lmin, lmax);
  *rout = ClampOutput(LeafOutput(rg, rhe, p, rcnt, L.parent_output), rmin, rmax);
  if ((monotone > 0 && *lout > *rout) || (monotone < 0 && *lout < *rout)) return ninf;
  const double gain = FB_ADD(LeafGainGivenOutput(lg, lhe, p, *lout), LeafGainGivenOutput(rg, rhe, p, *rout));
  if (!(gain > L.min_gain_shift)) return ninf;
  const double above = FB_SUB(gain, L.min_gain_shift);
  return (monotone != 0 && L.mono_factor != 1.0) ? FB_MUL(above, L.mono_factor) : above;
}

// Numerical threshold search of one feature: one forward prefix over the non-missing bins serves
// both scan directions (see ScanRank in fb/split_math.h).
void CPUTreeLearner::ScanNumerical(const LeafState& leaf, int f, const LeafScanInfo& L, SplitRecord* best) const {
  const FeatureMeta& m = ds_->feature_meta[f];
  const int nb = m.num_bin;
  // The common case - real-valued bins of an unbundled feature without a missing bin, no forced or random threshold -
  // reads the leaf's histogram in place: the same candidates in the same order with the same arithmetic as the general
  // scan below (one pass, default direction left), without its per-call scratch arrays.
  if (!quant_ && !m.bundled && !(m.missing_type != static_cast<int>(MissingType::None) && nb > 2) && !(sp_.extra_trees && nb > 2) &&
      !(forced_bin_ >= 0 && f == forced_feature_) && !mono_advanced_) {
    const double* hist = leaf.hist.data() + 2 * static_cast<size_t>(m.hist_offset);
    double best_gain = -std::numeric_limits<double>::infinity(); int best_t = -1;
    double best_lg = 0, best_lh = 0; int best_lc = 0;
    const double ninf = -std::numeric_limits<double>::infinity();
    const int n = nb - 1;
    if (sp_.lambda_l1 <= 0.0 && sp_.max_delta_step <= 0.0 && sp_.path_smooth <= 0.0 && sp_.use_mc == 0 && m.monotone == 0 && n > 0) {
      static thread_local std::vector<double> buf;
      if (buf.size() < 4 * static_cast<size_t>(n)) buf.resize(4 * static_cast<size_t>(n));
      double* PG = buf.data(); double* PH = PG + n; double* PC = PH + n; double* G = PC + n;
      double pg = 0, ph = 0; int pc = 0;
      for (int t = 0; t < n; ++t) {
        pg += hist[2 * t]; ph += hist[2 * t + 1]; pc += BinCountEstimate(hist[2 * t + 1], L.cnt_factor);
        PG[t] = pg; PH[t] = ph; PC[t] = pc;
      }
      PlainGainPass(n, PG, PH, PC, L.sum_g, L.sum_h, L.num_data, sp_.min_data_in_leaf, sp_.min_sum_hessian_in_leaf, sp_.lambda_l2, L.min_gain_shift, G);
      for (int t = 0; t < n; ++t) if (G[t] != ninf && G[t] >= best_gain) { best_gain = G[t]; best_t = t; }   // equal gains: the higher threshold ranks first (ScanRank, pass 0)
      if (best_t >= 0) { best_lg = PG[best_t]; best_lh = PH[best_t]; best_lc = static_cast<int>(PC[best_t]); }
    } else {
      double pg = 0, ph = 0; int pc = 0;
      for (int t = 0; t < n; ++t) {
        pg += hist[2 * t]; ph += hist[2 * t + 1]; pc += BinCountEstimate(hist[2 * t + 1], L.cnt_factor);
        double lo, ro;
        const double gain = EvalCandidate(pg, ph, pc, L, sp_, m.monotone, &lo, &ro);
        if (gain == ninf) continue;
        if (gain >= best_gain) { best_gain = gain; best_t = t; best_lg = pg; best_lh = ph; best_lc = pc; }
      }
    }
    if (best_t >= 0) {
      SplitRecord cand; InitSplitRecord(&cand);
      cand.gain = best_gain; cand.feature = f; cand.threshold = best_t; cand.default_left = 1;
      cand.left_g = best_lg; cand.left_h = best_lh; cand.right_g = FB_SUB(L.sum_g, best_lg); cand.right_h = FB_SUB(L.sum_h, best_lh);
      cand.left_gi = 0; cand.left_hi = 0; cand.left_cnt = best_lc; cand.right_cnt = L.num_data - best_lc; cand.monotone = m.monotone;
      cand.left_out = ChildOutput(cand.left_g, FB_ADD(cand.left_h, kEpsilon), sp_, cand.left_cnt, L);
      cand.right_out = ChildOutput(cand.right_g, FB_ADD(cand.right_h, kEpsilon), sp_, cand.right_cnt, L);
      cand.gain = FB_MUL(cand.gain, static_cast<double>(m.penalty));
      if (SplitBetter(cand.gain, ds_->feature_meta[cand.feature].real_index, cand.threshold, best->gain,
                      best->feature >= 0 ? ds_->feature_meta[best->feature].real_index : -1, best->threshold)) *best = cand;
    }
    return;
  }
  auto slot = [&](int b) { return m.bundled ? m.hist_offset + (b < m.most_freq_bin ? b : b - 1) : m.hist_offset + b; };
  // per-bin values (integers when quantized)
  // scratch per worker thread: four arrays of nb values, zeroed (no allocation per call)
  static thread_local std::vector<int64_t> scratch_i; static thread_local std::vector<double> scratch_d;
  if (scratch_i.size() < 2 * static_cast<size_t>(nb)) { scratch_i.resize(2 * static_cast<size_t>(nb)); scratch_d.resize(2 * static_cast<size_t>(nb)); }
  std::fill(scratch_i.begin(), scratch_i.begin() + 2 * nb, 0); std::fill(scratch_d.begin(), scratch_d.begin() + 2 * nb, 0.0);
  int64_t* gi = scratch_i.data(); int64_t* hi = gi + nb; double* gd = scratch_d.data(); double* hd = gd + nb;
  if (quant_) {
    int64_t og = 0, oh = 0;
    for (int b = 0; b < nb; ++b) if (!(m.bundled && b == m.most_freq_bin)) { gi[b] = leaf.hist_i[2 * slot(b)]; hi[b] = leaf.hist_i[2 * slot(b) + 1]; og += gi[b]; oh += hi[b]; }
    if (m.bundled) { gi[m.most_freq_bin] = L.sum_gi - og; hi[m.most_freq_bin] = L.sum_hi - oh; }
  } else {
    double og = 0, oh = 0;
    for (int b = 0; b < nb; ++b) if (!(m.bundled && b == m.most_freq_bin)) { gd[b] = leaf.hist[2 * slot(b)]; hd[b] = leaf.hist[2 * slot(b) + 1]; og += gd[b]; oh += hd[b]; }
    if (m.bundled) { gd[m.most_freq_bin] = L.sum_g - og; hd[m.most_freq_bin] = L.sum_h - oh; }
  }
  int skip = -1;
  const bool two_pass = m.missing_type != static_cast<int>(MissingType::None) && nb > 2;
  if (two_pass) skip = m.missing_type == static_cast<int>(MissingType::Zero) ? m.default_bin : nb - 1;
  auto binh = [&](int b) { return quant_ ? FB_MUL(static_cast<double>(hi[b]), L.h_scale) : hd[b]; };
  int64_t mgi = 0, mhi = 0; double mgd = 0, mhd = 0; int mcnt = 0;
  if (skip >= 0) { mgi = gi[skip]; mhi = hi[skip]; mgd = gd[skip]; mhd = hd[skip]; mcnt = BinCountEstimate(binh(skip), L.cnt_factor); }
  int rand_t = -1;
  if (sp_.extra_trees && nb > 2) rand_t = ExtraTreesThreshold(static_cast<uint32_t>(cfg_.extra_seed), cur_tree_index_, leaf.id, m.real_index, nb);
  if (forced_bin_ >= 0 && f == forced_feature_) rand_t = forced_bin_;
  double best_gain = -std::numeric_limits<double>::infinity(); int best_rank = 1 << 30;
  SplitRecord cand; InitSplitRecord(&cand);
  // advanced monotone bounds: per threshold the output range of either child from the neighbours that its part of the
  // cell touches. A neighbour across feature f itself bounds both children at every threshold; a neighbour across
  // another feature touches the left child when its cell starts at or below the threshold and the right child when it
  // ends above it, so the left bounds tighten with a growing threshold and the right bounds loosen.
  static thread_local std::vector<double> adv;   // [lmin | lmax | rmin | rmax][nb]
  const bool advanced = mono_advanced_ && nb >= 2;
  if (advanced) {
    const double inf = std::numeric_limits<double>::infinity();
    adv.assign(4 * static_cast<size_t>(nb), 0.0);
    double* lmin = adv.data(); double* lmax = lmin + nb; double* rmin = lmax + nb; double* rmax = rmin + nb;
    for (int t = 0; t < nb; ++t) { lmin[t] = rmin[t] = -inf; lmax[t] = rmax[t] = inf; }
    for (const LeafState::Neighbour& q : leaf.neighbours) {
      const bool upper = q.dir > 0;   // this leaf lies below the neighbour: the neighbour's output bounds it from above
      int l_from = 0, r_to = nb - 1;  // left child touched for t >= l_from, right child for t <= r_to
      if (q.sep != f) { l_from = q.box[2 * f]; r_to = static_cast<int>(q.box[2 * f + 1]) - 1; }
      for (int t = std::max(0, l_from); t < nb; ++t) { if (upper) lmax[t] = std::min(lmax[t], q.output); else lmin[t] = std::max(lmin[t], q.output); }
      for (int t = 0; t <= std::min(nb - 1, r_to); ++t) { if (upper) rmax[t] = std::min(rmax[t], q.output); else rmin[t] = std::max(rmin[t], q.output); }
    }
  }
  double best_bounds[4] = {L.min_c, L.max_c, L.min_c, L.max_c};
  int64_t pgi = 0, phi = 0; double pgd = 0, phd = 0; int pc = 0;
  for (int t = 0; t <= nb - 2; ++t) {
    if (t != skip) { pgi += gi[t]; phi += hi[t]; pgd += gd[t]; phd += hd[t]; pc += BinCountEstimate(binh(t), L.cnt_factor); }
    if (rand_t >= 0 && t != rand_t) continue;
    for (int pass = 0; pass < (two_pass ? 2 : 1); ++pass) {
      if (t == skip && pass == 1 && m.missing_type == static_cast<int>(MissingType::Zero)) continue;
      int64_t lgi = pgi, lhi = phi; double lg, lh; int lc = pc;
      if (pass == 0 && skip >= 0) { lgi += mgi; lhi += mhi; lc += mcnt; }
      if (quant_) { lg = FB_MUL(static_cast<double>(lgi), L.g_scale); lh = FB_MUL(static_cast<double>(lhi), L.h_scale); }
      else { lg = pgd + ((pass == 0 && skip >= 0) ? mgd : 0.0); lh = phd + ((pass == 0 && skip >= 0) ? mhd : 0.0); }
      double lo, ro;
      const double gain = advanced ? EvalCandidateBounded(lg, lh, lc, L, sp_, m.monotone, adv[t], adv[nb + t], adv[2 * nb + t], adv[3 * nb + t], &lo, &ro)
                                   : EvalCandidate(lg, lh, lc, L, sp_, m.monotone, &lo, &ro);
      if (gain == -std::numeric_limits<double>::infinity()) continue;
      const int rank = ScanRank(pass, t, nb);
      if (gain > best_gain || (gain == best_gain && rank < best_rank)) {
        if (advanced) { best_bounds[0] = adv[t]; best_bounds[1] = adv[nb + t]; best_bounds[2] = adv[2 * nb + t]; best_bounds[3] = adv[3 * nb + t]; }
        best_gain = gain; best_rank = rank;
        cand.gain = gain; cand.feature = f; cand.threshold = t; cand.default_left = pass == 0 ? 1 : 0;
        cand.left_g = lg; cand.left_h = lh; cand.right_g = FB_SUB(L.sum_g, lg); cand.right_h = FB_SUB(L.sum_h, lh);
        cand.left_out = lo; cand.right_out = ro; cand.left_gi = lgi; cand.left_hi = lhi;
        cand.left_cnt = lc; cand.right_cnt = L.num_data - lc; cand.monotone = m.monotone;
      }
    }
  }
  if (cand.feature >= 0) {
    if (advanced) {
      cand.left_out = ClampOutput(LeafOutput(cand.left_g, FB_ADD(cand.left_h, kEpsilon), sp_, cand.left_cnt, L.parent_output), best_bounds[0], best_bounds[1]);
      cand.right_out = ClampOutput(LeafOutput(cand.right_g, FB_ADD(cand.right_h, kEpsilon), sp_, cand.right_cnt, L.parent_output), best_bounds[2], best_bounds[3]);
    } else {
      cand.left_out = ChildOutput(cand.left_g, FB_ADD(cand.left_h, kEpsilon), sp_, cand.left_cnt, L);
      cand.right_out = ChildOutput(cand.right_g, FB_ADD(cand.right_h, kEpsilon), sp_, cand.right_cnt, L);
    }
    cand.gain = FB_MUL(cand.gain, static_cast<double>(m.penalty));
    if (SplitBetter(cand.gain, ds_->feature_meta[cand.feature].real_index, cand.threshold, best->gain,
                    best->feature >= 0 ? ds_->feature_meta[best->feature].real_index : -1, best->threshold)) *best = cand;
  }
}

// Categorical search: one-vs-rest for few categories, otherwise categories sorted by
// sum_g / (sum_h + cat_smooth) and scanned from both ends (many-vs-many).
void CPUTreeLearner::ScanCategorical(const LeafState& leaf, int f, const LeafScanInfo& L, SplitRecord* best) const {
  const FeatureMeta& m = ds_->feature_meta[f];
  const int nb = m.num_bin;
  if (nb > 256) return;
  auto slot = [&](int b) { return m.bundled ? m.hist_offset + (b < m.most_freq_bin ? b : b - 1) : m.hist_offset + b; };
  std::vector<double> g(nb, 0), h(nb, 0);
  std::vector<int64_t> gi(nb, 0), hi(nb, 0);   // quantized: integer sums ride along so that the children keep exact totals
  double og = 0, oh = 0; int64_t ogi = 0, ohi = 0;
  for (int b = 0; b < nb; ++b) if (!(m.bundled && b == m.most_freq_bin)) {
    if (quant_) {
      gi[b] = leaf.hist_i[2 * slot(b)]; hi[b] = leaf.hist_i[2 * slot(b) + 1]; ogi += gi[b]; ohi += hi[b];
      g[b] = FB_MUL(static_cast<double>(gi[b]), L.g_scale); h[b] = FB_MUL(static_cast<double>(hi[b]), L.h_scale);
    } else { g[b] = leaf.hist[2 * slot(b)]; h[b] = leaf.hist[2 * slot(b) + 1]; }
    og = FB_ADD(og, g[b]); oh = FB_ADD(oh, h[b]);
  }
  if (m.bundled) {
    const int q = m.most_freq_bin;
    if (quant_) { gi[q] = L.sum_gi - ogi; hi[q] = L.sum_hi - ohi; g[q] = FB_MUL(static_cast<double>(gi[q]), L.g_scale); h[q] = FB_MUL(static_cast<double>(hi[q]), L.h_scale); }
    else { g[q] = FB_SUB(L.sum_g, og); h[q] = FB_SUB(L.sum_h, oh); }
  }
  SplitParams p = sp_; p.lambda_l2 = FB_ADD(p.lambda_l2, sp_.cat_l2);
  SplitRecord cand; InitSplitRecord(&cand);
  double best_gain = -std::numeric_limits<double>::infinity();
  auto consider = [&](double lg, double lh, int64_t lgi, int64_t lhi, int lc, const std::vector<int>& bins_left) {
    double lo, ro;
    double gain = EvalCandidate(lg, lh, lc, L, p, 0, &lo, &ro);
    if (gain > best_gain) {
      best_gain = gain; cand.gain = gain; cand.feature = f; cand.is_categorical = 1; cand.threshold = 0; cand.default_left = 0;
      cand.left_g = lg; cand.left_h = lh; cand.right_g = FB_SUB(L.sum_g, lg); cand.right_h = FB_SUB(L.sum_h, lh); cand.left_out = lo; cand.right_out = ro;
      cand.left_gi = lgi; cand.left_hi = lhi;
      cand.left_cnt = lc; cand.right_cnt = L.num_data - lc;
      for (int i = 0; i < 8; ++i) cand.cat_bitset[i] = 0;
      for (int b : bins_left) cand.cat_bitset[b >> 5] |= (1u << (b & 31));
      cand.num_cat_bins = static_cast<int>(bins_left.size());
    }
  };
  if (nb <= sp_.max_cat_to_onehot) {
    for (int b = 1; b < nb; ++b) {   // bin 0 (NaN / other) always goes right
      int c = BinCountEstimate(h[b], L.cnt_factor);
      consider(g[b], h[b], gi[b], hi[b], c, {b});
    }
  } else {
    std::vector<int> cats;
    for (int b = 1; b < nb; ++b) if (BinCountEstimate(h[b], L.cnt_factor) >= sp_.cat_smooth) cats.push_back(b);
    auto ratio = [&](int b) { return FB_DIV(g[b], FB_ADD(h[b], sp_.cat_smooth)); };
    std::stable_sort(cats.begin(), cats.end(), [&](int a, int b) { return ratio(a) < ratio(b); });
    const int used = static_cast<int>(cats.size());
    const int max_num = std::min(sp_.max_cat_threshold, (used + 1) / 2);
    for (int dir = 0; dir < 2; ++dir) {
      double lg = 0, lh = 0; int64_t lgi = 0, lhi = 0; int lc = 0, grp = 0; std::vector<int> left;
      for (int k = 0; k < used && k < max_num; ++k) {
        int b = dir == 0 ? cats[k] : cats[used - 1 - k];
        lg = FB_ADD(lg, g[b]); lh = FB_ADD(lh, h[b]); lgi += gi[b]; lhi += hi[b];
        int c = BinCountEstimate(h[b], L.cnt_factor); lc += c; grp += c; left.push_back(b);
        if (grp < sp_.min_data_per_group) continue;
        grp = 0;
        consider(lg, lh, lgi, lhi, lc, left);
      }
    }
  }
  if (cand.feature >= 0) {
    cand.left_out = ChildOutput(cand.left_g, FB_ADD(cand.left_h, kEpsilon), p, cand.left_cnt, L);
    cand.right_out = ChildOutput(cand.right_g, FB_ADD(cand.right_h, kEpsilon), p, cand.right_cnt, L);
    cand.gain = FB_MUL(cand.gain, static_cast<double>(m.penalty));
    if (SplitBetter(cand.gain, m.real_index, 0, best->gain, best->feature >= 0 ? ds_->feature_meta[best->feature].real_index : -1, best->threshold)) *best = cand;
  }
}

void CPUTreeLearner::SyncBestSplit(SplitRecord* rec) const {
  if (!(parallel_data_ || parallel_feature_ || parallel_voting_)) return;
  std::vector<char> all; Network::Gather(rec, sizeof(SplitRecord), &all);
  const SplitRecord* r = reinterpret_cast<const SplitRecord*>(all.data());
  SplitRecord bestr; InitSplitRecord(&bestr);
  for (int k = 0; k < Network::world(); ++k) {
    const int fa = r[k].feature >= 0 ? ds_->feature_meta[r[k].feature].real_index : -1;
    const int fb_ = bestr.feature >= 0 ? ds_->feature_meta[bestr.feature].real_index : -1;
    if (SplitBetter(r[k].gain, fa, r[k].threshold, bestr.gain, fb_, bestr.threshold)) bestr = r[k];
  }
  *rec = bestr;
}

// Everything FindBestSplit settles before the features are scanned: false when the leaf cannot be split at all.
bool CPUTreeLearner::PrepareLeafScan(LeafState* leaf, int leaf_id, int tree_index, LeafScanInfo* Lout, std::vector<int8_t>* mask_out) {
  leaf->id = leaf_id;
  InitSplitRecord(&leaf->best);
  if (!leaf->has_hist) ConstructHistogram(leaf);   // dropped by the histogram pool
  TouchHistogram(leaf);
  if (sp_.max_depth > 0 && leaf->depth >= sp_.max_depth) return false;
  const int64_t n_global = leaf->global_count;
  if (n_global < 2LL * sp_.min_data_in_leaf) return false;
  LeafScanInfo& L = *Lout;
  L.sum_g = leaf->sum_g; L.sum_h = leaf->sum_h; L.sum_gi = leaf->sum_gi; L.sum_hi = leaf->sum_hi;
  L.num_data = static_cast<int>(n_global); L.parent_output = leaf->output; L.min_c = leaf->min_constraint; L.max_c = leaf->max_constraint;
  L.g_scale = quant_ ? qs_.g_scale : 1.0; L.h_scale = quant_ ? qs_.h_scale : 1.0;
  L.mono_factor = MonotonePenaltyFactor(leaf->depth, sp_.monotone_penalty);
  L.cnt_factor = FB_DIV(static_cast<double>(L.num_data), L.sum_h);
  L.min_gain_shift = FB_ADD(LeafGainGivenOutput(L.sum_g, FB_ADD(L.sum_h, 2 * kEpsilon), sp_, leaf->output), sp_.min_gain_to_split);
  if (sp_.max_delta_step <= 0.0 && sp_.path_smooth <= 0.0)
    L.min_gain_shift = FB_ADD(LeafGain(L.sum_g, FB_ADD(L.sum_h, 2 * kEpsilon), sp_, L.num_data, leaf->output), sp_.min_gain_to_split);
  if (mono_advanced_) {
    leaf->neighbours.clear();
    for (int l = 0; l < mono_num_leaves_; ++l) {
      if (l == leaf_id || leaves_[l].box.empty()) continue;
      int sep = -1; const int r = RelateLeaves(leaf_id, l, &sep);
      if (r != 0) leaf->neighbours.push_back({leaves_[l].output, r, sep, leaves_[l].box.data()});
    }
  }
  *mask_out = col_sampler_.by_node() ? col_sampler_.SampleByNode(tree_index, leaf_id + 1000003 * leaf->depth, &leaf->path) : col_sampler_.used_by_tree();
  if (forced_feature_ >= 0) { mask_out->assign(mask_out->size(), 0); (*mask_out)[forced_feature_] = 1; }
  return true;
}

// The per-feature records of one leaf merged in feature order into its best split (SplitBetter is a total order, so the
// result does not depend on which thread scanned which feature).
void CPUTreeLearner::FinishLeafScan(LeafState* leaf, const LeafScanInfo& L, SplitRecord* per) {
  SplitRecord best; InitSplitRecord(&best);
  for (int f = 0; f < ds_->num_features; ++f) {
    SplitRecord& r = per[f];
    if (r.feature < 0) continue;
    if (!cegb_coupled_.empty() || !cegb_lazy_.empty()) { r.gain -= CegbFeaturePenalty(f, *leaf); if (!(r.gain > 0.0)) continue; }
    if (SplitBetter(r.gain, ds_->feature_meta[r.feature].real_index, r.threshold, best.gain, best.feature >= 0 ? ds_->feature_meta[best.feature].real_index : -1, best.threshold)) best = r;
  }
  // Parity: src/treelearner/cost_effective_gradient_boosting.hpp (DeltaGain: tradeoff * penalty_split * rows of the leaf)
  if (best.feature >= 0 && sp_.cegb_split > 0.0) best.gain -= sp_.cegb_split * static_cast<double>(L.num_data);
  SyncBestSplit(&best);
  leaf->best = best;
}

// Several leaves searched in one parallel region (the two children of a split, the children of a whole level): the
// tasks are (leaf, feature) pairs. Same records, same merge order and the same sequence of cross-rank exchanges as one
// FindBestSplit call per leaf in the order given.
void CPUTreeLearner::FindBestSplitMany(const std::vector<int>& ids, int tree_index) {
  if (ids.size() <= 1 || parallel_voting_ || forced_feature_ >= 0) { for (int id : ids) FindBestSplit(&leaves_[id], id, tree_index); return; }
  ScopedTimer timer("CPUTreeLearner::FindBestSplit");
  const int nf = ds_->num_features, nj = static_cast<int>(ids.size());
  std::vector<LeafScanInfo> Ls(nj); std::vector<std::vector<int8_t>> masks(nj); std::vector<char> active(nj, 0);
  for (int j = 0; j < nj; ++j) active[j] = PrepareLeafScan(&leaves_[ids[j]], ids[j], tree_index, &Ls[j], &masks[j]) ? 1 : 0;
  std::vector<SplitRecord> per(static_cast<size_t>(nj) * nf);
  const bool spread = omp_get_max_threads() > 1 && static_cast<int64_t>(nj) * nf >= 4 && static_cast<int64_t>(nj) * ds_->num_total_bin >= 1024;
  const int tasks = nj * nf;
#pragma omp parallel for schedule(dynamic, 1) num_threads(omp_get_max_threads()) if (spread)
  for (int t = 0; t < tasks; ++t) {
    const int j = t / nf, f = t % nf;
    SplitRecord* rec = &per[static_cast<size_t>(t)];
    InitSplitRecord(rec);
    if (!active[j] || !masks[j][f] || !FeatureOwned(f)) continue;
    const LeafState& leaf = leaves_[ids[j]];
    if (ds_->feature_meta[f].bin_type == static_cast<int>(BinType::Numerical)) ScanNumerical(leaf, f, Ls[j], rec);
    else ScanCategorical(leaf, f, Ls[j], rec);
  }
  for (int j = 0; j < nj; ++j) if (active[j]) FinishLeafScan(&leaves_[ids[j]], Ls[j], &per[static_cast<size_t>(j) * nf]);
}

void CPUTreeLearner::FindBestSplit(LeafState* leaf, int leaf_id, int tree_index) {
  ScopedTimer timer("CPUTreeLearner::FindBestSplit");
  LeafScanInfo L; std::vector<int8_t> mask;
  if (!PrepareLeafScan(leaf, leaf_id, tree_index, &L, &mask)) return;

  if (parallel_voting_) {
    // PV-Tree: local top-k by local gain, global vote, reduce only the voted features.
    LeafScanInfo Lloc = L;
    double lg = 0, lh = 0; int64_t lgi = 0, lhi = 0;
    // local totals from any one feature's bins
    { const FeatureMeta& m0 = ds_->feature_meta[0]; const int g0 = m0.group;
      for (int b = 0; b < ds_->group_num_bin[g0]; ++b) { int s = ds_->group_bin_start[g0] + b;
        if (quant_) { lgi += leaf->hist_i[2 * s]; lhi += leaf->hist_i[2 * s + 1]; } else { lg += leaf->hist[2 * s]; lh += leaf->hist[2 * s + 1]; } } }
    if (quant_) { lg = lgi * qs_.g_scale; lh = lhi * qs_.h_scale; }
    Lloc.sum_g = lg; Lloc.sum_h = lh; Lloc.sum_gi = lgi; Lloc.sum_hi = lhi; Lloc.num_data = leaf->count;
    Lloc.cnt_factor = lh > 0 ? leaf->count / lh : 0;
    Lloc.min_gain_shift = LeafGain(lg, lh + 2 * kEpsilon, sp_, leaf->count, leaf->output) + sp_.min_gain_to_split;
    SplitParams save = sp_;
    sp_.min_data_in_leaf = std::max(1, sp_.min_data_in_leaf / Network::world());
    sp_.min_sum_hessian_in_leaf = sp_.min_sum_hessian_in_leaf / Network::world();
    std::vector<std::pair<double, int>> local;
    for (int f = 0; f < ds_->num_features; ++f) {
      if (!mask[f]) continue;
      SplitRecord r; InitSplitRecord(&r);
      if (ds_->feature_meta[f].bin_type == static_cast<int>(BinType::Numerical)) ScanNumerical(*leaf, f, Lloc, &r); else ScanCategorical(*leaf, f, Lloc, &r);
      if (r.feature >= 0) local.emplace_back(r.gain, f);
    }
    sp_ = save;
    std::stable_sort(local.begin(), local.end(), [](const std::pair<double, int>& a, const std::pair<double, int>& b) { return a.first > b.first; });
    const int k = cfg_.top_k;
    std::vector<int32_t> mine(k, -1);
    for (int i = 0; i < k && i < static_cast<int>(local.size()); ++i) mine[i] = local[i].second;
    std::vector<char> all; Network::Gather(mine.data(), k * sizeof(int32_t), &all);
    const int32_t* v = reinterpret_cast<const int32_t*>(all.data());
    std::vector<int> votes(ds_->num_features, 0);
    for (int i = 0; i < k * Network::world(); ++i) if (v[i] >= 0) votes[v[i]]++;
    std::vector<int> order(ds_->num_features); std::iota(order.begin(), order.end(), 0);
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return votes[a] > votes[b]; });
    voted_.assign(ds_->num_features, 0);
    for (int i = 0; i < 2 * k && i < ds_->num_features; ++i) if (votes[order[i]] > 0) voted_[order[i]] = 1;
    // reduce voted features' slots only
    std::vector<int> slots;
    for (int f = 0; f < ds_->num_features; ++f) if (voted_[f]) {
      const FeatureMeta& m = ds_->feature_meta[f]; const int n = m.bundled ? m.num_bin - 1 : m.num_bin;
      for (int b = 0; b < n; ++b) slots.push_back(m.hist_offset + b);
    }
    if (quant_) { std::vector<int64_t> buf(2 * slots.size()); for (size_t i = 0; i < slots.size(); ++i) { buf[2 * i] = leaf->hist_i[2 * slots[i]]; buf[2 * i + 1] = leaf->hist_i[2 * slots[i] + 1]; }
      Network::SumInt64(buf.data(), static_cast<int64_t>(buf.size()));
      voted_hist_i_.assign(leaf->hist_i.size(), 0); for (size_t i = 0; i < slots.size(); ++i) { voted_hist_i_[2 * slots[i]] = buf[2 * i]; voted_hist_i_[2 * slots[i] + 1] = buf[2 * i + 1]; }
    } else { std::vector<double> buf(2 * slots.size()); for (size_t i = 0; i < slots.size(); ++i) { buf[2 * i] = leaf->hist[2 * slots[i]]; buf[2 * i + 1] = leaf->hist[2 * slots[i] + 1]; }
      Network::SumDouble(buf.data(), static_cast<int64_t>(buf.size()));
      voted_hist_.assign(leaf->hist.size(), 0.0); for (size_t i = 0; i < slots.size(); ++i) { voted_hist_[2 * slots[i]] = buf[2 * i]; voted_hist_[2 * slots[i] + 1] = buf[2 * i + 1]; }
    }
    LeafState global = *leaf;   // copy with reduced bins of the voted features
    if (quant_) global.hist_i = voted_hist_i_; else global.hist = voted_hist_;
    SplitRecord best; InitSplitRecord(&best);
    for (int f = 0; f < ds_->num_features; ++f) {
      if (!voted_[f] || f % Network::world() != Network::rank()) continue;
      if (ds_->feature_meta[f].bin_type == static_cast<int>(BinType::Numerical)) ScanNumerical(global, f, L, &best); else ScanCategorical(global, f, L, &best);
    }
    if (best.feature >= 0 && sp_.cegb_split > 0.0) best.gain -= sp_.cegb_split * static_cast<double>(L.num_data);
    SyncBestSplit(&best);
    leaf->best = best;
    return;
  }

  // one record per feature on the worker threads: the whole team or the calling thread alone (a region with a smaller
  // team than the last makes the runtime end and later restart its workers)
  std::vector<SplitRecord> per(ds_->num_features);
  const bool spread = omp_get_max_threads() > 1 && ds_->num_features >= 4 && ds_->num_total_bin >= 1024;
#pragma omp parallel for schedule(dynamic, 1) num_threads(omp_get_max_threads()) if (spread)
  for (int f = 0; f < ds_->num_features; ++f) {
    InitSplitRecord(&per[f]);
    if (!mask[f] || !FeatureOwned(f)) continue;
    if (ds_->feature_meta[f].bin_type == static_cast<int>(BinType::Numerical)) ScanNumerical(*leaf, f, L, &per[f]);
    else ScanCategorical(*leaf, f, L, &per[f]);
  }
  FinishLeafScan(leaf, L, per.data());
}

int CPUTreeLearner::ApplySplit(Tree* tree, int leaf_id) {
  ScopedTimer timer("CPUTreeLearner::ApplySplit");
  LeafState& P = leaves_[leaf_id];
  const SplitRecord s = P.best;
  if (!cegb_coupled_.empty() || !cegb_lazy_.empty()) CegbAfterSplit(s.feature, P);   // before the window is partitioned: the whole leaf passes the split
  const FeatureMeta& m = ds_->feature_meta[s.feature];
  const BinMapper& bm = *ds_->mappers[m.real_index];
  if (DebugFlags::Get().splits)
    Log::Info("[split] leaf %d depth %d feature %d bin %d gain %.9g left (n=%d g=%.9g h=%.9g out=%.9g) right (n=%d g=%.9g h=%.9g out=%.9g)%s", leaf_id, P.depth,
              m.real_index, s.threshold, s.gain, s.left_cnt, s.left_g, s.left_h, s.left_out, s.right_cnt, s.right_g, s.right_h, s.right_out, s.is_categorical ? " categorical" : "");
  // stable partition of the leaf's window
  data_size_t* idx = indices_.data() + P.begin;
  int nl = 0, nr = 0;
  const int nan_bin = m.num_bin - 1;
  if (!s.is_categorical && !m.bundled && ds_->bin_bytes == 1) {
    // the usual case, without a branch per row: both destinations are written and only one cursor moves (idx[nl] never
    // runs ahead of the row being read)
    const uint8_t* col = ds_->bins8.data() + m.group; const size_t stride = static_cast<size_t>(ds_->row_stride);
    const int miss_bin = m.missing_type == 1 ? m.default_bin : (m.missing_type == 2 ? nan_bin : -1);
    const int thr = s.threshold; const int miss_left = s.default_left != 0 ? 1 : 0;
    data_size_t* right_out = tmp_.data();
    for (int k = 0; k < P.count; ++k) {
      const data_size_t i = idx[k];
      const int fbin = col[static_cast<size_t>(i) * stride];
      const int left = fbin == miss_bin ? miss_left : (fbin <= thr ? 1 : 0);
      idx[nl] = i; right_out[nr] = i;
      nl += left; nr += 1 - left;
    }
  } else {
    for (int k = 0; k < P.count; ++k) {
      const data_size_t i = idx[k];
      const int fbin = ds_->FeatureBin(i, s.feature);
      bool left;
      if (s.is_categorical) left = (s.cat_bitset[fbin >> 5] >> (fbin & 31)) & 1;
      else if ((m.missing_type == 1 && fbin == m.default_bin) || (m.missing_type == 2 && fbin == nan_bin)) left = s.default_left != 0;
      else left = fbin <= s.threshold;
      if (left) idx[nl++] = i; else tmp_[nr++] = i;
    }
  }
  std::copy(tmp_.begin(), tmp_.begin() + nr, idx + nl);
  int64_t cnts[2] = {nl, nr};
  if (parallel_data_ || parallel_voting_) Network::SumInt64(cnts, 2);
  const int gl = static_cast<int>(cnts[0]), gr = static_cast<int>(cnts[1]);
  int right_id;
  if (s.is_categorical) {
    std::vector<uint32_t> inner(s.cat_bitset, s.cat_bitset + 8);
    while (inner.size() > 1 && inner.back() == 0) inner.pop_back();
    std::vector<uint32_t> real;
    for (int b = 0; b < m.num_bin; ++b) if ((s.cat_bitset[b >> 5] >> (b & 31)) & 1) {
      int cat = bm.bin_2_categorical[b]; if (cat < 0) continue;
      if (static_cast<int>(real.size()) <= (cat >> 5)) real.resize((cat >> 5) + 1, 0);
      real[cat >> 5] |= (1u << (cat & 31));
    }
    if (real.empty()) real.push_back(0);
    right_id = tree->SplitCategorical(leaf_id, s.feature, m.real_index, inner.data(), static_cast<int>(inner.size()), real.data(),
                                      static_cast<int>(real.size()), s.left_out, s.right_out, gl, gr, s.left_h, s.right_h,
                                      static_cast<float>(s.gain), m.missing_type);
  } else {
    right_id = tree->Split(leaf_id, s.feature, m.real_index, static_cast<uint32_t>(s.threshold), bm.BinToValue(s.threshold),
                           s.left_out, s.right_out, gl, gr, s.left_h, s.right_h, static_cast<float>(s.gain), m.missing_type, s.default_left != 0);
  }
  if (static_cast<int>(leaves_.size()) <= right_id) leaves_.resize(right_id + 1);
  LeafState& Lf = leaves_[leaf_id];     // reference may have moved after resize
  LeafState parent_copy;                // keeps the parent's histogram for the subtraction
  parent_copy.hist.swap(Lf.hist); parent_copy.hist_i.swap(Lf.hist_i);
  LeafState& R = leaves_[right_id];
  R = LeafState();
  R.id = right_id; Lf.id = leaf_id;
  R.begin = Lf.begin + nl; R.count = nr; Lf.count = nl;
  R.depth = Lf.depth + 1; Lf.depth += 1;
  { const int rf = ds_->feature_meta[s.feature].real_index; if (std::find(Lf.path.begin(), Lf.path.end(), rf) == Lf.path.end()) Lf.path.push_back(rf); R.path = Lf.path; }
  R.sum_g = s.right_g; R.sum_h = s.right_h; R.sum_gi = Lf.sum_gi - s.left_gi; R.sum_hi = Lf.sum_hi - s.left_hi;
  Lf.sum_g = s.left_g; Lf.sum_h = s.left_h; Lf.sum_gi = s.left_gi; Lf.sum_hi = s.left_hi;
  R.output = s.right_out; Lf.output = s.left_out;
  R.global_count = gr; Lf.global_count = gl;
  // monotone (basic): children inherit the parent's bounds, tightened at the mid point
  R.min_constraint = Lf.min_constraint; R.max_constraint = Lf.max_constraint;
  mono_dirty_.clear();
  if (mono_intermediate_) {
    R.box = Lf.box;
    if (!s.is_categorical) { Lf.box[2 * s.feature + 1] = static_cast<uint16_t>(s.threshold); R.box[2 * s.feature] = static_cast<uint16_t>(s.threshold + 1); }
    if (mono_advanced_) {   // a child is bounded by what its own cell touches, not by everything the parent's cell touched
      Lf.min_constraint = R.min_constraint = -std::numeric_limits<double>::infinity();
      Lf.max_constraint = R.max_constraint = std::numeric_limits<double>::infinity();
    }
    mono_num_leaves_ = tree->num_leaves;
    TightenMonotoneBounds(tree, leaf_id, right_id);
  } else if (s.monotone != 0) {
    const double mid = (s.left_out + s.right_out) / 2.0;
    if (s.monotone > 0) { Lf.max_constraint = std::min(Lf.max_constraint, mid); R.min_constraint = std::max(R.min_constraint, mid); }
    else { Lf.min_constraint = std::max(Lf.min_constraint, mid); R.max_constraint = std::min(R.max_constraint, mid); }
  }
  // histogram of the smaller child from data, the larger by subtraction. Smaller is decided on
  // GLOBAL counts so that every rank constructs the same child.
  LeafState* smaller = gl <= gr ? &Lf : &R;
  LeafState* larger = gl <= gr ? &R : &Lf;
  const bool parent_kept = quant_ ? !parent_copy.hist_i.empty() : !parent_copy.hist.empty();
  ConstructHistogram(smaller);
  if (parent_kept) SubtractHistogram(&parent_copy, *smaller, larger);
  else ConstructHistogram(larger);   // the pool dropped the parent's histogram: no subtraction to be had
  TouchHistogram(smaller); TouchHistogram(larger);
  if (hist_pool_cap_ > 0) EnforceHistogramPool(tree->num_leaves, leaf_id, right_id);
  return right_id;
}

// monotone_constraints_method=intermediate. Two leaves constrain one another when their cells (boxes in bin space)
// touch along a monotone feature: disjoint in that feature and overlapping in every other one, so that a point can move
// from one leaf to the other by changing that feature alone. The leaf on the lower side (for an increasing feature)
// must not exceed the other's output. After a split the two new leaves are checked against every leaf of the tree
// (and against one another): the lower leaf's upper bound drops to the upper leaf's output and the upper leaf's lower
// bound rises to the lower leaf's output. Older leaves whose range shrank are listed in mono_dirty_; their best
// split was found under the wider range and is searched again by the caller. Bounds only tighten, and an output, once
// set, lies inside its leaf's bounds, so every pair stays ordered. Missing-value bins are not part of the cells.
// Parity: src/treelearner/monotone_constraints.hpp (IntermediateLeafConstraints: bounds from the outputs of the
// contiguous leaves, found there by walking up and down the tree from the split leaf).
// +1: leaf a lies below leaf b along a monotone feature (a's output must not exceed b's), -1: above, 0: the two cells do
// not touch along one feature (apart in two features, or separated by categorical splits only). *sep = that feature.
int CPUTreeLearner::RelateLeaves(int a, int b, int* sep_out) const {
  const int nf = ds_->num_features;
  const uint16_t* A = leaves_[a].box.data(); const uint16_t* B = leaves_[b].box.data();
  int sep = -1, dir = 0;
  for (int f = 0; f < nf; ++f) {
    const bool a_below = A[2 * f + 1] < B[2 * f], b_below = B[2 * f + 1] < A[2 * f];
    if (!a_below && !b_below) continue;
    if (sep >= 0) return 0;
    sep = f; dir = a_below ? 1 : -1;
  }
  *sep_out = sep;
  if (sep < 0) return 0;
  const int mono = ds_->feature_meta[sep].monotone;
  return mono == 0 ? 0 : (mono > 0 ? dir : -dir);
}

void CPUTreeLearner::TightenMonotoneBounds(const Tree* tree, int left_id, int right_id) {
  auto relate = [&](int a, int b) { int sep; return RelateLeaves(a, b, &sep); };
  auto order = [&](int lower, int upper, bool lower_is_new, bool upper_is_new) {
    LeafState& lo = leaves_[lower]; LeafState& up = leaves_[upper];
    if (up.output < lo.max_constraint) { lo.max_constraint = up.output; if (!lower_is_new) mono_dirty_.push_back(lower); }
    if (lo.output > up.min_constraint) { up.min_constraint = lo.output; if (!upper_is_new) mono_dirty_.push_back(upper); }
    // advanced: an older leaf's bounds are per threshold, and a new neighbour can tighten one of them without moving the
    // leaf's overall range, so every older leaf that touches a new one is searched again
    if (mono_advanced_) { if (!lower_is_new) mono_dirty_.push_back(lower); if (!upper_is_new) mono_dirty_.push_back(upper); }
  };
  { const int r = relate(left_id, right_id); if (r > 0) order(left_id, right_id, true, true); else if (r < 0) order(right_id, left_id, true, true); }
  for (int c : {left_id, right_id}) {
    for (int l = 0; l < tree->num_leaves; ++l) {
      if (l == left_id || l == right_id) continue;
      const int r = relate(c, l);
      if (r > 0) order(c, l, true, false); else if (r < 0) order(l, c, false, true);
    }
  }
  std::sort(mono_dirty_.begin(), mono_dirty_.end());
  mono_dirty_.erase(std::unique(mono_dirty_.begin(), mono_dirty_.end()), mono_dirty_.end());
}

void CPUTreeLearner::EnforceHistogramPool(int num_leaves, int keep_a, int keep_b) {
  int held = 0;
  for (int l = 0; l < num_leaves; ++l) held += leaves_[l].has_hist ? 1 : 0;
  while (held > hist_pool_cap_) {
    int victim = -1;
    for (int l = 0; l < num_leaves; ++l)
      if (l != keep_a && l != keep_b && leaves_[l].has_hist && (victim < 0 || leaves_[l].hist_stamp < leaves_[victim].hist_stamp)) victim = l;
    if (victim < 0) break;
    DropHistogram(&leaves_[victim]); --held;
  }
}

double CPUTreeLearner::CegbFeaturePenalty(int inner_feature, const LeafState& leaf) const {
  const int real = ds_->feature_meta[inner_feature].real_index;
  double pen = 0.0;
  if (!cegb_coupled_.empty() && !cegb_feature_used_[real]) pen += cfg_.cegb_tradeoff * cegb_coupled_[real];
  if (!cegb_lazy_.empty() && cegb_lazy_[real] > 0.0) {
    const std::vector<bool>& paid = cegb_row_paid_[real];
    data_size_t unpaid = 0;
    for (data_size_t k = 0; k < leaf.count; ++k) unpaid += paid[indices_[leaf.begin + k]] ? 0 : 1;
    pen += cfg_.cegb_tradeoff * cegb_lazy_[real] * static_cast<double>(unpaid);
  }
  return pen;
}

void CPUTreeLearner::CegbAfterSplit(int inner_feature, const LeafState& leaf) {
  const int real = ds_->feature_meta[inner_feature].real_index;
  if (!cegb_coupled_.empty()) cegb_feature_used_[real] = 1;
  if (!cegb_lazy_.empty() && cegb_lazy_[real] > 0.0) {
    std::vector<bool>& paid = cegb_row_paid_[real];
    for (data_size_t k = 0; k < leaf.count; ++k) paid[indices_[leaf.begin + k]] = true;
  }
}

Tree* CPUTreeLearner::Train(const score_t* grad, const score_t* hess, int tree_index) {
  ScopedTimer timer("CPUTreeLearner::Train");
  grad_ = grad; hess_ = hess; cur_tree_index_ = tree_index;
  col_sampler_.ResetByTree(tree_index);
  if (quant_) Quantize(grad, hess, tree_index);
  std::unique_ptr<Tree> tree(new Tree(cfg_.num_leaves, false, false));
  leaves_.clear(); leaves_.resize(1);
  LeafState& root = leaves_[0];
  const data_size_t n = use_bag_ ? static_cast<data_size_t>(bag_.size()) : ds_->num_data;
  if (use_bag_) std::copy(bag_.begin(), bag_.end(), indices_.begin()); else std::iota(indices_.begin(), indices_.end(), 0);
  root.begin = 0; root.count = n;
  if (quant_) {
    int64_t sg = 0, sh = 0;
    for (data_size_t k = 0; k < n; ++k) { int32_t w = gh_packed_[indices_[k]]; sg += UnpackG(w); sh += UnpackH(w); }
    int64_t s[3] = {sg, sh, n};
    if (parallel_data_ || parallel_voting_) Network::SumInt64(s, 3);
    root.sum_gi = s[0]; root.sum_hi = s[1]; root.global_count = s[2];
    root.sum_g = FB_MUL(static_cast<double>(s[0]), qs_.g_scale); root.sum_h = FB_MUL(static_cast<double>(s[1]), qs_.h_scale);
  } else {
    double sg = 0, sh = 0;
    for (data_size_t k = 0; k < n; ++k) { sg += grad[indices_[k]]; sh += hess[indices_[k]]; }
    double s[2] = {sg, sh}; int64_t c = n;
    if (parallel_data_ || parallel_voting_) { Network::SumDouble(s, 2); Network::SumInt64(&c, 1); }
    root.sum_g = s[0]; root.sum_h = s[1]; root.global_count = c;
  }
  root.output = LeafOutput(root.sum_g, FB_ADD(root.sum_h, 2 * kEpsilon), sp_, static_cast<int>(root.global_count), 0.0);
  if (mono_intermediate_) {
    mono_num_leaves_ = 1;
    root.box.resize(2 * static_cast<size_t>(ds_->num_features));
    for (int f = 0; f < ds_->num_features; ++f) { root.box[2 * f] = 0; root.box[2 * f + 1] = static_cast<uint16_t>(std::min(65535, ds_->feature_meta[f].num_bin - 1)); }
  }
  tree->leaf_value[0] = root.output; tree->leaf_count[0] = static_cast<int>(root.global_count); tree->leaf_weight[0] = root.sum_h;
  ConstructHistogram(&root);
  FindBestSplit(&root, 0, tree_index);
  if (!forced_.empty()) ForceSplits(tree.get(), tree_index);

  if (cfg_.grow_policy == "leaf") {
    while (tree->num_leaves < cfg_.num_leaves) {
      int best_leaf = -1;
      for (int l = 0; l < tree->num_leaves; ++l) {
        const SplitRecord& b = leaves_[l].best;
        if (b.feature < 0 || !(b.gain > 0.0)) continue;
        if (best_leaf < 0 || b.gain > leaves_[best_leaf].best.gain) best_leaf = l;
      }
      if (best_leaf < 0) break;
      int right = ApplySplit(tree.get(), best_leaf);
      const std::vector<int> dirty = mono_dirty_;   // leaves whose monotone range the split tightened
      FindBestSplitMany({best_leaf, right}, tree_index);
      for (int d : dirty) FindBestSplit(&leaves_[d], d, tree_index);
    }
  } else {
    std::vector<int> frontier(tree->num_leaves); std::iota(frontier.begin(), frontier.end(), 0);   // more than the root after forced splits
    while (tree->num_leaves < cfg_.num_leaves && !frontier.empty()) {
      std::vector<int> cand;
      for (int l : frontier) if (leaves_[l].best.feature >= 0 && leaves_[l].best.gain > 0.0) cand.push_back(l);
      if (cand.empty()) break;
      const int budget = cfg_.num_leaves - tree->num_leaves;
      if (static_cast<int>(cand.size()) > budget) {
        std::stable_sort(cand.begin(), cand.end(), [&](int a, int b) {
          if (leaves_[a].best.gain != leaves_[b].best.gain) return leaves_[a].best.gain > leaves_[b].best.gain;
          return a < b; });
        cand.resize(budget);
      }
      std::sort(cand.begin(), cand.end());   // a level's splits are always applied in ascending leaf order
      std::vector<int> next;
      std::vector<char> stale(mono_intermediate_ ? leaves_.size() + 2 * cand.size() : 0, 0);
      for (int l : cand) {
        if (mono_intermediate_ && stale[l]) {   // an earlier split of this level tightened the leaf's monotone range
          FindBestSplit(&leaves_[l], l, tree_index);
          if (leaves_[l].best.feature < 0 || !(leaves_[l].best.gain > 0.0)) continue;
        }
        int r = ApplySplit(tree.get(), l); next.push_back(l); next.push_back(r);
        for (int d : mono_dirty_) if (d < static_cast<int>(stale.size())) stale[d] = 1;
      }
      FindBestSplitMany(next, tree_index);
      frontier.swap(next);
    }
  }
  if (quant_ && cfg_.quant_train_renew_leaf && tree->num_leaves > 1) {
    // leaf values from the unquantized gradients of the rows in each leaf
    std::vector<double> sums(2 * static_cast<size_t>(tree->num_leaves), 0.0);
    for (int l = 0; l < tree->num_leaves; ++l) {
      const data_size_t* idx = indices_.data() + leaves_[l].begin;
      double g = 0, h = 0;
      for (int k = 0; k < leaves_[l].count; ++k) { g += grad[idx[k]]; h += hess[idx[k]]; }
      sums[2 * l] = g; sums[2 * l + 1] = h;
    }
    if (parallel_data_ || parallel_voting_) Network::SumDouble(sums.data(), static_cast<int64_t>(sums.size()));
    // Monotone constraints: with the basic method a leaf's range does not depend on other leaves' outputs, so the renewed
    // output is clamped into it; with the other methods the ranges are the neighbours' (old) outputs and renewing would
    // break the order, so the outputs found during growth stay.
    if (!(sp_.use_mc != 0 && mono_intermediate_))
      for (int l = 0; l < tree->num_leaves; ++l) {
        double out = LeafOutputRaw(sums[2 * l], sums[2 * l + 1] + kEpsilon, sp_);
        if (sp_.use_mc != 0) out = ClampOutput(out, leaves_[l].min_constraint, leaves_[l].max_constraint);
        tree->SetLeafOutput(l, out);
      }
  }
  return tree.release();
}

void CPUTreeLearner::AddPredictionToScore(const Tree* tree, double* score) const {
  for (int l = 0; l < tree->num_leaves; ++l) {
    const double v = tree->leaf_value[l];
    const data_size_t* idx = indices_.data() + leaves_[l].begin;
    for (int k = 0; k < leaves_[l].count; ++k) score[idx[k]] += v;
  }
}

void CPUTreeLearner::RenewTreeOutput(Tree* tree, const ObjectiveFunction* obj, std::function<double(const label_t*, int)> residual,
                                     data_size_t, const data_size_t*, data_size_t, const double* score) const {
  if (obj == nullptr || !obj->IsRenewTreeOutput()) return;
  std::vector<double> outs(tree->num_leaves, 0.0); std::vector<double> have(tree->num_leaves, 0.0);
  for (int l = 0; l < tree->num_leaves; ++l) {
    if (leaves_[l].count == 0) continue;
    outs[l] = obj->RenewTreeOutput(tree->leaf_value[l], score, indices_.data() + leaves_[l].begin, leaves_[l].count);
    have[l] = 1.0;
  }
  if (Network::active() && (parallel_data_ || parallel_voting_)) {
    Network::SumDouble(outs.data(), tree->num_leaves); Network::SumDouble(have.data(), tree->num_leaves);
    for (int l = 0; l < tree->num_leaves; ++l) if (have[l] > 0) outs[l] /= have[l];
  }
  for (int l = 0; l < tree->num_leaves; ++l) if (have[l] > 0) tree->SetLeafOutput(l, outs[l]);
  (void)residual;
}

Tree* CPUTreeLearner::FitByExistingTree(const Tree* old_tree, const score_t* grad, const score_t* hess) const {
  // Route every row down the existing structure, then recompute leaf outputs from the new gradients.
  std::unique_ptr<Tree> tree(new Tree(*old_tree));
  std::vector<double> sg(tree->num_leaves, 0.0), sh(tree->num_leaves, 0.0);
  for (data_size_t i = 0; i < ds_->num_data; ++i) {
    int node = 0;
    if (tree->num_leaves > 1) {
      while (node >= 0) {
        const int f = ds_->used_feature_map[tree->split_feature[node]];
        const FeatureMeta& m = ds_->feature_meta[f];
        const BinMapper& bm = *ds_->mappers[m.real_index];
        const int fbin = ds_->FeatureBin(i, f);
        int thr_bin = bm.bin_type == BinType::Numerical ? bm.ValueToBin(tree->threshold[node]) : 0;
        if (tree->decision_type[node] & kCategoricalMask) {
          int cat = bm.bin_2_categorical[fbin];
          int ci = static_cast<int>(tree->threshold[node]); int lo = tree->cat_boundaries[ci], nn = tree->cat_boundaries[ci + 1] - lo;
          bool left = cat >= 0 && (cat >> 5) < nn && ((tree->cat_threshold[lo + (cat >> 5)] >> (cat & 31)) & 1);
          node = left ? tree->left_child[node] : tree->right_child[node];
        } else {
          const int mt = Tree::MissingTypeOf(tree->decision_type[node]);
          if ((mt == 1 && fbin == m.default_bin) || (mt == 2 && fbin == m.num_bin - 1 && m.missing_type == 2))
            node = (tree->decision_type[node] & kDefaultLeftMask) ? tree->left_child[node] : tree->right_child[node];
          else node = fbin <= thr_bin ? tree->left_child[node] : tree->right_child[node];
        }
      }
    } else node = ~0;
    sg[~node] += grad[i]; sh[~node] += hess[i];
  }
  if (Network::active()) { Network::SumDouble(sg.data(), tree->num_leaves); Network::SumDouble(sh.data(), tree->num_leaves); }
  for (int l = 0; l < tree->num_leaves; ++l) {
    double out = LeafOutputRaw(sg[l], sh[l] + kEpsilon, sp_);
    double old = tree->leaf_value[l];
    tree->SetLeafOutput(l, cfg_.refit_decay_rate * old + (1.0 - cfg_.refit_decay_rate) * out * tree->shrinkage);
  }
  return tree.release();
}

}  // namespace

TreeLearner* CreateCPUTreeLearner(const Config& cfg) { return new CPUTreeLearner(cfg); }

}  // namespace fb
