// Boosting driver. See fb/gbdt.h for the parity notes.
#include "fb/gbdt.h"

#include <numeric>

namespace fb {

GBDT::~GBDT() {}

// FALCATA_DEBUG=dump: every split of a finished tree, in node order (the same line for the host and the device learner)
static void DumpTree(const Tree& t, size_t index) {
  Log::Info("[dump] tree %d: %d leaves, shrinkage %.6g", static_cast<int>(index), t.num_leaves, t.shrinkage);
  for (int s = 0; s + 1 < t.num_leaves; ++s)
    Log::Info("[dump]   node %d: feature %d %s %.17g (bin %u) gain %.9g rows %d -> left %d right %d%s", s, t.split_feature[s],
              (t.decision_type[s] & kCategoricalMask) ? "in set" : "<=", t.threshold[s], s < static_cast<int>(t.threshold_in_bin.size()) ? t.threshold_in_bin[s] : 0u,
              static_cast<double>(t.split_gain[s]), s < static_cast<int>(t.internal_count.size()) ? t.internal_count[s] : -1, t.left_child[s], t.right_child[s],
              (t.decision_type[s] & kDefaultLeftMask) ? " default-left" : "");
  for (int l = 0; l < t.num_leaves; ++l) Log::Info("[dump]   leaf %d: value %.17g rows %d", l, t.leaf_value[l], l < static_cast<int>(t.leaf_count.size()) ? t.leaf_count[l] : -1);
}

void GBDT::Init(const Config& cfg, const Dataset* train, ObjectiveFunction* obj, const std::vector<std::string>& metric_names) {
  config_ = cfg; train_ = train; objective_ = obj; metric_names_ = metric_names;
  if (DebugFlags::Get().maxsplits > 0 && config_.num_leaves > DebugFlags::Get().maxsplits + 1) {
    Log::Warning("FALCATA_DEBUG maxsplits=%d: num_leaves lowered from %d to %d", DebugFlags::Get().maxsplits, config_.num_leaves, DebugFlags::Get().maxsplits + 1);
    config_.num_leaves = DebugFlags::Get().maxsplits + 1;
  }
  is_dart_ = cfg.boosting == "dart"; is_rf_ = cfg.boosting == "rf";
  is_cuda_ = cfg.is_cuda;
  num_class_ = cfg.num_class;
  num_tree_per_iteration_ = obj != nullptr ? obj->NumModelPerIteration() : std::max(1, cfg.num_class);
  shrinkage_rate_ = is_rf_ ? 1.0 : cfg.learning_rate;
  average_output_ = is_rf_;
  drop_rand_ = Random(cfg.drop_seed);
  iter_ = 0;
  if (train != nullptr) {
    max_feature_idx_ = train->num_total_features - 1;
    feature_names_ = train->feature_names;
    feature_infos_.clear();
    for (int j = 0; j < train->num_total_features; ++j)
      feature_infos_.push_back((train->mappers[j] == nullptr || train->mappers[j]->is_trivial) ? "none" : train->mappers[j]->InfoString());
    const size_t total = static_cast<size_t>(train->num_data) * num_tree_per_iteration_;
    class_need_train_.assign(num_tree_per_iteration_, true);
    if (obj != nullptr) for (int k = 0; k < num_tree_per_iteration_; ++k) class_need_train_[k] = obj->ClassNeedTrain(k);
    init_scores_.assign(num_tree_per_iteration_, 0.0);
    // Linear trees on a device booster: the trees grow on the device, the leaf regressions are solved on the host from the
    // raw values the Dataset keeps, and the scores take the difference by row. One GPU, no row sampling (the host does
    // not see the device's bags), host-resident bins and raw values; everything else trains on the host learner.
    const bool sampled_rows = cfg.data_sample_strategy == "goss" || (cfg.bagging_freq > 0 && (cfg.bagging_fraction < 1.0 || cfg.pos_bagging_fraction < 1.0 || cfg.neg_bagging_fraction < 1.0));
    if (cfg.linear_tree && is_cuda_ && (Network::active() || sampled_rows || is_dart_ || is_rf_ || !train->has_raw() || !train->has_host_bins())) {
      Log::Warning("linear_tree with several ranks, row sampling, dart or rf (or without host-resident raw values and bins) trains on the host learner");
      is_cuda_ = false; config_.is_cuda = false; config_.device_type = "cpu";
    }
    if (is_cuda_ && train->max_group_bin > 256) {
      // the device engine keeps one byte per feature group; wider groups (max_bin above 255) are trained by the host learner
      if (!train->has_host_bins()) Log::Fatal("max_bin above 255 needs host-resident bins (the device engine stores one byte per feature group): build the Dataset from host data");
      Log::Warning("max_bin above 255: the device engine stores one byte per feature group, training runs on the host learner");
      is_cuda_ = false; config_.is_cuda = false; config_.device_type = "cpu";
    }
    if ((!cfg.cegb_penalty_feature_coupled.empty() || !cfg.cegb_penalty_feature_lazy.empty()) && is_cuda_) {
      Log::Warning("Per-feature CEGB penalties (cegb_penalty_feature_coupled / _lazy) train on the host learner");
      is_cuda_ = false; config_.is_cuda = false; config_.device_type = "cpu";
    }
    if (!cfg.monotone_vec.empty() && cfg.monotone_constraints_method != "basic" && is_cuda_) {
      Log::Warning("monotone_constraints_method=%s trains on the host learner (the device engine has the basic method)", cfg.monotone_constraints_method.c_str());
      is_cuda_ = false; config_.is_cuda = false; config_.device_type = "cpu";
    }
    if (!cfg.forcedsplits_filename.empty() && is_cuda_ && Network::active() && cfg.tree_learner != "serial") {
      Log::Warning("forcedsplits_filename with several GPUs trains on the host learner (the device engine forces splits on one GPU)");
      is_cuda_ = false; config_.is_cuda = false; config_.device_type = "cpu";
    }
    if (cfg.linear_tree && !train->has_raw()) Log::Fatal("linear_tree needs the raw feature values: build the Dataset from host data with linear_tree=true in its params");
    if (is_rf_ && is_cuda_ && (obj == nullptr || obj->IsRenewTreeOutput())) {
      Log::Warning("boosting=rf with an objective that renews its leaf outputs (or without an objective) trains on the host learner");
      is_cuda_ = false; config_.is_cuda = false; config_.device_type = "cpu";
    }
    if (is_cuda_) {
      ScopedTimer t("GBDT::CreateDeviceEngine");
      engine_.reset(CreateDeviceEngine(config_, train, obj, num_tree_per_iteration_));
    } else {
      learner_.reset(CreateCPUTreeLearner(config_));
      learner_->Init(train, config_);
      train_score_.assign(total, 0.0);
      if (!train->metadata.init_score.empty()) {
        if (train->metadata.init_score.size() != total) Log::Fatal("init_score size does not match num_data * num_class");
        std::copy(train->metadata.init_score.begin(), train->metadata.init_score.end(), train_score_.begin());
      }
      grad_.resize(total); hess_.resize(total);
    }
    metrics_.clear(); metrics_.emplace_back();
    ScopedTimer tm("GBDT::MetricInit");
    for (auto& name : metric_names_) { std::unique_ptr<Metric> m(CreateMetric(name, config_)); if (m) { m->Init(train->metadata, train->num_data); metrics_[0].push_back(std::move(m)); } }
    is_goss_ = cfg.data_sample_strategy == "goss";
    is_bagging_ = !is_goss_ && cfg.bagging_freq > 0 && (cfg.bagging_fraction < 1.0 || cfg.pos_bagging_fraction < 1.0 || cfg.neg_bagging_fraction < 1.0);
    if (engine_ && is_bagging_) engine_->SetBagging(cfg.bagging_fraction, cfg.bagging_freq, cfg.bagging_seed);
    if (!engine_) bag_indices_.resize(train->num_data);   // the device engine draws its own bags
  }
}

// Parity: src/boosting/gbdt.cpp (GBDT::ResetTrainingData: new learner state and score updater, scores replayed tree by tree).
void GBDT::ResetTrainingData(const Config& cfg, const Dataset* train, ObjectiveFunction* obj, const std::vector<std::string>& metric_names) {
  // the existing trees are replayed on the new rows by bin index: that is only meaningful when both datasets bin alike
  if (train_ != nullptr && train != train_ && !models_.empty() && !train_->CheckAlign(*train))
    Log::Fatal("Cannot reset training data: the new dataset's bin mappers differ from the old one's (construct it with reference= the original training data)");
  std::vector<std::unique_ptr<Tree>> models = std::move(models_);
  const int iter = iter_;
  valid_.clear(); valid_score_.clear();
  models_.clear();
  Init(cfg, train, obj, metric_names);
  models_ = std::move(models); iter_ = iter;
  if (!models_.empty()) boosted_from_average_ = true;   // the first tree carries the start score
  const int K = num_tree_per_iteration_;
  for (size_t t = 0; t < models_.size(); ++t) {
    const int k = static_cast<int>(t % K);
    if (engine_) engine_->AddTreeToScores(*models_[t], k, 1.0);
    else AddTreeScore(models_[t].get(), train_, train_score_.data() + static_cast<size_t>(k) * train_->num_data, 1.0);
  }
}

void GBDT::ResetConfig(const Config& cfg) {
  config_.learning_rate = cfg.learning_rate; shrinkage_rate_ = is_rf_ ? 1.0 : cfg.learning_rate;
  Config merged = config_;
  merged.min_data_in_leaf = cfg.min_data_in_leaf; merged.lambda_l1 = cfg.lambda_l1; merged.lambda_l2 = cfg.lambda_l2;
  merged.num_leaves = cfg.num_leaves; merged.max_depth = cfg.max_depth; merged.feature_fraction = cfg.feature_fraction;
  merged.bagging_fraction = cfg.bagging_fraction; merged.bagging_freq = cfg.bagging_freq; merged.min_gain_to_split = cfg.min_gain_to_split;
  merged.min_sum_hessian_in_leaf = cfg.min_sum_hessian_in_leaf;
  config_ = merged;
  if (learner_) learner_->ResetConfig(config_);
  is_bagging_ = !is_goss_ && config_.bagging_freq > 0 && config_.bagging_fraction < 1.0;
}

void GBDT::AddValidData(const Dataset* valid) {
  valid_.push_back(valid);
  metrics_.emplace_back();
  for (auto& name : metric_names_) { std::unique_ptr<Metric> m(CreateMetric(name, config_)); if (m) { m->Init(valid->metadata, valid->num_data); metrics_.back().push_back(std::move(m)); } }
  if (engine_) { engine_->AddValid(valid); return; }
  const size_t total = static_cast<size_t>(valid->num_data) * num_tree_per_iteration_;
  valid_score_.emplace_back(total, 0.0);
  auto& vs = valid_score_.back();
  if (!valid->metadata.init_score.empty()) std::copy(valid->metadata.init_score.begin(), valid->metadata.init_score.end(), vs.begin());
  // bring the new validation scores up to date with the existing model
  for (int k = 0; k < num_tree_per_iteration_; ++k) if (boosted_from_average_ && models_.empty()) for (data_size_t i = 0; i < valid->num_data; ++i) vs[static_cast<size_t>(k) * valid->num_data + i] += init_scores_[k];
  for (size_t t = 0; t < models_.size(); ++t) AddTreeScore(models_[t].get(), valid, vs.data() + static_cast<size_t>(t % num_tree_per_iteration_) * valid->num_data, 1.0);
}

// score[i] += scale * tree(row i), rows routed on binned data.
void GBDT::AddTreeScore(const Tree* tree, const Dataset* ds, double* score, double scale) const {
  if (tree->num_leaves <= 1) { const double v = tree->leaf_value[0] * scale; for (data_size_t i = 0; i < ds->num_data; ++i) score[i] += v; return; }
  if (!ds->has_host_bins()) Log::Fatal("Host traversal needs host-resident bins");
  if (tree->is_linear && !ds->has_raw()) Log::Fatal("A linear tree needs the raw feature values of the dataset it scores (linear_tree=true in the Dataset params)");
#pragma omp parallel for schedule(static) num_threads(RowThreads(ds->num_data))
  for (data_size_t i = 0; i < ds->num_data; ++i) {
    int node = 0;
    while (node >= 0) {
      const int f = tree->split_feature_inner[node];
      const FeatureMeta& m = ds->feature_meta[f];
      node = tree->DecideBin(ds->FeatureBin(i, f), node, m.default_bin, m.num_bin - 1);
    }
    const int leaf = ~node;
    if (!tree->is_linear) { score[i] += scale * tree->leaf_value[leaf]; continue; }
    double out = tree->leaf_const[leaf];
    const float* row = ds->raw.data() + static_cast<size_t>(i) * ds->num_total_features;
    const auto& fs = tree->leaf_features[leaf];
    for (size_t k = 0; k < fs.size(); ++k) {
      const float v = row[fs[k]];
      if (std::isnan(v)) { out = tree->leaf_value[leaf]; break; }
      out += tree->leaf_coeff[leaf][k] * static_cast<double>(v);
    }
    score[i] += scale * out;
  }
}

namespace {
// Solves A x = b for a small dense symmetric system by elimination with partial pivoting; false when singular.
bool SolveDense(std::vector<double>* a_io, std::vector<double>* b_io, int n) {
  std::vector<double>& a = *a_io; std::vector<double>& b = *b_io;
  for (int c = 0; c < n; ++c) {
    int piv = c; double best = std::fabs(a[static_cast<size_t>(c) * n + c]);
    for (int r = c + 1; r < n; ++r) { const double v = std::fabs(a[static_cast<size_t>(r) * n + c]); if (v > best) { best = v; piv = r; } }
    if (!(best > 1e-12)) return false;
    if (piv != c) { for (int k = 0; k < n; ++k) std::swap(a[static_cast<size_t>(c) * n + k], a[static_cast<size_t>(piv) * n + k]); std::swap(b[c], b[piv]); }
    const double inv = 1.0 / a[static_cast<size_t>(c) * n + c];
    for (int r = c + 1; r < n; ++r) {
      const double f = a[static_cast<size_t>(r) * n + c] * inv;
      if (f == 0.0) continue;
      for (int k = c; k < n; ++k) a[static_cast<size_t>(r) * n + k] -= f * a[static_cast<size_t>(c) * n + k];
      b[r] -= f * b[c];
    }
  }
  for (int c = n - 1; c >= 0; --c) {
    double v = b[c];
    for (int k = c + 1; k < n; ++k) v -= a[static_cast<size_t>(c) * n + k] * b[k];
    b[c] = v / a[static_cast<size_t>(c) * n + c];
    if (!std::isfinite(b[c])) return false;
  }
  return true;
}
}  // namespace

// Piecewise-linear leaves: for every leaf, a second-order fit of the leaf's rows on the numerical features of its
// root path, coefficients = -(X^T H X + lambda I)^-1 X^T g with an unpenalised intercept. Rows with a missing value
// in a path feature stay on the constant output (kept in leaf_value). The first tree stays constant.
// Parity: src/treelearner/linear_tree_learner.cpp (CalculateLinear: path features, per-leaf normal equations,
// linear_lambda on the diagonal, fall back to the constant when a leaf has too few rows).
void GBDT::FitLinearLeaves(Tree* tree, const float* grad, const float* hess, bool constant_only) const {
  const int nl = tree->num_leaves;
  tree->is_linear = true;
  tree->leaf_const.assign(tree->leaf_value.begin(), tree->leaf_value.end());
  tree->leaf_coeff.assign(tree->leaf_value.size(), {}); tree->leaf_features.assign(tree->leaf_value.size(), {}); tree->leaf_features_inner.assign(tree->leaf_value.size(), {});
  if (constant_only || nl <= 1) return;
  const Dataset* ds = train_;
  if (!ds->has_raw()) Log::Fatal("linear_tree needs the raw feature values: build the Dataset from host data with linear_tree=true in its params");
  // numerical features on the path of every leaf
  std::vector<std::vector<int>> path(nl);
  {
    std::vector<std::pair<int, std::vector<int>>> stack; stack.push_back({0, {}});
    while (!stack.empty()) {
      auto cur = std::move(stack.back()); stack.pop_back();
      const int node = cur.first;
      if (node < 0) { std::sort(cur.second.begin(), cur.second.end()); cur.second.erase(std::unique(cur.second.begin(), cur.second.end()), cur.second.end()); path[~node] = std::move(cur.second); continue; }
      std::vector<int> f = cur.second;
      if (!(tree->decision_type[node] & kCategoricalMask)) f.push_back(tree->split_feature_inner[node]);
      stack.push_back({tree->left_child[node], f}); stack.push_back({tree->right_child[node], std::move(f)});
    }
  }
  // leaf of every fitting row (the bag when one is drawn)
  const bool bagged = (is_bagging_ || is_goss_) && bag_cnt_ > 0 && bag_cnt_ < ds->num_data;
  const data_size_t m = bagged ? bag_cnt_ : ds->num_data;
  std::vector<int> leaf_of(m);
#pragma omp parallel for schedule(static) num_threads(TeamThreads())
  for (data_size_t t = 0; t < m; ++t) {
    const data_size_t i = bagged ? bag_indices_[t] : t;
    int node = 0;
    while (node >= 0) {
      const int f = tree->split_feature_inner[node];
      const FeatureMeta& fm = ds->feature_meta[f];
      node = tree->DecideBin(ds->FeatureBin(i, f), node, fm.default_bin, fm.num_bin - 1);
    }
    leaf_of[t] = ~node;
  }
  std::vector<std::vector<data_size_t>> rows(nl);
  for (data_size_t t = 0; t < m; ++t) rows[leaf_of[t]].push_back(bagged ? bag_indices_[t] : t);
  const int ncol = ds->num_total_features;
  const double lambda = config_.linear_lambda;
#pragma omp parallel for schedule(dynamic) num_threads(TeamThreads())
  for (int leaf = 0; leaf < nl; ++leaf) {
    const int d = static_cast<int>(path[leaf].size());
    if (d == 0) continue;
    std::vector<int> real(d);
    for (int k = 0; k < d; ++k) real[k] = ds->real_feature_idx[path[leaf][k]];
    const int dim = d + 1;
    std::vector<double> A(static_cast<size_t>(dim) * dim, 0.0), b(dim, 0.0), x(dim);
    data_size_t used = 0;
    for (data_size_t i : rows[leaf]) {
      const float* r = ds->raw.data() + static_cast<size_t>(i) * ncol;
      bool nan = false;
      for (int k = 0; k < d; ++k) { x[k] = r[real[k]]; if (std::isnan(x[k])) { nan = true; break; } }
      if (nan) continue;
      x[d] = 1.0;
      const double g = grad[i], h = hess[i];
      for (int p = 0; p < dim; ++p) { b[p] -= g * x[p]; const double hx = h * x[p]; for (int q = p; q < dim; ++q) A[static_cast<size_t>(p) * dim + q] += hx * x[q]; }
      ++used;
    }
    if (used < static_cast<data_size_t>(dim)) continue;   // too few rows: the constant stays
    for (int p = 0; p < dim; ++p) for (int q = 0; q < p; ++q) A[static_cast<size_t>(p) * dim + q] = A[static_cast<size_t>(q) * dim + p];
    for (int p = 0; p < d; ++p) A[static_cast<size_t>(p) * dim + p] += lambda;
    if (!SolveDense(&A, &b, dim)) continue;
    std::vector<double> coeff; std::vector<int> feats, inner;
    for (int k = 0; k < d; ++k) {
      if (std::fabs(b[k]) <= kZeroThreshold) continue;
      coeff.push_back(b[k]); feats.push_back(real[k]); inner.push_back(path[leaf][k]);
    }
    tree->leaf_const[leaf] = b[d]; tree->leaf_coeff[leaf] = std::move(coeff); tree->leaf_features[leaf] = std::move(feats); tree->leaf_features_inner[leaf] = std::move(inner);
  }
}

// Linear leaves for trees that the device engine has just grown (and already added to its scores with constant leaves):
// the round's gradients come down, the regressions are solved on the host as for a host-grown tree, and every data set's
// scores take (linear tree - constant tree) by row. The first round's trees stay constant, as on the host.
void GBDT::FitLinearLeavesOnDeviceTrees(std::vector<std::unique_ptr<Tree>>* trees) {
  const int K = num_tree_per_iteration_;
  const data_size_t n = train_->num_data;
  const bool first_round = models_.size() < static_cast<size_t>(K);
  std::vector<float> hg, hh, delta;
  for (int k = 0; k < K && k < static_cast<int>(trees->size()); ++k) {
    Tree* tree = (*trees)[k].get();
    if (tree->num_leaves <= 1) continue;               // a constant tree stays a plain tree, as on the host
    if (first_round) { FitLinearLeaves(tree, nullptr, nullptr, true); continue; }
    const Tree constant = *tree;                       // what the device scores hold for this tree
    hg.resize(n); hh.resize(n);
    engine_->DownloadGradients(k, hg.data(), hh.data());
    tree->Shrink(1.0 / shrinkage_rate_);               // the regressions are solved on the unshrunk outputs
    FitLinearLeaves(tree, hg.data(), hh.data(), false);
    tree->Shrink(shrinkage_rate_);
    auto push_difference = [&](const Dataset* ds, int data_idx) {
      if (!ds->has_host_bins() || !ds->has_raw()) Log::Fatal("linear_tree on a device booster needs host-resident bins and raw values in every data set (build them from host data with linear_tree=true)");
      std::vector<double> d(static_cast<size_t>(ds->num_data), 0.0);
      AddTreeScore(tree, ds, d.data(), 1.0);
      AddTreeScore(&constant, ds, d.data(), -1.0);
      delta.assign(d.begin(), d.end());
      engine_->AddRowValuesToScores(data_idx, k, delta.data());
    };
    push_difference(train_, 0);
    for (size_t v = 0; v < valid_.size(); ++v) push_difference(valid_[v], static_cast<int>(v) + 1);
  }
}

void GBDT::BoostFromAverage(int k, double* out) {
  *out = 0.0;
  if (models_.empty() && !boosted_from_average_ && objective_ != nullptr && config_.boost_from_average && train_->metadata.init_score.empty()) {
    double init = objective_->BoostFromScore(k);
    if (std::fabs(init) > kEpsilon) { *out = init; Log::Info("Start training from score %f", init); }
  }
}

void GBDT::Bagging(int iter, const float* grad, const float* hess) {
  const data_size_t n = train_->num_data;
  if (is_goss_) {
    // gradient-based one-side sampling: keep the top_rate largest |g*h|, sample other_rate of the rest
    if (iter < static_cast<int>(1.0 / config_.learning_rate)) { learner_->SetBaggingData(nullptr, 0); bag_cnt_ = n; return; }
    std::vector<float> mag(n, 0.f);
    for (int k = 0; k < num_tree_per_iteration_; ++k) for (data_size_t i = 0; i < n; ++i) mag[i] += std::fabs(grad[static_cast<size_t>(k) * n + i] * hess[static_cast<size_t>(k) * n + i]);
    const data_size_t top_k = std::max<data_size_t>(1, static_cast<data_size_t>(config_.top_rate * n));
    const data_size_t other_k = static_cast<data_size_t>(config_.other_rate * n);
    std::vector<float> tmp(mag); std::nth_element(tmp.begin(), tmp.begin() + (top_k - 1), tmp.end(), std::greater<float>());
    const float thr = tmp[top_k - 1];
    const float multiply = static_cast<float>(n - top_k) / std::max<data_size_t>(1, other_k);
    // the small-gradient rows are kept independently with probability other_k / (n - top_k): a draw keyed on the
    // global row id, so the device engine and any rank count make the same choice
    data_size_t cnt = 0;
    const double prob = n > top_k ? static_cast<double>(other_k) / static_cast<double>(n - top_k) : 0.0;
    float* g = const_cast<float*>(grad); float* h = const_cast<float*>(hess);
    for (data_size_t i = 0; i < n; ++i) {
      if (mag[i] >= thr) { bag_indices_[cnt++] = i; continue; }
      const float u = U01From24(Philox4x32_10(static_cast<uint32_t>(train_->global_row_offset + i), static_cast<uint32_t>(iter), 0x60550000u, 0, static_cast<uint32_t>(config_.bagging_seed), 0x1234u).v[0]);
      if (static_cast<double>(u) < prob) {
        bag_indices_[cnt++] = i;
        for (int k = 0; k < num_tree_per_iteration_; ++k) { g[static_cast<size_t>(k) * n + i] *= multiply; h[static_cast<size_t>(k) * n + i] *= multiply; }
      }
    }
    bag_cnt_ = cnt;
    learner_->SetBaggingData(bag_indices_.data(), bag_cnt_);
    return;
  }
  if (!is_bagging_) { bag_cnt_ = n; return; }
  if (iter % config_.bagging_freq != 0 && bag_cnt_ > 0) return;   // keep the previous bag
  const bool balanced = config_.pos_bagging_fraction < 1.0 || config_.neg_bagging_fraction < 1.0;
  const uint32_t round = static_cast<uint32_t>(iter / config_.bagging_freq);
  data_size_t cnt = 0;
  if (config_.bagging_by_query && !train_->metadata.query_boundaries.empty()) {
    const auto& qb = train_->metadata.query_boundaries;
    for (data_size_t q = 0; q + 1 < static_cast<data_size_t>(qb.size()); ++q) {
      const float u = U01From24(Philox4x32_10(static_cast<uint32_t>(q), round, 0xBA660000u, 1, static_cast<uint32_t>(config_.bagging_seed), 0x9876u).v[0]);
      if (u < config_.bagging_fraction) for (data_size_t i = qb[q]; i < qb[q + 1]; ++i) bag_indices_[cnt++] = i;
    }
  } else {
    for (data_size_t i = 0; i < n; ++i) {
      const float u = U01From24(Philox4x32_10(static_cast<uint32_t>(train_->global_row_offset + i), round, 0xBA660000u, 0, static_cast<uint32_t>(config_.bagging_seed), 0x9876u).v[0]);
      double frac = config_.bagging_fraction;
      if (balanced) frac = train_->metadata.label[i] > 0 ? config_.pos_bagging_fraction : config_.neg_bagging_fraction;
      if (u < frac) bag_indices_[cnt++] = i;
    }
  }
  bag_cnt_ = cnt;
  learner_->SetBaggingData(bag_indices_.data(), bag_cnt_);
}

bool GBDT::CheckDivergence(const float* grad, int64_t n) {
  // every 32 iterations after 64: a 50x growth of the gradient norm since the start is reported
  if (iter_ < 64 && first_grad_norm_ >= 0) return false;
  if (iter_ % 32 != 0 && first_grad_norm_ >= 0) return false;
  double s = 0; for (int64_t i = 0; i < n; ++i) s += static_cast<double>(grad[i]) * grad[i];
  const double norm = std::sqrt(s / std::max<int64_t>(1, n));
  if (first_grad_norm_ < 0) { first_grad_norm_ = norm; return false; }
  if (!std::isfinite(norm) || (first_grad_norm_ > 0 && norm > 50.0 * first_grad_norm_)) {
    Log::Warning("Gradient norm grew from %g to %g: training may be diverging (lower learning_rate or set max_delta_step)", first_grad_norm_, norm);
    return true;
  }
  return false;
}

void GBDT::DartDropTrees() {
  drop_index_.clear();
  const int iters = current_iteration();
  const bool skip = drop_rand_.NextFloat() < config_.skip_drop;
  if (!skip && iters > 0) {
    double rate = config_.drop_rate;
    if (!config_.uniform_drop) {
      double inv_avg = sum_weight_ > 0 ? iters / sum_weight_ : 1.0;
      if (config_.max_drop > 0) rate = std::min(rate, config_.max_drop * inv_avg / std::max(1.0, sum_weight_));
      for (int i = 0; i < iters; ++i) if (drop_rand_.NextFloat() < rate * tree_weight_[i] * inv_avg) { drop_index_.push_back(i); if (config_.max_drop > 0 && static_cast<int>(drop_index_.size()) >= config_.max_drop) break; }
    } else {
      if (config_.max_drop > 0) rate = std::min(rate, config_.max_drop / static_cast<double>(iters));
      for (int i = 0; i < iters; ++i) if (drop_rand_.NextFloat() < rate) { drop_index_.push_back(i); if (config_.max_drop > 0 && static_cast<int>(drop_index_.size()) >= config_.max_drop) break; }
    }
  }
  for (int i : drop_index_) for (int k = 0; k < num_tree_per_iteration_; ++k) {
    const Tree* t = models_[static_cast<size_t>(i) * num_tree_per_iteration_ + k].get();
    if (engine_) engine_->AddTreeToScores(*t, k, -1.0, 1);   // device scores: the training rows only, the validation scores keep the tree until it is rescaled
    else AddTreeScore(t, train_, train_score_.data() + static_cast<size_t>(k) * train_->num_data, -1.0);
  }
  const double k = static_cast<double>(drop_index_.size());
  if (!config_.xgboost_dart_mode) shrinkage_rate_ = config_.learning_rate / (1.0 + k);
  else shrinkage_rate_ = drop_index_.empty() ? config_.learning_rate : config_.learning_rate / (config_.learning_rate + k);
}

void GBDT::DartNormalize() {
  const double k = static_cast<double>(drop_index_.size());
  for (int i : drop_index_) for (int c = 0; c < num_tree_per_iteration_; ++c) {
    Tree* t = models_[static_cast<size_t>(i) * num_tree_per_iteration_ + c].get();
    // validation scores still contain the full old tree; train scores contain none of it
    const double factor = config_.xgboost_dart_mode ? k / (k + config_.learning_rate) : k / (k + 1.0);
    if (engine_) {
      engine_->AddTreeToScores(*t, c, factor - 1.0, 2);
      t->Shrink(factor);
      engine_->AddTreeToScores(*t, c, 1.0, 1);
    } else {
      for (size_t v = 0; v < valid_.size(); ++v) AddTreeScore(t, valid_[v], valid_score_[v].data() + static_cast<size_t>(c) * valid_[v]->num_data, factor - 1.0);
      t->Shrink(factor);
      AddTreeScore(t, train_, train_score_.data() + static_cast<size_t>(c) * train_->num_data, 1.0);
    }
    if (!config_.uniform_drop && c == 0) { sum_weight_ -= tree_weight_[i] * (1.0 - factor); tree_weight_[i] *= factor; }
  }
  if (!config_.uniform_drop) { tree_weight_.push_back(shrinkage_rate_); sum_weight_ += shrinkage_rate_; }
}

void GBDT::UpdateScore(const Tree* tree, int k) {
  const data_size_t n = train_->num_data;
  double* ts = train_score_.data() + static_cast<size_t>(k) * n;
  if (tree->num_leaves > 1 && !(is_bagging_ || is_goss_) && !tree->is_linear) learner_->AddPredictionToScore(tree, ts);
  else AddTreeScore(tree, train_, ts, 1.0);   // bagging: out-of-bag rows need the traversal
  for (size_t v = 0; v < valid_.size(); ++v) AddTreeScore(tree, valid_[v], valid_score_[v].data() + static_cast<size_t>(k) * valid_[v]->num_data, 1.0);
}

bool GBDT::TrainOneIter(const float* grad_in, const float* hess_in) {
  ScopedTimer timer("GBDT::TrainOneIter");
  const int K = num_tree_per_iteration_;
  std::vector<double> inits(K, 0.0);
  if (grad_in == nullptr || hess_in == nullptr) {
    if (objective_ == nullptr) Log::Fatal("No objective function provided and no custom gradients given");
    ScopedTimer t("GBDT::BoostFromAverage");
    for (int k = 0; k < K; ++k) BoostFromAverage(k, &inits[k]);
  }
  if (models_.empty() && !boosted_from_average_) {
    boosted_from_average_ = true;
    for (int k = 0; k < K; ++k) {
      init_scores_[k] = inits[k];
      if (inits[k] == 0.0) continue;
      if (engine_) engine_->AddConstantToScores(inits[k], k);
      else {
        double* ts = train_score_.data() + static_cast<size_t>(k) * train_->num_data;
        for (data_size_t i = 0; i < train_->num_data; ++i) ts[i] += inits[k];
        for (size_t v = 0; v < valid_.size(); ++v) { double* vs = valid_score_[v].data() + static_cast<size_t>(k) * valid_[v]->num_data; for (data_size_t i = 0; i < valid_[v]->num_data; ++i) vs[i] += inits[k]; }
      }
    }
  } else {
    std::fill(inits.begin(), inits.end(), 0.0);
  }

  if (engine_) {
    std::vector<std::unique_ptr<Tree>> trees; bool all_const = false;
    ScopedTimer te("GBDT::EngineIter");
    if (is_dart_) DartDropTrees();   // the dropped trees leave the device's training scores; sets this round's shrinkage
    if (is_rf_) {
      // Random forest on the device: every tree is trained on the gradients at the start score (computed once on the
      // host and handed to the engine as this round's gradients), with shrinkage 1; the device scores hold the running
      // mean of the trees' outputs: s <- m s, the engine adds the new tree, s <- (s + start score) / (m + 1).
      const data_size_t n = train_->num_data;
      if (grad_in == nullptr) {
        if (rf_init_scores_.empty()) {
          rf_init_scores_.assign(static_cast<size_t>(n) * K, 0.0);
          for (int k = 0; k < K; ++k) for (data_size_t i = 0; i < n; ++i) rf_init_scores_[static_cast<size_t>(k) * n + i] = init_scores_[k];
          grad_.resize(static_cast<size_t>(n) * K); hess_.resize(static_cast<size_t>(n) * K);
          objective_->GetGradients(rf_init_scores_.data(), grad_.data(), hess_.data());
          engine_->UploadGradients(grad_.data(), hess_.data(), &rf_dev_grad_, &rf_dev_hess_);   // the engine reads device memory only
        }
        grad_in = rf_dev_grad_; hess_in = rf_dev_hess_;
      }
      const double m = static_cast<double>(iter_);
      engine_->ScaleScores(m, {});
      std::vector<double> zeros(K, 0.0);
      engine_->TrainOneIter(grad_in, hess_in, iter_, 1.0, zeros, &trees, &all_const);
      if (all_const) { if (m > 0.0) engine_->ScaleScores(1.0 / m, {}); }   // nothing was added: back to the mean of the m trees
      else {
        std::vector<double> bias(K, 0.0);
        for (int k = 0; k < K; ++k) bias[k] = init_scores_[k] / (m + 1.0);
        engine_->ScaleScores(1.0 / (m + 1.0), bias);
      }
      if (!all_const) for (int k = 0; k < K && k < static_cast<int>(trees.size()); ++k) if (std::fabs(init_scores_[k]) > kEpsilon) trees[k]->AddBias(init_scores_[k]);
    } else {
      engine_->TrainOneIter(grad_in, hess_in, iter_, shrinkage_rate_, inits, &trees, &all_const);
    }
    if (all_const) {
      if (is_dart_)   // nothing was learnt this round: the dropped trees go back into the training scores as they were
        for (int i : drop_index_) for (int k = 0; k < K; ++k) engine_->AddTreeToScores(*models_[static_cast<size_t>(i) * K + k], k, 1.0, 1);
      Log::Warning("Stopped training because there are no more leaves that meet the split requirements");
      if (models_.empty()) for (auto& t : trees) models_.push_back(std::move(t));
      return true;
    }
    if (config_.linear_tree) FitLinearLeavesOnDeviceTrees(&trees);
    for (auto& t : trees) { if (DebugFlags::Get().dump) DumpTree(*t, models_.size()); models_.push_back(std::move(t)); }
    if (is_dart_) DartNormalize();
    ++iter_;
    return false;
  }

  const data_size_t n = train_->num_data;
  if (is_dart_) DartDropTrees();
  const float* grad = grad_in; const float* hess = hess_in;
  if (grad == nullptr) {
    if (is_rf_) {
      if (iter_ == 0 || rf_init_scores_.empty()) {
        rf_init_scores_.assign(static_cast<size_t>(n) * K, 0.0);
        for (int k = 0; k < K; ++k) for (data_size_t i = 0; i < n; ++i) rf_init_scores_[static_cast<size_t>(k) * n + i] = init_scores_[k];
        objective_->GetGradients(rf_init_scores_.data(), grad_.data(), hess_.data());
      }
    } else {
      objective_->GetGradients(train_score_.data(), grad_.data(), hess_.data());
    }
    grad = grad_.data(); hess = hess_.data();
  } else {
    std::copy(grad_in, grad_in + static_cast<size_t>(n) * K, grad_.begin()); std::copy(hess_in, hess_in + static_cast<size_t>(n) * K, hess_.begin());
    grad = grad_.data(); hess = hess_.data();
  }
  CheckDivergence(grad, static_cast<int64_t>(n) * K);
  Bagging(iter_, grad, hess);
  bool should_continue = false;
  for (int k = 0; k < K; ++k) {
    std::unique_ptr<Tree> tree(new Tree(2));
    if (class_need_train_[k] && train_->num_features > 0) {
      tree.reset(learner_->Train(grad + static_cast<size_t>(k) * n, hess + static_cast<size_t>(k) * n, iter_ * K + k));
    }
    if (tree->num_leaves > 1) {
      should_continue = true;
      if (objective_ != nullptr && objective_->IsRenewTreeOutput()) {
        std::vector<double> sc(train_score_.begin() + static_cast<size_t>(k) * n, train_score_.begin() + static_cast<size_t>(k + 1) * n);
        if (is_rf_) std::fill(sc.begin(), sc.end(), init_scores_[k]);
        learner_->RenewTreeOutput(tree.get(), objective_, nullptr, n, bag_indices_.data(), bag_cnt_, sc.data());
      }
      if (config_.linear_tree) FitLinearLeaves(tree.get(), grad + static_cast<size_t>(k) * n, hess + static_cast<size_t>(k) * n, models_.size() < static_cast<size_t>(K));
      tree->Shrink(shrinkage_rate_);
      if (is_rf_) {
        // forests average: train/valid scores hold the running mean
        const double m = static_cast<double>(iter_);
        double* ts = train_score_.data() + static_cast<size_t>(k) * n;
        if (std::fabs(init_scores_[k]) > kEpsilon) tree->AddBias(init_scores_[k]);
        for (data_size_t i = 0; i < n; ++i) ts[i] *= m;
        for (size_t v = 0; v < valid_.size(); ++v) { double* vs = valid_score_[v].data() + static_cast<size_t>(k) * valid_[v]->num_data; for (data_size_t i = 0; i < valid_[v]->num_data; ++i) vs[i] *= m; }
        AddTreeScore(tree.get(), train_, ts, 1.0);
        for (size_t v = 0; v < valid_.size(); ++v) AddTreeScore(tree.get(), valid_[v], valid_score_[v].data() + static_cast<size_t>(k) * valid_[v]->num_data, 1.0);
        for (data_size_t i = 0; i < n; ++i) ts[i] /= (m + 1);
        for (size_t v = 0; v < valid_.size(); ++v) { double* vs = valid_score_[v].data() + static_cast<size_t>(k) * valid_[v]->num_data; for (data_size_t i = 0; i < valid_[v]->num_data; ++i) vs[i] /= (m + 1); }
      } else {
        UpdateScore(tree.get(), k);
        if (std::fabs(inits[k]) > kEpsilon) tree->AddBias(inits[k]);
      }
    } else {
      // constant tree: keeps the model aligned (one tree per class per iteration)
      if (models_.size() < static_cast<size_t>(K)) {
        double out = 0.0;
        if (!class_need_train_[k] && objective_ != nullptr) out = objective_->BoostFromScore(k); else out = inits[k];
        tree->AsConstantTree(out);
        if (!class_need_train_[k]) { double* ts = train_score_.data() + static_cast<size_t>(k) * n; for (data_size_t i = 0; i < n; ++i) ts[i] += out; }
      } else tree->AsConstantTree(0.0);
    }
    if (DebugFlags::Get().dump) DumpTree(*tree, models_.size());
    models_.push_back(std::move(tree));
  }
  if (!should_continue) {
    Log::Warning("Stopped training because there are no more leaves that meet the split requirements");
    if (models_.size() > static_cast<size_t>(K)) for (int k = 0; k < K; ++k) models_.pop_back();
    return true;
  }
  if (is_dart_) DartNormalize();
  ++iter_;
  return false;
}

void GBDT::RollbackOneIter() {
  if (iter_ <= 0) return;
  const int K = num_tree_per_iteration_;
  for (int k = 0; k < K; ++k) {
    const Tree* t = models_[models_.size() - K + k].get();
    if (engine_) engine_->AddTreeToScores(*t, k, -1.0);
    else {
      AddTreeScore(t, train_, train_score_.data() + static_cast<size_t>(k) * train_->num_data, -1.0);
      for (size_t v = 0; v < valid_.size(); ++v) AddTreeScore(t, valid_[v], valid_score_[v].data() + static_cast<size_t>(k) * valid_[v]->num_data, -1.0);
    }
  }
  for (int k = 0; k < K; ++k) models_.pop_back();
  --iter_;
}

std::vector<std::string> GBDT::EvalNames() const {
  std::vector<std::string> out;
  if (!metrics_.empty()) for (auto& m : metrics_[0]) for (auto& s : m->Names()) out.push_back(s);
  return out;
}
std::vector<bool> GBDT::EvalHigherBetter() const {
  std::vector<bool> out;
  if (!metrics_.empty()) for (auto& m : metrics_[0]) for (size_t i = 0; i < m->Names().size(); ++i) out.push_back(m->HigherBetter());
  return out;
}

std::vector<double> GBDT::GetEval(int data_idx) const {
  std::vector<double> out;
  if (data_idx < 0 || data_idx >= static_cast<int>(metrics_.size())) return out;
  const Dataset* ds = data_idx == 0 ? train_ : valid_[data_idx - 1];
  std::vector<double> host;
  const double* score = nullptr;
  bool host_ready = false;
  for (auto& m : metrics_[data_idx]) {
    if (engine_) {
      bool ok = false;
      auto names = m->Names();
      std::vector<double> v = engine_->EvalMetric(data_idx, names[0].substr(0, names[0].find('@')), &ok);
      if (ok && v.size() == names.size()) { out.insert(out.end(), v.begin(), v.end()); continue; }
      if (!host_ready) { host.resize(static_cast<size_t>(ds->num_data) * num_tree_per_iteration_); engine_->CopyScoresToHost(data_idx, host.data()); host_ready = true; }
      score = host.data();
    } else score = data_idx == 0 ? train_score_.data() : valid_score_[data_idx - 1].data();
    auto v = m->Eval(score, objective_);
    out.insert(out.end(), v.begin(), v.end());
  }
  return out;
}

int64_t GBDT::GetNumPredict(int data_idx) const {
  const Dataset* ds = data_idx == 0 ? train_ : valid_[data_idx - 1];
  return static_cast<int64_t>(ds->num_data) * num_tree_per_iteration_;
}

void GBDT::GetPredictAt(int data_idx, double* out) const {
  const Dataset* ds = data_idx == 0 ? train_ : valid_[data_idx - 1];
  const data_size_t n = ds->num_data; const int K = num_tree_per_iteration_;
  std::vector<double> host;
  const double* score;
  if (engine_) { host.resize(static_cast<size_t>(n) * K); engine_->CopyScoresToHost(data_idx, host.data()); score = host.data(); }
  else score = data_idx == 0 ? train_score_.data() : valid_score_[data_idx - 1].data();
  std::vector<double> raw(K), conv(K);
  for (data_size_t i = 0; i < n; ++i) {
    for (int k = 0; k < K; ++k) raw[k] = score[static_cast<size_t>(k) * n + i];
    if (objective_ != nullptr) objective_->ConvertOutput(raw.data(), conv.data()); else conv = raw;
    for (int k = 0; k < K; ++k) out[static_cast<size_t>(k) * n + i] = conv[k];
  }
}

void GBDT::RefitTree(const int* leaf_preds, int nrow, int ncol) {
  if (learner_ == nullptr) Log::Fatal("refit runs on the host learner (device_type=cpu)");
  if (nrow != train_->num_data || ncol != static_cast<int>(models_.size())) Log::Fatal("leaf prediction shape does not match");
  const int K = num_tree_per_iteration_; const data_size_t n = train_->num_data;
  std::fill(train_score_.begin(), train_score_.end(), 0.0);
  if (!train_->metadata.init_score.empty()) std::copy(train_->metadata.init_score.begin(), train_->metadata.init_score.end(), train_score_.begin());
  const int iters = static_cast<int>(models_.size()) / K;
  for (int it = 0; it < iters; ++it) {
    objective_->GetGradients(train_score_.data(), grad_.data(), hess_.data());
    for (int k = 0; k < K; ++k) {
      const int ti = it * K + k;
      Tree* t = models_[ti].get();
      std::vector<double> sg(t->num_leaves, 0.0), sh(t->num_leaves, 0.0);
      for (data_size_t i = 0; i < n; ++i) { const int leaf = leaf_preds[static_cast<size_t>(i) * ncol + ti]; sg[leaf] += grad_[static_cast<size_t>(k) * n + i]; sh[leaf] += hess_[static_cast<size_t>(k) * n + i]; }
      for (int l = 0; l < t->num_leaves; ++l) {
        const double out = -sg[l] / (sh[l] + config_.lambda_l2 + kEpsilon);
        t->SetLeafOutput(l, config_.refit_decay_rate * t->leaf_value[l] + (1.0 - config_.refit_decay_rate) * out * t->shrinkage);
      }
      double* ts = train_score_.data() + static_cast<size_t>(k) * n;
      for (data_size_t i = 0; i < n; ++i) ts[i] += t->leaf_value[leaf_preds[static_cast<size_t>(i) * ncol + ti]];
    }
  }
}

void GBDT::ShuffleModels(int start, int end) {
  const int K = num_tree_per_iteration_; const int iters = static_cast<int>(models_.size()) / K;
  start = std::max(0, start); if (end <= 0 || end > iters) end = iters;
  std::vector<int> idx(iters); std::iota(idx.begin(), idx.end(), 0);
  Random r(17);
  for (int i = start; i < end - 1; ++i) { int j = r.NextInt(i + 1, end); std::swap(idx[i], idx[j]); }
  std::vector<std::unique_ptr<Tree>> old; old.swap(models_);
  for (int i = 0; i < iters; ++i) for (int k = 0; k < K; ++k) models_.push_back(std::move(old[static_cast<size_t>(idx[i]) * K + k]));
}

void GBDT::MergeFrom(const GBDT* other) {
  std::vector<std::unique_ptr<Tree>> merged;
  for (auto& t : other->models_) merged.emplace_back(new Tree(*t));
  for (auto& t : models_) merged.push_back(std::move(t));
  models_.swap(merged);
}

// ------------------------------------------------------------ prediction ----
int GBDT::NumPredictOneRow(int predict_type, int start_iter, int num_iter) const {
  const int K = num_tree_per_iteration_; int iters = static_cast<int>(models_.size()) / K;
  start_iter = std::max(0, std::min(start_iter, iters));
  int use = num_iter > 0 ? std::min(num_iter, iters - start_iter) : iters - start_iter;
  if (predict_type == 2) return use * K;
  if (predict_type == 3) {
    // every prediction entry point sizes its output through here, outside any parallel region
    if (falb_without_stats_)
      Log::Fatal("Feature contributions need the per-node counts, which this binary model was saved without; save it with with_stats=true or use the text model");
    return K * (max_feature_idx_ + 2);
  }
  return K;
}

PredictParams PredictParams::FromString(const char* parameter) {
  PredictParams pp;
  if (parameter == nullptr || *parameter == 0) return pp;
  auto m = Config::Str2Map(parameter);
  auto truthy = [](const std::string& v) { return v == "true" || v == "1" || v == "True" || v == "+"; };
  if (m.count("pred_early_stop")) pp.early_stop = truthy(m["pred_early_stop"]);
  if (m.count("pred_early_stop_freq")) pp.early_stop_freq = std::max(1, atoi(m["pred_early_stop_freq"].c_str()));
  if (m.count("pred_early_stop_margin")) pp.early_stop_margin = ParseDouble(m["pred_early_stop_margin"]);
  if (m.count("predict_disable_shape_check")) pp.disable_shape_check = truthy(m["predict_disable_shape_check"]);
  return pp;
}

void GBDT::PredictRow(const double* row, int predict_type, int start_iter, int num_iter, double* out, const PredictParams& pp) const {
  const int K = num_tree_per_iteration_; int iters = static_cast<int>(models_.size()) / K;
  start_iter = std::max(0, std::min(start_iter, iters));
  const int use = num_iter > 0 ? std::min(num_iter, iters - start_iter) : iters - start_iter;
  const int begin = start_iter * K, end = (start_iter + use) * K;
  if (predict_type == 2) { for (int t = begin; t < end; ++t) out[t - begin] = models_[t]->LeafIndex(row); return; }
  if (predict_type == 3) {
    const int nf = max_feature_idx_ + 1;
    std::fill(out, out + static_cast<size_t>(K) * (nf + 1), 0.0);
    for (int t = begin; t < end; ++t) models_[t]->PredictContrib(row, nf, out + static_cast<size_t>(t % K) * (nf + 1));
    return;
  }
  std::vector<double> raw(K, 0.0);
  const bool early = pp.early_stop && predict_type == 0 && (K > 1 || (objective_ && std::string(objective_->GetName()) == "binary"));
  for (int t = begin; t < end; ++t) {
    raw[t % K] += models_[t]->Predict(row);
    if (early && ((t - begin + 1) % (pp.early_stop_freq * K) == 0)) {
      double margin;
      if (K == 1) margin = 2.0 * std::fabs(raw[0]);
      else { std::vector<double> s(raw); std::partial_sort(s.begin(), s.begin() + 2, s.end(), std::greater<double>()); margin = s[0] - s[1]; }
      if (margin > pp.early_stop_margin) break;
    }
  }
  if (average_output_ && use > 0) for (int k = 0; k < K; ++k) raw[k] /= use;
  if (predict_type == 1 || objective_ == nullptr) { for (int k = 0; k < K; ++k) out[k] = raw[k]; }
  else objective_->ConvertOutput(raw.data(), out);
}

void GBDT::PredictMat(const void* data, int dtype, int nrow, int ncol, bool row_major, int predict_type, int start_iter, int num_iter, double* out, const PredictParams& pp) const {
  const int per = NumPredictOneRow(predict_type, start_iter, num_iter);
  if (ncol <= max_feature_idx_ && !pp.disable_shape_check)
    Log::Fatal("The number of features in data (%d) is not the same as it was in training data (%d)", ncol, max_feature_idx_ + 1);
#pragma omp parallel num_threads(TeamThreads())
  {
    std::vector<double> row(std::max(ncol, max_feature_idx_ + 1), 0.0);
#pragma omp for schedule(static)
    for (int i = 0; i < nrow; ++i) {
      for (int j = 0; j < ncol; ++j) {
        const size_t src = row_major ? static_cast<size_t>(i) * ncol + j : static_cast<size_t>(j) * nrow + i;
        switch (dtype) {
          case kF32: row[j] = static_cast<const float*>(data)[src]; break;
          case kF64: row[j] = static_cast<const double*>(data)[src]; break;
          case kI8: row[j] = static_cast<const int8_t*>(data)[src]; break;
          case kI16: row[j] = static_cast<const int16_t*>(data)[src]; break;
          case kU8: row[j] = static_cast<const uint8_t*>(data)[src]; break;
          case kU16: row[j] = static_cast<const uint16_t*>(data)[src]; break;
          case kI32: row[j] = static_cast<const int32_t*>(data)[src]; break;
          default: row[j] = 0.0;
        }
      }
      PredictRow(row.data(), predict_type, start_iter, num_iter, out + static_cast<size_t>(i) * per, pp);
    }
  }
}

double GBDT::UpperBound() const { double s = 0; for (auto& t : models_) { double m = t->leaf_value[0]; for (int l = 1; l < t->num_leaves; ++l) m = std::max(m, t->leaf_value[l]); s += m; } return s; }
double GBDT::LowerBound() const { double s = 0; for (auto& t : models_) { double m = t->leaf_value[0]; for (int l = 1; l < t->num_leaves; ++l) m = std::min(m, t->leaf_value[l]); s += m; } return s; }

}  // namespace fb
