// Host objective functions. Formulas follow the reference semantics:
//   regression family : src/objective/regression_objective.hpp:L94-752
//   binary            : src/objective/binary_objective.hpp:L22-196
//   multiclass / OVA  : src/objective/multiclass_objective.hpp:L25-263
//   cross entropy     : src/objective/xentropy_objective.hpp:L45-277
//   lambdarank/xendcg : src/objective/rank_objective.hpp:L26-459
#include "fb/objective.h"
#include "fb/learner.h"
#include "fb/kinds.h"

#include <numeric>

namespace fb {

namespace {

inline double Sign(double x) { return (x > 0) - (x < 0); }

// Weighted percentile of values[idx[k]] over a subset. alpha in [0,1].
template <typename GetV, typename GetW>
double WeightedPercentile(int cnt, double alpha, GetV getv, GetW getw, bool weighted) {
  if (cnt <= 0) return 0.0;
  std::vector<int> order(cnt); std::iota(order.begin(), order.end(), 0);
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return getv(a) < getv(b); });
  if (!weighted) {
    if (cnt == 1) return getv(order[0]);
    const double pos = alpha * (cnt - 1);   // linear interpolation between order statistics
    int lo = static_cast<int>(std::floor(pos)); int hi = std::min(cnt - 1, lo + 1);
    double frac = pos - lo;
    return getv(order[lo]) * (1 - frac) + getv(order[hi]) * frac;
  }
  double total = 0; for (int i = 0; i < cnt; ++i) total += getw(i);
  double thr = alpha * total, acc = 0;
  for (int k = 0; k < cnt; ++k) { acc += getw(order[k]); if (acc >= thr) return getv(order[k]); }
  return getv(order[cnt - 1]);
}

class RegressionBase : public ObjectiveFunction {
 public:
  explicit RegressionBase(const Config& cfg) : sqrt_(cfg.reg_sqrt), cfg_(cfg) {}
  void Init(const Metadata& md, data_size_t n) override {
    n_ = n; label_ = md.label.data(); weights_ = md.weights.empty() ? nullptr : md.weights.data();
    if (sqrt_) { trans_.resize(n); for (data_size_t i = 0; i < n; ++i) trans_[i] = static_cast<label_t>(Sign(label_[i]) * std::sqrt(std::fabs(label_[i]))); label_ = trans_.data(); }
  }
  void ConvertOutput(const double* in, double* out) const override { out[0] = sqrt_ ? Sign(in[0]) * in[0] * in[0] : in[0]; }
  std::string ToString() const override { std::string s = GetName(); if (sqrt_) s += " sqrt"; return s; }
  double MeanLabel() const {
    // fixed-point integer accumulation: the sum does not depend on the order or on how rows are
    // sharded over ranks, so the init score is bit-identical at any rank count
    const double kScale = 1048576.0;
    int64_t acc[2] = {0, 0}; double sw = 0;
    for (data_size_t i = 0; i < n_; ++i) {
      const double w = weights_ ? weights_[i] : 1.0;
      acc[0] += llround(static_cast<double>(label_[i]) * w * kScale); sw += w;
    }
    acc[1] = llround(sw * kScale);
    Network::SumInt64(acc, 2);
    return acc[1] != 0 ? static_cast<double>(acc[0]) / static_cast<double>(acc[1]) : 0.0;
  }
  double PercentileLabel(double alpha) const {
    return WeightedPercentile(n_, alpha, [&](int i) { return static_cast<double>(label_[i]); }, [&](int i) { return static_cast<double>(weights_[i]); }, weights_ != nullptr);
  }
 protected:
  bool sqrt_; Config cfg_;
  data_size_t n_ = 0; const label_t* label_ = nullptr; const label_t* weights_ = nullptr;
  std::vector<label_t> trans_;
};

class RegressionL2 : public RegressionBase {
 public:
  using RegressionBase::RegressionBase;
  const char* GetName() const override { return "regression"; }
  void GetGradients(const double* s, score_t* g, score_t* h) const override {
#pragma omp parallel for schedule(static) num_threads(RowThreads(n_))
    for (data_size_t i = 0; i < n_; ++i) { const double w = weights_ ? weights_[i] : 1.0; g[i] = static_cast<score_t>((s[i] - label_[i]) * w); h[i] = static_cast<score_t>(w); }
  }
  bool IsConstantHessian() const override { return weights_ == nullptr; }
  double BoostFromScore(int) const override { return MeanLabel(); }
  int DeviceKind() const override { return kObjL2; }
};

class RegressionL1 : public RegressionBase {
 public:
  using RegressionBase::RegressionBase;
  const char* GetName() const override { return "regression_l1"; }
  void GetGradients(const double* s, score_t* g, score_t* h) const override {
    for (data_size_t i = 0; i < n_; ++i) { const double w = weights_ ? weights_[i] : 1.0; g[i] = static_cast<score_t>(Sign(s[i] - label_[i]) * w); h[i] = static_cast<score_t>(w); }
  }
  bool IsConstantHessian() const override { return weights_ == nullptr; }
  bool IsRenewTreeOutput() const override { return true; }
  double BoostFromScore(int) const override { return PercentileLabel(0.5); }
  double RenewTreeOutput(double, const double* score, const data_size_t* idx, int cnt) const override {
    return WeightedPercentile(cnt, 0.5, [&](int k) { return static_cast<double>(label_[idx[k]]) - score[idx[k]]; }, [&](int k) { return static_cast<double>(weights_[idx[k]]); }, weights_ != nullptr);
  }
  int DeviceKind() const override { return kObjL1; }
};

class RegressionHuber : public RegressionBase {
 public:
  explicit RegressionHuber(const Config& cfg) : RegressionBase(cfg), alpha_(cfg.alpha) {}
  const char* GetName() const override { return "huber"; }
  void GetGradients(const double* s, score_t* g, score_t* h) const override {
    for (data_size_t i = 0; i < n_; ++i) {
      const double w = weights_ ? weights_[i] : 1.0, d = s[i] - label_[i];
      g[i] = static_cast<score_t>((std::fabs(d) <= alpha_ ? d : Sign(d) * alpha_) * w); h[i] = static_cast<score_t>(w);
    }
  }
  bool IsConstantHessian() const override { return weights_ == nullptr; }
  double BoostFromScore(int) const override { return MeanLabel(); }
  int DeviceKind() const override { return kObjHuber; }
  double DeviceParam(int) const override { return alpha_; }
 private:
  double alpha_;
};

class RegressionFair : public RegressionBase {
 public:
  explicit RegressionFair(const Config& cfg) : RegressionBase(cfg), c_(cfg.fair_c) {}
  const char* GetName() const override { return "fair"; }
  void GetGradients(const double* s, score_t* g, score_t* h) const override {
    for (data_size_t i = 0; i < n_; ++i) {
      const double w = weights_ ? weights_[i] : 1.0, x = s[i] - label_[i], d = std::fabs(x) + c_;
      g[i] = static_cast<score_t>(c_ * x / d * w); h[i] = static_cast<score_t>(c_ * c_ / (d * d) * w);
    }
  }
  int DeviceKind() const override { return kObjFair; }
  double DeviceParam(int) const override { return c_; }
 private:
  double c_;
};

class RegressionPoisson : public RegressionBase {
 public:
  explicit RegressionPoisson(const Config& cfg) : RegressionBase(cfg), mds_(cfg.poisson_max_delta_step) { sqrt_ = false; }
  const char* GetName() const override { return "poisson"; }
  void Init(const Metadata& md, data_size_t n) override {
    RegressionBase::Init(md, n);
    for (data_size_t i = 0; i < n; ++i) if (label_[i] < 0) Log::Fatal("[poisson]: at least one target label is negative");
  }
  void GetGradients(const double* s, score_t* g, score_t* h) const override {
    const double em = std::exp(mds_);
    for (data_size_t i = 0; i < n_; ++i) {
      const double w = weights_ ? weights_[i] : 1.0, e = std::exp(s[i]);
      g[i] = static_cast<score_t>((e - label_[i]) * w); h[i] = static_cast<score_t>(e * em * w);
    }
  }
  void ConvertOutput(const double* in, double* out) const override { out[0] = std::exp(in[0]); }
  double BoostFromScore(int) const override { return std::log(std::max(1e-10, MeanLabel())); }
  int DeviceKind() const override { return kObjPoisson; }
  double DeviceParam(int) const override { return mds_; }
 protected:
  double mds_;
};

class RegressionQuantile : public RegressionBase {
 public:
  explicit RegressionQuantile(const Config& cfg) : RegressionBase(cfg), alpha_(cfg.alpha) {}
  const char* GetName() const override { return "quantile"; }
  void GetGradients(const double* s, score_t* g, score_t* h) const override {
    for (data_size_t i = 0; i < n_; ++i) {
      const double w = weights_ ? weights_[i] : 1.0, d = s[i] - label_[i];
      g[i] = static_cast<score_t>((d >= 0 ? (1.0 - alpha_) : -alpha_) * w); h[i] = static_cast<score_t>(w);
    }
  }
  bool IsConstantHessian() const override { return weights_ == nullptr; }
  bool IsRenewTreeOutput() const override { return true; }
  double BoostFromScore(int) const override { return PercentileLabel(alpha_); }
  double RenewTreeOutput(double, const double* score, const data_size_t* idx, int cnt) const override {
    return WeightedPercentile(cnt, alpha_, [&](int k) { return static_cast<double>(label_[idx[k]]) - score[idx[k]]; }, [&](int k) { return static_cast<double>(weights_[idx[k]]); }, weights_ != nullptr);
  }
  int DeviceKind() const override { return kObjQuantile; }
  double DeviceParam(int) const override { return alpha_; }
 private:
  double alpha_;
};

class RegressionMAPE : public RegressionBase {
 public:
  using RegressionBase::RegressionBase;
  const char* GetName() const override { return "mape"; }
  void Init(const Metadata& md, data_size_t n) override {
    RegressionBase::Init(md, n);
    lw_.resize(n);
    for (data_size_t i = 0; i < n; ++i) lw_[i] = static_cast<label_t>((weights_ ? weights_[i] : 1.0) / std::max(1.0, std::fabs(static_cast<double>(label_[i]))));
  }
  void GetGradients(const double* s, score_t* g, score_t* h) const override {
    for (data_size_t i = 0; i < n_; ++i) { g[i] = static_cast<score_t>(Sign(s[i] - label_[i]) * lw_[i]); h[i] = weights_ ? weights_[i] : 1.0f; }
  }
  bool IsRenewTreeOutput() const override { return true; }
  double BoostFromScore(int) const override {
    return WeightedPercentile(n_, 0.5, [&](int i) { return static_cast<double>(label_[i]); }, [&](int i) { return static_cast<double>(lw_[i]); }, true);
  }
  double RenewTreeOutput(double, const double* score, const data_size_t* idx, int cnt) const override {
    return WeightedPercentile(cnt, 0.5, [&](int k) { return static_cast<double>(label_[idx[k]]) - score[idx[k]]; }, [&](int k) { return static_cast<double>(lw_[idx[k]]); }, true);
  }
  int DeviceKind() const override { return kObjMape; }
 private:
  std::vector<label_t> lw_;
};

class RegressionGamma : public RegressionPoisson {
 public:
  using RegressionPoisson::RegressionPoisson;
  const char* GetName() const override { return "gamma"; }
  void GetGradients(const double* s, score_t* g, score_t* h) const override {
    for (data_size_t i = 0; i < n_; ++i) {
      const double w = weights_ ? weights_[i] : 1.0, e = std::exp(-s[i]);
      g[i] = static_cast<score_t>((1.0 - label_[i] * e) * w); h[i] = static_cast<score_t>(label_[i] * e * w);
    }
  }
  int DeviceKind() const override { return kObjGamma; }
};

class RegressionTweedie : public RegressionPoisson {
 public:
  explicit RegressionTweedie(const Config& cfg) : RegressionPoisson(cfg), rho_(cfg.tweedie_variance_power) {}
  const char* GetName() const override { return "tweedie"; }
  void GetGradients(const double* s, score_t* g, score_t* h) const override {
    for (data_size_t i = 0; i < n_; ++i) {
      const double w = weights_ ? weights_[i] : 1.0, e1 = std::exp((1 - rho_) * s[i]), e2 = std::exp((2 - rho_) * s[i]);
      g[i] = static_cast<score_t>((-label_[i] * e1 + e2) * w); h[i] = static_cast<score_t>((-label_[i] * (1 - rho_) * e1 + (2 - rho_) * e2) * w);
    }
  }
  int DeviceKind() const override { return kObjTweedie; }
  double DeviceParam(int) const override { return rho_; }
 private:
  double rho_;
};

class BinaryLogloss : public ObjectiveFunction {
 public:
  explicit BinaryLogloss(const Config& cfg, std::function<bool(label_t)> is_pos = nullptr)
      : sigmoid_(cfg.sigmoid), unbalance_(cfg.is_unbalance), spw_(cfg.scale_pos_weight), is_pos_(is_pos) {
    if (sigmoid_ <= 0.0) Log::Fatal("Sigmoid parameter %f should be greater than zero", sigmoid_);
    if (unbalance_ && std::fabs(spw_ - 1.0) > 1e-6) Log::Fatal("Cannot set is_unbalance and scale_pos_weight at the same time");
    if (!is_pos_) is_pos_ = [](label_t l) { return l > 0; };
  }
  const char* GetName() const override { return "binary"; }
  void Init(const Metadata& md, data_size_t n) override {
    n_ = n; label_ = md.label.data(); weights_ = md.weights.empty() ? nullptr : md.weights.data();
    int64_t cnt[2] = {0, 0};
    { int64_t c0 = 0, c1 = 0;
#pragma omp parallel for schedule(static) reduction(+ : c0, c1) num_threads(TeamThreads())
      for (data_size_t i = 0; i < n; ++i) { if (is_pos_(label_[i])) ++c0; else ++c1; }
      cnt[0] = c0; cnt[1] = c1; }
    Network::SumInt64(cnt, 2);
    need_train_ = true;
    if (cnt[0] == 0 || cnt[1] == 0) { Log::Warning("Contains only one class"); need_train_ = false; }
    Log::Info("Number of positive: %lld, number of negative: %lld", static_cast<long long>(cnt[0]), static_cast<long long>(cnt[1]));
    const double ratio = static_cast<double>(std::max(cnt[0], cnt[1])) / std::max<int64_t>(1, std::min(cnt[0], cnt[1]));
    if (need_train_ && ratio > 100.0 && !unbalance_ && spw_ == 1.0)
      Log::Warning("Extreme class imbalance (%.0f:1): consider is_unbalance=true or scale_pos_weight", ratio);
    lw_[0] = lw_[1] = 1.0;   // [negative, positive]
    if (unbalance_ && cnt[0] > 0 && cnt[1] > 0) { if (cnt[0] > cnt[1]) lw_[0] = static_cast<double>(cnt[0]) / cnt[1]; else lw_[1] = static_cast<double>(cnt[1]) / cnt[0]; }
    lw_[1] *= spw_;
    num_pos_ = cnt[0]; num_neg_ = cnt[1];
  }
  void GetGradients(const double* s, score_t* g, score_t* h) const override {
    if (!need_train_) { for (data_size_t i = 0; i < n_; ++i) { g[i] = 0; h[i] = 0; } return; }
#pragma omp parallel for schedule(static) num_threads(RowThreads(n_))
    for (data_size_t i = 0; i < n_; ++i) {
      const bool pos = is_pos_(label_[i]); const double y = pos ? 1.0 : -1.0, lw = lw_[pos ? 1 : 0] * (weights_ ? weights_[i] : 1.0);
      const double r = -y * sigmoid_ / (1.0 + std::exp(y * sigmoid_ * s[i])), ar = std::fabs(r);
      g[i] = static_cast<score_t>(r * lw); h[i] = static_cast<score_t>(ar * (sigmoid_ - ar) * lw);
    }
  }
  double BoostFromScore(int) const override {
    // weighted positive rate through exact integer sums (rank-count independent)
    const double kScale = 1048576.0;
    int64_t acc[2] = {0, 0};
    { int64_t a0 = 0, a1 = 0;   // integer sums: the thread split cannot change the result
#pragma omp parallel for schedule(static) reduction(+ : a0, a1) num_threads(RowThreads(n_))
      for (data_size_t i = 0; i < n_; ++i) { const int64_t w = weights_ ? llround(weights_[i] * kScale) : 1048576; if (is_pos_(label_[i])) a0 += w; a1 += w; }
      acc[0] = a0; acc[1] = a1; }
    Network::SumInt64(acc, 2);
    double p = acc[1] ? static_cast<double>(acc[0]) / static_cast<double>(acc[1]) : 0.5;
    p = std::min(std::max(p, 1e-15), 1.0 - 1e-15);
    const double init = std::log(p / (1.0 - p)) / sigmoid_;
    Log::Info("[binary:BoostFromScore]: pavg=%f -> initscore=%f", p, init);
    return init;
  }
  bool ClassNeedTrain(int) const override { return need_train_; }
  void ConvertOutput(const double* in, double* out) const override { out[0] = 1.0 / (1.0 + std::exp(-sigmoid_ * in[0])); }
  std::string ToString() const override { return std::string("binary sigmoid:") + DoubleToStrG(sigmoid_); }
  int DeviceKind() const override { return kObjBinary; }
  double DeviceParam(int i) const override { return i == 0 ? sigmoid_ : (i == 1 ? lw_[0] : lw_[1]); }
 private:
  double sigmoid_; bool unbalance_; double spw_; std::function<bool(label_t)> is_pos_;
  data_size_t n_ = 0; const label_t* label_ = nullptr; const label_t* weights_ = nullptr;
  bool need_train_ = true; double lw_[2]; int64_t num_pos_ = 0, num_neg_ = 0;
};

// Several regression targets at once: num_class carries the number of targets, labels are [target][row], every round
// grows one L2 tree per target. Parity: src/objective/multi_regression_objective.hpp (MultiRegressionL2).
class MultiRegressionL2 : public ObjectiveFunction {
 public:
  explicit MultiRegressionL2(const Config& cfg) : k_(cfg.num_class) {
    if (k_ <= 1) Log::Fatal("multi_regression requires num_class > 1 (num_class carries the number of targets)");
  }
  const char* GetName() const override { return "multi_regression"; }
  void Init(const Metadata& md, data_size_t n) override {
    n_ = n; label_ = md.label.data(); weights_ = md.weights.empty() ? nullptr : md.weights.data();
    if (md.label.size() != static_cast<size_t>(n) * k_)
      Log::Fatal("multi_regression with num_class=%d expects %zu label values (num_data * num_class, target-major), but got %zu. Pass y as a 2D array of shape [num_data, num_class].",
                 k_, static_cast<size_t>(n) * k_, md.label.size());
    std::vector<double> sums(k_ + 1, 0.0);
    for (data_size_t i = 0; i < n; ++i) sums[k_] += weights_ ? weights_[i] : 1.0;
    for (int t = 0; t < k_; ++t) {
      const label_t* y = label_ + static_cast<size_t>(t) * n;
      double s = 0.0;
#pragma omp parallel for schedule(static) reduction(+ : s) num_threads(RowThreads(n))
      for (data_size_t i = 0; i < n; ++i) s += y[i] * (weights_ ? weights_[i] : 1.0);
      sums[t] = s;
    }
    Network::SumDouble(sums.data(), k_ + 1);
    means_.assign(k_, 0.0);
    for (int t = 0; t < k_; ++t) means_[t] = sums[t] / std::max(sums[k_], kEpsilon);
  }
  int DeviceKind() const override { return kObjMultiReg; }
  void GetGradients(const double* s, score_t* g, score_t* h) const override {
    const int64_t total = static_cast<int64_t>(n_) * k_;
#pragma omp parallel for schedule(static) num_threads(RowThreads(n_))
    for (int64_t o = 0; o < total; ++o) {
      const double w = weights_ ? weights_[o % n_] : 1.0;
      g[o] = static_cast<score_t>((s[o] - label_[o]) * w); h[o] = static_cast<score_t>(w);
    }
  }
  void ConvertOutput(const double* in, double* out) const override { for (int t = 0; t < k_; ++t) out[t] = in[t]; }
  std::string ToString() const override { return std::string(GetName()) + " num_class:" + std::to_string(k_); }
  int NumModelPerIteration() const override { return k_; }
  bool IsConstantHessian() const override { return weights_ == nullptr; }
  double BoostFromScore(int t) const override { return means_[t]; }

 private:
  int k_; data_size_t n_ = 0; const label_t* label_ = nullptr; const label_t* weights_ = nullptr; std::vector<double> means_;
};

class MulticlassSoftmax : public ObjectiveFunction {
 public:
  explicit MulticlassSoftmax(const Config& cfg) : k_(cfg.num_class) { factor_ = static_cast<double>(k_) / (k_ - 1.0); }
  const char* GetName() const override { return "multiclass"; }
  void Init(const Metadata& md, data_size_t n) override {
    n_ = n; label_ = md.label.data(); weights_ = md.weights.empty() ? nullptr : md.weights.data();
    li_.resize(n); std::vector<double> prob(2 * k_, 0.0);
    for (data_size_t i = 0; i < n; ++i) {
      li_[i] = static_cast<int>(label_[i]);
      if (li_[i] < 0 || li_[i] >= k_) Log::Fatal("Label must be in [0, %d), but found %d in label", k_, li_[i]);
      prob[li_[i]] += weights_ ? weights_[i] : 1.0; prob[k_ + li_[i]] += 1;
    }
    Network::SumDouble(prob.data(), 2 * k_);
    double sw = 0; for (int c = 0; c < k_; ++c) sw += prob[c];
    class_init_.assign(k_, 0.0);
    for (int c = 0; c < k_; ++c) class_init_[c] = prob[c] / std::max(sw, kEpsilon);
  }
  void GetGradients(const double* s, score_t* g, score_t* h) const override {
#pragma omp parallel for schedule(static) num_threads(RowThreads(n_))
    for (data_size_t i = 0; i < n_; ++i) {
      std::vector<double> p(k_);
      double mx = s[i]; for (int c = 1; c < k_; ++c) mx = std::max(mx, s[static_cast<size_t>(c) * n_ + i]);
      double sum = 0; for (int c = 0; c < k_; ++c) { p[c] = std::exp(s[static_cast<size_t>(c) * n_ + i] - mx); sum += p[c]; }
      const double w = weights_ ? weights_[i] : 1.0;
      for (int c = 0; c < k_; ++c) {
        const double pc = p[c] / sum; const size_t o = static_cast<size_t>(c) * n_ + i;
        g[o] = static_cast<score_t>((pc - (li_[i] == c ? 1.0 : 0.0)) * w); h[o] = static_cast<score_t>(factor_ * pc * (1.0 - pc) * w);
      }
    }
  }
  double BoostFromScore(int c) const override { return std::log(std::max(kEpsilon, class_init_[c])); }
  bool ClassNeedTrain(int c) const override { return !(std::fabs(class_init_[c]) <= kEpsilon || std::fabs(class_init_[c]) >= 1.0 - kEpsilon); }
  int NumModelPerIteration() const override { return k_; }
  int NumPredictOneRow() const override { return k_; }
  void ConvertOutput(const double* in, double* out) const override {
    double mx = in[0]; for (int c = 1; c < k_; ++c) mx = std::max(mx, in[c]);
    double sum = 0; for (int c = 0; c < k_; ++c) { out[c] = std::exp(in[c] - mx); sum += out[c]; }
    for (int c = 0; c < k_; ++c) out[c] /= sum;
  }
  std::string ToString() const override { return std::string("multiclass num_class:") + std::to_string(k_); }
  int DeviceKind() const override { return kObjMulticlass; }
 private:
  int k_; double factor_; data_size_t n_ = 0; const label_t* label_ = nullptr; const label_t* weights_ = nullptr;
  std::vector<int> li_; std::vector<double> class_init_;
};

class MulticlassOVA : public ObjectiveFunction {
 public:
  explicit MulticlassOVA(const Config& cfg) : k_(cfg.num_class), sigmoid_(cfg.sigmoid) {
    for (int c = 0; c < k_; ++c) bin_.emplace_back(new BinaryLogloss(cfg, [c](label_t l) { return static_cast<int>(l) == c; }));
  }
  const char* GetName() const override { return "multiclassova"; }
  void Init(const Metadata& md, data_size_t n) override { n_ = n; for (auto& b : bin_) b->Init(md, n); }
  void GetGradients(const double* s, score_t* g, score_t* h) const override {
    for (int c = 0; c < k_; ++c) bin_[c]->GetGradients(s + static_cast<size_t>(c) * n_, g + static_cast<size_t>(c) * n_, h + static_cast<size_t>(c) * n_);
  }
  double BoostFromScore(int c) const override { return bin_[c]->BoostFromScore(0); }
  bool ClassNeedTrain(int c) const override { return bin_[c]->ClassNeedTrain(0); }
  int NumModelPerIteration() const override { return k_; }
  int NumPredictOneRow() const override { return k_; }
  void ConvertOutput(const double* in, double* out) const override { for (int c = 0; c < k_; ++c) out[c] = 1.0 / (1.0 + std::exp(-sigmoid_ * in[c])); }
  std::string ToString() const override { return std::string("multiclassova num_class:") + std::to_string(k_) + " sigmoid:" + DoubleToStrG(sigmoid_); }
  int DeviceKind() const override { return kObjMulticlassOVA; }
  double DeviceParam(int) const override { return sigmoid_; }
 private:
  int k_; double sigmoid_; data_size_t n_ = 0; std::vector<std::unique_ptr<BinaryLogloss>> bin_;
};

class CrossEntropy : public ObjectiveFunction {
 public:
  explicit CrossEntropy(const Config&) {}
  const char* GetName() const override { return "cross_entropy"; }
  void Init(const Metadata& md, data_size_t n) override {
    n_ = n; label_ = md.label.data(); weights_ = md.weights.empty() ? nullptr : md.weights.data();
    for (data_size_t i = 0; i < n; ++i) if (label_[i] < 0 || label_[i] > 1) Log::Fatal("[cross_entropy]: labels must be in [0, 1]");
  }
  void GetGradients(const double* s, score_t* g, score_t* h) const override {
    for (data_size_t i = 0; i < n_; ++i) { const double z = 1.0 / (1.0 + std::exp(-s[i])), w = weights_ ? weights_[i] : 1.0; g[i] = static_cast<score_t>((z - label_[i]) * w); h[i] = static_cast<score_t>(z * (1 - z) * w); }
  }
  double BoostFromScore(int) const override {
    double a[2] = {0, 0}; for (data_size_t i = 0; i < n_; ++i) { const double w = weights_ ? weights_[i] : 1.0; a[0] += label_[i] * w; a[1] += w; }
    Network::SumDouble(a, 2);
    double p = std::min(std::max(a[0] / a[1], kEpsilon), 1 - kEpsilon); return std::log(p / (1 - p));
  }
  void ConvertOutput(const double* in, double* out) const override { out[0] = 1.0 / (1.0 + std::exp(-in[0])); }
  std::string ToString() const override { return "cross_entropy"; }
  int DeviceKind() const override { return kObjXent; }
 private:
  data_size_t n_ = 0; const label_t* label_ = nullptr; const label_t* weights_ = nullptr;
};

class CrossEntropyLambda : public ObjectiveFunction {
 public:
  explicit CrossEntropyLambda(const Config&) {}
  const char* GetName() const override { return "cross_entropy_lambda"; }
  void Init(const Metadata& md, data_size_t n) override { n_ = n; label_ = md.label.data(); weights_ = md.weights.empty() ? nullptr : md.weights.data(); }
  void GetGradients(const double* s, score_t* g, score_t* h) const override {
    for (data_size_t i = 0; i < n_; ++i) {
      const double w = weights_ ? weights_[i] : 1.0, y = label_[i], epf = std::exp(s[i]), hhat = std::log1p(epf);
      const double z = 1.0 - std::exp(-w * hhat), enf = 1.0 / epf;
      g[i] = static_cast<score_t>((1.0 - y / z) * w / (1.0 + enf));
      const double c = 1.0 / (1.0 - z), d = 1.0 + epf, a = w * epf / (d * d), b = (c / ((c - 1) * (c - 1))) * (1.0 + w * epf - c);
      h[i] = static_cast<score_t>(a * (1.0 + y * b));
    }
  }
  double BoostFromScore(int) const override {
    double a[2] = {0, 0}; for (data_size_t i = 0; i < n_; ++i) { const double w = weights_ ? weights_[i] : 1.0; a[0] += label_[i] * w; a[1] += w; }
    Network::SumDouble(a, 2);
    double havg = a[0] / a[1]; return std::log(std::expm1(std::max(havg, kEpsilon)));
  }
  void ConvertOutput(const double* in, double* out) const override { out[0] = std::log1p(std::exp(in[0])); }
  std::string ToString() const override { return "cross_entropy_lambda"; }
  int DeviceKind() const override { return kObjXentLambda; }
 private:
  data_size_t n_ = 0; const label_t* label_ = nullptr; const label_t* weights_ = nullptr;
};

class LambdarankNDCG : public ObjectiveFunction {
 public:
  explicit LambdarankNDCG(const Config& cfg) : sigmoid_(cfg.sigmoid), norm_(cfg.lambdarank_norm), trunc_(cfg.lambdarank_truncation_level), gains_(cfg.label_gain_vec) {
    if (sigmoid_ <= 0.0) Log::Fatal("Sigmoid param %f should be greater than zero", sigmoid_);
  }
  const char* GetName() const override { return "lambdarank"; }
  bool NeedQueries() const override { return true; }
  void Init(const Metadata& md, data_size_t n) override {
    n_ = n; label_ = md.label.data(); weights_ = md.weights.empty() ? nullptr : md.weights.data();
    if (md.query_boundaries.empty()) Log::Fatal("Ranking tasks require query information");
    qb_ = md.query_boundaries.data(); nq_ = md.num_queries();
    inv_max_dcg_.resize(nq_);
    for (data_size_t q = 0; q < nq_; ++q) {
      for (data_size_t i = qb_[q]; i < qb_[q + 1]; ++i) if (static_cast<size_t>(label_[i]) >= gains_.size() || label_[i] < 0) Log::Fatal("Label %f is not in the label_gain range", label_[i]);
      double m = DCG::MaxDCGAtK(trunc_, label_ + qb_[q], qb_[q + 1] - qb_[q], gains_);
      inv_max_dcg_[q] = m > 0 ? 1.0 / m : 0.0;
    }
    int maxn = 0; for (data_size_t q = 0; q < nq_; ++q) maxn = std::max(maxn, qb_[q + 1] - qb_[q]);
    discount_ = DCG::Discounts(maxn + 1);
  }
  void GetGradients(const double* s, score_t* g, score_t* h) const override {
#pragma omp parallel for schedule(guided) num_threads(TeamThreads())
    for (data_size_t q = 0; q < nq_; ++q) OneQuery(q, s + qb_[q], g + qb_[q], h + qb_[q]);
    if (weights_) for (data_size_t i = 0; i < n_; ++i) { g[i] *= weights_[i]; h[i] *= weights_[i]; }
  }
  void OneQuery(data_size_t q, const double* s, score_t* g, score_t* h) const {
    const int cnt = qb_[q + 1] - qb_[q]; const label_t* lab = label_ + qb_[q];
    std::vector<double> lg(cnt, 0.0), lh(cnt, 0.0);
    std::vector<int> order(cnt); std::iota(order.begin(), order.end(), 0);
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return s[a] > s[b]; });
    const double inv = inv_max_dcg_[q];
    double sum_lambda = 0.0;
    double best = s[order[0]], worst = s[order[cnt - 1]];
    for (int i = 0; i < cnt - 1 && i < trunc_; ++i) {
      for (int j = i + 1; j < cnt; ++j) {
        const int a = order[i], b = order[j];
        if (lab[a] == lab[b]) continue;
        int hi, lo, hr, lr;
        if (lab[a] > lab[b]) { hi = a; hr = i; lo = b; lr = j; } else { hi = b; hr = j; lo = a; lr = i; }
        const double ds = s[hi] - s[lo];
        const double dcg_gap = gains_[static_cast<int>(lab[hi])] - gains_[static_cast<int>(lab[lo])];
        const double pd = std::fabs(discount_[hr] - discount_[lr]);
        double delta = dcg_gap * pd * inv;
        if (norm_ && best != worst) delta /= (0.01 + std::fabs(ds));
        const double rho = 1.0 / (1.0 + std::exp(sigmoid_ * ds));
        const double pl = -sigmoid_ * delta * rho, ph = sigmoid_ * sigmoid_ * delta * rho * (1.0 - rho);
        lg[lo] -= pl; lh[lo] += ph; lg[hi] += pl; lh[hi] += ph;
        sum_lambda -= 2 * pl;
      }
    }
    if (norm_ && sum_lambda > 0) { const double f = std::log2(1 + sum_lambda) / sum_lambda; for (int i = 0; i < cnt; ++i) { lg[i] *= f; lh[i] *= f; } }
    for (int i = 0; i < cnt; ++i) { g[i] = static_cast<score_t>(lg[i]); h[i] = static_cast<score_t>(lh[i]); }
  }
  std::string ToString() const override { return "lambdarank"; }
  int DeviceKind() const override { return kObjLambdarank; }
  double DeviceParam(int i) const override { return i == 0 ? sigmoid_ : (i == 1 ? (norm_ ? 1.0 : 0.0) : trunc_); }
 private:
  double sigmoid_; bool norm_; int trunc_; std::vector<double> gains_;
  data_size_t n_ = 0, nq_ = 0; const label_t* label_ = nullptr; const label_t* weights_ = nullptr; const data_size_t* qb_ = nullptr;
  std::vector<double> inv_max_dcg_, discount_;
};

class RankXENDCG : public ObjectiveFunction {
 public:
  explicit RankXENDCG(const Config& cfg) : seed_(cfg.objective_seed) {}
  const char* GetName() const override { return "rank_xendcg"; }
  bool NeedQueries() const override { return true; }
  void Init(const Metadata& md, data_size_t n) override {
    n_ = n; label_ = md.label.data(); weights_ = md.weights.empty() ? nullptr : md.weights.data();
    if (md.query_boundaries.empty()) Log::Fatal("Ranking tasks require query information");
    qb_ = md.query_boundaries.data(); nq_ = md.num_queries(); iter_ = 0;
  }
  void GetGradients(const double* s, score_t* g, score_t* h) const override {
    const uint32_t it = iter_++;
    for (data_size_t q = 0; q < nq_; ++q) {
      const int cnt = qb_[q + 1] - qb_[q]; const double* sc = s + qb_[q]; const label_t* lab = label_ + qb_[q];
      score_t* gg = g + qb_[q]; score_t* hh = h + qb_[q];
      if (cnt <= 1) { for (int i = 0; i < cnt; ++i) { gg[i] = 0; hh[i] = 0; } continue; }
      std::vector<double> rho(cnt), params(cnt);
      double mx = sc[0]; for (int i = 1; i < cnt; ++i) mx = std::max(mx, sc[i]);
      double sum = 0; for (int i = 0; i < cnt; ++i) { rho[i] = std::exp(sc[i] - mx); sum += rho[i]; }
      for (int i = 0; i < cnt; ++i) rho[i] /= sum;
      double inv_denom = 0;
      for (int i = 0; i < cnt; ++i) {
        const double u = U01From24(Philox4x32_10(static_cast<uint32_t>(qb_[q] + i), it, 0x1234u, 0x5678u, static_cast<uint32_t>(seed_), 0xABCDu).v[0]);
        params[i] = std::pow(2.0, static_cast<int>(lab[i])) - u; inv_denom += params[i];
      }
      inv_denom = 1.0 / std::max(kEpsilon, inv_denom);
      double sum_l1 = 0; std::vector<double> l1(cnt);
      for (int i = 0; i < cnt; ++i) { l1[i] = -params[i] * inv_denom + rho[i]; params[i] = l1[i] / (1.0 - rho[i]); sum_l1 += params[i]; }
      double sum_l2 = 0; std::vector<double> l2(cnt);
      for (int i = 0; i < cnt; ++i) { l2[i] = rho[i] * (sum_l1 - params[i]); params[i] = l2[i] / (1.0 - rho[i]); sum_l2 += params[i]; }
      for (int i = 0; i < cnt; ++i) { gg[i] = static_cast<score_t>(l1[i] + l2[i] + rho[i] * (sum_l2 - params[i])); hh[i] = static_cast<score_t>(rho[i] * (1.0 - rho[i])); }
    }
    if (weights_) for (data_size_t i = 0; i < n_; ++i) { g[i] *= weights_[i]; h[i] *= weights_[i]; }
  }
  std::string ToString() const override { return "rank_xendcg"; }
  // the device kernel makes the same draws: parameter 0 is the seed; the engine counts the rounds itself
  int DeviceKind() const override { return kObjXendcg; }
  double DeviceParam(int i) const override { return i == 0 ? static_cast<double>(seed_) : 0.0; }
 private:
  int seed_; mutable uint32_t iter_ = 0;
  data_size_t n_ = 0, nq_ = 0; const label_t* label_ = nullptr; const label_t* weights_ = nullptr; const data_size_t* qb_ = nullptr;
};

}  // namespace

ObjectiveFunction* CreateObjective(const std::string& name, const Config& cfg) {
  if (name == "regression") return new RegressionL2(cfg);
  if (name == "regression_l1") return new RegressionL1(cfg);
  if (name == "huber") return new RegressionHuber(cfg);
  if (name == "fair") return new RegressionFair(cfg);
  if (name == "poisson") return new RegressionPoisson(cfg);
  if (name == "quantile") return new RegressionQuantile(cfg);
  if (name == "mape") return new RegressionMAPE(cfg);
  if (name == "gamma") return new RegressionGamma(cfg);
  if (name == "tweedie") return new RegressionTweedie(cfg);
  if (name == "binary") return new BinaryLogloss(cfg);
  if (name == "multiclass") return new MulticlassSoftmax(cfg);
  if (name == "multi_regression") return new MultiRegressionL2(cfg);
  if (name == "multiclassova") return new MulticlassOVA(cfg);
  if (name == "cross_entropy") return new CrossEntropy(cfg);
  if (name == "cross_entropy_lambda") return new CrossEntropyLambda(cfg);
  if (name == "lambdarank") return new LambdarankNDCG(cfg);
  if (name == "rank_xendcg") return new RankXENDCG(cfg);
  if (name == "custom") return nullptr;
  Log::Fatal("Unknown objective type name: %s", name.c_str());
}

ObjectiveFunction* CreateObjectiveFromModelString(const std::string& str, Config* cfg) {
  auto toks = SplitAny(str, " ");
  if (toks.empty()) return nullptr;
  std::string name = Config::ParseObjectiveAlias(toks[0]);
  for (size_t i = 1; i < toks.size(); ++i) {
    auto kv = Split(toks[i], ':');
    if (kv.size() == 2) {
      if (kv[0] == "sigmoid") cfg->sigmoid = ParseDouble(kv[1]);
      else if (kv[0] == "num_class") cfg->num_class = atoi(kv[1].c_str());
    } else if (toks[i] == "sqrt") cfg->reg_sqrt = true;
  }
  cfg->objective = name;
  if (name == "custom") return nullptr;
  return CreateObjective(name, *cfg);
}

}  // namespace fb
