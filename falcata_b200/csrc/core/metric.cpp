// Host evaluation metrics and DCG helpers.
// Parity: src/metric/regression_metric.hpp, binary_metric.hpp (logloss, error, AUC, average
// precision), multiclass_metric.hpp (multi_logloss, multi_error, auc_mu), rank_metric.hpp
// (ndcg@k), map_metric.hpp, xentropy_metric.hpp, dcg_calculator.cpp:L34-174.
// Sums go through Network so that every rank reports the global value.
#include "fb/objective.h"
#include "fb/learner.h"

#include <numeric>

namespace fb {

std::vector<double> DCG::Discounts(int n) { std::vector<double> d(n); for (int i = 0; i < n; ++i) d[i] = 1.0 / std::log2(2.0 + i); return d; }

double DCG::MaxDCGAtK(int k, const label_t* label, int n, const std::vector<double>& gains) {
  std::vector<int> cnt(gains.size(), 0);
  for (int i = 0; i < n; ++i) cnt[static_cast<int>(label[i])]++;
  double ret = 0; int top = static_cast<int>(gains.size()) - 1; if (k > n) k = n;
  for (int j = 0; j < k; ++j) { while (top > 0 && cnt[top] <= 0) --top; ret += gains[top] / std::log2(2.0 + j); cnt[top]--; }
  return ret;
}

void DCG::CalMaxDCG(const std::vector<int>& ks, const label_t* label, int n, const std::vector<double>& gains, std::vector<double>* out) {
  out->resize(ks.size());
  for (size_t i = 0; i < ks.size(); ++i) (*out)[i] = MaxDCGAtK(ks[i], label, n, gains);
}

void DCG::CalDCG(const std::vector<int>& ks, const label_t* label, const double* score, int n, const std::vector<double>& gains, std::vector<double>* out) {
  std::vector<int> order(n); std::iota(order.begin(), order.end(), 0);
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return score[a] > score[b]; });
  out->resize(ks.size());
  double cur = 0; int left = 0;
  for (size_t i = 0; i < ks.size(); ++i) {
    int k = std::min(ks[i], n);
    for (int j = left; j < k; ++j) cur += gains[static_cast<int>(label[order[j]])] / std::log2(2.0 + j);
    (*out)[i] = cur; left = std::max(left, k);
  }
}

namespace {

struct MetricBase : public Metric {
  data_size_t n_ = 0; const label_t* label_ = nullptr; const label_t* weights_ = nullptr; double sum_w_ = 0;
  const Metadata* md_ = nullptr;
  void Init(const Metadata& md, data_size_t n) override {
    md_ = &md; n_ = n; label_ = md.label.data(); weights_ = md.weights.empty() ? nullptr : md.weights.data();
    sum_w_ = 0; if (weights_) for (data_size_t i = 0; i < n; ++i) sum_w_ += weights_[i]; else sum_w_ = n;
    Network::SumDouble(&sum_w_, 1);
  }
};

// pointwise metric: loss(label, converted score)
template <typename Loss>
struct Pointwise : public MetricBase {
  Config cfg_; std::string name_; bool convert_; bool sqrt_out_;
  Pointwise(const Config& c, const char* name, bool convert, bool sqrt_out = false) : cfg_(c), name_(name), convert_(convert), sqrt_out_(sqrt_out) {}
  std::vector<std::string> Names() const override { return {name_}; }
  bool HigherBetter() const override { return Loss::kHigherBetter; }
  std::vector<double> Eval(const double* score, const ObjectiveFunction* obj) const override {
    double s = 0;
    // several regression targets (multi_regression): labels and scores are [target][row]; the loss is averaged over both
    const int targets = (md_ != nullptr && n_ > 0 && md_->label.size() > static_cast<size_t>(n_) && obj != nullptr && obj->NumModelPerIteration() > 1)
                            ? static_cast<int>(md_->label.size() / static_cast<size_t>(n_)) : 1;
    const int64_t total = static_cast<int64_t>(n_) * targets;
#pragma omp parallel for schedule(static) reduction(+ : s) num_threads(RowThreads(n_))
    for (int64_t i = 0; i < total; ++i) {
      double v = score[i];
      if (convert_ && obj != nullptr && targets == 1) obj->ConvertOutput(&score[i], &v);
      s += Loss::Point(label_[i], v, cfg_) * (weights_ ? weights_[i % n_] : 1.0);
    }
    Network::SumDouble(&s, 1);
    double r = s / (sum_w_ * targets);
    return {sqrt_out_ ? std::sqrt(r) : r};
  }
};

struct L2Loss { static constexpr bool kHigherBetter = false; static double Point(double y, double s, const Config&) { return (s - y) * (s - y); } };
struct L1Loss { static constexpr bool kHigherBetter = false; static double Point(double y, double s, const Config&) { return std::fabs(s - y); } };
struct QuantileLoss { static constexpr bool kHigherBetter = false; static double Point(double y, double s, const Config& c) { double d = y - s; return d >= 0 ? c.alpha * d : (c.alpha - 1) * d; } };
struct HuberLoss { static constexpr bool kHigherBetter = false; static double Point(double y, double s, const Config& c) { double d = s - y; return std::fabs(d) <= c.alpha ? 0.5 * d * d : c.alpha * (std::fabs(d) - 0.5 * c.alpha); } };
struct FairLoss { static constexpr bool kHigherBetter = false; static double Point(double y, double s, const Config& c) { double x = std::fabs(s - y); return c.fair_c * x - c.fair_c * c.fair_c * std::log1p(x / c.fair_c); } };
struct PoissonLoss { static constexpr bool kHigherBetter = false; static double Point(double y, double s, const Config&) { if (s < 1e-10) s = 1e-10; return s - y * std::log(s); } };
struct MapeLoss { static constexpr bool kHigherBetter = false; static double Point(double y, double s, const Config&) { return std::fabs(y - s) / std::max(1.0, std::fabs(y)); } };
struct GammaLoss { static constexpr bool kHigherBetter = false; static double Point(double y, double s, const Config&) { double psi = 1.0, theta = -1.0 / s, a = psi, b = -std::log(-theta), c = 1.0 / psi * std::log(y / psi) - std::log(y) - 0; return -((y * theta - b) / a + c); } };
struct GammaDevLoss { static constexpr bool kHigherBetter = false; static double Point(double y, double s, const Config&) { double e = 1e-9, t = y / (s + e); return 2 * (t - std::log(t + 1e-300) - 1); } };
struct TweedieLoss { static constexpr bool kHigherBetter = false; static double Point(double y, double s, const Config& c) { double rho = c.tweedie_variance_power; if (s < 1e-10) s = 1e-10; double a = y * std::exp((1 - rho) * std::log(s)) / (1 - rho), b = std::exp((2 - rho) * std::log(s)) / (2 - rho); return -a + b; } };
struct BinLogloss { static constexpr bool kHigherBetter = false; static double Point(double y, double p, const Config&) { if (y <= 0) { return 1 - p > kEpsilon ? -std::log(1 - p) : -std::log(kEpsilon); } return p > kEpsilon ? -std::log(p) : -std::log(kEpsilon); } };
struct BinError { static constexpr bool kHigherBetter = false; static double Point(double y, double p, const Config&) { return p <= 0.5 ? (y > 0 ? 1.0 : 0.0) : (y > 0 ? 0.0 : 1.0); } };
struct XentLoss { static constexpr bool kHigherBetter = false; static double Point(double y, double p, const Config&) { auto lg = [](double x) { return std::log(std::max(x, kEpsilon)); }; return -(y * lg(p) + (1 - y) * lg(1 - p)); } };
struct KLDivLoss { static constexpr bool kHigherBetter = false; static double Point(double y, double p, const Config& c) { auto lg = [](double x) { return std::log(std::max(x, kEpsilon)); }; double ent = 0; if (y > 0) ent += y * lg(y); if (y < 1) ent += (1 - y) * lg(1 - y); return ent + XentLoss::Point(y, p, c); } };

struct R2Metric : public MetricBase {
  std::vector<std::string> Names() const override { return {"r2"}; }
  bool HigherBetter() const override { return true; }
  std::vector<double> Eval(const double* score, const ObjectiveFunction* obj) const override {
    double a[3] = {0, 0, 0};
    for (data_size_t i = 0; i < n_; ++i) { double w = weights_ ? weights_[i] : 1.0; a[0] += label_[i] * w; }
    Network::SumDouble(a, 1); const double mean = a[0] / sum_w_;
    for (data_size_t i = 0; i < n_; ++i) { double v = score[i]; if (obj) obj->ConvertOutput(&score[i], &v); double w = weights_ ? weights_[i] : 1.0; a[1] += w * (label_[i] - v) * (label_[i] - v); a[2] += w * (label_[i] - mean) * (label_[i] - mean); }
    Network::SumDouble(a + 1, 2);
    return {a[2] > 0 ? 1.0 - a[1] / a[2] : 0.0};
  }
};

struct AUCMetric : public MetricBase {
  std::vector<std::string> Names() const override { return {"auc"}; }
  bool HigherBetter() const override { return true; }
  std::vector<double> Eval(const double* score, const ObjectiveFunction*) const override {
    // gather (score, label, weight) of all ranks, then the usual sorted sweep with tie groups
    std::vector<double> s(score, score + n_); std::vector<double> y(n_), w(n_);
    for (data_size_t i = 0; i < n_; ++i) { y[i] = label_[i] > 0 ? 1.0 : 0.0; w[i] = weights_ ? weights_[i] : 1.0; }
    if (Network::active()) {
      int64_t cnt = n_; std::vector<char> all; Network::Gather(&cnt, 8, &all);
      const int64_t* c = reinterpret_cast<const int64_t*>(all.data()); int64_t mx = 0; for (int r = 0; r < Network::world(); ++r) mx = std::max(mx, c[r]);
      auto gather = [&](std::vector<double>* v) {
        std::vector<double> pad(*v); pad.resize(mx, 0.0); std::vector<char> buf; Network::Gather(pad.data(), mx * 8, &buf);
        std::vector<double> out; const double* p = reinterpret_cast<const double*>(buf.data());
        for (int r = 0; r < Network::world(); ++r) out.insert(out.end(), p + r * mx, p + r * mx + c[r]);
        v->swap(out);
      };
      gather(&s); gather(&y); gather(&w);
    }
    const size_t n = s.size();
    std::vector<size_t> order(n); std::iota(order.begin(), order.end(), 0);
    std::stable_sort(order.begin(), order.end(), [&](size_t a, size_t b) { return s[a] > s[b]; });
    double sum_pos = 0, accum = 0, cur_pos = 0, cur_neg = 0, total_pos = 0;
    double thr = n ? s[order[0]] : 0;
    for (size_t k = 0; k < n; ++k) {
      const size_t i = order[k];
      if (s[i] != thr) { thr = s[i]; accum += cur_neg * (cur_pos * 0.5 + sum_pos); sum_pos += cur_pos; cur_neg = cur_pos = 0; }
      cur_neg += (1 - y[i]) * w[i]; cur_pos += y[i] * w[i];
    }
    accum += cur_neg * (cur_pos * 0.5 + sum_pos); sum_pos += cur_pos; total_pos = sum_pos;
    double sw = 0; for (size_t i = 0; i < n; ++i) sw += w[i];
    double total_neg = sw - total_pos;
    if (total_pos <= 0 || total_neg <= 0) return {1.0};
    return {accum / (total_pos * total_neg)};
  }
};

struct AveragePrecision : public MetricBase {
  std::vector<std::string> Names() const override { return {"average_precision"}; }
  bool HigherBetter() const override { return true; }
  std::vector<double> Eval(const double* score, const ObjectiveFunction*) const override {
    std::vector<int> order(n_); std::iota(order.begin(), order.end(), 0);
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return score[a] > score[b]; });
    double tp = 0, seen = 0, ap = 0, total_pos = 0;
    for (data_size_t i = 0; i < n_; ++i) if (label_[i] > 0) total_pos += weights_ ? weights_[i] : 1.0;
    for (int k = 0; k < n_; ++k) { int i = order[k]; double w = weights_ ? weights_[i] : 1.0; seen += w; if (label_[i] > 0) { tp += w; ap += w * tp / seen; } }
    return {total_pos > 0 ? ap / total_pos : 1.0};
  }
};

struct MultiLogloss : public MetricBase {
  int k_; explicit MultiLogloss(const Config& c) : k_(c.num_class) {}
  std::vector<std::string> Names() const override { return {"multi_logloss"}; }
  bool HigherBetter() const override { return false; }
  std::vector<double> Eval(const double* score, const ObjectiveFunction* obj) const override {
    double s = 0;
#pragma omp parallel for schedule(static) reduction(+ : s) num_threads(RowThreads(n_))
    for (data_size_t i = 0; i < n_; ++i) {
      std::vector<double> raw(k_), p(k_);
      for (int c = 0; c < k_; ++c) raw[c] = score[static_cast<size_t>(c) * n_ + i];
      if (obj) obj->ConvertOutput(raw.data(), p.data()); else p = raw;
      double pc = p[static_cast<int>(label_[i])];
      s += (pc > kEpsilon ? -std::log(pc) : -std::log(kEpsilon)) * (weights_ ? weights_[i] : 1.0);
    }
    Network::SumDouble(&s, 1);
    return {s / sum_w_};
  }
};

struct MultiError : public MetricBase {
  int k_, topk_; explicit MultiError(const Config& c) : k_(c.num_class), topk_(c.multi_error_top_k) {}
  std::vector<std::string> Names() const override { return {topk_ == 1 ? std::string("multi_error") : "multi_error@" + std::to_string(topk_)}; }
  bool HigherBetter() const override { return false; }
  std::vector<double> Eval(const double* score, const ObjectiveFunction*) const override {
    double s = 0;
    for (data_size_t i = 0; i < n_; ++i) {
      const int y = static_cast<int>(label_[i]); const double sy = score[static_cast<size_t>(y) * n_ + i]; int larger = 0;
      for (int c = 0; c < k_; ++c) if (score[static_cast<size_t>(c) * n_ + i] >= sy) ++larger;
      if (larger > topk_) s += weights_ ? weights_[i] : 1.0;
    }
    Network::SumDouble(&s, 1);
    return {s / sum_w_};
  }
};

// AUC-mu (Kleiman & Page, 2019): the mean over class pairs (i, j) of the probability that a row of class i lies farther
// on i's side of the pair's separating direction than a row of class j, ties counting one half. With partition weights
// W (default: 1 off the diagonal, 0 on it), v = W[i] - W[j] and the signed distance of row a is (v[i] - v[j]) * <v, raw
// scores of a>. Row weights multiply pair counts. Parity: src/metric/multiclass_metric.hpp (AucMuMetric).
struct AucMu : public MetricBase {
  int k_; std::vector<double> w_;   // [k x k]
  explicit AucMu(const Config& c) : k_(c.num_class) {
    w_.assign(static_cast<size_t>(k_) * k_, 1.0);
    for (int i = 0; i < k_; ++i) w_[static_cast<size_t>(i) * k_ + i] = 0.0;
    if (!c.auc_mu_weights.empty()) {
      std::vector<double> given;
      for (auto& t : SplitAny(c.auc_mu_weights, ",")) { const std::string s = Trim(t); if (!s.empty()) given.push_back(atof(s.c_str())); }
      if (given.size() != w_.size()) Log::Fatal("auc_mu_weights must have %d elements, but found %d", k_ * k_, static_cast<int>(given.size()));
      for (int i = 0; i < k_; ++i) {
        if (std::fabs(given[static_cast<size_t>(i) * k_ + i]) > kEpsilon) Log::Warning("AUC-mu matrix must have zeros on diagonal. Overwriting value in position %d of auc_mu_weights with 0.", i * k_ + i);
        given[static_cast<size_t>(i) * k_ + i] = 0.0;
      }
      w_ = given;
    }
  }
  std::vector<std::string> Names() const override { return {"auc_mu"}; }
  bool HigherBetter() const override { return true; }
  std::vector<double> Eval(const double* score, const ObjectiveFunction*) const override {
    std::vector<std::vector<int>> rows_of(k_);
    for (data_size_t a = 0; a < n_; ++a) {
      const int y = static_cast<int>(label_[a]);
      if (y < 0 || y >= k_) Log::Fatal("Label must be in [0, %d), but found %d in label", k_, y);
      rows_of[y].push_back(a);
    }
    double total = 0.0;
    std::vector<double> v(k_);
    struct Item { double d; double w; int is_i; };
    std::vector<Item> items;
    for (int i = 0; i < k_; ++i) {
      for (int j = i + 1; j < k_; ++j) {
        for (int m = 0; m < k_; ++m) v[m] = w_[static_cast<size_t>(i) * k_ + m] - w_[static_cast<size_t>(j) * k_ + m];
        const double t1 = v[i] - v[j];
        items.clear();
        double wi = 0.0, wj = 0.0;
        for (int side = 0; side < 2; ++side) {
          for (int a : rows_of[side == 0 ? i : j]) {
            double dot = 0.0;
            for (int m = 0; m < k_; ++m) dot += v[m] * score[static_cast<size_t>(m) * n_ + a];
            const double w = weights_ ? weights_[a] : 1.0;
            items.push_back({t1 * dot, w, side == 0 ? 1 : 0});
            (side == 0 ? wi : wj) += w;
          }
        }
        if (wi <= 0.0 || wj <= 0.0) continue;   // a class without rows adds nothing for its pairs
        std::sort(items.begin(), items.end(), [](const Item& a, const Item& b) { return a.d < b.d; });
        // walk the distances upwards in groups of (near-)equal distance: a class-i row beats all class-j weight strictly
        // below its group and half of the class-j weight inside it
        double below_j = 0.0, s = 0.0;
        for (size_t b = 0; b < items.size();) {
          size_t e = b; double gi = 0.0, gj = 0.0;
          while (e < items.size() && std::fabs(items[e].d - items[b].d) < kEpsilon) { if (items[e].is_i) gi += items[e].w; else gj += items[e].w; ++e; }
          s += gi * (below_j + 0.5 * gj);
          below_j += gj;
          b = e;
        }
        total += s / (wi * wj);
      }
    }
    return {k_ > 1 ? 2.0 * total / (static_cast<double>(k_) * (k_ - 1)) : 1.0};
  }
};

struct NDCGMetric : public MetricBase {
  std::vector<int> ks_; std::vector<double> gains_;
  explicit NDCGMetric(const Config& c) : ks_(c.eval_at_vec), gains_(c.label_gain_vec) {}
  std::vector<std::string> Names() const override { std::vector<std::string> r; for (int k : ks_) r.push_back("ndcg@" + std::to_string(k)); return r; }
  bool HigherBetter() const override { return true; }
  std::vector<double> Eval(const double* score, const ObjectiveFunction*) const override {
    if (md_->query_boundaries.empty()) Log::Fatal("The NDCG metric requires query information");
    const data_size_t nq = md_->num_queries(); const data_size_t* qb = md_->query_boundaries.data();
    std::vector<double> acc(ks_.size() + 1, 0.0);
    for (data_size_t q = 0; q < nq; ++q) {
      const int cnt = qb[q + 1] - qb[q]; std::vector<double> mx, dcg;
      DCG::CalMaxDCG(ks_, label_ + qb[q], cnt, gains_, &mx);
      const double qw = md_->query_weights.empty() ? 1.0 : md_->query_weights[q];
      if (mx.empty() || mx[0] <= 0) { for (size_t j = 0; j < ks_.size(); ++j) acc[j] += qw; }
      else { DCG::CalDCG(ks_, label_ + qb[q], score + qb[q], cnt, gains_, &dcg); for (size_t j = 0; j < ks_.size(); ++j) acc[j] += qw * dcg[j] / mx[j]; }
      acc[ks_.size()] += qw;
    }
    Network::SumDouble(acc.data(), static_cast<int64_t>(acc.size()));
    std::vector<double> out(ks_.size()); for (size_t j = 0; j < ks_.size(); ++j) out[j] = acc[j] / acc[ks_.size()];
    return out;
  }
};

struct MAPMetric : public MetricBase {
  std::vector<int> ks_; explicit MAPMetric(const Config& c) : ks_(c.eval_at_vec) {}
  std::vector<std::string> Names() const override { std::vector<std::string> r; for (int k : ks_) r.push_back("map@" + std::to_string(k)); return r; }
  bool HigherBetter() const override { return true; }
  std::vector<double> Eval(const double* score, const ObjectiveFunction*) const override {
    if (md_->query_boundaries.empty()) Log::Fatal("The MAP metric requires query information");
    const data_size_t nq = md_->num_queries(); const data_size_t* qb = md_->query_boundaries.data();
    std::vector<double> acc(ks_.size() + 1, 0.0);
    for (data_size_t q = 0; q < nq; ++q) {
      const int cnt = qb[q + 1] - qb[q]; const double* s = score + qb[q]; const label_t* lab = label_ + qb[q];
      std::vector<int> order(cnt); std::iota(order.begin(), order.end(), 0);
      std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return s[a] > s[b]; });
      int npos = 0; for (int i = 0; i < cnt; ++i) if (lab[i] > 0.5f) ++npos;
      for (size_t j = 0; j < ks_.size(); ++j) {
        int k = std::min(ks_[j], cnt), hit = 0; double ap = 0;
        for (int i = 0; i < k; ++i) if (lab[order[i]] > 0.5f) { ++hit; ap += static_cast<double>(hit) / (i + 1); }
        acc[j] += npos > 0 ? ap / std::min(npos, k) : 1.0;
      }
      acc[ks_.size()] += 1.0;
    }
    Network::SumDouble(acc.data(), static_cast<int64_t>(acc.size()));
    std::vector<double> out(ks_.size()); for (size_t j = 0; j < ks_.size(); ++j) out[j] = acc[j] / acc[ks_.size()];
    return out;
  }
};

}  // namespace

Metric* CreateMetric(const std::string& name, const Config& cfg) {
  if (name == "l2") return new Pointwise<L2Loss>(cfg, "l2", true);
  if (name == "rmse") return new Pointwise<L2Loss>(cfg, "rmse", true, true);
  if (name == "l1") return new Pointwise<L1Loss>(cfg, "l1", true);
  if (name == "quantile") return new Pointwise<QuantileLoss>(cfg, "quantile", true);
  if (name == "huber") return new Pointwise<HuberLoss>(cfg, "huber", true);
  if (name == "fair") return new Pointwise<FairLoss>(cfg, "fair", true);
  if (name == "poisson") return new Pointwise<PoissonLoss>(cfg, "poisson", true);
  if (name == "mape") return new Pointwise<MapeLoss>(cfg, "mape", true);
  if (name == "gamma") return new Pointwise<GammaLoss>(cfg, "gamma", true);
  if (name == "gamma_deviance") return new Pointwise<GammaDevLoss>(cfg, "gamma_deviance", true);
  if (name == "tweedie") return new Pointwise<TweedieLoss>(cfg, "tweedie", true);
  if (name == "r2") return new R2Metric();
  if (name == "binary_logloss") return new Pointwise<BinLogloss>(cfg, "binary_logloss", true);
  if (name == "binary_error") return new Pointwise<BinError>(cfg, "binary_error", true);
  if (name == "auc") return new AUCMetric();
  if (name == "average_precision") return new AveragePrecision();
  if (name == "multi_logloss") return new MultiLogloss(cfg);
  if (name == "multi_error") return new MultiError(cfg);
  if (name == "auc_mu") return new AucMu(cfg);
  if (name == "cross_entropy") return new Pointwise<XentLoss>(cfg, "cross_entropy", true);
  if (name == "cross_entropy_lambda") return new Pointwise<XentLoss>(cfg, "cross_entropy_lambda", true);
  if (name == "kullback_leibler") return new Pointwise<KLDivLoss>(cfg, "kullback_leibler", true);
  if (name == "ndcg") return new NDCGMetric(cfg);
  if (name == "map") return new MAPMetric(cfg);
  Log::Warning("Unknown metric %s is ignored", name.c_str());
  return nullptr;
}

}  // namespace fb
