// Native unit tests of the core library (plain asserts, no framework): value formatting, binning (order invariance, 32- and
// 64-bit sort, zero and NaN bins, categorical bins, serialisation), linear leaves, candidate limits and tie order, forced-split
// files, tree text round
// trip, single-row prediction, counter-based random numbers, quantization, and the best-first order keys of the
// device level controller checked against a brute-force best-first growth.
// Parity: tests/cpp_tests/ (test_common.cpp, test_serialize.cpp, test_single_row.cpp) of the reference.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <functional>
#include <map>
#include <queue>
#include <string>
#include <vector>

#include "fb/bin.h"
#include "fb/common.h"
#include "fb/config.h"
#include "fb/learner.h"
#include "fb/split_math.h"
#include "fb/tree.h"

using namespace fb;

static int g_failed = 0, g_checks = 0;
#define CHECK(cond) do { ++g_checks; if (!(cond)) { ++g_failed; fprintf(stderr, "FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); } } while (0)

static void TestFormatting() {
  const double vals[] = {0.1, -3.25, 1e-300, 12345678.9012345678, 1.0 / 3.0, 5e22};
  for (double v : vals) CHECK(atof(DoubleToStr17(v).c_str()) == v);   // 17 significant digits round-trip a double
  const auto parts = Split("a,b,,c", ',');
  CHECK(parts.size() == 4 && parts[0] == "a" && parts[2].empty() && parts[3] == "c");
}

static void TestPhilox() {
  const Philox4 a = Philox4x32_10(1, 2, 3, 4, 5, 6), b = Philox4x32_10(1, 2, 3, 4, 5, 6), c = Philox4x32_10(2, 2, 3, 4, 5, 6);
  CHECK(memcmp(&a, &b, sizeof(a)) == 0);
  CHECK(memcmp(&a, &c, sizeof(a)) != 0);
  double mean = 0; const int n = 20000;
  for (int i = 0; i < n; ++i) { const float u = U01From24(Philox4x32_10(i, 0, 0, 0, 7, 9).v[0]); CHECK(u >= 0.f && u < 1.f); mean += u; }
  CHECK(std::fabs(mean / n - 0.5) < 0.01);
}

static void TestQuantizeRow() {
  // stochastic rounding is unbiased and stays inside the signed 16-bit / unsigned 16-bit lanes
  const float g = 0.37f, h = 0.21f, inv_g = 1.f / 0.25f, inv_h = 1.f / 0.25f;
  double sg = 0, sh = 0; const int n = 40000;
  for (int i = 0; i < n; ++i) {
    const int32_t w = QuantizeRow(g, h, inv_g, inv_h, true, 11u, 3u, static_cast<uint64_t>(i));
    sg += UnpackG(w); sh += UnpackH(w);
    CHECK(UnpackG(w) == 1 || UnpackG(w) == 2);
  }
  CHECK(std::fabs(sg / n - g * inv_g) < 0.02 && std::fabs(sh / n - h * inv_h) < 0.02);
  CHECK(UnpackG(PackGH(-5, 9)) == -5 && UnpackH(PackGH(-5, 9)) == 9);
}

static void TestBinMapper() {
  std::vector<double> v;
  for (int i = 0; i < 1000; ++i) v.push_back((i * 37 % 1000) / 10.0);
  Config cfg;
  BinMapper bm;
  bm.FindBin(v.data(), static_cast<int>(v.size()), 1000, 16, 3, 20, true, BinType::Numerical, true, false, {});
  CHECK(bm.num_bin >= 2 && bm.num_bin <= 16 && !bm.is_trivial);
  int prev = -1;
  for (double x = 0.0; x < 100.0; x += 0.5) { const int b = static_cast<int>(bm.ValueToBin(x)); CHECK(b >= prev && b < bm.num_bin); prev = b; }
  CHECK(static_cast<int>(bm.ValueToBin(std::nan(""))) < bm.num_bin);
}

static void TestTreeRoundTripAndPredict() {
  Tree t(4);
  const int r1 = t.Split(0, 0, 0, 3, 0.5, -1.0, 2.0, 60, 40, 6.0, 4.0, 10.f, 0, true);
  const int r2 = t.Split(r1, 1, 2, 5, -1.25, 0.25, 4.0, 30, 10, 3.0, 1.0, 5.f, 2, false);
  CHECK(r1 == 1 && r2 == 2 && t.num_leaves == 3);
  double row_a[3] = {0.4, 0.0, 9.0}, row_b[3] = {0.6, 0.0, -2.0}, row_c[3] = {0.6, 0.0, 7.0}, row_d[3] = {0.6, 0.0, std::nan("")};
  CHECK(t.Predict(row_a) == -1.0 && t.Predict(row_b) == 0.25 && t.Predict(row_c) == 4.0);
  CHECK(t.Predict(row_d) == 4.0);   // missing_type NaN with default right
  const std::string text = t.ToString();
  size_t used = 0;
  Tree u(text.c_str(), &used);
  CHECK(u.num_leaves == 3 && u.ToString() == text);
  CHECK(u.Predict(row_a) == -1.0 && u.Predict(row_b) == 0.25 && u.Predict(row_c) == 4.0 && u.Predict(row_d) == 4.0);
  t.Shrink(0.5);
  CHECK(t.Predict(row_c) == 2.0 && t.shrinkage == 0.5);
}

static void TestSplitMath() {
  SplitParams p; memset(&p, 0, sizeof(p));
  p.lambda_l2 = 1.0; p.min_data_in_leaf = 1;
  CHECK(LeafOutput(-6.0, 2.0, p, 10, 0.0) == 2.0);
  CHECK(LeafGain(-6.0, 2.0, p, 10, 0.0) == 12.0);
  p.lambda_l1 = 1.0;
  CHECK(ThresholdL1(-6.0, 1.0) == -5.0 && LeafOutput(-6.0, 2.0, p, 10, 0.0) == 5.0 / 3.0);
  // monotone ranges clamp the children and a violated order rejects the candidate
  p.lambda_l1 = 0.0; p.use_mc = 1;
  double gain, lo, ro;
  CHECK(SplitGain(-4.0, 1.0, 4.0, 1.0, p, 5, 5, 0.0, +1, -1.0, 1.0, &gain, &lo, &ro) == false);   // left 2 > right -2 under +1
  CHECK(SplitGain(4.0, 1.0, -4.0, 1.0, p, 5, 5, 0.0, +1, -1.0, 1.0, &gain, &lo, &ro) == true);
  CHECK(lo == -1.0 && ro == 1.0);   // clamped from -2 / +2
}

static void TestConfig() {
  Config cfg;
  cfg.Set(Config::Str2Map("n_estimators=37 num_leaf=15 eta=0.25 quant_mode=none monotone_constraints=1,-1,0 min_data=7 objective=binary"), false);
  CHECK(cfg.num_iterations == 37 && cfg.num_leaves == 15 && cfg.learning_rate == 0.25 && cfg.min_data_in_leaf == 7);
  CHECK(cfg.quant == QuantMode::None && cfg.objective == "binary");
  Config q; q.Set(Config::Str2Map("quant_mode=fixedpoint quant_bins=64"), false);
  CHECK(q.quant == QuantMode::FixedPoint && q.quant_bins == 64);
  CHECK(cfg.monotone_vec.size() == 3 && cfg.monotone_vec[0] == 1 && cfg.monotone_vec[1] == -1 && cfg.monotone_vec[2] == 0);
  Config depth; depth.Set(Config::Str2Map("num_leaves=255 max_depth=4"), false);
  CHECK(depth.num_leaves == 16);   // a depth cap bounds the leaf count
  bool threw = false;
  try { Config bad; bad.Set(Config::Str2Map("grow_policy=sideways"), false); } catch (const std::exception&) { threw = true; }
  CHECK(threw);
  threw = false;   // quantized training and monotone constraints combine on the host learner only
  try { Config bad; bad.Set(Config::Str2Map("quant_mode=stochastic monotone_constraints=1,0 device_type=cuda"), true); } catch (const std::exception&) { threw = true; }
  CHECK(threw);
  threw = false;
  try { Config ok; ok.Set(Config::Str2Map("quant_mode=stochastic monotone_constraints=1,0 device_type=cpu"), false); } catch (const std::exception&) { threw = true; }
  CHECK(!threw);
}

// Best-first growth over a random gain tree, against the rule of the level controller: a node is split while fewer
// than B evaluated nodes sort strictly before it by the order key; replaying best-first over the split nodes must
// then give exactly the best-first tree.
static void TestLeafwiseKeys() {
  typedef std::vector<int> Path;
  for (int seed = 0; seed < 60; ++seed) {
    std::map<Path, double> gains;
    auto gain = [&](const Path& v) {
      auto it = gains.find(v);
      if (it != gains.end()) return it->second;
      uint32_t h = 2166136261u ^ static_cast<uint32_t>(seed * 7919);
      for (int b : v) h = (h ^ static_cast<uint32_t>(b + 1)) * 16777619u;
      const Philox4 r = Philox4x32_10(h, static_cast<uint32_t>(v.size()), 0, 0, 17, 23);
      double g = U01From24(r.v[0]) * std::pow(seed % 2 ? 0.9 : 0.6, static_cast<double>(v.size()));
      if (U01From24(r.v[1]) < 0.1) g = -1.0;
      gains[v] = g; return g;
    };
    const int B = 3 + seed % 40;
    auto best_first = [&](const std::map<Path, int>* allowed) {
      std::vector<Path> picked;
      std::priority_queue<std::pair<double, Path>> pq; pq.push({gain(Path()), Path()});
      while (!pq.empty() && static_cast<int>(picked.size()) < B) {
        const auto top = pq.top(); pq.pop();
        if (!(top.first > 0.0)) break;
        if (allowed != nullptr && !allowed->count(top.second)) continue;   // not split on the "device": unsplittable
        picked.push_back(top.second);
        for (int c = 0; c < 2; ++c) { Path ch = top.second; ch.push_back(c); pq.push({gain(ch), ch}); }
      }
      std::sort(picked.begin(), picked.end());
      return picked;
    };
    const std::vector<Path> ref = best_first(nullptr);
    // level-wise over-growth with the key rule
    std::map<Path, std::vector<double>> key_of, pkey_of;
    pkey_of[Path()] = std::vector<double>(4, 1.0 / 0.0);
    std::vector<std::vector<double>> all_keys;
    std::map<Path, int> split;
    std::vector<Path> frontier = {Path()};
    while (!frontier.empty() && split.size() < 4000) {
      std::vector<Path> cand;
      for (const Path& v : frontier) {
        const double g = gain(v);
        if (!(g > 0.0)) continue;
        std::vector<double> k(4);
        LeafwiseChildKey(pkey_of[v].data(), g, k.data());
        key_of[v] = k; all_keys.push_back(k); cand.push_back(v);
      }
      std::vector<Path> next;
      for (const Path& v : cand) {
        int before = 0;
        for (const auto& k : all_keys) before += LeafwiseKeyBefore(k.data(), key_of[v].data()) ? 1 : 0;
        if (before >= B) continue;
        split[v] = 1;
        for (int c = 0; c < 2; ++c) { Path ch = v; ch.push_back(c); pkey_of[ch] = key_of[v]; next.push_back(ch); }
      }
      frontier.swap(next);
    }
    CHECK(best_first(&split) == ref);
    CHECK(split.size() <= 4 * ref.size() + 4);   // the growth cap of the device learner is 4 x the leaf budget
  }
}

// Fixed-point quantizer extras: the error feedback carries what rounding dropped into the next round, saturation is not
// fed back, and the robust scale re-anchors only below a small outlier cluster that an empty octave separates from the rest.
static void TestFixedPointExtras() {
  // feedback: a value of 0.3 levels rounds to 0, 0, 0, 1 ... so that the long-run mean is 0.3 levels
  int8_t res[2] = {0, 0};
  long long sum_g = 0, sum_h = 0;
  const int rounds = 1000;
  for (int r = 0; r < rounds; ++r) { const int32_t w = QuantizeRowFeedback(0.3f, 0.3f, 1.0f, 1.0f, 0, res); sum_g += UnpackG(w); sum_h += UnpackH(w); }
  CHECK(std::fabs(static_cast<double>(sum_g) / rounds - 0.3) < 0.01);
  CHECK(std::fabs(static_cast<double>(sum_h) / rounds - 0.3) < 0.01);
  long long plain = 0;
  for (int r = 0; r < rounds; ++r) plain += UnpackG(QuantizeRowFeedback(0.3f, 0.3f, 1.0f, 1.0f, 0, nullptr));
  CHECK(plain == 0);                                               // without feedback the 0.3 is lost every round
  res[0] = res[1] = 0;
  const int32_t sat = QuantizeRowFeedback(-100.0f, 1.0f, 1.0f, 1.0f, 32, res);
  CHECK(UnpackG(sat) == -32 && res[1] == 0);                       // saturated, and the saturation is not carried
  // robust scale: 1000 rows around 1e-3 .. 2e-3 and 5 rows at 1.0
  std::vector<long long> hist(kQuantMagBuckets, 0);
  for (int i = 0; i < 1000; ++i) ++hist[QuantMagBucket(1e-3f + 1e-6f * i, 1.0f)];
  for (int i = 0; i < 5; ++i) ++hist[QuantMagBucket(1.0f - 0.01f * i, 1.0f)];
  const float anchor = RobustGradAnchor(hist.data(), 1005, 1.0f);
  CHECK(anchor < 1.0f && anchor >= 2e-3f * 0.99f && anchor < 2.1e-3f);   // the upper edge of the bulk's top bucket
  // the same bulk without a gap below the top (magnitudes spread over every octave): nothing moves
  std::fill(hist.begin(), hist.end(), 0);
  for (int i = 0; i < 2000; ++i) ++hist[QuantMagBucket(std::pow(2.0f, -10.0f * i / 2000.0f), 1.0f)];
  CHECK(RobustGradAnchor(hist.data(), 2000, 1.0f) == 1.0f);
  // many large values are not outliers
  std::fill(hist.begin(), hist.end(), 0);
  for (int i = 0; i < 1000; ++i) ++hist[QuantMagBucket(1e-3f, 1.0f)];
  for (int i = 0; i < 200; ++i) ++hist[QuantMagBucket(1.0f, 1.0f)];
  CHECK(RobustGradAnchor(hist.data(), 1200, 1.0f) == 1.0f);
  // monotone penalty factor: forbidden near the root, towards 1 with depth
  CHECK(MonotonePenaltyFactor(0, 0.0) == 1.0);
  CHECK(MonotonePenaltyFactor(0, 2.0) < 1e-10 && MonotonePenaltyFactor(1, 2.0) < 1e-10);
  CHECK(std::fabs(MonotonePenaltyFactor(2, 2.0) - 0.5) < 1e-9 && std::fabs(MonotonePenaltyFactor(3, 2.0) - 0.75) < 1e-9);
  CHECK(std::fabs(MonotonePenaltyFactor(2, 0.5) - (1.0 - 0.5 / 4.0)) < 1e-9);
}

// Bin finding does not depend on the order of the sample, takes the 32-bit sort for values that are exact floats and the
// 64-bit sort otherwise (both must order alike), keeps zero in a bin of its own and gives NaN the last bin.
static void TestBinFindingInvariants() {
  std::vector<double> base;
  uint32_t s = 12345u;
  for (int i = 0; i < 20000; ++i) { s = s * 1664525u + 1013904223u; base.push_back(static_cast<double>(static_cast<float>((static_cast<double>(s >> 8) / 16777216.0 - 0.5) * 8.0))); }
  auto bounds_of = [](std::vector<double> v, int max_bin) {
    BinMapper bm; bm.FindBin(v.data(), static_cast<int>(v.size()), v.size(), max_bin, 3, 20, true, BinType::Numerical, true, false, {});
    return bm.bin_upper_bound;
  };
  const std::vector<double> sorted_bounds = bounds_of(base, 63);
  std::vector<double> shuffled = base;
  for (size_t i = shuffled.size() - 1; i > 0; --i) { s = s * 1664525u + 1013904223u; std::swap(shuffled[i], shuffled[s % (i + 1)]); }
  CHECK(bounds_of(shuffled, 63) == sorted_bounds);
  // the same sample scaled by (1 + 2^-40) is no longer made of exact floats and takes the 64-bit sort; the order of the
  // values is the same, so every value must land in the bin it had before
  std::vector<double> scaled = shuffled; for (double& x : scaled) x *= 1.0 + 1.0 / 1099511627776.0;
  BinMapper m32, m64;
  { std::vector<double> c = shuffled; m32.FindBin(c.data(), static_cast<int>(c.size()), c.size(), 63, 3, 20, true, BinType::Numerical, true, false, {}); }
  { std::vector<double> c = scaled; m64.FindBin(c.data(), static_cast<int>(c.size()), c.size(), 63, 3, 20, true, BinType::Numerical, true, false, {}); }
  CHECK(m32.num_bin == m64.num_bin);
  int moved = 0; for (size_t i = 0; i < shuffled.size(); ++i) if (m32.ValueToBin(shuffled[i]) != m64.ValueToBin(scaled[i])) ++moved;
  CHECK(moved == 0);
  // zeros that are not in the sample (sparse input) get their own bin between the negative and the positive values
  std::vector<double> sparse; for (int i = 0; i < 300; ++i) sparse.push_back(i % 2 ? 1.0 + i : -1.0 - i);
  BinMapper z; z.FindBin(sparse.data(), 300, 3000, 32, 3, 20, true, BinType::Numerical, true, false, {});
  CHECK(z.ValueToBin(0.0) == z.default_bin && z.ValueToBin(-1e-40) == z.default_bin && z.ValueToBin(2.0) > z.default_bin && z.ValueToBin(-2.0) < z.default_bin);
  CHECK(z.most_freq_bin == z.default_bin && z.sparse_rate > 0.85);
  // NaN in the sample: the last bin is the missing bin
  std::vector<double> nanv = base; for (size_t i = 0; i < nanv.size(); i += 10) nanv[i] = std::nan("");
  BinMapper m; m.FindBin(nanv.data(), static_cast<int>(nanv.size()), nanv.size(), 63, 3, 20, true, BinType::Numerical, true, false, {});
  CHECK(m.missing_type == MissingType::NaN && static_cast<int>(m.ValueToBin(std::nan(""))) == m.num_bin - 1 && std::isnan(m.bin_upper_bound.back()));
  // serialisation round trip
  std::vector<char> buf; m.Serialize(&buf);
  BinMapper back; back.Deserialize(buf.data());
  CHECK(back.num_bin == m.num_bin && back.missing_type == m.missing_type && back.default_bin == m.default_bin && back.most_freq_bin == m.most_freq_bin);
  for (double x : {-3.0, -0.1, 0.0, 0.1, 2.5}) CHECK(back.ValueToBin(x) == m.ValueToBin(x));
}

// Categorical bins: categories by frequency, rare ones and negatives in bin 0.
static void TestCategoricalBins() {
  std::vector<double> v;
  for (int i = 0; i < 1000; ++i) v.push_back(i % 10 < 6 ? 3.0 : (i % 10 < 9 ? 7.0 : 11.0));
  v.push_back(-1.0); v.push_back(42.0);
  BinMapper bm; bm.FindBin(v.data(), static_cast<int>(v.size()), v.size(), 16, 1, 1, false, BinType::Categorical, true, false, {});
  CHECK(bm.bin_type == BinType::Categorical && bm.num_bin >= 3);
  CHECK(bm.ValueToBin(3.0) == 1 && bm.ValueToBin(7.0) == 2);           // by count
  CHECK(bm.ValueToBin(-1.0) == 0 && bm.ValueToBin(12345.0) == 0 && bm.ValueToBin(std::nan("")) == 0);
}

// Linear leaves: prediction, shrinkage and the fallback to the constant for rows with a missing regressor.
static void TestLinearLeaves() {
  Tree t(2);
  t.Split(0, 0, 0, 3, 0.5, 1.0, 2.0, 60, 40, 6.0, 4.0, 10.f, 0, true);
  t.is_linear = true;
  t.leaf_const = {0.5, 2.0}; t.leaf_coeff = {{2.0, -1.0}, {}}; t.leaf_features = {{1, 2}, {}}; t.leaf_features_inner = {{1, 2}, {}};
  double left[3] = {0.0, 3.0, 4.0}, right[3] = {1.0, 3.0, 4.0}, missing[3] = {0.0, std::nan(""), 4.0};
  CHECK(t.Predict(left) == 0.5 + 2.0 * 3.0 - 4.0);
  CHECK(t.Predict(right) == 2.0);
  CHECK(t.Predict(missing) == 1.0);                                    // the leaf's constant output
  t.Shrink(0.5);
  CHECK(t.Predict(left) == 0.5 * (0.5 + 2.0 * 3.0 - 4.0) && t.Predict(missing) == 0.5);
  size_t used = 0; const std::string text = t.ToString();
  Tree u(text.c_str(), &used);
  CHECK(u.is_linear && u.Predict(left) == t.Predict(left) && u.ToString() == text);
}

// Monotone penalty factor and the candidate evaluation's size limits.
static void TestCandidateLimits() {
  CHECK(MonotonePenaltyFactor(3, 0.0) == 1.0);
  CHECK(MonotonePenaltyFactor(0, 2.0) == kEpsilon && MonotonePenaltyFactor(1, 2.0) == kEpsilon);   // forbidden above the penalty's depth
  CHECK(MonotonePenaltyFactor(2, 2.0) > 0.4 && MonotonePenaltyFactor(2, 2.0) < MonotonePenaltyFactor(5, 2.0) && MonotonePenaltyFactor(20, 2.0) <= 1.0 + kEpsilon);
  SplitParams p; memset(&p, 0, sizeof(p)); p.min_data_in_leaf = 10; p.min_sum_hessian_in_leaf = 1e-3;
  LeafScanInfo L; memset(&L, 0, sizeof(L));
  L.sum_g = 0.0; L.sum_h = 100.0; L.num_data = 100; L.cnt_factor = 1.0; L.g_scale = L.h_scale = 1.0; L.mono_factor = 1.0;
  L.min_c = -1.0 / 0.0; L.max_c = 1.0 / 0.0; L.min_gain_shift = LeafGain(0.0, 100.0 + 2 * kEpsilon, p, 100, 0.0);
  double lo, ro;
  CHECK(EvalCandidate(-5.0, 9.0, 9, L, p, 0, &lo, &ro) == -1.0 / 0.0);    // nine rows on the left: below min_data_in_leaf
  CHECK(EvalCandidate(-5.0, 95.0, 95, L, p, 0, &lo, &ro) == -1.0 / 0.0);  // five rows on the right
  const double g = EvalCandidate(-30.0, 50.0, 50, L, p, 0, &lo, &ro);
  CHECK(g > 0.0 && std::fabs(g - (900.0 / (50.0 + kEpsilon) * 2)) < 1e-6);
  CHECK(BinCountEstimate(2.49, 1.0) == 2 && BinCountEstimate(2.5, 1.0) == 3);
  // tie order of splits: higher gain, then lower feature, then lower threshold
  CHECK(SplitBetter(1.0, 3, 5, 0.5, 1, 1) && !SplitBetter(0.5, 1, 1, 1.0, 3, 5));
  CHECK(SplitBetter(1.0, 1, 9, 1.0, 2, 0) && SplitBetter(1.0, 2, 3, 1.0, 2, 4) && !SplitBetter(1.0, 2, 4, 1.0, 2, 4));
  CHECK(!SplitBetter(5.0, -1, 0, -1.0 / 0.0, -1, 0) && SplitBetter(-5.0, 0, 0, 1.0, -1, 0));
}

// Forced-split files and the debugging switches' parser.
static void TestForcedSplitFile() {
  const char* path = "core_tests_forced.json";
  FILE* f = fopen(path, "w");
  fputs("{ \"feature\": 3, \"threshold\": 0.25,\n  \"left\": {\"feature\": 4, \"threshold\": -0.5},\n  \"right\": {\"feature\": 1, \"threshold\": 0, \"right\": {\"feature\": 0, \"threshold\": 7}} }", f);
  fclose(f);
  const std::vector<ForcedSplitNode> nodes = LoadForcedSplitsFile(path);
  remove(path);
  CHECK(nodes.size() == 4 && nodes[0].feature == 3 && nodes[0].threshold == 0.25);
  CHECK(nodes[0].left == 1 && nodes[1].feature == 4 && nodes[1].left == -1 && nodes[1].right == -1);
  CHECK(nodes[0].right == 2 && nodes[2].feature == 1 && nodes[2].right == 3 && nodes[3].feature == 0 && nodes[3].threshold == 7.0);
  CHECK(LoadForcedSplitsFile("").empty());
}

int main() {
  TestBinFindingInvariants();
  TestCategoricalBins();
  TestLinearLeaves();
  TestCandidateLimits();
  TestForcedSplitFile();
  TestFixedPointExtras();
  TestFormatting();
  TestPhilox();
  TestQuantizeRow();
  TestBinMapper();
  TestTreeRoundTripAndPredict();
  TestSplitMath();
  TestConfig();
  TestLeafwiseKeys();
  printf("%d checks, %d failed\n", g_checks, g_failed);
  return g_failed == 0 ? 0 : 1;
}
