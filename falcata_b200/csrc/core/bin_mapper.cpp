// Bin boundary search for one feature from a value sample.
// Parity (semantics, not code): src/io/bin.cpp:L81-160 (greedy equal-frequency search with
// big-count values), L247-303 (zero gets its own bin), L316-511 (FindBin: missing type,
// distinct values, categorical by frequency, trivial-feature filter, default/most-freq bin).
#include "fb/bin.h"

#include <cstring>

#include <numeric>

namespace fb {

namespace {

// Smallest double strictly above the midpoint is not needed: values <= bound go left, and the
// bound is the midpoint of two distinct sampled values, nudged up when rounding collapsed it.
inline double UpperBoundBetween(double lo, double hi) {
  double mid = (lo + hi) / 2.0;
  if (!(mid >= lo) || mid >= hi) mid = lo;   // adjacent doubles: keep lo as the inclusive bound
  return mid;
}

// Boundaries over one sign side. `vals`/`cnts` are ascending distinct values with their counts.
std::vector<double> GreedyBounds(const double* vals, const int* cnts, int n, int max_bin, size_t total, int min_data_in_bin) {
  std::vector<double> bounds;
  if (max_bin <= 0 || n == 0) return bounds;
  if (n <= max_bin) {
    int acc = 0;
    for (int i = 0; i < n - 1; ++i) {
      acc += cnts[i];
      if (acc >= min_data_in_bin) { bounds.push_back(UpperBoundBetween(vals[i], vals[i + 1])); acc = 0; }
    }
    bounds.push_back(std::numeric_limits<double>::infinity());
    return bounds;
  }
  if (min_data_in_bin > 0) max_bin = std::max(1, std::min(max_bin, static_cast<int>(total / min_data_in_bin)));
  double mean_size = static_cast<double>(total) / max_bin;
  std::vector<char> big(n, 0);
  int rest_bins = max_bin; size_t rest_cnt = total;
  for (int i = 0; i < n; ++i) if (cnts[i] >= mean_size) { big[i] = 1; --rest_bins; rest_cnt -= cnts[i]; }
  mean_size = rest_bins > 0 ? static_cast<double>(rest_cnt) / rest_bins : std::numeric_limits<double>::infinity();
  std::vector<double> hi_of_bin, lo_of_next;
  int acc = 0, bins_made = 0;
  for (int i = 0; i < n - 1; ++i) {
    if (!big[i]) rest_cnt -= cnts[i];
    acc += cnts[i];
    bool close = big[i] || acc >= mean_size || (big[i + 1] && acc >= std::max(1.0, mean_size * 0.5));
    if (close) {
      hi_of_bin.push_back(vals[i]); lo_of_next.push_back(vals[i + 1]);
      ++bins_made; acc = 0;
      if (bins_made >= max_bin - 1) break;
      if (!big[i]) { --rest_bins; mean_size = rest_bins > 0 ? static_cast<double>(rest_cnt) / rest_bins : std::numeric_limits<double>::infinity(); }
    }
  }
  for (size_t i = 0; i < hi_of_bin.size(); ++i) {
    double b = UpperBoundBetween(hi_of_bin[i], lo_of_next[i]);
    if (bounds.empty() || b > bounds.back()) bounds.push_back(b);
  }
  bounds.push_back(std::numeric_limits<double>::infinity());
  return bounds;
}

// Zero keeps a bin of its own, (-kZeroThreshold, kZeroThreshold]; negatives and positives get
// bin budgets proportional to their sample counts.
std::vector<double> BoundsZeroOwnBin(const std::vector<double>& vals, const std::vector<int>& cnts, int max_bin,
                                     size_t total, int min_data_in_bin) {
  const int n = static_cast<int>(vals.size());
  int n_neg = 0; size_t cnt_neg = 0, cnt_pos = 0, cnt_zero = 0;
  int first_pos = n;
  for (int i = 0; i < n; ++i) {
    if (vals[i] <= -kZeroThreshold) { ++n_neg; cnt_neg += cnts[i]; }
    else if (vals[i] > kZeroThreshold) { if (first_pos == n) first_pos = i; cnt_pos += cnts[i]; }
    else cnt_zero += cnts[i];
  }
  const int n_pos = n - first_pos;
  std::vector<double> bounds;
  int budget = max_bin - 1;  // one bin is the zero bin
  int neg_bins = 0;
  if (n_neg > 0) {
    double share = static_cast<double>(cnt_neg) / std::max<size_t>(1, cnt_neg + cnt_pos);
    neg_bins = std::max(1, static_cast<int>(share * budget));
    if (n_pos > 0) neg_bins = std::min(neg_bins, budget - 1);
    neg_bins = std::max(1, neg_bins);
    auto nb = GreedyBounds(vals.data(), cnts.data(), n_neg, neg_bins, cnt_neg, min_data_in_bin);
    if (!nb.empty()) nb.back() = -kZeroThreshold;   // the last negative bin ends just below zero
    bounds = nb;
  }
  int pos_bins = budget - static_cast<int>(bounds.size());
  if (n_pos > 0 && pos_bins > 0) {
    bounds.push_back(kZeroThreshold);               // zero bin
    auto pb = GreedyBounds(vals.data() + first_pos, cnts.data() + first_pos, n_pos, pos_bins, cnt_pos, min_data_in_bin);
    bounds.insert(bounds.end(), pb.begin(), pb.end());
  } else {
    bounds.push_back(std::numeric_limits<double>::infinity());  // zero (and any positives) share the last bin
  }
  (void)cnt_zero;
  return bounds;
}

inline bool NearlyEqualOrdered(double a, double b) {
  // a <= b assumed; equal or adjacent representable doubles are merged. Neighbouring doubles differ by at most
  // 2.3e-16 of their magnitude, so a wider gap settles the question without the library call.
  if (b - a > std::fabs(a) * 2.3e-16 + 1e-300) return false;
  return b <= std::nextafter(a, std::numeric_limits<double>::infinity());
}

}  // namespace

namespace {
// Ascending sort of finite doubles. Large inputs take an LSD radix sort on the order-preserving integer image
// of the IEEE bits, over the bit range that actually differs between the keys (values that came from float32 share
// their low 29 mantissa bits) in 12-bit digits, with all digit histograms counted in one read and the two key
// buffers kept per thread: about twice as fast as eight 8-bit passes on the 200k-value columns of a bin sample,
// which is where ingest spends its host time.
void SortValues(double* v, int n) {
  if (n < 4096) { std::sort(v, v + n); return; }
  if (std::is_sorted(v, v + n)) return;
  {
    // values that are exactly single-precision floats (a float32 matrix, the usual input) sort as 32-bit keys: three
    // 11-bit passes over arrays of half the size. Floats and doubles order alike (signed zeros included), so the result
    // is the one of the 64-bit path below.
    static thread_local std::vector<uint32_t> tl_fa, tl_fb;
    std::vector<uint32_t>& fa = tl_fa; std::vector<uint32_t>& fb32 = tl_fb;
    if (fa.size() < static_cast<size_t>(n)) { fa.resize(n); fb32.resize(n); }
    bool exact = true;
    for (int i = 0; i < n; ++i) {
      const float f = static_cast<float>(v[i]);
      if (static_cast<double>(f) != v[i]) { exact = false; break; }
      uint32_t u; memcpy(&u, &f, 4); fa[i] = (u >> 31) ? ~u : (u | 0x80000000u);
    }
    if (exact) {
      constexpr int kD = 11, kR = 1 << kD;
      uint32_t count[3][kR + 1] = {};
      for (int i = 0; i < n; ++i) { const uint32_t u = fa[i]; ++count[0][(u & (kR - 1)) + 1]; ++count[1][((u >> kD) & (kR - 1)) + 1]; ++count[2][(u >> (2 * kD)) + 1]; }
      uint32_t* src = fa.data(); uint32_t* dst = fb32.data();
      for (int p = 0; p < 3; ++p) {
        uint32_t* c = count[p];
        const int shift = p * kD;
        if (c[((src[0] >> shift) & (kR - 1)) + 1] == static_cast<uint32_t>(n)) continue;   // all keys share this digit
        for (int d = 0; d < kR; ++d) c[d + 1] += c[d];
        for (int i = 0; i < n; ++i) dst[c[(src[i] >> shift) & (kR - 1)]++] = src[i];
        std::swap(src, dst);
      }
      for (int i = 0; i < n; ++i) { uint32_t u = src[i]; u = (u >> 31) ? (u & 0x7FFFFFFFu) : ~u; float f; memcpy(&f, &u, 4); v[i] = static_cast<double>(f); }
      return;
    }
  }
  static thread_local std::vector<uint64_t> tl_a, tl_b;
  std::vector<uint64_t>& a = tl_a; std::vector<uint64_t>& b = tl_b;
  if (a.size() < static_cast<size_t>(n)) { a.resize(n); b.resize(n); }
  uint64_t all_or = 0, all_and = ~0ull;
  for (int i = 0; i < n; ++i) { uint64_t u; memcpy(&u, &v[i], 8); u = (u >> 63) ? ~u : (u | 0x8000000000000000ull); a[i] = u; all_or |= u; all_and &= u; }
  const uint64_t diff = all_or ^ all_and;
  if (diff == 0) return;
  const int lo = __builtin_ctzll(diff), hi = 63 - __builtin_clzll(diff);
  constexpr int kDigit = 12, kRadix = 1 << kDigit;
  const int passes = (hi - lo + 1 + kDigit - 1) / kDigit;
  std::vector<uint32_t> count(static_cast<size_t>(passes) * (kRadix + 1), 0);
  for (int i = 0; i < n; ++i) {
    const uint64_t u = a[i] >> lo;
    for (int p = 0; p < passes; ++p) ++count[static_cast<size_t>(p) * (kRadix + 1) + ((u >> (p * kDigit)) & (kRadix - 1)) + 1];
  }
  uint64_t* src = a.data(); uint64_t* dst = b.data();
  for (int p = 0; p < passes; ++p) {
    uint32_t* c = count.data() + static_cast<size_t>(p) * (kRadix + 1);
    const int shift = lo + p * kDigit;
    if (c[((src[0] >> shift) & (kRadix - 1)) + 1] == static_cast<uint32_t>(n)) continue;   // all keys share this digit
    for (int d = 0; d < kRadix; ++d) c[d + 1] += c[d];
    for (int i = 0; i < n; ++i) dst[c[(src[i] >> shift) & (kRadix - 1)]++] = src[i];
    std::swap(src, dst);
  }
  for (int i = 0; i < n; ++i) { uint64_t u = src[i]; u = (u >> 63) ? (u & 0x7FFFFFFFFFFFFFFFull) : ~u; memcpy(&v[i], &u, 8); }
}
}  // namespace

void BinMapper::FindBin(double* values, int num_values, size_t total_sample_cnt, int max_bin, int min_data_in_bin,
                        int min_split_data, bool pre_filter, BinType type, bool use_missing, bool zero_as_missing,
                        const std::vector<double>& forced_upper_bounds) {
  bin_type = type;
  default_bin = 0;
  // NaNs are moved out first.
  int na_cnt = 0, m = 0;
  for (int i = 0; i < num_values; ++i) { if (std::isnan(values[i])) ++na_cnt; else values[m++] = values[i]; }
  num_values = m;
  if (!use_missing) missing_type = MissingType::None;
  else if (zero_as_missing) missing_type = MissingType::Zero;
  else missing_type = na_cnt > 0 ? MissingType::NaN : MissingType::None;
  const size_t zero_cnt = total_sample_cnt - static_cast<size_t>(num_values) - static_cast<size_t>(na_cnt);

  SortValues(values, num_values);
  // distinct values with their counts (adjacent doubles merge into the larger one); the implicit zeros of the sample
  // enter once, between the negative and the positive values. Written through raw indices: with a continuous feature
  // nearly every sampled value is distinct and the loop runs once per value.
  std::vector<double> dv(static_cast<size_t>(num_values) + 2); std::vector<int> dc(static_cast<size_t>(num_values) + 2);
  int top = -1;   // index of the last distinct value
  bool zero_pushed = false;
  auto push_zero = [&] {
    if (!zero_pushed && zero_cnt > 0) {
      if (top >= 0 && dv[top] == 0.0) dc[top] += static_cast<int>(zero_cnt);
      else { ++top; dv[top] = 0.0; dc[top] = static_cast<int>(zero_cnt); }
    }
    zero_pushed = true;
  };
  if (num_values == 0 || values[0] > 0.0) push_zero();
  for (int i = 0; i < num_values; ++i) {
    const double x = values[i];
    if (!zero_pushed && x > 0.0) push_zero();
    if (top >= 0) {
      const double last = dv[top];
      if (last != 0.0 && NearlyEqualOrdered(last, x)) { dv[top] = x; ++dc[top]; continue; }
      if (last == x) { ++dc[top]; continue; }
    }
    ++top; dv[top] = x; dc[top] = 1;
  }
  if (!zero_pushed) push_zero();
  if (top < 0) { top = 0; dv[0] = 0.0; dc[0] = static_cast<int>(total_sample_cnt); }
  dv.resize(static_cast<size_t>(top) + 1); dc.resize(static_cast<size_t>(top) + 1);
  min_val = dv.front(); max_val = dv.back();
  const int nd = static_cast<int>(dv.size());
  std::vector<int> cnt_in_bin;

  if (type == BinType::Numerical) {
    std::vector<double> ub;
    if (!forced_upper_bounds.empty()) {
      ub = forced_upper_bounds;
      std::sort(ub.begin(), ub.end());
      ub.push_back(std::numeric_limits<double>::infinity());
      if (static_cast<int>(ub.size()) > max_bin - (missing_type == MissingType::NaN ? 1 : 0)) ub.resize(max_bin - (missing_type == MissingType::NaN ? 1 : 0)), ub.back() = std::numeric_limits<double>::infinity();
    } else if (missing_type == MissingType::Zero) {
      ub = BoundsZeroOwnBin(dv, dc, max_bin, total_sample_cnt - na_cnt, min_data_in_bin);
      if (ub.size() == 2) missing_type = MissingType::None;
    } else if (missing_type == MissingType::None) {
      ub = BoundsZeroOwnBin(dv, dc, max_bin, total_sample_cnt - na_cnt, min_data_in_bin);
    } else {
      ub = BoundsZeroOwnBin(dv, dc, max_bin - 1, total_sample_cnt - na_cnt, min_data_in_bin);
      ub.push_back(std::numeric_limits<double>::quiet_NaN());
    }
    bin_upper_bound = ub;
    num_bin = static_cast<int>(ub.size());
    cnt_in_bin.assign(num_bin, 0);
    int b = 0;
    for (int i = 0; i < nd; ++i) {
      while (b < num_bin - 1 && !(dv[i] <= bin_upper_bound[b])) ++b;
      cnt_in_bin[b] += dc[i];
    }
    if (missing_type == MissingType::NaN) cnt_in_bin[num_bin - 1] = na_cnt;
    FB_CHECK(num_bin <= max_bin);
  } else {
    // categorical: by count, keep until 99% of the non-NaN mass or max_bin; bin 0 = NaN/other/negative
    std::vector<int> ci; std::vector<int> cc;
    int neg_or_na = na_cnt;
    for (int i = 0; i < nd; ++i) {
      int v = static_cast<int>(dv[i]);
      if (v < 0) { neg_or_na += dc[i]; continue; }
      if (!ci.empty() && ci.back() == v) cc.back() += dc[i]; else { ci.push_back(v); cc.push_back(dc[i]); }
    }
    std::vector<int> order(ci.size());
    std::iota(order.begin(), order.end(), 0);
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return cc[a] > cc[b]; });
    size_t mass = 0; for (int c : cc) mass += c;
    const size_t cut = static_cast<size_t>(0.99 * static_cast<double>(mass));
    bin_2_categorical.clear(); categorical_2_bin.clear();
    bin_2_categorical.push_back(-1); cnt_in_bin.push_back(0);
    size_t used = 0;
    int cap = std::min(max_bin, static_cast<int>(ci.size()) + 1);
    for (size_t k = 0; k < order.size(); ++k) {
      if (static_cast<int>(bin_2_categorical.size()) >= cap) break;
      if (used >= cut && k > 0) break;
      int idx = order[k];
      categorical_2_bin[ci[idx]] = static_cast<int>(bin_2_categorical.size());
      bin_2_categorical.push_back(ci[idx]);
      cnt_in_bin.push_back(cc[idx]);
      used += cc[idx];
    }
    num_bin = static_cast<int>(bin_2_categorical.size());
    cnt_in_bin[0] = static_cast<int>(total_sample_cnt - used);
    missing_type = (cnt_in_bin[0] > 0 && use_missing) ? MissingType::NaN : MissingType::None;
    (void)neg_or_na;
  }

  is_trivial = num_bin <= 1;
  if (!is_trivial && pre_filter && min_split_data > 0) {
    // No threshold can leave >= min_split_data on both sides -> unusable feature.
    bool usable = false; int left = 0; int total = 0;
    for (int c : cnt_in_bin) total += c;
    if (type == BinType::Numerical) {
      for (int i = 0; i < num_bin - 1; ++i) { left += cnt_in_bin[i]; if (left >= min_split_data && total - left >= min_split_data) { usable = true; break; } }
    } else {
      for (int i = 0; i < num_bin; ++i) { if (cnt_in_bin[i] >= min_split_data && total - cnt_in_bin[i] >= min_split_data) { usable = true; break; } }
    }
    if (!usable) is_trivial = true;
  }
  if (!is_trivial) {
    default_bin = ValueToBin(0.0);
    most_freq_bin = static_cast<int>(std::max_element(cnt_in_bin.begin(), cnt_in_bin.end()) - cnt_in_bin.begin());
    double top_share = static_cast<double>(cnt_in_bin[most_freq_bin]) / std::max<size_t>(1, total_sample_cnt);
    if (most_freq_bin != default_bin && top_share < kSparseThreshold) most_freq_bin = default_bin;
    sparse_rate = static_cast<double>(cnt_in_bin[most_freq_bin]) / std::max<size_t>(1, total_sample_cnt);
  } else {
    sparse_rate = 1.0; most_freq_bin = 0;
  }
}

std::string BinMapper::InfoString() const {
  if (bin_type == BinType::Categorical) {
    std::string s;
    for (size_t i = 1; i < bin_2_categorical.size(); ++i) { if (i > 1) s += ":"; s += std::to_string(bin_2_categorical[i]); }
    if (s.empty()) s = "none";
    return s;
  }
  return "[" + DoubleToStr17(min_val) + ":" + DoubleToStr17(max_val) + "]";
}

void BinMapper::Serialize(std::vector<char>* out) const {
  auto put = [&](const void* p, size_t n) { const char* c = static_cast<const char*>(p); out->insert(out->end(), c, c + n); };
  int32_t hdr[6] = {num_bin, static_cast<int>(missing_type), static_cast<int>(bin_type), is_trivial ? 1 : 0, default_bin, most_freq_bin};
  put(hdr, sizeof(hdr));
  double d[3] = {sparse_rate, min_val, max_val};
  put(d, sizeof(d));
  int32_t nu = static_cast<int32_t>(bin_upper_bound.size()), nc = static_cast<int32_t>(bin_2_categorical.size());
  put(&nu, 4); put(&nc, 4);
  put(bin_upper_bound.data(), nu * sizeof(double));
  put(bin_2_categorical.data(), nc * sizeof(int));
}

const char* BinMapper::Deserialize(const char* p) {
  int32_t hdr[6]; memcpy(hdr, p, sizeof(hdr)); p += sizeof(hdr);
  num_bin = hdr[0]; missing_type = static_cast<MissingType>(hdr[1]); bin_type = static_cast<BinType>(hdr[2]);
  is_trivial = hdr[3] != 0; default_bin = hdr[4]; most_freq_bin = hdr[5];
  double d[3]; memcpy(d, p, sizeof(d)); p += sizeof(d);
  sparse_rate = d[0]; min_val = d[1]; max_val = d[2];
  int32_t nu, nc; memcpy(&nu, p, 4); p += 4; memcpy(&nc, p, 4); p += 4;
  bin_upper_bound.resize(nu); memcpy(bin_upper_bound.data(), p, nu * sizeof(double)); p += nu * sizeof(double);
  bin_2_categorical.resize(nc); memcpy(bin_2_categorical.data(), p, nc * sizeof(int)); p += nc * sizeof(int);
  categorical_2_bin.clear();
  for (int i = 1; i < nc; ++i) categorical_2_bin[bin_2_categorical[i]] = i;
  return p;
}

}  // namespace fb
