// Host dataset: schema construction from a sample (bin mappers + exclusive feature bundling),
// dense row push, metadata, schema (de)serialisation, binary dataset files and row subsets.
// Parity (semantics): src/io/dataset_loader.cpp:L607-768, src/io/dataset.cpp:L125-262 (greedy
// conflict-bounded grouping), L414-531 (two orderings, fewer groups wins), L533-676 (Construct),
// L1298-1356 (CopySubrow); src/io/metadata.cpp.
#include "fb/dataset.h"
#include "fb/learner.h"

#include <omp.h>

#include <cstdio>
#include <fstream>
#include <numeric>

namespace fb {

Dataset::~Dataset() { if (device != nullptr) FreeDeviceDataset(device); }

void Metadata::SetGroup(const int32_t* sizes, data_size_t n) {
  query_boundaries.clear();
  if (sizes == nullptr || n == 0) return;
  query_boundaries.resize(n + 1);
  query_boundaries[0] = 0;
  for (data_size_t i = 0; i < n; ++i) query_boundaries[i + 1] = query_boundaries[i] + sizes[i];
  if (num_data > 0 && query_boundaries.back() != num_data)
    Log::Fatal("Sum of query counts (%d) differs from the number of rows (%d)", query_boundaries.back(), num_data);
  UpdateQueryWeights();
}

void Metadata::UpdateQueryWeights() {
  query_weights.clear();
  if (weights.empty() || query_boundaries.empty()) return;
  data_size_t nq = num_queries();
  query_weights.resize(nq);
  for (data_size_t q = 0; q < nq; ++q) {
    double s = 0; for (data_size_t i = query_boundaries[q]; i < query_boundaries[q + 1]; ++i) s += weights[i];
    query_weights[q] = static_cast<label_t>(s / std::max(1, query_boundaries[q + 1] - query_boundaries[q]));
  }
}

namespace {

struct BitSet {
  std::vector<uint64_t> w;
  explicit BitSet(int n) : w((n + 63) / 64, 0) {}
  inline bool Get(int i) const { return (w[i >> 6] >> (i & 63)) & 1; }
  inline void Set(int i) { w[i >> 6] |= (1ull << (i & 63)); }
};

// Greedy bundling over features in `order`. `nz[f]` lists the sample rows where feature f is away
// from its most frequent bin. A feature joins a group when the added conflicts keep the group's
// total under `max_conflict` and under half of the feature's own non-default count.
std::vector<std::vector<int>> BundleGreedy(const std::vector<int>& order, const std::vector<std::vector<int>>& nz,
                                           const std::vector<int>& nbins, int ns, int max_conflict, int max_group_bins,
                                           int seed) {
  std::vector<std::vector<int>> groups;
  std::vector<BitSet> marks;
  std::vector<int> conflicts, bins, nzcnt;
  Random rnd(seed);
  const int kSearch = 100;
  for (int f : order) {
    const int fcnt = static_cast<int>(nz[f].size());
    int best = -1;
    std::vector<int> cand;
    for (int g = 0; g < static_cast<int>(groups.size()); ++g)
      if (bins[g] + nbins[f] - 1 <= max_group_bins) cand.push_back(g);
    if (static_cast<int>(cand.size()) > kSearch) {
      // keep the most recent group plus a random subset
      std::vector<int> pick; pick.push_back(cand.back()); cand.pop_back();
      auto idx = rnd.Sample(static_cast<int>(cand.size()), kSearch - 1);
      for (int i : idx) pick.push_back(cand[i]);
      cand.swap(pick);
    }
    for (int g : cand) {
      const int room = max_conflict - conflicts[g];
      const int allow = std::min(room, fcnt / 2);
      if (allow < 0) continue;
      int c = 0; bool ok = true;
      for (int r : nz[f]) { if (marks[g].Get(r)) { if (++c > allow) { ok = false; break; } } }
      if (ok) { best = g; conflicts[g] += c; break; }
    }
    if (best < 0) {
      groups.emplace_back(); marks.emplace_back(ns); conflicts.push_back(0); bins.push_back(1); nzcnt.push_back(0);
      best = static_cast<int>(groups.size()) - 1;
    }
    groups[best].push_back(f);
    bins[best] += nbins[f] - 1;
    for (int r : nz[f]) marks[best].Set(r);
  }
  return groups;
}

template <typename T>
inline double ReadAs(const void* p, size_t i) { return static_cast<double>(static_cast<const T*>(p)[i]); }

inline double HalfToDouble(uint16_t h) {
  uint32_t sign = (h >> 15) & 1, exp = (h >> 10) & 0x1F, man = h & 0x3FF;
  double v;
  if (exp == 0) v = std::ldexp(static_cast<double>(man), -24);
  else if (exp == 31) v = man ? std::numeric_limits<double>::quiet_NaN() : std::numeric_limits<double>::infinity();
  else v = std::ldexp(static_cast<double>(man | 0x400), static_cast<int>(exp) - 25);
  return sign ? -v : v;
}

inline double ReadValue(const void* data, int dtype, size_t i) {
  switch (dtype) {
    case kF32: return ReadAs<float>(data, i);
    case kF64: return ReadAs<double>(data, i);
    case kI8: return ReadAs<int8_t>(data, i);
    case kI16: return ReadAs<int16_t>(data, i);
    case kU8: return ReadAs<uint8_t>(data, i);
    case kU16: return ReadAs<uint16_t>(data, i);
    case kI32: return ReadAs<int32_t>(data, i);
    case kF16: return HalfToDouble(static_cast<const uint16_t*>(data)[i]);
    default: Log::Fatal("Unsupported dtype code %d", dtype);
  }
}

}  // namespace

void Dataset::ConstructSchema(const double* sample, int ns, int ncol, int64_t total_rows, const Config& cfg,
                              const std::vector<int>& categorical) {
  ConstructSchemaTyped(sample, kF64, ns, ncol, total_rows, cfg, categorical);
}

void Dataset::ConstructSchemaTyped(const void* sample, int dtype, int ns, int ncol, int64_t total_rows, const Config& cfg,
                                   const std::vector<int>& categorical) {
  ScopedTimer timer("Dataset::ConstructSchema");
  num_total_features = ncol;
  max_bin_param = cfg.max_bin;
  keep_raw = cfg.linear_tree;
  categorical_features = categorical;
  std::vector<char> is_cat(ncol, 0);
  for (int c : categorical) if (c >= 0 && c < ncol) is_cat[c] = 1;
  mappers.clear(); mappers.resize(ncol);
  const int min_split_data = total_rows > 0
      ? static_cast<int>(static_cast<double>(cfg.min_data_in_leaf) * ns / static_cast<double>(total_rows)) : 0;
  // One bin search per feature, independent of each other: tiles of adjacent columns go to the host cores, and a
  // tile's rows are read in order (the sample is row-major, so a single column on its own would stride by a row).
  // The rows where a feature leaves its most frequent bin are collected in the same pass, for the bundling below.
  // narrow data: one column per task keeps every core busy; wide data: up to 16 columns per task
  // Several ranks holding the SAME sample (the global one, gathered by row id) split the bin search by feature: tile t
  // belongs to rank t % world, the finished mappers are all-gathered, and every rank ends up with the same schema as a
  // single process would. Parity: src/io/dataset_loader.cpp:L672-759 (features striped over machines, mappers gathered).
  const bool split_search = cfg.distributed_bin_finding && Network::active() && ncol >= 2;
  const int my_rank = split_search ? Network::rank() : 0, nranks = split_search ? Network::world() : 1;
  const int threads = std::max(1, omp_get_max_threads());
  const int kTile = split_search ? std::max(1, std::min(16, ncol / (4 * threads * nranks))) : std::max(1, std::min(16, ncol / (4 * threads)));
  const int ntiles = (ncol + kTile - 1) / kTile;
  std::vector<std::vector<int>> nz_by_col(cfg.enable_bundle ? ncol : 0);
#pragma omp parallel for schedule(dynamic, 1) num_threads(TeamThreads())
  for (int t = 0; t < ntiles; ++t) {
    if (t % nranks != my_rank) continue;
    const int j0 = t * kTile, j1 = std::min(ncol, j0 + kTile), w = j1 - j0;
    std::vector<std::vector<double>> cols(w, std::vector<double>(ns));
    std::vector<int> m(w, 0);
    for (int i = 0; i < ns; ++i) {
      for (int c = 0; c < w; ++c) {
        const double v = ReadValue(sample, dtype, static_cast<size_t>(i) * ncol + j0 + c);
        if (std::isnan(v) || std::fabs(v) > kZeroThreshold) cols[c][m[c]++] = v;
      }
    }
    for (int c = 0; c < w; ++c) {
      const int j = j0 + c;
      int mb = cfg.max_bin;
      if (j < static_cast<int>(cfg.max_bin_by_feature_vec.size())) mb = cfg.max_bin_by_feature_vec[j];
      mappers[j].reset(new BinMapper());
      mappers[j]->FindBin(cols[c].data(), m[c], ns, mb, cfg.min_data_in_bin, min_split_data, cfg.feature_pre_filter,
                          is_cat[j] ? BinType::Categorical : BinType::Numerical, cfg.use_missing, cfg.zero_as_missing, {});
    }
    if (cfg.enable_bundle && !split_search) {
      for (int i = 0; i < ns; ++i) {
        for (int c = 0; c < w; ++c) {
          const BinMapper& bm = *mappers[j0 + c];
          if (bm.is_trivial || bm.sparse_rate < 0.5) continue;   // dense features never share a bundle
          if (bm.ValueToBin(ReadValue(sample, dtype, static_cast<size_t>(i) * ncol + j0 + c)) != bm.most_freq_bin) nz_by_col[j0 + c].push_back(i);
        }
      }
    }
  }
  if (split_search) {
    // all-gather of the mappers: sizes first, then the serialised stripes padded to the largest
    std::vector<char> mine;
    for (int t = my_rank; t < ntiles; t += nranks)
      for (int j = t * kTile; j < std::min(ncol, (t + 1) * kTile); ++j) mappers[j]->Serialize(&mine);
    int64_t my_size = static_cast<int64_t>(mine.size());
    std::vector<char> sizes_raw; Network::Gather(&my_size, sizeof(int64_t), &sizes_raw);
    const int64_t* sizes = reinterpret_cast<const int64_t*>(sizes_raw.data());
    int64_t cap = 8; for (int r = 0; r < nranks; ++r) cap = std::max(cap, sizes[r]);
    mine.resize(static_cast<size_t>(cap), 0);
    std::vector<char> all; Network::Gather(mine.data(), cap, &all);
    for (int r = 0; r < nranks; ++r) {
      if (r == my_rank) continue;
      const char* p = all.data() + static_cast<size_t>(r) * cap;
      for (int t = r; t < ntiles; t += nranks)
        for (int j = t * kTile; j < std::min(ncol, (t + 1) * kTile); ++j) { mappers[j].reset(new BinMapper()); p = mappers[j]->Deserialize(p); }
    }
    if (cfg.enable_bundle) {
      // rows where a sparse feature leaves its most frequent bin, for the bundling below (needs every mapper)
#pragma omp parallel for schedule(dynamic, 8) num_threads(TeamThreads())
      for (int j = 0; j < ncol; ++j) {
        const BinMapper& bm = *mappers[j];
        if (bm.is_trivial || bm.sparse_rate < 0.5) continue;
        for (int i = 0; i < ns; ++i) if (bm.ValueToBin(ReadValue(sample, dtype, static_cast<size_t>(i) * ncol + j)) != bm.most_freq_bin) nz_by_col[j].push_back(i);
      }
    }
  }
  used_feature_map.assign(ncol, -1);
  real_feature_idx.clear();
  for (int j = 0; j < ncol; ++j) if (!mappers[j]->is_trivial) { used_feature_map[j] = static_cast<int>(real_feature_idx.size()); real_feature_idx.push_back(j); }
  num_features = static_cast<int>(real_feature_idx.size());
  if (num_features == 0) Log::Warning("There are no meaningful features which satisfy the provided configuration");
  if (feature_names.empty()) { for (int j = 0; j < ncol; ++j) feature_names.push_back("Column_" + std::to_string(j)); }

  // ---- exclusive feature bundling on the sample ----
  std::vector<std::vector<int>> groups;
  bool try_bundle = cfg.enable_bundle && num_features > 1;
  if (try_bundle) {
    std::vector<std::vector<int>> nz(num_features);
    std::vector<int> nbins(num_features);
    bool any_sparse = false;
    for (int f = 0; f < num_features; ++f) {
      const BinMapper& bm = *mappers[real_feature_idx[f]];
      nbins[f] = bm.num_bin;
      if (bm.sparse_rate >= 0.5) any_sparse = true;
    }
    if (any_sparse) {
      for (int f = 0; f < num_features; ++f) nz[f].swap(nz_by_col[real_feature_idx[f]]);
      const int max_conflict = ns / 10000;
      std::vector<int> order1;   // only sparse features are offered to the bundler; dense ones stay alone
      for (int f = 0; f < num_features; ++f) if (mappers[real_feature_idx[f]]->sparse_rate >= 0.5) order1.push_back(f);
      std::vector<int> order2 = order1;
      std::stable_sort(order2.begin(), order2.end(), [&](int a, int b) { return nz[a].size() > nz[b].size(); });
      auto g1 = BundleGreedy(order1, nz, nbins, ns, max_conflict, 256, static_cast<int>(total_rows & 0x7fffffff));
      auto g2 = BundleGreedy(order2, nz, nbins, ns, max_conflict, 256, static_cast<int>(total_rows & 0x7fffffff));
      groups = g2.size() < g1.size() ? g2 : g1;
      for (int f = 0; f < num_features; ++f) if (mappers[real_feature_idx[f]]->sparse_rate < 0.5) groups.push_back({f});
      // dense features (sparse_rate small) gain nothing from a bundle slot: keep them alone
      std::vector<std::vector<int>> cleaned;
      for (auto& g : groups) {
        if (g.size() == 1) { cleaned.push_back(g); continue; }
        std::vector<int> keep;
        for (int f : g) { if (mappers[real_feature_idx[f]]->sparse_rate < 0.5) cleaned.push_back({f}); else keep.push_back(f); }
        if (!keep.empty()) cleaned.push_back(keep);
      }
      groups.swap(cleaned);
      for (auto& g : groups) std::sort(g.begin(), g.end());
      std::sort(groups.begin(), groups.end(), [](const std::vector<int>& a, const std::vector<int>& b) { return a[0] < b[0]; });
    }
  }
  if (groups.empty()) { for (int f = 0; f < num_features; ++f) groups.push_back({f}); }
  BuildGroups(groups, cfg);
}

void Dataset::BuildGroups(const std::vector<std::vector<int>>& groups, const Config& cfg) {
  group_features = groups;
  num_groups = static_cast<int>(groups.size());
  group_bin_start.assign(num_groups, 0); group_num_bin.assign(num_groups, 0);
  feature_meta.assign(num_features, FeatureMeta());
  int total = 0; max_group_bin = 0;
  for (int g = 0; g < num_groups; ++g) {
    group_bin_start[g] = total;
    const bool multi = groups[g].size() > 1;
    int gb = multi ? 1 : 0;
    for (int f : groups[g]) {
      const BinMapper& bm = *mappers[real_feature_idx[f]];
      FeatureMeta& m = feature_meta[f];
      m.num_bin = bm.num_bin; m.missing_type = static_cast<int>(bm.missing_type); m.default_bin = bm.default_bin;
      m.most_freq_bin = bm.most_freq_bin; m.bundled = multi ? 1 : 0; m.bin_type = static_cast<int>(bm.bin_type);
      m.group = g; m.group_offset = multi ? gb : 0; m.hist_offset = total + (multi ? gb : 0);
      m.real_index = real_feature_idx[f];
      m.monotone = (m.real_index < static_cast<int>(cfg.monotone_vec.size())) ? cfg.monotone_vec[m.real_index] : 0;
      m.penalty = (m.real_index < static_cast<int>(cfg.feature_contri_vec.size())) ? static_cast<float>(cfg.feature_contri_vec[m.real_index]) : 1.0f;
      gb += multi ? bm.num_bin - 1 : bm.num_bin;
    }
    group_num_bin[g] = gb;
    max_group_bin = std::max(max_group_bin, gb);
    total += gb;
  }
  num_total_bin = total;
  bin_bytes = max_group_bin > 256 ? 2 : 1;
  row_stride = num_groups;
}

void Dataset::CopySchemaFrom(const Dataset& ref) {
  num_total_features = ref.num_total_features; num_features = ref.num_features; num_groups = ref.num_groups;
  num_total_bin = ref.num_total_bin; max_group_bin = ref.max_group_bin; max_bin_param = ref.max_bin_param;
  mappers.clear();
  for (auto& m : ref.mappers) mappers.emplace_back(new BinMapper(*m));
  used_feature_map = ref.used_feature_map; real_feature_idx = ref.real_feature_idx;
  group_features = ref.group_features; group_bin_start = ref.group_bin_start; group_num_bin = ref.group_num_bin;
  feature_meta = ref.feature_meta; feature_names = ref.feature_names; categorical_features = ref.categorical_features;
  bin_bytes = ref.bin_bytes; row_stride = ref.num_groups; keep_raw = ref.keep_raw;
}

void Dataset::AddFeaturesFrom(const Dataset& other) {
  if (other.num_data != num_data) Log::Fatal("Cannot add features from a dataset with %d rows to one with %d rows", other.num_data, num_data);
  if (!has_host_bins() || !other.has_host_bins()) Log::Fatal("AddFeaturesFrom needs host-resident bins in both datasets");
  if (device != nullptr) { FreeDeviceDataset(device); device = nullptr; }   // a device copy would be stale
  const int f0 = num_features, t0 = num_total_features, g0 = num_groups, b0 = num_total_bin;
  for (const auto& m : other.mappers) mappers.emplace_back(m ? new BinMapper(*m) : nullptr);
  for (int u : other.used_feature_map) used_feature_map.push_back(u < 0 ? -1 : u + f0);
  for (int r : other.real_feature_idx) real_feature_idx.push_back(r + t0);
  for (const auto& g : other.group_features) { std::vector<int> v; for (int f : g) v.push_back(f + f0); group_features.push_back(std::move(v)); }
  for (int s : other.group_bin_start) group_bin_start.push_back(s + b0);
  group_num_bin.insert(group_num_bin.end(), other.group_num_bin.begin(), other.group_num_bin.end());
  for (FeatureMeta m : other.feature_meta) { m.hist_offset += b0; m.group += g0; m.real_index += t0; feature_meta.push_back(m); }
  if (!feature_names.empty() || !other.feature_names.empty()) {
    std::vector<std::string> names = feature_names;
    for (int j = static_cast<int>(names.size()); j < t0; ++j) names.push_back("Column_" + std::to_string(j));
    for (int j = 0; j < other.num_total_features; ++j) {
      // a default name ("Column_<j>") moves with the column's new position; a given name is kept
      const bool given = j < static_cast<int>(other.feature_names.size()) && other.feature_names[j] != "Column_" + std::to_string(j);
      names.push_back(given ? other.feature_names[j] : "Column_" + std::to_string(t0 + j));
    }
    feature_names.swap(names);
  }
  for (int c : other.categorical_features) categorical_features.push_back(c + t0);
  // bin columns: rows of [this groups | other groups], in the wider of the two element types
  const int ng = g0 + other.num_groups;
  const bool wide = bin_bytes == 2 || other.bin_bytes == 2;
  auto cell = [](const Dataset& d, data_size_t i, int g) { return d.bin_bytes == 1 ? static_cast<int>(d.bins8[static_cast<size_t>(i) * d.row_stride + g]) : static_cast<int>(d.bins16[static_cast<size_t>(i) * d.row_stride + g]); };
  std::vector<uint8_t> n8; std::vector<uint16_t> n16;
  if (wide) n16.assign(static_cast<size_t>(num_data) * ng, 0); else n8.assign(static_cast<size_t>(num_data) * ng, 0);
  for (data_size_t i = 0; i < num_data; ++i) {
    for (int g = 0; g < g0; ++g) { const int v = cell(*this, i, g); if (wide) n16[static_cast<size_t>(i) * ng + g] = static_cast<uint16_t>(v); else n8[static_cast<size_t>(i) * ng + g] = static_cast<uint8_t>(v); }
    for (int g = 0; g < other.num_groups; ++g) { const int v = cell(other, i, g); if (wide) n16[static_cast<size_t>(i) * ng + g0 + g] = static_cast<uint16_t>(v); else n8[static_cast<size_t>(i) * ng + g0 + g] = static_cast<uint8_t>(v); }
  }
  bins8.swap(n8); bins16.swap(n16); bin_bytes = wide ? 2 : 1; row_stride = ng;
  if (has_raw() && other.has_raw()) {
    std::vector<float> r(static_cast<size_t>(num_data) * (t0 + other.num_total_features));
    for (data_size_t i = 0; i < num_data; ++i) {
      std::copy(raw.begin() + static_cast<size_t>(i) * t0, raw.begin() + static_cast<size_t>(i + 1) * t0, r.begin() + static_cast<size_t>(i) * (t0 + other.num_total_features));
      std::copy(other.raw.begin() + static_cast<size_t>(i) * other.num_total_features, other.raw.begin() + static_cast<size_t>(i + 1) * other.num_total_features,
                r.begin() + static_cast<size_t>(i) * (t0 + other.num_total_features) + t0);
    }
    raw.swap(r);
  } else { raw.clear(); keep_raw = false; }
  num_features += other.num_features; num_total_features += other.num_total_features; num_groups = ng; num_total_bin += other.num_total_bin;
  max_group_bin = std::max(max_group_bin, other.max_group_bin);
}

void Dataset::AllocateRows(data_size_t n) {
  num_data = n; metadata.num_data = n;
  if (global_num_data == 0) global_num_data = n;
  if (bin_bytes == 1) bins8.assign(static_cast<size_t>(n) * row_stride, 0); else bins16.assign(static_cast<size_t>(n) * row_stride, 0);
  if (keep_raw) raw.assign(static_cast<size_t>(n) * num_total_features, 0.f);
}

void Dataset::PushDense(const void* data, int dtype, data_size_t n, int ncol, bool row_major, data_size_t row_begin) {
  if (ncol != num_total_features) Log::Fatal("The number of columns (%d) differs from the dataset's (%d)", ncol, num_total_features);
  if (keep_raw && !raw.empty()) {
#pragma omp parallel for schedule(static) num_threads(TeamThreads())
    for (data_size_t i = 0; i < n; ++i)
      for (int j = 0; j < ncol; ++j)
        raw[static_cast<size_t>(row_begin + i) * ncol + j] = static_cast<float>(ReadValue(data, dtype, row_major ? static_cast<size_t>(i) * ncol + j : static_cast<size_t>(j) * n + i));
  }
#pragma omp parallel for schedule(static) num_threads(TeamThreads())
  for (data_size_t i = 0; i < n; ++i) {
    const size_t out = static_cast<size_t>(row_begin + i) * row_stride;
    for (int g = 0; g < num_groups; ++g) {
      int gb = 0;
      const auto& feats = group_features[g];
      if (feats.size() == 1) {
        const int j = real_feature_idx[feats[0]];
        const size_t src = row_major ? static_cast<size_t>(i) * ncol + j : static_cast<size_t>(j) * n + i;
        gb = mappers[j]->ValueToBin(ReadValue(data, dtype, src));
      } else {
        for (int f : feats) {
          const int j = real_feature_idx[f];
          const size_t src = row_major ? static_cast<size_t>(i) * ncol + j : static_cast<size_t>(j) * n + i;
          const int b = mappers[j]->ValueToBin(ReadValue(data, dtype, src));
          const FeatureMeta& m = feature_meta[f];
          if (b != m.most_freq_bin) gb = m.group_offset + (b > m.most_freq_bin ? b - 1 : b);   // later features win conflicts
        }
      }
      if (bin_bytes == 1) bins8[out + g] = static_cast<uint8_t>(gb); else bins16[out + g] = static_cast<uint16_t>(gb);
    }
  }
}

std::string Dataset::FeatureInfos() const {
  std::string s;
  for (int j = 0; j < num_total_features; ++j) {
    if (j) s += " ";
    s += (mappers[j] == nullptr || mappers[j]->is_trivial) ? std::string("none") : mappers[j]->InfoString();
  }
  return s;
}

void Dataset::SerializeSchema(std::vector<char>* out) const {
  auto put = [&](const void* p, size_t n) { const char* c = static_cast<const char*>(p); out->insert(out->end(), c, c + n); };
  int32_t hdr[3] = {num_total_features, num_groups, max_bin_param};
  put(hdr, sizeof(hdr));
  for (int j = 0; j < num_total_features; ++j) mappers[j]->Serialize(out);
  for (int g = 0; g < num_groups; ++g) {
    int32_t n = static_cast<int32_t>(group_features[g].size()); put(&n, 4);
    put(group_features[g].data(), n * sizeof(int));
  }
  int32_t nc = static_cast<int32_t>(categorical_features.size()); put(&nc, 4);
  put(categorical_features.data(), nc * sizeof(int));
  for (int j = 0; j < num_total_features; ++j) { int32_t l = static_cast<int32_t>(feature_names[j].size()); put(&l, 4); put(feature_names[j].data(), l); }
}

void Dataset::DeserializeSchema(const char* p, size_t n, const Config& cfg) {
  const char* end = p + n;
  int32_t hdr[3]; memcpy(hdr, p, sizeof(hdr)); p += sizeof(hdr);
  num_total_features = hdr[0]; int ng = hdr[1]; max_bin_param = hdr[2];
  mappers.clear(); mappers.resize(num_total_features);
  for (int j = 0; j < num_total_features; ++j) { mappers[j].reset(new BinMapper()); p = mappers[j]->Deserialize(p); }
  used_feature_map.assign(num_total_features, -1); real_feature_idx.clear();
  for (int j = 0; j < num_total_features; ++j) if (!mappers[j]->is_trivial) { used_feature_map[j] = static_cast<int>(real_feature_idx.size()); real_feature_idx.push_back(j); }
  num_features = static_cast<int>(real_feature_idx.size());
  std::vector<std::vector<int>> groups(ng);
  for (int g = 0; g < ng; ++g) { int32_t c; memcpy(&c, p, 4); p += 4; groups[g].resize(c); memcpy(groups[g].data(), p, c * sizeof(int)); p += c * sizeof(int); }
  int32_t nc; memcpy(&nc, p, 4); p += 4;
  categorical_features.resize(nc); memcpy(categorical_features.data(), p, nc * sizeof(int)); p += nc * sizeof(int);
  feature_names.clear();
  for (int j = 0; j < num_total_features; ++j) { int32_t l; memcpy(&l, p, 4); p += 4; feature_names.emplace_back(p, l); p += l; }
  FB_CHECK(p <= end);
  BuildGroups(groups, cfg);
}

void Dataset::SaveBinary(const std::string& path) const {
  if (!has_host_bins()) Log::Fatal("save_binary needs host-resident bins");
  std::ofstream f(path, std::ios::binary);
  if (!f) Log::Fatal("Cannot open %s for writing", path.c_str());
  const char magic[8] = {'F', 'B', 'D', 'S', 'B', 'I', 'N', '1'};
  f.write(magic, 8);
  std::vector<char> schema; SerializeSchema(&schema);
  int64_t sz = static_cast<int64_t>(schema.size());
  f.write(reinterpret_cast<const char*>(&sz), 8); f.write(schema.data(), sz);
  int32_t h[2] = {num_data, bin_bytes};
  f.write(reinterpret_cast<const char*>(h), sizeof(h));
  if (bin_bytes == 1) f.write(reinterpret_cast<const char*>(bins8.data()), bins8.size()); else f.write(reinterpret_cast<const char*>(bins16.data()), bins16.size() * 2);
  auto putvec = [&](const void* p, int64_t n, size_t es) { f.write(reinterpret_cast<const char*>(&n), 8); f.write(static_cast<const char*>(p), n * es); };
  putvec(metadata.label.data(), metadata.label.size(), sizeof(label_t));
  putvec(metadata.weights.data(), metadata.weights.size(), sizeof(label_t));
  putvec(metadata.query_boundaries.data(), metadata.query_boundaries.size(), sizeof(data_size_t));
  putvec(metadata.init_score.data(), metadata.init_score.size(), sizeof(double));
}

Dataset* Dataset::LoadBinary(const std::string& path) {
  std::ifstream f(path, std::ios::binary);
  if (!f) Log::Fatal("Cannot open %s", path.c_str());
  char magic[8]; f.read(magic, 8);
  if (memcmp(magic, "FBDSBIN1", 8) != 0) return nullptr;
  int64_t sz; f.read(reinterpret_cast<char*>(&sz), 8);
  std::vector<char> schema(sz); f.read(schema.data(), sz);
  std::unique_ptr<Dataset> ds(new Dataset());
  Config cfg;
  ds->DeserializeSchema(schema.data(), schema.size(), cfg);
  int32_t h[2]; f.read(reinterpret_cast<char*>(h), sizeof(h));
  ds->bin_bytes = h[1];
  ds->AllocateRows(h[0]);
  if (ds->bin_bytes == 1) f.read(reinterpret_cast<char*>(ds->bins8.data()), ds->bins8.size()); else f.read(reinterpret_cast<char*>(ds->bins16.data()), ds->bins16.size() * 2);
  auto getvec = [&](auto* v) { int64_t n; f.read(reinterpret_cast<char*>(&n), 8); v->resize(n); f.read(reinterpret_cast<char*>(v->data()), n * sizeof((*v)[0])); };
  getvec(&ds->metadata.label); getvec(&ds->metadata.weights); getvec(&ds->metadata.query_boundaries); getvec(&ds->metadata.init_score);
  ds->metadata.UpdateQueryWeights();
  return ds.release();
}

Dataset* Dataset::Subset(const data_size_t* idx, data_size_t n) const {
  if (!has_host_bins()) Log::Fatal("Subset needs host-resident bins");
  std::unique_ptr<Dataset> ds(new Dataset());
  ds->CopySchemaFrom(*this);
  ds->AllocateRows(n);
  for (data_size_t i = 0; i < n; ++i) {
    const size_t s = static_cast<size_t>(idx[i]) * row_stride, d = static_cast<size_t>(i) * row_stride;
    if (bin_bytes == 1) memcpy(&ds->bins8[d], &bins8[s], row_stride); else memcpy(&ds->bins16[d], &bins16[s], row_stride * 2);
    if (has_raw()) memcpy(&ds->raw[static_cast<size_t>(i) * num_total_features], &raw[static_cast<size_t>(idx[i]) * num_total_features], sizeof(float) * num_total_features);
  }
  if (!metadata.label.empty()) {
    const size_t targets = num_data > 0 ? std::max<size_t>(1, metadata.label.size() / static_cast<size_t>(num_data)) : 1;   // [target][row]
    ds->metadata.label.resize(static_cast<size_t>(n) * targets);
    for (size_t t = 0; t < targets; ++t)
      for (data_size_t i = 0; i < n; ++i) ds->metadata.label[t * n + i] = metadata.label[t * num_data + idx[i]];
  }
  if (!metadata.weights.empty()) { ds->metadata.weights.resize(n); for (data_size_t i = 0; i < n; ++i) ds->metadata.weights[i] = metadata.weights[idx[i]]; }
  if (!metadata.init_score.empty()) {
    int k = static_cast<int>(metadata.init_score.size() / num_data);
    ds->metadata.init_score.resize(static_cast<size_t>(k) * n);
    for (int c = 0; c < k; ++c) for (data_size_t i = 0; i < n; ++i) ds->metadata.init_score[static_cast<size_t>(c) * n + i] = metadata.init_score[static_cast<size_t>(c) * num_data + idx[i]];
  }
  if (!metadata.query_boundaries.empty()) {
    // rows of a subset are expected to keep whole queries together, in order
    std::vector<int32_t> sizes; data_size_t q = 0, cur = 0;
    for (data_size_t i = 0; i < n; ++i) {
      while (idx[i] >= metadata.query_boundaries[q + 1]) { if (cur) sizes.push_back(cur); cur = 0; ++q; }
      ++cur;
    }
    if (cur) sizes.push_back(cur);
    ds->metadata.SetGroup(sizes.data(), static_cast<data_size_t>(sizes.size()));
  }
  return ds.release();
}

bool Dataset::CheckAlign(const Dataset& o) const {
  if (num_total_features != o.num_total_features || num_features != o.num_features || num_groups != o.num_groups || num_total_bin != o.num_total_bin) return false;
  if (used_feature_map != o.used_feature_map || group_bin_start != o.group_bin_start || group_features != o.group_features) return false;
  for (int f = 0; f < num_total_features; ++f) {
    const BinMapper* a = mappers[f].get(); const BinMapper* b = o.mappers[f].get();
    if ((a == nullptr) != (b == nullptr)) return false;
    if (a == nullptr) continue;
    if (a->num_bin != b->num_bin || a->bin_type != b->bin_type || a->missing_type != b->missing_type || a->default_bin != b->default_bin ||
        a->most_freq_bin != b->most_freq_bin || a->is_trivial != b->is_trivial) return false;
    if (a->bin_type == BinType::Numerical) {
      if (a->bin_upper_bound.size() != b->bin_upper_bound.size()) return false;
      for (size_t k = 0; k < a->bin_upper_bound.size(); ++k) {
        const double x = a->bin_upper_bound[k], y = b->bin_upper_bound[k];
        if (!(x == y || (std::isnan(x) && std::isnan(y)))) return false;
      }
    } else if (a->bin_2_categorical != b->bin_2_categorical) return false;
  }
  return true;
}

}  // namespace fb
