// Text data files: CSV / TSV / LibSVM with optional header; label / weight / group / ignore
// columns by index or "name:"; side files <data>.weight, <data>.query, <data>.init.
// Parity: src/io/parser.cpp (format detection), src/io/dataset_loader.cpp:L216 (LoadFromFile),
// src/io/metadata.cpp (side files).
#include "fb/dataset.h"
#include "fb/learner.h"

#include <fstream>

namespace fb {

namespace {

enum class Fmt { CSV, TSV, LIBSVM };

Fmt Detect(const std::vector<std::string>& lines) {
  int comma = 0, tab = 0, colon = 0;
  for (auto& l : lines) { for (char c : l) { if (c == ',') ++comma; else if (c == '\t') ++tab; else if (c == ':') ++colon; } }
  if (colon > 0 && comma == 0) return Fmt::LIBSVM;
  if (tab > 0 && comma == 0) return Fmt::TSV;
  if (comma > 0) return Fmt::CSV;
  return colon > 0 ? Fmt::LIBSVM : Fmt::TSV;
}

int ResolveColumn(const std::string& spec, const std::vector<std::string>& header) {
  std::string s = Trim(spec);
  if (s.empty()) return -1;
  if (StartsWith(s, "name:")) { std::string n = s.substr(5); for (size_t i = 0; i < header.size(); ++i) if (header[i] == n) return static_cast<int>(i); Log::Fatal("Could not find column %s in the data file header", n.c_str()); }
  return atoi(s.c_str());
}

std::vector<double> ReadSideFile(const std::string& path) {
  std::vector<double> v; std::ifstream f(path);
  if (!f) return v;
  std::string line; while (std::getline(f, line)) { line = Trim(line); if (!line.empty()) v.push_back(ParseDouble(line)); }
  return v;
}

}  // namespace

void ParseDataFile(const std::string& path, const Config& cfg, int force_num_features, ParsedFile* out) {
  std::ifstream f(path);
  if (!f) Log::Fatal("Data file %s doesn't exist", path.c_str());
  std::vector<std::string> lines; std::string line;
  while (std::getline(f, line)) { if (!line.empty() && line.back() == '\r') line.pop_back(); if (!Trim(line).empty()) lines.push_back(line); }
  if (lines.empty()) Log::Fatal("Data file %s is empty", path.c_str());
  std::vector<std::string> header;
  std::vector<std::string> probe(lines.begin() + (cfg.header ? 1 : 0), lines.begin() + std::min<size_t>(lines.size(), 32));
  const Fmt fmt = Detect(probe.empty() ? lines : probe);
  const char delim = fmt == Fmt::CSV ? ',' : '\t';
  if (cfg.header) { header = fmt == Fmt::LIBSVM ? SplitAny(lines[0], " \t") : Split(lines[0], delim); for (auto& h : header) h = Trim(h); lines.erase(lines.begin()); }
  int label_col = cfg.label_column.empty() ? 0 : ResolveColumn(cfg.label_column, header);
  int weight_col = ResolveColumn(cfg.weight_column, header), group_col = ResolveColumn(cfg.group_column, header);
  std::vector<int> ignore; for (auto& t : SplitAny(cfg.ignore_column, ",")) { int c = ResolveColumn(t, header); if (c >= 0) ignore.push_back(c); }
  // weight/group/ignore indices do not count the label column (reference convention)
  auto shift = [&](int c) { return (c >= 0 && label_col >= 0 && c >= label_col && !StartsWith(Trim(cfg.weight_column), "name:")) ? c + 1 : c; };
  if (!StartsWith(Trim(cfg.weight_column), "name:")) weight_col = shift(weight_col);
  if (!StartsWith(Trim(cfg.group_column), "name:") && group_col >= 0 && label_col >= 0 && group_col >= label_col) group_col += 1;

  const data_size_t n = static_cast<data_size_t>(lines.size());
  std::vector<float> label(n, 0.f), weight; std::vector<double> groupv;
  std::vector<std::vector<std::pair<int, double>>> rows(n);
  int ncol_raw = 0;
  for (data_size_t i = 0; i < n; ++i) {
    if (fmt == Fmt::LIBSVM) {
      auto toks = SplitAny(lines[i], " \t");
      size_t k = 0;
      if (!toks.empty() && toks[0].find(':') == std::string::npos) { label[i] = static_cast<float>(ParseDouble(toks[0])); k = 1; }
      for (; k < toks.size(); ++k) { size_t c = toks[k].find(':'); if (c == std::string::npos) continue; int idx = atoi(toks[k].substr(0, c).c_str()); double v = ParseDouble(toks[k].substr(c + 1)); rows[i].emplace_back(idx, v); ncol_raw = std::max(ncol_raw, idx + 1); }
    } else {
      auto toks = Split(lines[i], delim);
      ncol_raw = std::max<int>(ncol_raw, static_cast<int>(toks.size()));
      for (int c = 0; c < static_cast<int>(toks.size()); ++c) {
        std::string t = Trim(toks[c]);
        double v = (t.empty() || ToLower(t) == "na" || ToLower(t) == "nan" || ToLower(t) == "null") ? std::numeric_limits<double>::quiet_NaN() : ParseDouble(t);
        if (c == label_col) label[i] = static_cast<float>(v);
        else if (c == weight_col) { weight.resize(n, 1.f); weight[i] = static_cast<float>(v); }
        else if (c == group_col) { groupv.resize(n, 0); groupv[i] = v; }
        else rows[i].emplace_back(c, v);
      }
    }
  }
  // map raw columns to feature indices (dropping label / weight / group / ignored columns)
  std::vector<int> col2feat(ncol_raw, -1); int nfeat = 0;
  std::vector<std::string> names;
  for (int c = 0; c < ncol_raw; ++c) {
    if (fmt != Fmt::LIBSVM && (c == label_col || c == weight_col || c == group_col)) continue;
    if (std::find(ignore.begin(), ignore.end(), c) != ignore.end()) continue;
    col2feat[c] = nfeat++;
    names.push_back(c < static_cast<int>(header.size()) ? header[c] : "Column_" + std::to_string(nfeat - 1));
  }
  if (force_num_features > 0) nfeat = force_num_features;
  std::vector<double> dense(static_cast<size_t>(n) * nfeat, 0.0);
  for (data_size_t i = 0; i < n; ++i) for (auto& kv : rows[i]) { if (kv.first < ncol_raw && col2feat[kv.first] >= 0 && col2feat[kv.first] < nfeat) dense[static_cast<size_t>(i) * nfeat + col2feat[kv.first]] = kv.second; }
  out->num_rows = n; out->num_features = nfeat; out->dense.swap(dense); out->label.swap(label); out->weight.swap(weight); out->group_ids.swap(groupv);
  out->names.swap(names); out->has_header = !header.empty();
}

Dataset* LoadDatasetFromFile(const std::string& path, const Config& cfg, const Dataset* reference) {
  ParsedFile pf;
  ParseDataFile(path, cfg, reference != nullptr ? reference->num_total_features : 0, &pf);
  const data_size_t n = pf.num_rows; const int nfeat = pf.num_features;
  std::vector<double>& dense = pf.dense; std::vector<float>& label = pf.label; std::vector<float>& weight = pf.weight; std::vector<double>& groupv = pf.group_ids;
  std::vector<std::string>& names = pf.names;
  std::unique_ptr<Dataset> ds(new Dataset());
  // Several processes over the TCP mesh (the command line's distributed mode), training data only: with pre_partition
  // every process has read its own rows and the bin sample is the concatenation of every process's sample in rank order;
  // without it every process has read the whole file, draws the same sample and keeps its block of consecutive rows. Either
  // way all processes find the same bin boundaries, and the rows carry their global numbers.
  // Feature-parallel training is the exception: every process keeps all rows.
  const bool distributed = reference == nullptr && SocketNetworkActive() && Network::active() && cfg.tree_learner != "feature";
  data_size_t keep_begin = 0, keep_end = n; int64_t global_offset = 0, global_total = n;
  if (distributed) {
    if (!groupv.empty() && !cfg.pre_partition) Log::Fatal("Distributed ranking data must be pre-partitioned by query (pre_partition=true, one file per machine)");
    const int W = Network::world(), R = Network::rank();
    if (cfg.pre_partition) {
      GatherRowCounts(n, &global_offset, &global_total);
    } else {
      keep_begin = static_cast<data_size_t>(static_cast<int64_t>(n) * R / W); keep_end = static_cast<data_size_t>(static_cast<int64_t>(n) * (R + 1) / W);
      global_offset = keep_begin; global_total = n;
    }
  }
  if (reference != nullptr) ds->CopySchemaFrom(*reference);
  else {
    Random rnd(cfg.data_random_seed);
    int want = std::min<int>(n, cfg.bin_construct_sample_cnt);
    if (distributed && cfg.pre_partition) want = static_cast<int>(std::min<int64_t>(n, (static_cast<int64_t>(cfg.bin_construct_sample_cnt) * n + global_total - 1) / std::max<int64_t>(1, global_total)));
    auto idx = rnd.Sample(n, want);
    std::vector<double> sample(idx.size() * static_cast<size_t>(nfeat));
    for (size_t r = 0; r < idx.size(); ++r) memcpy(&sample[r * nfeat], &dense[static_cast<size_t>(idx[r]) * nfeat], nfeat * sizeof(double));
    if (distributed && cfg.pre_partition) { AllGatherSampleRows(&sample, nfeat); idx.resize(sample.size() / std::max(1, nfeat)); }
    std::vector<int> cats;
    for (auto& t : SplitAny(cfg.categorical_feature, ",")) { std::string s = Trim(t); if (StartsWith(s, "name:")) { for (size_t k = 0; k < names.size(); ++k) if (names[k] == s.substr(5)) cats.push_back(static_cast<int>(k)); } else if (!s.empty()) cats.push_back(atoi(s.c_str())); }
    if (pf.has_header) ds->feature_names = names;
    ds->ConstructSchema(sample.data(), static_cast<int>(idx.size()), nfeat, distributed ? global_total : n, cfg, cats);
  }
  if (distributed && (keep_begin != 0 || keep_end != n)) {
    // this process's block of the shared file
    const data_size_t m = keep_end - keep_begin;
    ds->global_num_data = global_total; ds->global_row_offset = global_offset;
    ds->AllocateRows(m);
    ds->PushDense(dense.data() + static_cast<size_t>(keep_begin) * nfeat, kF64, m, nfeat, true, 0);
    ds->metadata.label.assign(label.begin() + keep_begin, label.begin() + keep_end);
    if (!weight.empty()) ds->metadata.SetWeights(weight.data() + keep_begin, m);
    return ds.release();
  }
  if (distributed) { ds->global_num_data = global_total; ds->global_row_offset = global_offset; }
  ds->AllocateRows(n);
  ds->PushDense(dense.data(), kF64, n, nfeat, true, 0);
  ds->metadata.label = label;
  if (!weight.empty()) ds->metadata.SetWeights(weight.data(), n);
  if (!groupv.empty()) {
    std::vector<int32_t> sizes; double cur = groupv[0]; int cnt = 0;
    for (data_size_t i = 0; i < n; ++i) { if (groupv[i] != cur) { sizes.push_back(cnt); cnt = 0; cur = groupv[i]; } ++cnt; }
    sizes.push_back(cnt);
    ds->metadata.SetGroup(sizes.data(), static_cast<data_size_t>(sizes.size()));
  }
  auto w = ReadSideFile(path + ".weight");
  if (!w.empty()) { std::vector<float> wf(w.begin(), w.end()); ds->metadata.SetWeights(wf.data(), static_cast<data_size_t>(wf.size())); }
  auto q = ReadSideFile(path + ".query");
  if (!q.empty()) { std::vector<int32_t> sizes(q.begin(), q.end()); ds->metadata.SetGroup(sizes.data(), static_cast<data_size_t>(sizes.size())); }
  auto init = ReadSideFile(path + ".init");
  if (!init.empty()) ds->metadata.SetInitScore(init.data(), static_cast<int64_t>(init.size()));
  return ds.release();
}

}  // namespace fb
