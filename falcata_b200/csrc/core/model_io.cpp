// Model serialisation: LightGBM-compatible v4 text format (writer + reader), JSON dump, if-else
// C++ export, feature importance, and the FALB sectioned binary container.
// Parity: src/boosting/gbdt_model_text.cpp:L315-422 (save), L435-639 (load), L641-675 (importance),
// L1-313 (JSON / if-else); src/boosting/falb.h:L35-114 + gbdt_model_binary.cpp (binary container:
// magic, version, section table, per-section compression with a byte-plane shuffle).
#include "fb/gbdt.h"

#include <unordered_map>
#include <zlib.h>

namespace fb {

std::vector<double> GBDT::FeatureImportance(int num_iter, int importance_type) const {
  int n = static_cast<int>(models_.size());
  if (num_iter > 0) n = std::min(n, num_iter * num_tree_per_iteration_);
  std::vector<double> imp(max_feature_idx_ + 1, 0.0);
  for (int t = 0; t < n; ++t) for (int s = 0; s < models_[t]->num_leaves - 1; ++s) {
    if (models_[t]->split_gain[s] <= 0) continue;
    const int f = models_[t]->split_feature[s];
    if (f < 0 || f > max_feature_idx_) continue;
    imp[f] += importance_type == 0 ? 1.0 : models_[t]->split_gain[s];
  }
  return imp;
}

std::string GBDT::SaveModelToString(int start_iter, int num_iter, int importance_type) const {
  std::string s;
  s += "tree\n";
  s += "version=v4\n";
  s += "num_class=" + std::to_string(num_class_) + "\n";
  s += "num_tree_per_iteration=" + std::to_string(num_tree_per_iteration_) + "\n";
  s += "label_index=" + std::to_string(label_idx_) + "\n";
  s += "max_feature_idx=" + std::to_string(max_feature_idx_) + "\n";
  if (objective_ != nullptr) s += "objective=" + objective_->ToString() + "\n";
  if (average_output_) s += "average_output\n";
  s += "feature_names=";
  for (size_t i = 0; i < feature_names_.size(); ++i) { if (i) s += " "; s += feature_names_[i]; }
  s += "\n";
  if (!config_.monotone_vec.empty()) { s += "monotone_constraints="; for (size_t i = 0; i < config_.monotone_vec.size(); ++i) { if (i) s += " "; s += std::to_string(static_cast<int>(config_.monotone_vec[i])); } s += "\n"; }
  s += "feature_infos=";
  for (size_t i = 0; i < feature_infos_.size(); ++i) { if (i) s += " "; s += feature_infos_[i]; }
  s += "\n";
  const int K = num_tree_per_iteration_;
  int used = static_cast<int>(models_.size()); const int total_iter = used / std::max(1, K);
  start_iter = std::max(0, std::min(start_iter, total_iter));
  if (num_iter > 0) used = std::min((start_iter + num_iter) * K, used);
  const int start_model = start_iter * K;
  std::vector<std::string> blocks;
  for (int i = start_model; i < used; ++i) blocks.push_back("Tree=" + std::to_string(i - start_model) + "\n" + models_[i]->ToString() + "\n");
  s += "tree_sizes=";
  for (size_t i = 0; i < blocks.size(); ++i) { if (i) s += " "; s += std::to_string(blocks[i].size()); }
  s += "\n\n";
  for (auto& b : blocks) s += b;
  s += "end of trees\n";
  auto imp = FeatureImportance(num_iter, importance_type);
  std::vector<std::pair<size_t, std::string>> pairs;
  for (size_t i = 0; i < imp.size(); ++i) { size_t v = static_cast<size_t>(imp[i]); if (v > 0 && i < feature_names_.size()) pairs.emplace_back(v, feature_names_[i]); }
  std::stable_sort(pairs.begin(), pairs.end(), [](const std::pair<size_t, std::string>& a, const std::pair<size_t, std::string>& b) { return a.first > b.first; });
  s += "\nfeature_importances:\n";
  for (auto& p : pairs) s += p.second + "=" + std::to_string(p.first) + "\n";
  // one "[key: value]" line per parameter, an empty line, then the end marker
  const std::string dump = Trim(train_ != nullptr || loaded_parameter_.empty() ? config_.ToString() : loaded_parameter_);
  s += "\nparameters:\n" + dump + "\n\nend of parameters\n";
  return s;
}

bool GBDT::LoadModelFromString(const char* str, size_t len) {
  models_.clear();
  std::string text(str, len);
  size_t pos = 0;
  std::unordered_map<std::string, std::string> kv;
  // header: lines up to the first "Tree=" line or "end of trees"
  while (pos < text.size()) {
    size_t eol = text.find('\n', pos);
    if (eol == std::string::npos) eol = text.size();
    std::string line = Trim(text.substr(pos, eol - pos));
    if (StartsWith(line, "Tree=") || line == "end of trees") break;
    pos = eol + 1;
    if (line.empty()) continue;
    size_t eq = line.find('=');
    if (eq != std::string::npos) kv[line.substr(0, eq)] = line.substr(eq + 1); else kv[line] = "";
  }
  if (!kv.count("num_class") || !kv.count("max_feature_idx")) { Log::Fatal("Model file doesn't specify num_class / max_feature_idx"); }
  num_class_ = atoi(kv["num_class"].c_str());
  num_tree_per_iteration_ = kv.count("num_tree_per_iteration") ? atoi(kv["num_tree_per_iteration"].c_str()) : num_class_;
  label_idx_ = kv.count("label_index") ? atoi(kv["label_index"].c_str()) : 0;
  max_feature_idx_ = atoi(kv["max_feature_idx"].c_str());
  average_output_ = kv.count("average_output") > 0;
  feature_names_ = kv.count("feature_names") ? SplitAny(kv["feature_names"], " ") : std::vector<std::string>();
  if (static_cast<int>(feature_names_.size()) != max_feature_idx_ + 1) Log::Fatal("Wrong size of feature_names");
  feature_infos_ = kv.count("feature_infos") ? SplitAny(kv["feature_infos"], " ") : std::vector<std::string>(max_feature_idx_ + 1, "none");
  if (kv.count("monotone_constraints")) { config_.monotone_vec.clear(); for (int v : ParseNumArray<int>(kv["monotone_constraints"])) config_.monotone_vec.push_back(static_cast<int8_t>(v)); }
  config_.num_class = num_class_;
  if (kv.count("objective")) { loaded_objective_.reset(CreateObjectiveFromModelString(kv["objective"], &config_)); objective_ = loaded_objective_.get(); }
  // trees
  while (pos < text.size()) {
    size_t eol = text.find('\n', pos);
    if (eol == std::string::npos) eol = text.size();
    std::string line = Trim(text.substr(pos, eol - pos));
    if (line == "end of trees") { pos = eol + 1; break; }
    if (StartsWith(line, "Tree=")) {
      pos = eol + 1;
      size_t used = 0;
      models_.emplace_back(new Tree(text.c_str() + pos, &used));
      pos += used;
    } else pos = eol + 1;
  }
  size_t pp = text.find("\nparameters:\n", pos > 0 ? pos - 1 : 0);
  if (pp != std::string::npos) {
    size_t b = pp + 13, e = text.find("\nend of parameters", b);
    if (e != std::string::npos) {
      loaded_parameter_ = Trim(text.substr(b, e - b));
      // recover the parameters that prediction depends on
      for (auto& ln : SplitAny(loaded_parameter_, "\n")) {
        std::string t = Trim(ln);
        if (t.size() < 3 || t[0] != '[') continue;
        size_t c = t.find(": ");
        if (c == std::string::npos) continue;
        std::string k = t.substr(1, c - 1), v = t.substr(c + 2, t.size() - c - 3);
        if (k == "learning_rate") config_.learning_rate = ParseDouble(v);
        else if (k == "pred_early_stop") config_.pred_early_stop = v == "1";
      }
    }
  }
  iter_ = static_cast<int>(models_.size()) / std::max(1, num_tree_per_iteration_);
  return true;
}

std::string GBDT::DumpModel(int start_iter, int num_iter, int importance_type) const {
  std::ostringstream os;
  os << "{\"name\":\"tree\",\n\"version\":\"v4\",\n\"num_class\":" << num_class_ << ",\n\"num_tree_per_iteration\":" << num_tree_per_iteration_
     << ",\n\"label_index\":" << label_idx_ << ",\n\"max_feature_idx\":" << max_feature_idx_ << ",\n";
  if (objective_) os << "\"objective\":\"" << objective_->ToString() << "\",\n";
  os << "\"average_output\":" << (average_output_ ? "true" : "false") << ",\n\"feature_names\":[";
  for (size_t i = 0; i < feature_names_.size(); ++i) os << (i ? "," : "") << "\"" << feature_names_[i] << "\"";
  os << "],\n\"monotone_constraints\":[";
  for (size_t i = 0; i < config_.monotone_vec.size(); ++i) os << (i ? "," : "") << static_cast<int>(config_.monotone_vec[i]);
  os << "],\n\"feature_infos\":{";
  bool first = true;
  for (size_t i = 0; i < feature_infos_.size(); ++i) {
    const std::string& fi = feature_infos_[i];
    if (fi == "none") continue;
    os << (first ? "" : ",") << "\"" << feature_names_[i] << "\":{"; first = false;
    if (fi.size() > 2 && fi[0] == '[') { auto mm = Split(fi.substr(1, fi.size() - 2), ':'); os << "\"min_value\":" << mm[0] << ",\"max_value\":" << (mm.size() > 1 ? mm[1] : mm[0]) << ",\"values\":[]}"; }
    else { os << "\"min_value\":0,\"max_value\":0,\"values\":["; auto vs = Split(fi, ':'); for (size_t k = 0; k < vs.size(); ++k) os << (k ? "," : "") << vs[k]; os << "]}"; }
  }
  os << "},\n\"tree_info\":[";
  const int K = num_tree_per_iteration_;
  int used = static_cast<int>(models_.size()); const int total_iter = used / std::max(1, K);
  start_iter = std::max(0, std::min(start_iter, total_iter));
  if (num_iter > 0) used = std::min((start_iter + num_iter) * K, used);
  for (int i = start_iter * K; i < used; ++i) os << (i > start_iter * K ? "," : "") << "{\"tree_index\":" << i << "," << models_[i]->ToJSON() << "}";
  os << "],\n\"feature_importances\":{";
  auto imp = FeatureImportance(num_iter, importance_type);
  first = true;
  for (size_t i = 0; i < imp.size(); ++i) if (static_cast<size_t>(imp[i]) > 0) { os << (first ? "" : ",") << "\"" << feature_names_[i] << "\":" << static_cast<size_t>(imp[i]); first = false; }
  os << "}\n}\n";
  return os.str();
}

std::string GBDT::ModelToIfElse(int num_iter) const {
  std::ostringstream os;
  int n = static_cast<int>(models_.size());
  if (num_iter > 0) n = std::min(n, num_iter * num_tree_per_iteration_);
  os << "#include <cmath>\n#include <cstdint>\nnamespace falcata_model {\n";
  os << "static inline bool CatIn(const uint32_t* bits, int n, int pos) { int i = pos / 32; return i < n && ((bits[i] >> (pos % 32)) & 1); }\n";
  for (int i = 0; i < n; ++i) os << models_[i]->ToIfElse(i, false);
  os << "double (*PredictTreePtr[])(const double*) = {";
  for (int i = 0; i < n; ++i) os << (i ? "," : "") << "PredictTree" << i;
  os << "};\nvoid PredictRaw(const double* features, double* output) {\n  for (int k = 0; k < " << num_tree_per_iteration_ << "; ++k) output[k] = 0.0;\n";
  os << "  for (int i = 0; i < " << n << "; ++i) output[i % " << num_tree_per_iteration_ << "] += PredictTreePtr[i](features);\n";
  if (average_output_) os << "  for (int k = 0; k < " << num_tree_per_iteration_ << "; ++k) output[k] /= " << std::max(1, n / num_tree_per_iteration_) << ";\n";
  os << "}\n}  // namespace falcata_model\n";
  return os.str();
}

// ------------------------------------------------------------------ FALB ----
// The reference's binary model container, read and written byte-compatibly (src/boosting/falb.h:L35-114,
// src/boosting/gbdt_model_binary.cpp). Layout, all little-endian:
//   0  "FALB" | 4 u32 version (1) | 8 u64 required-capability flags | 16 u64 tree count | 24 u32 section count | 28 u32 pad
//   32 section table: {u32 id, u32 dtype, u32 codec, u32 shuffle, u64 offset, u64 stored_len, u64 raw_len} per section
//   then the section payloads, each 8-byte aligned.
// A payload is raw (codec 0) or zlib (codec 2; 1 is reserved and rejected); `shuffle` > 1 means that the
// decoded bytes are byte planes of items of that width. Sections: the model's text header with no tree
// bodies (metadata, parsed by the text loader), a fixed-width per-tree index, structure-of-arrays node
// and leaf data narrowed to the smallest integer type that fits, per-feature threshold dictionaries, and
// optionally categorical sets, node statistics and diagnostics. Linear trees are not representable
// (their flag bit is reserved) and are refused. Every read is checked against the real buffer length.
namespace {

constexpr uint32_t kFalbVersion = 1;
enum : uint64_t { kFalbHasStats = 1ull << 0, kFalbHasDiagnostics = 1ull << 1, kFalbHasCategorical = 1ull << 2, kFalbHasLinear = 1ull << 3,
                  kFalbKnownFlags = kFalbHasStats | kFalbHasDiagnostics | kFalbHasCategorical };
enum FalbSectionId : uint32_t { kSecMeta = 1, kSecTreeIndex = 2, kSecSplitFeature = 3, kSecThresholdIdx = 4, kSecDictOffsets = 5, kSecDictValues = 6,
                                kSecDecisionType = 7, kSecLeftChild = 8, kSecRightChild = 9, kSecLeafValue = 10, kSecCatBoundaries = 11,
                                kSecCatThreshold = 12, kSecStats = 13, kSecDiagnostics = 14 };
enum FalbDType : uint32_t { kDtBytes = 0, kDtU8 = 1, kDtU16 = 2, kDtU32 = 3, kDtI8 = 4, kDtI16 = 5, kDtI32 = 6, kDtF32 = 7, kDtF64 = 8, kDtU64 = 9 };
enum FalbCodec : uint32_t { kCodecRaw = 0, kCodecReserved = 1, kCodecZlib = 2 };

#pragma pack(push, 1)
struct FalbEntry { uint32_t id, dtype, codec, shuffle; uint64_t offset, stored_len, raw_len; };
struct FalbTreeRecord { uint32_t num_leaves, num_cat; int32_t max_depth; uint32_t leaf_dim; uint64_t node_offset, leaf_offset, cat_boundary_offset, cat_threshold_offset; double shrinkage; };
#pragma pack(pop)
static_assert(sizeof(FalbEntry) == 40 && sizeof(FalbTreeRecord) == 56, "FALB on-disk records");

size_t DTypeWidth(uint32_t d) {
  switch (d) { case kDtU8: case kDtI8: case kDtBytes: return 1; case kDtU16: case kDtI16: return 2; case kDtU32: case kDtI32: case kDtF32: return 4; default: return 8; }
}
uint32_t NarrowestUnsigned(uint64_t max_value) { return max_value <= 0xFFu ? kDtU8 : max_value <= 0xFFFFu ? kDtU16 : max_value <= 0xFFFFFFFFull ? kDtU32 : kDtU64; }

struct Bytes {
  std::vector<char> b;
  template <typename T> void Put(const T& v) { const char* p = reinterpret_cast<const char*>(&v); b.insert(b.end(), p, p + sizeof(T)); }
  void PutRaw(const void* p, size_t n) { if (n) { const char* c = static_cast<const char*>(p); b.insert(b.end(), c, c + n); } }
  // one integer, narrowed to the section's element type
  void PutAs(uint32_t dtype, long long v) {
    switch (dtype) {
      case kDtU8: Put(static_cast<uint8_t>(v)); break; case kDtU16: Put(static_cast<uint16_t>(v)); break; case kDtU32: Put(static_cast<uint32_t>(v)); break;
      case kDtI8: Put(static_cast<int8_t>(v)); break; case kDtI16: Put(static_cast<int16_t>(v)); break; case kDtI32: Put(static_cast<int32_t>(v)); break;
      default: Log::Fatal("FALB: cannot write integers as dtype %u", dtype);
    }
  }
};

// A window of untrusted bytes: nothing is read without a range check first.
struct View {
  const char* p = nullptr; uint64_t n = 0;
  void Require(uint64_t off, uint64_t count, uint64_t width, const char* what) const {
    if ((width != 0 && count > UINT64_MAX / width) || off > n || count * width > n - off)
      Log::Fatal("FALB: corrupt model -- %s needs %llu items of %llu bytes at offset %llu of a %llu-byte block", what, static_cast<unsigned long long>(count),
                 static_cast<unsigned long long>(width), static_cast<unsigned long long>(off), static_cast<unsigned long long>(n));
  }
  template <typename T> T At(uint64_t off, const char* what) const { Require(off, 1, sizeof(T), what); T v; memcpy(&v, p + off, sizeof(T)); return v; }
  // `count` integers of element type `dtype` starting at element `first`, widened to T
  template <typename T> void Ints(uint32_t dtype, uint64_t first, uint64_t count, const char* what, std::vector<T>* out) const {
    const size_t w = DTypeWidth(dtype);
    if (dtype != kDtU8 && dtype != kDtU16 && dtype != kDtU32 && dtype != kDtI8 && dtype != kDtI16 && dtype != kDtI32)
      Log::Fatal("FALB: %s has element type %u, which this build cannot read", what, dtype);
    Require(first * w, count, w, what);
    out->resize(count);
    const char* q = p + first * w;
    for (uint64_t i = 0; i < count; ++i, q += w) {
      switch (dtype) {
        case kDtU8: { uint8_t v; memcpy(&v, q, 1); (*out)[i] = static_cast<T>(v); break; } case kDtU16: { uint16_t v; memcpy(&v, q, 2); (*out)[i] = static_cast<T>(v); break; }
        case kDtU32: { uint32_t v; memcpy(&v, q, 4); (*out)[i] = static_cast<T>(v); break; } case kDtI8: { int8_t v; memcpy(&v, q, 1); (*out)[i] = static_cast<T>(v); break; }
        case kDtI16: { int16_t v; memcpy(&v, q, 2); (*out)[i] = static_cast<T>(v); break; } default: { int32_t v; memcpy(&v, q, 4); (*out)[i] = static_cast<T>(v); break; }
      }
    }
  }
  template <typename T> void Copy(uint64_t off, uint64_t count, const char* what, T* dst) const { Require(off, count, sizeof(T), what); if (count) memcpy(dst, p + off, count * sizeof(T)); }
};

struct PendingSection { FalbEntry e; std::vector<char> payload; };

// Encodes one section: byte-plane shuffle (multi-byte items) then zlib, kept only when it is smaller than the raw bytes.
void AddSection(std::vector<PendingSection>* out, uint32_t id, uint32_t dtype, std::vector<char>&& raw, size_t item, int level) {
  PendingSection s; s.e.id = id; s.e.dtype = dtype; s.e.codec = kCodecRaw; s.e.shuffle = 0; s.e.offset = 0; s.e.raw_len = s.e.stored_len = raw.size();
  s.payload = std::move(raw);
  if (level > 0 && !s.payload.empty()) {
    const size_t n = s.payload.size();
    std::vector<char> planes; const char* src = s.payload.data(); uint32_t shuffle = 0;
    if (item > 1 && n % item == 0) {
      planes.resize(n); const size_t cnt = n / item;
      for (size_t b = 0; b < item; ++b) for (size_t i = 0; i < cnt; ++i) planes[b * cnt + i] = s.payload[i * item + b];
      src = planes.data(); shuffle = static_cast<uint32_t>(item);
    }
    uLongf cap = compressBound(static_cast<uLong>(n)); std::vector<char> z(cap);
    if (compress2(reinterpret_cast<Bytef*>(z.data()), &cap, reinterpret_cast<const Bytef*>(src), static_cast<uLong>(n), level) != Z_OK) Log::Fatal("FALB: zlib compression failed");
    if (static_cast<size_t>(cap) < n) { z.resize(cap); s.payload = std::move(z); s.e.codec = kCodecZlib; s.e.shuffle = shuffle; s.e.stored_len = s.payload.size(); }
  }
  out->push_back(std::move(s));
}

}  // namespace

std::vector<char> GBDT::SaveModelToBinary(int start_iter, int num_iter, int importance_type, bool with_stats, bool with_diagnostics, bool f32_leaves, int compress_level) const {
  const int K = std::max(1, num_tree_per_iteration_);
  int used = static_cast<int>(models_.size()); const int total_iter = used / K;
  start_iter = std::max(0, std::min(start_iter, total_iter));
  if (num_iter > 0) used = std::min((start_iter + num_iter) * K, used);
  const int first = start_iter * K;
  const int num_trees = std::max(0, used - first);
  for (int t = first; t < used; ++t) if (models_[t]->is_linear) Log::Fatal("FALB version 1 cannot store linear trees; save this model as text (format='txt') instead");

  // metadata = the text model with an empty tree range (start past the last iteration, no end bound)
  const std::string meta = SaveModelToString(total_iter, 0, importance_type);

  // per-feature dictionaries of the thresholds that occur (sorted, exact doubles); categorical nodes keep their set index
  const int nfeat = max_feature_idx_ + 1;
  std::vector<std::vector<double>> dict(nfeat + 1);
  long long max_feature = 0, max_child = 0; size_t total_cat = 0;
  for (int t = first; t < used; ++t) {
    const Tree& T = *models_[t];
    total_cat += T.num_cat > 0 ? T.cat_threshold.size() : 0;
    for (int s = 0; s < T.num_leaves - 1; ++s) {
      max_feature = std::max<long long>(max_feature, T.split_feature[s]);
      max_child = std::max<long long>(max_child, std::max(std::abs(T.left_child[s]), std::abs(T.right_child[s])));
      if (T.decision_type[s] & kCategoricalMask) continue;
      const int f = T.split_feature[s];
      if (f >= 0 && f <= nfeat) dict[f].push_back(T.threshold[s]);
    }
  }
  size_t max_dict = 0;
  std::vector<uint32_t> dict_off(dict.size() + 1, 0); std::vector<double> dict_val;
  for (size_t f = 0; f < dict.size(); ++f) {
    auto& d = dict[f]; std::sort(d.begin(), d.end()); d.erase(std::unique(d.begin(), d.end()), d.end());
    dict_val.insert(dict_val.end(), d.begin(), d.end()); dict_off[f + 1] = static_cast<uint32_t>(dict_val.size()); max_dict = std::max(max_dict, d.size());
  }
  const uint32_t feat_dt = NarrowestUnsigned(static_cast<uint64_t>(max_feature));
  uint32_t thr_dt = NarrowestUnsigned(max_dict == 0 ? 0 : max_dict - 1); if (thr_dt == kDtU64) thr_dt = kDtU32;
  const uint32_t child_dt = max_child <= 127 ? kDtI8 : (max_child <= 32767 ? kDtI16 : kDtI32);
  const bool has_cat = total_cat > 0;

  std::vector<PendingSection> secs;
  { Bytes w; w.PutRaw(meta.data(), meta.size()); AddSection(&secs, kSecMeta, kDtBytes, std::move(w.b), 1, compress_level); }
  {
    Bytes w; uint64_t node_off = 0, leaf_off = 0, cb_off = 0, ct_off = 0;
    for (int t = first; t < used; ++t) {
      const Tree& T = *models_[t];
      FalbTreeRecord r; r.num_leaves = static_cast<uint32_t>(T.num_leaves); r.num_cat = static_cast<uint32_t>(T.num_cat); r.max_depth = -1 /* derived from the child arrays on load, never trusted */; r.leaf_dim = 1;
      r.node_offset = node_off; r.leaf_offset = leaf_off; r.cat_boundary_offset = cb_off; r.cat_threshold_offset = ct_off; r.shrinkage = T.shrinkage;
      w.Put(r);
      node_off += static_cast<uint64_t>(std::max(0, T.num_leaves - 1)); leaf_off += static_cast<uint64_t>(T.num_leaves);
      if (T.num_cat > 0) { cb_off += static_cast<uint64_t>(T.num_cat) + 1; ct_off += T.cat_threshold.size(); }
    }
    AddSection(&secs, kSecTreeIndex, kDtBytes, std::move(w.b), sizeof(FalbTreeRecord), compress_level);
  }
  {
    Bytes feat, thr, dec, lc, rc, lv;
    for (int t = first; t < used; ++t) {
      const Tree& T = *models_[t];
      for (int s = 0; s < T.num_leaves - 1; ++s) {
        feat.PutAs(feat_dt, T.split_feature[s]);
        long long code;
        if (T.decision_type[s] & kCategoricalMask) code = static_cast<long long>(T.threshold[s]);
        else { const auto& d = dict[T.split_feature[s]]; code = std::lower_bound(d.begin(), d.end(), T.threshold[s]) - d.begin(); }
        thr.PutAs(thr_dt, code);
        dec.Put(static_cast<int8_t>(T.decision_type[s]));
        lc.PutAs(child_dt, T.left_child[s]); rc.PutAs(child_dt, T.right_child[s]);
      }
      for (int l = 0; l < T.num_leaves; ++l) { if (f32_leaves) lv.Put(static_cast<float>(T.leaf_value[l])); else lv.Put(T.leaf_value[l]); }
    }
    AddSection(&secs, kSecSplitFeature, feat_dt, std::move(feat.b), DTypeWidth(feat_dt), compress_level);
    AddSection(&secs, kSecThresholdIdx, thr_dt, std::move(thr.b), DTypeWidth(thr_dt), compress_level);
    AddSection(&secs, kSecDecisionType, kDtI8, std::move(dec.b), 1, compress_level);
    AddSection(&secs, kSecLeftChild, child_dt, std::move(lc.b), DTypeWidth(child_dt), compress_level);
    AddSection(&secs, kSecRightChild, child_dt, std::move(rc.b), DTypeWidth(child_dt), compress_level);
    AddSection(&secs, kSecLeafValue, f32_leaves ? kDtF32 : kDtF64, std::move(lv.b), f32_leaves ? 4 : 8, compress_level);
  }
  {
    Bytes off, val; off.PutRaw(dict_off.data(), dict_off.size() * sizeof(uint32_t)); val.PutRaw(dict_val.data(), dict_val.size() * sizeof(double));
    AddSection(&secs, kSecDictOffsets, kDtU32, std::move(off.b), 4, compress_level);
    AddSection(&secs, kSecDictValues, kDtF64, std::move(val.b), 8, compress_level);
  }
  if (has_cat) {
    Bytes cb, ct;
    for (int t = first; t < used; ++t) {
      const Tree& T = *models_[t];
      if (T.num_cat <= 0) continue;
      for (int c = 0; c <= T.num_cat; ++c) cb.Put(static_cast<uint32_t>(T.cat_boundaries[c]));
      ct.PutRaw(T.cat_threshold.data(), T.cat_threshold.size() * sizeof(uint32_t));
    }
    AddSection(&secs, kSecCatBoundaries, kDtU32, std::move(cb.b), 4, compress_level);
    AddSection(&secs, kSecCatThreshold, kDtU32, std::move(ct.b), 4, compress_level);
  }
  if (with_stats) {   // four arrays back to back, each over all trees: leaf weights, leaf counts, internal weights, internal counts
    Bytes w;
    for (int t = first; t < used; ++t) w.PutRaw(models_[t]->leaf_weight.data(), sizeof(double) * models_[t]->num_leaves);
    for (int t = first; t < used; ++t) for (int l = 0; l < models_[t]->num_leaves; ++l) w.Put(static_cast<int32_t>(models_[t]->leaf_count[l]));
    for (int t = first; t < used; ++t) w.PutRaw(models_[t]->internal_weight.data(), sizeof(double) * std::max(0, models_[t]->num_leaves - 1));
    for (int t = first; t < used; ++t) for (int s = 0; s < models_[t]->num_leaves - 1; ++s) w.Put(static_cast<int32_t>(models_[t]->internal_count[s]));
    AddSection(&secs, kSecStats, kDtBytes, std::move(w.b), 8, compress_level);
  }
  if (with_diagnostics) {   // split gains (f32) of all trees, then internal values (f64) of all trees
    Bytes w;
    for (int t = first; t < used; ++t) w.PutRaw(models_[t]->split_gain.data(), sizeof(float) * std::max(0, models_[t]->num_leaves - 1));
    for (int t = first; t < used; ++t) w.PutRaw(models_[t]->internal_value.data(), sizeof(double) * std::max(0, models_[t]->num_leaves - 1));
    AddSection(&secs, kSecDiagnostics, kDtBytes, std::move(w.b), 8, compress_level);
  }

  uint64_t flags = 0;
  if (with_stats) flags |= kFalbHasStats;
  if (with_diagnostics) flags |= kFalbHasDiagnostics;
  if (has_cat) flags |= kFalbHasCategorical;
  Bytes out;
  out.PutRaw("FALB", 4); out.Put(kFalbVersion); out.Put(flags); out.Put(static_cast<uint64_t>(num_trees)); out.Put(static_cast<uint32_t>(secs.size())); out.Put(static_cast<uint32_t>(0));
  const size_t table = out.b.size();
  out.b.resize(table + secs.size() * sizeof(FalbEntry), 0);
  for (size_t i = 0; i < secs.size(); ++i) {
    while (out.b.size() % 8 != 0) out.b.push_back(0);
    secs[i].e.offset = out.b.size();
    out.PutRaw(secs[i].payload.data(), secs[i].payload.size());
    memcpy(out.b.data() + table + i * sizeof(FalbEntry), &secs[i].e, sizeof(FalbEntry));
  }
  return out.b;
}

bool GBDT::LoadModelFromBinary(const char* data, size_t len) {
  View file; file.p = data; file.n = len;
  if (len < 4 || memcmp(data, "FALB", 4) != 0) Log::Fatal("FALB: not a binary model (bad magic)");
  const uint32_t version = file.At<uint32_t>(4, "version");
  if (version != kFalbVersion) Log::Fatal("FALB: model version %u, this build reads version %u", version, kFalbVersion);
  const uint64_t flags = file.At<uint64_t>(8, "flags");
  if (flags & ~static_cast<uint64_t>(kFalbKnownFlags))
    Log::Fatal("FALB: the model requires capabilities this build does not have (flag bits 0x%llx)", static_cast<unsigned long long>(flags & ~static_cast<uint64_t>(kFalbKnownFlags)));
  const uint64_t num_trees = file.At<uint64_t>(16, "tree count");
  const uint32_t nsec = file.At<uint32_t>(24, "section count");
  file.Require(32, nsec, sizeof(FalbEntry), "section table");
  std::unordered_map<uint32_t, FalbEntry> table;
  for (uint32_t i = 0; i < nsec; ++i) {
    const FalbEntry e = file.At<FalbEntry>(32 + static_cast<uint64_t>(i) * sizeof(FalbEntry), "section entry");
    file.Require(e.offset, e.stored_len, 1, "section payload");
    table[e.id] = e;
  }
  std::unordered_map<uint32_t, std::vector<char>> decoded;
  auto entry = [&](uint32_t id) -> const FalbEntry& {
    auto it = table.find(id);
    if (it == table.end()) Log::Fatal("FALB: corrupt model -- section %u is missing", id);
    return it->second;
  };
  // A section as a checked window: raw payloads are viewed in place, compressed ones are decoded once.
  auto open = [&](uint32_t id) -> View {
    const FalbEntry& e = entry(id);
    View v;
    if (e.codec == kCodecRaw) { v.p = data + e.offset; v.n = e.stored_len; return v; }
    if (e.codec != kCodecZlib) Log::Fatal("FALB: section %u uses codec %u, which this build does not read", e.id, e.codec);
    auto it = decoded.find(id);
    if (it == decoded.end()) {
      if (e.raw_len > (1ull << 40)) Log::Fatal("FALB: corrupt model -- section %u declares an implausible size", e.id);
      std::vector<char> raw(static_cast<size_t>(e.raw_len)); uLongf got = static_cast<uLongf>(e.raw_len);
      const int rc = uncompress(reinterpret_cast<Bytef*>(raw.data()), &got, reinterpret_cast<const Bytef*>(data + e.offset), static_cast<uLong>(e.stored_len));
      if (rc != Z_OK || got != e.raw_len) Log::Fatal("FALB: corrupt model -- section %u does not decompress (%d)", e.id, rc);
      if (e.shuffle > 1) {
        if (raw.size() % e.shuffle != 0) Log::Fatal("FALB: corrupt model -- section %u is not a whole number of %u-byte items", e.id, e.shuffle);
        std::vector<char> flat(raw.size()); const size_t cnt = raw.size() / e.shuffle;
        for (size_t b = 0; b < e.shuffle; ++b) for (size_t i = 0; i < cnt; ++i) flat[i * e.shuffle + b] = raw[b * cnt + i];
        raw.swap(flat);
      }
      it = decoded.emplace(id, std::move(raw)).first;
    }
    v.p = it->second.data(); v.n = it->second.size();
    return v;
  };

  // metadata: the text loader reads the header and the parameter dump
  { const View m = open(kSecMeta); const std::string text(m.p, static_cast<size_t>(m.n)); if (!LoadModelFromString(text.c_str(), text.size())) Log::Fatal("FALB: the metadata block does not parse"); }
  models_.clear();

  const View doff = open(kSecDictOffsets), dval = open(kSecDictValues);
  std::vector<uint32_t> dict_off(static_cast<size_t>(doff.n / sizeof(uint32_t))); doff.Copy<uint32_t>(0, dict_off.size(), "dictionary offsets", dict_off.data());
  std::vector<double> dict_val(static_cast<size_t>(dval.n / sizeof(double))); dval.Copy<double>(0, dict_val.size(), "dictionary values", dict_val.data());
  const View idx = open(kSecTreeIndex);
  idx.Require(0, num_trees, sizeof(FalbTreeRecord), "tree index");
  const View sf = open(kSecSplitFeature), ti = open(kSecThresholdIdx), dt = open(kSecDecisionType), lc = open(kSecLeftChild), rc = open(kSecRightChild), lv = open(kSecLeafValue);
  const uint32_t sf_dt = entry(kSecSplitFeature).dtype, ti_dt = entry(kSecThresholdIdx).dtype, lc_dt = entry(kSecLeftChild).dtype, rc_dt = entry(kSecRightChild).dtype, lv_dt = entry(kSecLeafValue).dtype;
  if (lv_dt != kDtF32 && lv_dt != kDtF64) Log::Fatal("FALB: leaf values have element type %u, which this build cannot read", lv_dt);
  const bool has_cat = flags & kFalbHasCategorical, has_stats = flags & kFalbHasStats, has_diag = flags & kFalbHasDiagnostics;
  uint64_t total_nodes = 0, total_leaves = 0;
  for (uint64_t t = 0; t < num_trees; ++t) {
    const FalbTreeRecord r = idx.At<FalbTreeRecord>(t * sizeof(FalbTreeRecord), "tree record");
    if (r.num_leaves == 0 || r.num_leaves > (1u << 28)) Log::Fatal("FALB: corrupt model -- tree %llu has %u leaves", static_cast<unsigned long long>(t), r.num_leaves);
    total_nodes += r.num_leaves - 1; total_leaves += r.num_leaves;
  }
  View cbv, ctv, stv, dgv; uint32_t cb_dt = kDtU32;
  if (has_cat) { cbv = open(kSecCatBoundaries); ctv = open(kSecCatThreshold); cb_dt = entry(kSecCatBoundaries).dtype; }
  if (has_stats) stv = open(kSecStats);
  if (has_diag) dgv = open(kSecDiagnostics);
  models_.reserve(static_cast<size_t>(num_trees));
  for (uint64_t t = 0; t < num_trees; ++t) {
    const FalbTreeRecord r = idx.At<FalbTreeRecord>(t * sizeof(FalbTreeRecord), "tree record");
    if (r.leaf_dim != 1) Log::Fatal("FALB: tree %llu has leaf_dim %u; this build reads 1", static_cast<unsigned long long>(t), r.leaf_dim);
    const int nl = static_cast<int>(r.num_leaves), ni = nl - 1;
    std::unique_ptr<Tree> T(new Tree(std::max(2, nl), false, false));
    T->num_leaves = nl; T->num_cat = static_cast<int>(r.num_cat); T->shrinkage = r.shrinkage;
    std::vector<int> feat, left, right; std::vector<uint32_t> code; std::vector<int8_t> dec(ni);
    sf.Ints(sf_dt, r.node_offset, ni, "split_feature", &feat); lc.Ints(lc_dt, r.node_offset, ni, "left_child", &left); rc.Ints(rc_dt, r.node_offset, ni, "right_child", &right);
    ti.Ints(ti_dt, r.node_offset, ni, "threshold index", &code);
    dt.Copy<int8_t>(r.node_offset, ni, "decision_type", dec.data());
    for (int s = 0; s < ni; ++s) {
      const int f = feat[s];
      if (f < 0 || f > max_feature_idx_) Log::Fatal("FALB: corrupt model -- split feature %d out of range", f);
      T->split_feature[s] = f; T->split_feature_inner[s] = f; T->decision_type[s] = dec[s];
      if (left[s] >= ni || ~left[s] >= nl || right[s] >= ni || ~right[s] >= nl) Log::Fatal("FALB: corrupt model -- child index out of range in tree %llu", static_cast<unsigned long long>(t));
      T->left_child[s] = left[s]; T->right_child[s] = right[s];
      if (dec[s] & kCategoricalMask) { T->threshold[s] = static_cast<double>(code[s]); T->threshold_in_bin[s] = code[s]; continue; }
      if (static_cast<size_t>(f) + 1 >= dict_off.size()) Log::Fatal("FALB: corrupt model -- feature %d has no threshold dictionary", f);
      const uint64_t pos = static_cast<uint64_t>(dict_off[f]) + code[s];
      if (pos >= dict_off[f + 1] || pos >= dict_val.size()) Log::Fatal("FALB: corrupt model -- threshold index %u out of range for feature %d", code[s], f);
      T->threshold[s] = dict_val[pos];
    }
    if (lv_dt == kDtF32) { std::vector<float> v(nl); lv.Copy<float>(r.leaf_offset * sizeof(float), nl, "leaf_value", v.data()); for (int l = 0; l < nl; ++l) T->leaf_value[l] = v[l]; }
    else lv.Copy<double>(r.leaf_offset * sizeof(double), nl, "leaf_value", T->leaf_value.data());
    if (has_cat && r.num_cat > 0) {
      std::vector<int> cb; cbv.Ints(cb_dt, r.cat_boundary_offset, static_cast<uint64_t>(r.num_cat) + 1, "cat_boundaries", &cb);
      if (cb.back() < 0) Log::Fatal("FALB: corrupt model -- negative categorical boundary");
      std::vector<uint32_t> ct(static_cast<size_t>(cb.back())); ctv.Copy<uint32_t>(r.cat_threshold_offset * sizeof(uint32_t), ct.size(), "cat_threshold", ct.data());
      T->cat_boundaries = cb; T->cat_threshold = ct; T->cat_boundaries_inner = cb; T->cat_threshold_inner = ct;
    }
    if (has_stats) {
      const uint64_t lw0 = 0, lcnt0 = lw0 + total_leaves * sizeof(double), iw0 = lcnt0 + total_leaves * sizeof(int32_t), icnt0 = iw0 + total_nodes * sizeof(double);
      stv.Copy<double>(lw0 + r.leaf_offset * sizeof(double), nl, "leaf_weight", T->leaf_weight.data());
      stv.Copy<double>(iw0 + r.node_offset * sizeof(double), ni, "internal_weight", T->internal_weight.data());
      std::vector<int32_t> c(nl); stv.Copy<int32_t>(lcnt0 + r.leaf_offset * sizeof(int32_t), nl, "leaf_count", c.data()); for (int l = 0; l < nl; ++l) T->leaf_count[l] = c[l];
      c.resize(ni); stv.Copy<int32_t>(icnt0 + r.node_offset * sizeof(int32_t), ni, "internal_count", c.data()); for (int s = 0; s < ni; ++s) T->internal_count[s] = c[s];
    }
    if (has_diag) {
      dgv.Copy<float>(r.node_offset * sizeof(float), ni, "split_gain", T->split_gain.data());
      dgv.Copy<double>(total_nodes * sizeof(float) + r.node_offset * sizeof(double), ni, "internal_value", T->internal_value.data());
    }
    // parents and depths follow from the child arrays
    std::vector<int> depth(std::max(1, ni), 0);
    for (int s = 0; s < ni; ++s) for (int c : {T->left_child[s], T->right_child[s]}) {
      if (c >= 0) depth[c] = depth[s] + 1; else { T->leaf_parent[~c] = s; T->leaf_depth[~c] = depth[s] + 1; }
    }
    models_.push_back(std::move(T));
  }
  falb_without_stats_ = !has_stats;
  iter_ = static_cast<int>(models_.size()) / std::max(1, num_tree_per_iteration_);
  return true;
}

}  // namespace fb
