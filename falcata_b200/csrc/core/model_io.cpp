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
  if (train_ != nullptr || loaded_parameter_.empty()) {
    s += "\nparameters:\n" + config_.ToString() + "\nend of parameters\n";
  } else {
    s += "\nparameters:\n" + loaded_parameter_ + "\nend of parameters\n";
  }
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
// Container: "FALB" | u32 version | u32 flags | u32 num_sections | section table | payloads.
// Section table entry: u32 id | u32 dtype | u32 codec (0 raw, 1 zlib) | u32 shuffle (element size
// whose byte planes were transposed before compression, 0 = none) | u64 raw_bytes | u64 stored_bytes.
namespace {
enum FalbSection : uint32_t { kSecHeader = 1, kSecTreeIndex = 2, kSecInt = 3, kSecThreshold = 4, kSecLeaf = 5, kSecGain = 6, kSecInternal = 7, kSecCat = 8, kSecParams = 9, kSecLinear = 10 };
constexpr uint32_t kFalbFlagF32Leaves = 1;

struct ByteWriter {
  std::vector<char> b;
  template <typename T> void Put(T v) { const char* p = reinterpret_cast<const char*>(&v); b.insert(b.end(), p, p + sizeof(T)); }
  void PutBytes(const void* p, size_t n) { const char* c = static_cast<const char*>(p); b.insert(b.end(), c, c + n); }
  void PutStr(const std::string& s) { Put<uint32_t>(static_cast<uint32_t>(s.size())); PutBytes(s.data(), s.size()); }
};
struct ByteReader {
  const char* p; const char* end;
  ByteReader(const char* d, size_t n) : p(d), end(d + n) {}
  void Need(size_t n) const { if (static_cast<size_t>(end - p) < n) Log::Fatal("FALB: truncated input"); }
  template <typename T> T Get() { Need(sizeof(T)); T v; memcpy(&v, p, sizeof(T)); p += sizeof(T); return v; }
  std::string GetStr() { uint32_t n = Get<uint32_t>(); Need(n); std::string s(p, n); p += n; return s; }
  void GetBytes(void* dst, size_t n) { Need(n); memcpy(dst, p, n); p += n; }
};

std::vector<char> ShuffleBytes(const std::vector<char>& in, size_t es) {
  if (es <= 1 || in.size() % es != 0) return in;
  const size_t n = in.size() / es; std::vector<char> out(in.size());
  for (size_t i = 0; i < n; ++i) for (size_t b = 0; b < es; ++b) out[b * n + i] = in[i * es + b];
  return out;
}
std::vector<char> UnshuffleBytes(const std::vector<char>& in, size_t es) {
  if (es <= 1 || in.size() % es != 0) return in;
  const size_t n = in.size() / es; std::vector<char> out(in.size());
  for (size_t i = 0; i < n; ++i) for (size_t b = 0; b < es; ++b) out[i * es + b] = in[b * n + i];
  return out;
}
struct Section { uint32_t id, dtype, codec, shuffle; std::vector<char> raw; };

void AppendSection(ByteWriter* table, ByteWriter* payload, const Section& s) {
  std::vector<char> staged = s.shuffle ? ShuffleBytes(s.raw, s.shuffle) : s.raw;
  std::vector<char> stored; uint32_t codec = 0;
  if (!staged.empty()) {
    uLongf cap = compressBound(static_cast<uLong>(staged.size())); stored.resize(cap);
    if (compress2(reinterpret_cast<Bytef*>(stored.data()), &cap, reinterpret_cast<const Bytef*>(staged.data()), static_cast<uLong>(staged.size()), 6) == Z_OK && cap < staged.size()) { stored.resize(cap); codec = 1; }
    else stored = staged;
  }
  table->Put<uint32_t>(s.id); table->Put<uint32_t>(s.dtype); table->Put<uint32_t>(codec); table->Put<uint32_t>(s.shuffle);
  table->Put<uint64_t>(s.raw.size()); table->Put<uint64_t>(stored.size());
  payload->PutBytes(stored.data(), stored.size());
}
}  // namespace

std::vector<char> GBDT::SaveModelToBinary(int start_iter, int num_iter, bool f32_leaves) const {
  const int K = num_tree_per_iteration_;
  int used = static_cast<int>(models_.size()); const int total_iter = used / std::max(1, K);
  start_iter = std::max(0, std::min(start_iter, total_iter));
  if (num_iter > 0) used = std::min((start_iter + num_iter) * K, used);
  const int start_model = start_iter * K;
  ByteWriter hdr, index, ints, thr, leaf, gain, internal, cat, params, linear;
  hdr.Put<int32_t>(num_class_); hdr.Put<int32_t>(K); hdr.Put<int32_t>(label_idx_); hdr.Put<int32_t>(max_feature_idx_);
  hdr.Put<int32_t>(average_output_ ? 1 : 0); hdr.Put<int32_t>(used - start_model);
  hdr.PutStr(objective_ ? objective_->ToString() : std::string());
  hdr.Put<uint32_t>(static_cast<uint32_t>(feature_names_.size()));
  for (auto& s : feature_names_) hdr.PutStr(s);
  for (auto& s : feature_infos_) hdr.PutStr(s);
  hdr.Put<uint32_t>(static_cast<uint32_t>(config_.monotone_vec.size()));
  for (auto v : config_.monotone_vec) hdr.Put<int8_t>(v);
  // per-feature threshold dictionaries: thresholds repeat heavily across trees
  std::vector<std::vector<double>> dict(max_feature_idx_ + 1);
  for (int t = start_model; t < used; ++t) for (int s = 0; s < models_[t]->num_leaves - 1; ++s) if (!(models_[t]->decision_type[s] & kCategoricalMask)) dict[models_[t]->split_feature[s]].push_back(models_[t]->threshold[s]);
  for (auto& d : dict) { std::sort(d.begin(), d.end()); d.erase(std::unique(d.begin(), d.end()), d.end()); }
  for (auto& d : dict) { thr.Put<uint32_t>(static_cast<uint32_t>(d.size())); }
  for (auto& d : dict) thr.PutBytes(d.data(), d.size() * sizeof(double));
  for (int t = start_model; t < used; ++t) {
    const Tree& T = *models_[t]; const int nl = T.num_leaves, ni = nl - 1;
    index.Put<int32_t>(nl); index.Put<int32_t>(T.num_cat); index.Put<int32_t>(T.is_linear ? 1 : 0); index.Put<double>(T.shrinkage);
    for (int s = 0; s < ni; ++s) {
      ints.Put<int32_t>(T.split_feature[s]); ints.Put<int32_t>(T.left_child[s]); ints.Put<int32_t>(T.right_child[s]);
      ints.Put<int32_t>(T.decision_type[s]); ints.Put<int32_t>(T.internal_count[s]);
      uint32_t code;
      if (T.decision_type[s] & kCategoricalMask) code = static_cast<uint32_t>(T.threshold[s]);
      else { const auto& d = dict[T.split_feature[s]]; code = static_cast<uint32_t>(std::lower_bound(d.begin(), d.end(), T.threshold[s]) - d.begin()); }
      ints.Put<uint32_t>(code);
      gain.Put<float>(T.split_gain[s]);
      internal.Put<float>(static_cast<float>(T.internal_value[s])); internal.Put<float>(static_cast<float>(T.internal_weight[s]));
    }
    for (int l = 0; l < nl; ++l) {
      ints.Put<int32_t>(T.leaf_count[l]);
      if (f32_leaves) { leaf.Put<float>(static_cast<float>(T.leaf_value[l])); leaf.Put<float>(static_cast<float>(T.leaf_weight[l])); }
      else { leaf.Put<double>(T.leaf_value[l]); leaf.Put<double>(T.leaf_weight[l]); }
    }
    if (T.num_cat > 0) {
      for (int c = 0; c <= T.num_cat; ++c) cat.Put<int32_t>(T.cat_boundaries[c]);
      cat.Put<uint32_t>(static_cast<uint32_t>(T.cat_threshold.size()));
      for (auto v : T.cat_threshold) cat.Put<uint32_t>(v);
    }
    if (T.is_linear) {
      for (int l = 0; l < nl; ++l) {
        linear.Put<double>(T.leaf_const[l]); linear.Put<uint32_t>(static_cast<uint32_t>(T.leaf_coeff[l].size()));
        for (size_t k = 0; k < T.leaf_coeff[l].size(); ++k) { linear.Put<int32_t>(T.leaf_features[l][k]); linear.Put<double>(T.leaf_coeff[l][k]); }
      }
    }
  }
  params.PutStr(train_ != nullptr || loaded_parameter_.empty() ? config_.ToString() : loaded_parameter_);
  std::vector<Section> secs = {
      {kSecHeader, 0, 0, 0, hdr.b}, {kSecTreeIndex, 0, 0, 0, index.b}, {kSecInt, 1, 0, 4, ints.b}, {kSecThreshold, 2, 0, 0, thr.b},
      {kSecLeaf, f32_leaves ? 3u : 2u, 0, f32_leaves ? 4u : 8u, leaf.b}, {kSecGain, 3, 0, 4, gain.b}, {kSecInternal, 3, 0, 4, internal.b},
      {kSecCat, 1, 0, 4, cat.b}, {kSecParams, 0, 0, 0, params.b}, {kSecLinear, 0, 0, 0, linear.b}};
  ByteWriter out, table, payload;
  out.PutBytes("FALB", 4); out.Put<uint32_t>(1); out.Put<uint32_t>(f32_leaves ? kFalbFlagF32Leaves : 0); out.Put<uint32_t>(static_cast<uint32_t>(secs.size()));
  for (auto& s : secs) AppendSection(&table, &payload, s);
  out.PutBytes(table.b.data(), table.b.size()); out.PutBytes(payload.b.data(), payload.b.size());
  return out.b;
}

bool GBDT::LoadModelFromBinary(const char* data, size_t len) {
  ByteReader r(data, len);
  char magic[4]; r.GetBytes(magic, 4);
  if (memcmp(magic, "FALB", 4) != 0) return false;
  const uint32_t version = r.Get<uint32_t>(); if (version != 1) Log::Fatal("FALB: unsupported version %u", version);
  const uint32_t flags = r.Get<uint32_t>(); const uint32_t nsec = r.Get<uint32_t>();
  if (nsec > 64) Log::Fatal("FALB: implausible section count");
  struct Ent { uint32_t id, dtype, codec, shuffle; uint64_t raw, stored; };
  std::vector<Ent> ents(nsec);
  for (auto& e : ents) { e.id = r.Get<uint32_t>(); e.dtype = r.Get<uint32_t>(); e.codec = r.Get<uint32_t>(); e.shuffle = r.Get<uint32_t>(); e.raw = r.Get<uint64_t>(); e.stored = r.Get<uint64_t>(); }
  std::unordered_map<uint32_t, std::vector<char>> sec;
  for (auto& e : ents) {
    r.Need(e.stored);
    if (e.raw > (1ull << 34)) Log::Fatal("FALB: implausible section size");
    std::vector<char> staged;
    if (e.codec == 1) {
      staged.resize(e.raw); uLongf dl = static_cast<uLongf>(e.raw);
      if (uncompress(reinterpret_cast<Bytef*>(staged.data()), &dl, reinterpret_cast<const Bytef*>(r.p), static_cast<uLong>(e.stored)) != Z_OK || dl != e.raw) Log::Fatal("FALB: corrupt section %u", e.id);
    } else { if (e.stored != e.raw) Log::Fatal("FALB: raw section size mismatch"); staged.assign(r.p, r.p + e.stored); }
    r.p += e.stored;
    sec[e.id] = e.shuffle ? UnshuffleBytes(staged, e.shuffle) : staged;
  }
  const bool f32 = flags & kFalbFlagF32Leaves;
  ByteReader hdr(sec[kSecHeader].data(), sec[kSecHeader].size());
  num_class_ = hdr.Get<int32_t>(); num_tree_per_iteration_ = hdr.Get<int32_t>(); label_idx_ = hdr.Get<int32_t>(); max_feature_idx_ = hdr.Get<int32_t>();
  average_output_ = hdr.Get<int32_t>() != 0; const int ntree = hdr.Get<int32_t>();
  if (max_feature_idx_ < 0 || max_feature_idx_ > (1 << 26) || ntree < 0) Log::Fatal("FALB: corrupt header");
  const std::string objstr = hdr.GetStr();
  const uint32_t nf = hdr.Get<uint32_t>(); if (static_cast<int>(nf) != max_feature_idx_ + 1) Log::Fatal("FALB: feature name count mismatch");
  feature_names_.clear(); feature_infos_.clear();
  for (uint32_t i = 0; i < nf; ++i) feature_names_.push_back(hdr.GetStr());
  for (uint32_t i = 0; i < nf; ++i) feature_infos_.push_back(hdr.GetStr());
  const uint32_t nm = hdr.Get<uint32_t>(); config_.monotone_vec.clear(); for (uint32_t i = 0; i < nm; ++i) config_.monotone_vec.push_back(hdr.Get<int8_t>());
  config_.num_class = num_class_;
  if (!objstr.empty()) { loaded_objective_.reset(CreateObjectiveFromModelString(objstr, &config_)); objective_ = loaded_objective_.get(); }
  ByteReader thr(sec[kSecThreshold].data(), sec[kSecThreshold].size());
  std::vector<std::vector<double>> dict(nf);
  { std::vector<uint32_t> sizes(nf); for (auto& s : sizes) s = thr.Get<uint32_t>(); for (uint32_t f = 0; f < nf; ++f) { dict[f].resize(sizes[f]); thr.GetBytes(dict[f].data(), sizes[f] * sizeof(double)); } }
  ByteReader index(sec[kSecTreeIndex].data(), sec[kSecTreeIndex].size()), ints(sec[kSecInt].data(), sec[kSecInt].size()), leaf(sec[kSecLeaf].data(), sec[kSecLeaf].size()),
      gain(sec[kSecGain].data(), sec[kSecGain].size()), internal(sec[kSecInternal].data(), sec[kSecInternal].size()), cat(sec[kSecCat].data(), sec[kSecCat].size()),
      linear(sec[kSecLinear].data(), sec[kSecLinear].size());
  models_.clear();
  for (int t = 0; t < ntree; ++t) {
    const int nl = index.Get<int32_t>(), ncat = index.Get<int32_t>(); const bool lin = index.Get<int32_t>() != 0; const double shr = index.Get<double>();
    if (nl < 1 || nl > (1 << 24)) Log::Fatal("FALB: corrupt tree index");
    std::unique_ptr<Tree> T(new Tree(std::max(2, nl), false, lin));
    T->num_leaves = nl; T->num_cat = ncat; T->shrinkage = shr;
    for (int s = 0; s < nl - 1; ++s) {
      T->split_feature[s] = ints.Get<int32_t>(); T->split_feature_inner[s] = T->split_feature[s];
      T->left_child[s] = ints.Get<int32_t>(); T->right_child[s] = ints.Get<int32_t>();
      T->decision_type[s] = static_cast<int8_t>(ints.Get<int32_t>()); T->internal_count[s] = ints.Get<int32_t>();
      const uint32_t code = ints.Get<uint32_t>();
      if (T->split_feature[s] < 0 || T->split_feature[s] > max_feature_idx_) Log::Fatal("FALB: split feature out of range");
      if (T->decision_type[s] & kCategoricalMask) T->threshold[s] = static_cast<double>(code);
      else { const auto& d = dict[T->split_feature[s]]; if (code >= d.size()) Log::Fatal("FALB: threshold code out of range"); T->threshold[s] = d[code]; }
      T->split_gain[s] = gain.Get<float>(); T->internal_value[s] = internal.Get<float>(); T->internal_weight[s] = internal.Get<float>();
    }
    for (int l = 0; l < nl; ++l) {
      T->leaf_count[l] = ints.Get<int32_t>();
      if (f32) { T->leaf_value[l] = leaf.Get<float>(); T->leaf_weight[l] = leaf.Get<float>(); } else { T->leaf_value[l] = leaf.Get<double>(); T->leaf_weight[l] = leaf.Get<double>(); }
    }
    if (ncat > 0) {
      T->cat_boundaries.clear(); for (int c = 0; c <= ncat; ++c) T->cat_boundaries.push_back(cat.Get<int32_t>());
      const uint32_t n = cat.Get<uint32_t>(); T->cat_threshold.clear(); for (uint32_t i = 0; i < n; ++i) T->cat_threshold.push_back(cat.Get<uint32_t>());
    }
    if (lin) for (int l = 0; l < nl; ++l) {
      T->leaf_const[l] = linear.Get<double>(); const uint32_t n = linear.Get<uint32_t>();
      for (uint32_t k = 0; k < n; ++k) { T->leaf_features[l].push_back(linear.Get<int32_t>()); T->leaf_coeff[l].push_back(linear.Get<double>()); }
    }
    // parents / depths
    std::vector<int> depth(std::max(1, nl - 1), 0);
    for (int n = 0; n < nl - 1; ++n) for (int c : {T->left_child[n], T->right_child[n]}) {
      if (c >= 0) { if (c >= nl - 1) Log::Fatal("FALB: child index out of range"); depth[c] = depth[n] + 1; }
      else { if (~c >= nl) Log::Fatal("FALB: leaf index out of range"); T->leaf_parent[~c] = n; T->leaf_depth[~c] = depth[n] + 1; }
    }
    models_.push_back(std::move(T));
  }
  ByteReader params(sec[kSecParams].data(), sec[kSecParams].size());
  loaded_parameter_ = Trim(params.GetStr());
  iter_ = static_cast<int>(models_.size()) / std::max(1, num_tree_per_iteration_);
  return true;
}

}  // namespace fb
