// Parameter parsing, alias normalisation, resolution rules and conflict checks.
// Parity: src/io/config.cpp:L273-359 (Set), L361-401 (quant_mode resolution),
// L409-649 (conflict checks); include/Falcata/falcata_plan.h:L164-258 (plan grammar).
#include "fb/config.h"

#include <omp.h>

namespace fb {

const DebugFlags& DebugFlags::Get() {
  static const DebugFlags flags = [] {
    DebugFlags f;
    if (const char* e = getenv("FALCATA_DEBUG")) {
      std::string s(e); size_t pos = 0;
      while (pos <= s.size()) {
        size_t c = s.find(',', pos); if (c == std::string::npos) c = s.size();
        const std::string k = s.substr(pos, c - pos);
        if (k == "diag") f.diag = true; else if (k == "dump") f.dump = true; else if (k == "sync" || k == "syncpairs") f.sync = true; else if (k == "canary") f.canary = true;
        else if (k.rfind("maxsplits=", 0) == 0) f.maxsplits = std::max(0, atoi(k.c_str() + 10));
        else if (!k.empty()) Log::Warning("FALCATA_DEBUG: unknown key %s (diag, dump, sync, canary, maxsplits=N)", k.c_str());
        pos = c + 1;
      }
    }
    if (const char* e = getenv("FALCATA_DEBUG_SPLITS")) f.splits = e[0] != '\0' && e[0] != '0';
    if (const char* e = getenv("FALCATA_VERIFY")) f.verify = e[0] != '\0' && e[0] != '0';
    return f;
  }();
  return flags;
}

int TeamThreads() { return omp_get_max_threads(); }
int RowThreads(long long rows) { return rows >= 8192 ? TeamThreads() : 1; }


namespace {
template <typename T> void ParseInto(const std::string& v, T* out);
template <> void ParseInto<std::string>(const std::string& v, std::string* out) { *out = Trim(v); }
template <> void ParseInto<int>(const std::string& v, int* out) {
  std::string t = Trim(v);
  char* end = nullptr;
  double d = strtod(t.c_str(), &end);
  if (end == t.c_str()) Log::Fatal("Parameter value '%s' is not a number", v.c_str());
  *out = static_cast<int>(d);
}
template <> void ParseInto<double>(const std::string& v, double* out) { *out = ParseDouble(v); }
template <> void ParseInto<bool>(const std::string& v, bool* out) {
  std::string t = ToLower(Trim(v));
  if (t == "true" || t == "1" || t == "+" || t == "yes") *out = true;
  else if (t == "false" || t == "0" || t == "-" || t == "no") *out = false;
  else Log::Fatal("Parameter value '%s' is not a boolean", v.c_str());
}
std::string ValToStr(const std::string& v) { return v; }
std::string ValToStr(int v) { return std::to_string(v); }
std::string ValToStr(double v) { return DoubleToStrG(v); }
std::string ValToStr(bool v) { return v ? "1" : "0"; }
}  // namespace

const std::unordered_map<std::string, std::string>& Config::AliasTable() {
  static std::unordered_map<std::string, std::string> table = [] {
    std::unordered_map<std::string, std::string> t;
#define FB_ALIAS(type, name, def, aliases) \
    for (auto& a : SplitAny(aliases, ",")) t[a] = #name;
    FB_CONFIG_PARAMS(FB_ALIAS)
#undef FB_ALIAS
    return t;
  }();
  return table;
}

std::unordered_map<std::string, std::string> Config::Str2Map(const char* parameters) {
  std::unordered_map<std::string, std::string> out;
  if (parameters == nullptr) return out;
  for (auto& tok : SplitAny(parameters, " \t\n\r")) {
    size_t eq = tok.find('=');
    if (eq == std::string::npos) continue;
    std::string k = Trim(tok.substr(0, eq)), v = Trim(tok.substr(eq + 1));
    if (k.empty()) continue;
    if (out.count(k) == 0) out[k] = v;
    else Log::Warning("%s is set=%s, %s=%s will be ignored", k.c_str(), out[k].c_str(), k.c_str(), v.c_str());
  }
  NormalizeAliases(&out);
  return out;
}

void Config::NormalizeAliases(std::unordered_map<std::string, std::string>* params) {
  const auto& table = AliasTable();
  std::vector<std::pair<std::string, std::string>> moved;
  for (auto it = params->begin(); it != params->end();) {
    auto a = table.find(it->first);
    if (a != table.end()) { moved.emplace_back(a->second, it->second); it = params->erase(it); }
    else ++it;
  }
  for (auto& kv : moved) if (params->count(kv.first) == 0) (*params)[kv.first] = kv.second;
}

std::string Config::ParseObjectiveAlias(const std::string& in) {
  std::string n = ToLower(Trim(in));
  if (n == "regression" || n == "regression_l2" || n == "mean_squared_error" || n == "mse" || n == "l2" ||
      n == "l2_root" || n == "root_mean_squared_error" || n == "rmse") return "regression";
  if (n == "regression_l1" || n == "mean_absolute_error" || n == "l1" || n == "mae") return "regression_l1";
  if (n == "multiclass" || n == "softmax") return "multiclass";
  if (n == "multi_regression" || n == "multi_regression_l2" || n == "multiregression") return "multi_regression";
  if (n == "multiclassova" || n == "multiclass_ova" || n == "ova" || n == "ovr") return "multiclassova";
  if (n == "xentropy" || n == "cross_entropy") return "cross_entropy";
  if (n == "xentlambda" || n == "cross_entropy_lambda") return "cross_entropy_lambda";
  if (n == "mean_absolute_percentage_error" || n == "mape") return "mape";
  if (n == "rank_xendcg" || n == "xendcg" || n == "xe_ndcg" || n == "xe_ndcg_mart" || n == "xendcg_mart") return "rank_xendcg";
  if (n == "none" || n == "null" || n == "custom" || n == "na") return "custom";
  return n;
}

std::string Config::ParseMetricAlias(const std::string& in) {
  std::string n = ToLower(Trim(in));
  if (n == "regression" || n == "regression_l2" || n == "l2" || n == "mean_squared_error" || n == "mse") return "l2";
  if (n == "l2_root" || n == "root_mean_squared_error" || n == "rmse") return "rmse";
  if (n == "regression_l1" || n == "l1" || n == "mean_absolute_error" || n == "mae") return "l1";
  if (n == "binary_logloss" || n == "binary") return "binary_logloss";
  if (n == "ndcg" || n == "lambdarank" || n == "rank_xendcg" || n == "xendcg" || n == "xe_ndcg" || n == "xe_ndcg_mart" || n == "xendcg_mart") return "ndcg";
  if (n == "map" || n == "mean_average_precision") return "map";
  if (n == "multi_logloss" || n == "multiclass" || n == "softmax" || n == "multiclassova" || n == "multiclass_ova" || n == "ova" || n == "ovr") return "multi_logloss";
  if (n == "xentropy" || n == "cross_entropy") return "cross_entropy";
  if (n == "xentlambda" || n == "cross_entropy_lambda") return "cross_entropy_lambda";
  if (n == "kldiv" || n == "kullback_leibler") return "kullback_leibler";
  if (n == "mean_absolute_percentage_error" || n == "mape") return "mape";
  if (n == "none" || n == "null" || n == "custom" || n == "na") return "custom";
  return n;
}

void Config::Set(const std::unordered_map<std::string, std::string>& params_in, bool cuda_available) {
  std::unordered_map<std::string, std::string> params = params_in;
  NormalizeAliases(&params);
  // seeds derived from `seed` unless given explicitly
  if (params.count("seed")) {
    int s = 0; ParseInto(params["seed"], &s);
    Random rnd(s);
    const int hi = std::numeric_limits<int16_t>::max();
    data_random_seed = rnd.NextShort(0, hi);
    bagging_seed = rnd.NextShort(0, hi);
    drop_seed = rnd.NextShort(0, hi);
    feature_fraction_seed = rnd.NextShort(0, hi);
    objective_seed = rnd.NextShort(0, hi);
    extra_seed = rnd.NextShort(0, hi);
  }
#define FB_SET(type, name, def, aliases) \
  { auto it = params.find(#name); if (it != params.end()) { ParseInto<type>(it->second, &name); raw[#name] = it->second; } }
  FB_CONFIG_PARAMS(FB_SET)
#undef FB_SET
  for (auto& kv : params) {
    bool known = false;
#define FB_KNOWN(type, name, def, aliases) if (kv.first == #name) known = true;
    FB_CONFIG_PARAMS(FB_KNOWN)
#undef FB_KNOWN
    if (!known && kv.first != "config" && kv.first != "num_gpus") Log::Warning("Unknown parameter: %s", kv.first.c_str());
  }
  Resolve(cuda_available);
  CheckParamConflict();
}

void Config::Resolve(bool cuda_available) {
  objective = ParseObjectiveAlias(objective);
  boosting = ToLower(boosting);
  if (boosting == "gbrt") boosting = "gbdt";
  if (boosting == "random_forest") boosting = "rf";
  if (boosting == "goss") { boosting = "gbdt"; data_sample_strategy = "goss"; }
  tree_learner = ToLower(tree_learner);
  if (tree_learner == "feature_parallel") tree_learner = "feature";
  if (tree_learner == "data_parallel") tree_learner = "data";
  if (tree_learner == "voting_parallel") tree_learner = "voting";
  device_type = ToLower(device_type);
  if (device_type.empty()) device_type = cuda_available ? "cuda" : "cpu";
  if (device_type == "gpu") {
    // The OpenCL learner is not part of this build; the name is accepted and mapped.
    Log::Warning("device_type=gpu (OpenCL) is not built; using %s", cuda_available ? "cuda" : "cpu");
    device_type = cuda_available ? "cuda" : "cpu";
  }
  if (device_type != "cpu" && device_type != "cuda") Log::Fatal("Unknown device_type %s", device_type.c_str());
  is_cuda = device_type == "cuda";
  Log::ResetLevel(verbosity < 0 ? -1 : (verbosity == 0 ? 0 : (verbosity == 1 ? 1 : 2)));

  // quant_mode: auto -> stochastic iff use_quantized_grad, else none. deterministic=true on
  // CUDA maps to fixedpoint (order-independent integer sums).
  std::string qm = ToLower(quant_mode);
  if (qm == "auto") qm = use_quantized_grad ? (stochastic_rounding ? "stochastic" : "fixedpoint") : "none";
  if (qm == "none" && deterministic && is_cuda && raw.count("quant_mode") == 0) qm = "fixedpoint";
  if (qm == "none") quant = QuantMode::None;
  else if (qm == "stochastic") quant = QuantMode::Stochastic;
  else if (qm == "fixedpoint") quant = QuantMode::FixedPoint;
  else Log::Fatal("Unknown quant_mode %s (expected auto|none|stochastic|fixedpoint)", quant_mode.c_str());
  if (quant != QuantMode::None) {
    quant_bins_resolved = quant_bins > 0 ? quant_bins : (quant == QuantMode::Stochastic ? 4 : 64);
    quant_bins_from_auto = quant_bins <= 0;
    if (quant_bins_resolved < 2 || quant_bins_resolved > 65534) Log::Fatal("quant_bins must be in [2, 65534]");
    use_quantized_grad = true;
  }
  cuda_precision = ToLower(cuda_precision);
  if (cuda_precision != "fp64" && cuda_precision != "fp32") Log::Fatal("cuda_precision must be fp64 or fp32");

  // label_gain default 2^i - 1
  label_gain_vec.clear();
  if (!label_gain.empty()) label_gain_vec = ParseNumArray<double>(label_gain, ',');
  else { for (int i = 0; i < 31; ++i) label_gain_vec.push_back(static_cast<double>((1ll << i) - 1)); }
  eval_at_vec = ParseNumArray<int>(eval_at, ',');
  std::sort(eval_at_vec.begin(), eval_at_vec.end());
  metric_list.clear();
  {
    std::string m = metric;
    std::vector<std::string> seen;
    for (auto& tok : SplitAny(m, ",")) {
      std::string mm = ParseMetricAlias(tok);
      if (std::find(seen.begin(), seen.end(), mm) == seen.end()) seen.push_back(mm);
    }
    if (seen.empty() && objective != "custom") seen.push_back(ParseMetricAlias(objective));
    for (auto& mm : seen) if (mm != "custom") metric_list.push_back(mm);
  }
  monotone_vec.clear();
  for (auto v : ParseNumArray<int>(monotone_constraints, ',')) monotone_vec.push_back(static_cast<int8_t>(v));
  feature_contri_vec = ParseNumArray<double>(feature_contri, ',');
  max_bin_by_feature_vec = ParseNumArray<int>(max_bin_by_feature, ',');
  if (objective == "multiclass" || objective == "multiclassova" || objective == "multi_regression") num_tree_per_iteration = num_class;
  else num_tree_per_iteration = (objective == "custom" ? std::max(1, num_class) : 1);
}

void Config::CheckParamConflict() {
  if ((objective == "multiclass" || objective == "multiclassova") && num_class <= 1)
    Log::Fatal("Number of classes should be specified and greater than 1 for multiclass training");
  if (objective == "multi_regression" && num_class <= 1) Log::Fatal("multi_regression requires num_class > 1 (num_class carries the number of targets)");
  if (objective != "multiclass" && objective != "multiclassova" && objective != "multi_regression" && objective != "custom" && num_class != 1)
    Log::Fatal("Number of classes must be 1 for non-multiclass training");
  if (num_leaves < 2) Log::Fatal("num_leaves must be >= 2");
  if (num_leaves > 131072) Log::Fatal("num_leaves must be <= 131072");
  if (max_bin < 2) Log::Fatal("max_bin must be > 1");
  if (learning_rate <= 0.0) Log::Fatal("learning_rate must be > 0");
  if (feature_fraction <= 0.0 || feature_fraction > 1.0) Log::Fatal("feature_fraction must be in (0, 1]");
  if (bagging_fraction <= 0.0 || bagging_fraction > 1.0) Log::Fatal("bagging_fraction must be in (0, 1]");
  if (max_depth > 0) {
    double full = std::pow(2.0, max_depth);
    if (full < num_leaves) { num_leaves = static_cast<int>(full); }
  }
  // the host learner combines quantized gradients with both kinds of constraints; the device engine's quantized search does not
  if (quant != QuantMode::None && !monotone_vec.empty() && is_cuda)
    Log::Fatal("Quantized training does not support monotone constraints on device_type=cuda: disable one of them or use device_type=cpu");
  if (quant != QuantMode::None && !interaction_constraints.empty() && is_cuda)
    Log::Fatal("Quantized training does not support interaction constraints on device_type=cuda: disable one of them or use device_type=cpu");
  if (!monotone_vec.empty() && monotone_constraints_method != "basic" && monotone_constraints_method != "intermediate" && monotone_constraints_method != "advanced")
    Log::Fatal("Unknown monotone_constraints_method %s (basic, intermediate, advanced)", monotone_constraints_method.c_str());
  if (boosting == "rf") {
    if (!((bagging_freq > 0 && bagging_fraction < 1.0) || feature_fraction < 1.0))
      Log::Fatal("Random forest needs bagging (bagging_freq>0 and bagging_fraction<1) or feature_fraction<1");
  }
  if (data_sample_strategy == "goss" && (top_rate + other_rate > 1.0)) Log::Fatal("top_rate + other_rate must be <= 1 for GOSS");
  if (tree_learner != "serial" && tree_learner != "data" && tree_learner != "voting" && tree_learner != "feature")
    Log::Fatal("Unknown tree_learner %s", tree_learner.c_str());
  if (grow_policy != "level" && grow_policy != "leaf") Log::Fatal("grow_policy must be level or leaf");
  if (linear_tree && is_cuda) { Log::Warning("linear_tree runs its leaf solves on the host"); }
}

std::string Config::ToString() const {
  std::ostringstream os;
#define FB_STR(type, name, def, aliases) \
  if (std::string(#name) != "task" && std::string(#name) != "data" && std::string(#name) != "valid" && \
      std::string(#name) != "input_model" && std::string(#name) != "output_model" && std::string(#name) != "output_result") \
    os << "[" #name ": " << ValToStr(name) << "]\n";
  FB_CONFIG_PARAMS(FB_STR)
#undef FB_STR
  return os.str();
}

// ------------------------------------------------------------------ Plan ----
Plan Plan::FromString(const std::string& s) {
  Plan p;
  auto toks = SplitAny(s, ",");
  for (size_t i = 0; i < toks.size(); ++i) {
    std::string t = ToLower(Trim(toks[i]));
    if (t == "auto" || t.empty()) continue;
    size_t c = t.find(':');
    if (c == std::string::npos) Log::Fatal("cuda_plan entry '%s' is not key:on|off", t.c_str());
    std::string k = t.substr(0, c), v = t.substr(c + 1);
    bool on;
    if (v == "on" || v == "1" || v == "true") on = true;
    else if (v == "off" || v == "0" || v == "false") on = false;
    else Log::Fatal("cuda_plan value '%s' must be on or off", v.c_str());
#define FB_PK(name) if (k == #name) { p.name = on; continue; }
    FB_PK(hist_tc) FB_PK(device_controller) FB_PK(fused_tail) FB_PK(fused_scan)
    FB_PK(pack4) FB_PK(compact_view) FB_PK(gh_in_row) FB_PK(hist_lane) FB_PK(hist_lane_atomic) FB_PK(hist_lane_red) FB_PK(hist_float_red) FB_PK(robust_scale) FB_PK(quant_ef) FB_PK(col_major_part) FB_PK(bulk_root)
#undef FB_PK
    Log::Fatal("Unknown cuda_plan key '%s'", k.c_str());
  }
  return p;
}

std::string Plan::ToString() const {
  std::ostringstream os;
#define FB_PS(name) os << #name << ":" << (name ? "on" : "off") << " ";
  FB_PS(hist_tc) FB_PS(device_controller) FB_PS(fused_tail) FB_PS(fused_scan)
  FB_PS(pack4) FB_PS(compact_view) FB_PS(gh_in_row) FB_PS(hist_lane) FB_PS(hist_lane_atomic) FB_PS(hist_lane_red) FB_PS(hist_float_red) FB_PS(robust_scale) FB_PS(quant_ef) FB_PS(col_major_part) FB_PS(bulk_root)
#undef FB_PS
  return os.str();
}

}  // namespace fb
