// Tree model implementation. The text block layout follows the LightGBM v4 model format
// (parity: src/io/tree.cpp:L344-414 writer, L690-871 reader) so files interchange.
#include "fb/tree.h"

#include <functional>
#include <unordered_map>

namespace fb {

Tree::Tree(int max_leaves_in, bool /*track_branch*/, bool linear) : max_leaves(std::max(2, max_leaves_in)), is_linear(linear) {
  Resize(max_leaves);
  num_leaves = 1;
  leaf_value[0] = 0.0; leaf_weight[0] = 0.0; leaf_parent[0] = -1; leaf_depth[0] = 0; leaf_count[0] = 0;
  cat_boundaries.push_back(0); cat_boundaries_inner.push_back(0);
}

void Tree::Resize(int n) {
  left_child.resize(n - 1); right_child.resize(n - 1); split_feature_inner.resize(n - 1); split_feature.resize(n - 1);
  threshold_in_bin.resize(n - 1); threshold.resize(n - 1); decision_type.assign(n - 1, 0); split_gain.resize(n - 1);
  leaf_parent.resize(n); leaf_value.resize(n); leaf_weight.resize(n); leaf_count.resize(n);
  internal_value.resize(n - 1); internal_weight.resize(n - 1); internal_count.resize(n - 1); leaf_depth.resize(n);
  if (is_linear) { leaf_const.resize(n); leaf_coeff.resize(n); leaf_features.resize(n); leaf_features_inner.resize(n); }
}

void Tree::SplitCommon(int leaf, int feature_inner, int real_feature, double left_value, double right_value, int left_cnt,
                       int right_cnt, double left_weight, double right_weight, float gain) {
  if (num_leaves >= max_leaves) { max_leaves *= 2; Resize(max_leaves); }
  const int node = num_leaves - 1;
  const int parent = leaf_parent[leaf];
  if (parent >= 0) {
    if (left_child[parent] == ~leaf) left_child[parent] = node; else right_child[parent] = node;
  }
  split_feature_inner[node] = feature_inner; split_feature[node] = real_feature; split_gain[node] = gain;
  left_child[node] = ~leaf; right_child[node] = ~num_leaves;
  leaf_parent[leaf] = node; leaf_parent[num_leaves] = node;
  internal_weight[node] = left_weight + right_weight;
  internal_value[node] = leaf_value[leaf];
  internal_count[node] = left_cnt + right_cnt;
  leaf_value[leaf] = std::isnan(left_value) ? 0.0 : left_value;
  leaf_weight[leaf] = left_weight; leaf_count[leaf] = left_cnt;
  leaf_value[num_leaves] = std::isnan(right_value) ? 0.0 : right_value;
  leaf_weight[num_leaves] = right_weight; leaf_count[num_leaves] = right_cnt;
  leaf_depth[num_leaves] = leaf_depth[leaf] + 1; leaf_depth[leaf]++;
}

int Tree::Split(int leaf, int feature_inner, int real_feature, uint32_t threshold_bin, double threshold_double,
                double left_value, double right_value, int left_cnt, int right_cnt, double left_weight, double right_weight,
                float gain, int missing_type, bool default_left) {
  SplitCommon(leaf, feature_inner, real_feature, left_value, right_value, left_cnt, right_cnt, left_weight, right_weight, gain);
  const int node = num_leaves - 1;
  int8_t dt = 0;
  if (default_left) dt |= kDefaultLeftMask;
  SetMissingType(&dt, missing_type);
  decision_type[node] = dt;
  threshold_in_bin[node] = threshold_bin; threshold[node] = threshold_double;
  return num_leaves++;
}

int Tree::SplitCategorical(int leaf, int feature_inner, int real_feature, const uint32_t* thr_bin, int n_thr_bin,
                           const uint32_t* thr, int n_thr, double left_value, double right_value, int left_cnt, int right_cnt,
                           double left_weight, double right_weight, float gain, int missing_type) {
  SplitCommon(leaf, feature_inner, real_feature, left_value, right_value, left_cnt, right_cnt, left_weight, right_weight, gain);
  const int node = num_leaves - 1;
  int8_t dt = kCategoricalMask;
  SetMissingType(&dt, missing_type);
  decision_type[node] = dt;
  threshold_in_bin[node] = static_cast<uint32_t>(num_cat); threshold[node] = static_cast<double>(num_cat);
  ++num_cat;
  cat_boundaries.push_back(cat_boundaries.back() + n_thr);
  for (int i = 0; i < n_thr; ++i) cat_threshold.push_back(thr[i]);
  cat_boundaries_inner.push_back(cat_boundaries_inner.back() + n_thr_bin);
  for (int i = 0; i < n_thr_bin; ++i) cat_threshold_inner.push_back(thr_bin[i]);
  return num_leaves++;
}

void Tree::Shrink(double rate) {
  for (int i = 0; i < num_leaves; ++i) {
    leaf_value[i] *= rate;
    if (is_linear) { leaf_const[i] *= rate; for (auto& c : leaf_coeff[i]) c *= rate; }
  }
  for (int i = 0; i < num_leaves - 1; ++i) internal_value[i] *= rate;
  shrinkage *= rate;
}

void Tree::AddBias(double val) {
  for (int i = 0; i < num_leaves; ++i) { leaf_value[i] += val; if (is_linear) leaf_const[i] += val; }
  for (int i = 0; i < num_leaves - 1; ++i) internal_value[i] += val;
  shrinkage = 1.0;
}

void Tree::AsConstantTree(double val) { num_leaves = 1; shrinkage = 1.0; leaf_value[0] = val; if (is_linear) leaf_const[0] = val; }

int Tree::MaxDepth() const { int d = 0; for (int i = 0; i < num_leaves; ++i) d = std::max(d, leaf_depth[i]); return d; }

std::string Tree::ToString() const {
  std::string s;
  s += "num_leaves=" + std::to_string(num_leaves) + "\n";
  s += "num_cat=" + std::to_string(num_cat) + "\n";
  const int ni = num_leaves - 1;
  s += "split_feature=" + JoinInts(split_feature.data(), ni) + "\n";
  s += "split_gain=" + JoinDoublesG(split_gain.data(), ni) + "\n";
  s += "threshold=" + JoinDoubles17(threshold.data(), ni) + "\n";
  { std::vector<int> dt(ni); for (int i = 0; i < ni; ++i) dt[i] = decision_type[i]; s += "decision_type=" + JoinInts(dt.data(), ni) + "\n"; }
  s += "left_child=" + JoinInts(left_child.data(), ni) + "\n";
  s += "right_child=" + JoinInts(right_child.data(), ni) + "\n";
  s += "leaf_value=" + JoinDoubles17(leaf_value.data(), num_leaves) + "\n";
  s += "leaf_weight=" + JoinDoubles17(leaf_weight.data(), num_leaves) + "\n";
  s += "leaf_count=" + JoinInts(leaf_count.data(), num_leaves) + "\n";
  s += "internal_value=" + JoinDoublesG(internal_value.data(), ni) + "\n";
  s += "internal_weight=" + JoinDoublesG(internal_weight.data(), ni) + "\n";
  s += "internal_count=" + JoinInts(internal_count.data(), ni) + "\n";
  if (num_cat > 0) {
    s += "cat_boundaries=" + JoinInts(cat_boundaries.data(), num_cat + 1) + "\n";
    s += "cat_threshold=" + JoinInts(cat_threshold.data(), cat_threshold.size()) + "\n";
  }
  s += "is_linear=" + std::to_string(is_linear ? 1 : 0) + "\n";
  if (is_linear) {
    s += "leaf_const=" + JoinDoubles17(leaf_const.data(), num_leaves) + "\n";
    std::vector<int> nf(num_leaves);
    for (int i = 0; i < num_leaves; ++i) nf[i] = static_cast<int>(leaf_coeff[i].size());
    s += "num_features=" + JoinInts(nf.data(), num_leaves) + "\n";
    s += "leaf_features=";
    for (int i = 0; i < num_leaves; ++i) { if (nf[i] > 0) s += JoinInts(leaf_features[i].data(), leaf_features[i].size()) + " "; s += " "; }
    s += "\nleaf_coeff=";
    for (int i = 0; i < num_leaves; ++i) { if (nf[i] > 0) s += JoinDoubles17(leaf_coeff[i].data(), leaf_coeff[i].size()) + " "; s += " "; }
    s += "\n";
  }
  s += "shrinkage=" + DoubleToStrG(shrinkage) + "\n";
  s += "\n";
  return s;
}

Tree::Tree(const char* str, size_t* used_len) {
  // key=value lines until a blank line (or the next "Tree=" / "end of trees")
  std::unordered_map<std::string, std::string> kv;
  const char* p = str;
  while (*p) {
    const char* eol = strchr(p, '\n');
    size_t len = eol ? static_cast<size_t>(eol - p) : strlen(p);
    std::string line(p, len);
    if (!line.empty() && line.back() == '\r') line.pop_back();
    if (line.empty() || StartsWith(line, "Tree=") || StartsWith(line, "end of trees")) {
      if (line.empty()) p += len + (eol ? 1 : 0);
      if (!kv.empty() || !line.empty()) break;
      continue;
    }
    size_t eq = line.find('=');
    if (eq != std::string::npos) kv[line.substr(0, eq)] = line.substr(eq + 1);
    p += len + (eol ? 1 : 0);
  }
  if (used_len) *used_len = static_cast<size_t>(p - str);
  auto need = [&](const char* k) -> const std::string& {
    auto it = kv.find(k);
    if (it == kv.end()) Log::Fatal("Tree model string format error, should contain %s field", k);
    return it->second;
  };
  num_leaves = atoi(need("num_leaves").c_str());
  num_cat = kv.count("num_cat") ? atoi(kv["num_cat"].c_str()) : 0;
  is_linear = kv.count("is_linear") ? atoi(kv["is_linear"].c_str()) != 0 : false;
  shrinkage = kv.count("shrinkage") ? ParseDouble(kv["shrinkage"]) : 1.0;
  max_leaves = std::max(2, num_leaves);
  Resize(max_leaves);
  leaf_value = ParseNumArray<double>(need("leaf_value"));
  leaf_value.resize(max_leaves);
  if (num_leaves > 1) {
    const int ni = num_leaves - 1;
    left_child = ParseNumArray<int>(need("left_child")); right_child = ParseNumArray<int>(need("right_child"));
    split_feature = ParseNumArray<int>(need("split_feature"));
    threshold = ParseNumArray<double>(need("threshold"));
    { auto dt = ParseNumArray<int>(need("decision_type")); decision_type.assign(ni, 0); for (int i = 0; i < ni && i < static_cast<int>(dt.size()); ++i) decision_type[i] = static_cast<int8_t>(dt[i]); }
    if (kv.count("split_gain")) { auto g = ParseNumArray<double>(kv["split_gain"]); split_gain.assign(g.begin(), g.end()); } else split_gain.assign(ni, 0.f);
    if (kv.count("internal_count")) internal_count = ParseNumArray<int>(kv["internal_count"]); else internal_count.assign(ni, 0);
    if (kv.count("internal_value")) internal_value = ParseNumArray<double>(kv["internal_value"]); else internal_value.assign(ni, 0.0);
    if (kv.count("internal_weight")) internal_weight = ParseNumArray<double>(kv["internal_weight"]); else internal_weight.assign(ni, 0.0);
    if (kv.count("leaf_weight")) leaf_weight = ParseNumArray<double>(kv["leaf_weight"]); else leaf_weight.assign(num_leaves, 0.0);
    if (kv.count("leaf_count")) leaf_count = ParseNumArray<int>(kv["leaf_count"]); else leaf_count.assign(num_leaves, 0);
    split_feature_inner = split_feature;
    threshold_in_bin.assign(ni, 0);
    for (auto* v : {&left_child, &right_child, &split_feature, &split_feature_inner, &internal_count}) v->resize(ni);
    threshold.resize(ni); split_gain.resize(ni); internal_value.resize(ni); internal_weight.resize(ni);
    leaf_weight.resize(max_leaves); leaf_count.resize(max_leaves);
    if (num_cat > 0) {
      cat_boundaries = ParseNumArray<int>(need("cat_boundaries"));
      cat_threshold = ParseNumArray<uint32_t>(need("cat_threshold"));
    }
    // leaf parents and depths from the child arrays
    leaf_parent.assign(max_leaves, -1); leaf_depth.assign(max_leaves, 0);
    std::vector<int> depth(ni, 0);
    for (int n = 0; n < ni; ++n) {
      for (int c : {left_child[n], right_child[n]}) {
        if (c >= 0) depth[c] = depth[n] + 1; else { leaf_parent[~c] = n; leaf_depth[~c] = depth[n] + 1; }
      }
    }
  } else {
    leaf_weight.assign(max_leaves, 0.0); leaf_count.assign(max_leaves, 0);
  }
  if (cat_boundaries.empty()) cat_boundaries.push_back(0);
  cat_boundaries_inner.push_back(0);
  if (is_linear) {
    leaf_const = ParseNumArray<double>(need("leaf_const")); leaf_const.resize(max_leaves);
    auto nf = ParseNumArray<int>(need("num_features"));
    auto feats = ParseNumArray<int>(kv["leaf_features"]);
    auto coefs = ParseNumArray<double>(kv["leaf_coeff"]);
    leaf_coeff.assign(max_leaves, {}); leaf_features.assign(max_leaves, {}); leaf_features_inner.assign(max_leaves, {});
    size_t pos = 0;
    for (int i = 0; i < num_leaves; ++i) for (int k = 0; k < nf[i]; ++k, ++pos) { leaf_features[i].push_back(feats[pos]); leaf_coeff[i].push_back(coefs[pos]); }
  }
}

// --------------------------------------------------------------- JSON ----
std::string Tree::NodeToJSON(int index) const {
  std::ostringstream os;
  if (index >= 0) {
    os << "{\n\"split_index\":" << index << ",\n\"split_feature\":" << split_feature[index] << ",\n\"split_gain\":" << DoubleToStrG(split_gain[index]) << ",\n";
    if (decision_type[index] & kCategoricalMask) {
      int ci = static_cast<int>(threshold[index]);
      std::vector<int> cats;
      for (int i = cat_boundaries[ci]; i < cat_boundaries[ci + 1]; ++i)
        for (int b = 0; b < 32; ++b) if ((cat_threshold[i] >> b) & 1) cats.push_back((i - cat_boundaries[ci]) * 32 + b);
      os << "\"threshold\":\"" << JoinInts(cats.data(), cats.size(), "||") << "\",\n\"decision_type\":\"==\",\n";
    } else {
      os << "\"threshold\":" << DoubleToStr17(threshold[index]) << ",\n\"decision_type\":\"<=\",\n";
    }
    os << "\"default_left\":" << ((decision_type[index] & kDefaultLeftMask) ? "true" : "false") << ",\n";
    const char* mt[] = {"None", "Zero", "NaN", "NaN"};
    os << "\"missing_type\":\"" << mt[MissingTypeOf(decision_type[index])] << "\",\n";
    os << "\"internal_value\":" << DoubleToStr17(internal_value[index]) << ",\n\"internal_weight\":" << DoubleToStr17(internal_weight[index]) << ",\n\"internal_count\":" << internal_count[index] << ",\n";
    os << "\"left_child\":" << NodeToJSON(left_child[index]) << ",\n\"right_child\":" << NodeToJSON(right_child[index]) << "\n}";
  } else {
    int leaf = ~index;
    os << "{\n\"leaf_index\":" << leaf << ",\n\"leaf_value\":" << DoubleToStr17(leaf_value[leaf]) << ",\n\"leaf_weight\":" << DoubleToStr17(leaf_weight[leaf]) << ",\n\"leaf_count\":" << leaf_count[leaf] << "\n}";
  }
  return os.str();
}

std::string Tree::ToJSON() const {
  std::ostringstream os;
  os << "\"num_leaves\":" << num_leaves << ",\n\"num_cat\":" << num_cat << ",\n\"shrinkage\":" << DoubleToStrG(shrinkage) << ",\n";
  if (num_leaves == 1) os << "\"tree_structure\":{\"leaf_value\":" << DoubleToStr17(leaf_value[0]) << "}\n";
  else os << "\"tree_structure\":" << NodeToJSON(0) << "\n";
  return os.str();
}

// ------------------------------------------------------------ if-else ----
std::string Tree::NodeToIfElse(int index, bool leaf_idx) const {
  std::ostringstream os;
  if (index >= 0) {
    const int mt = MissingTypeOf(decision_type[index]);
    os << "fval = arr[" << split_feature[index] << "];";
    if (decision_type[index] & kCategoricalMask) {
      int ci = static_cast<int>(threshold[index]);
      os << "if (!std::isnan(fval) && fval >= 0 && CatIn(cat_threshold + " << cat_boundaries[ci] << ", " << (cat_boundaries[ci + 1] - cat_boundaries[ci]) << ", static_cast<int>(fval))) {";
    } else {
      const bool dl = decision_type[index] & kDefaultLeftMask;
      if (mt != 2) os << "if (std::isnan(fval)) fval = 0.0;";
      std::string miss = mt == 1 ? "(std::fabs(fval) <= 1e-35)" : (mt == 2 ? "std::isnan(fval)" : "false");
      os << "if ((" << miss << " && " << (dl ? "true" : "false") << ") || (!" << miss << " && fval <= " << DoubleToStr17(threshold[index]) << ")) {";
    }
    os << NodeToIfElse(left_child[index], leaf_idx) << " } else { " << NodeToIfElse(right_child[index], leaf_idx) << " }";
  } else {
    if (leaf_idx) os << "return " << (~index) << ";"; else os << "return " << DoubleToStr17(leaf_value[~index]) << ";";
  }
  return os.str();
}

std::string Tree::ToIfElse(int index, bool leaf_idx) const {
  std::ostringstream os;
  os << "double " << (leaf_idx ? "PredictTreeLeaf" : "PredictTree") << index << "(const double* arr) { ";
  if (num_cat > 0) os << "static const uint32_t cat_threshold[] = {" << JoinInts(cat_threshold.data(), cat_threshold.size(), ",") << "};";
  os << "double fval = 0.0; (void)fval; ";
  if (num_leaves <= 1) os << "return " << (leaf_idx ? std::string("0") : DoubleToStr17(leaf_value[0])) << ";";
  else os << NodeToIfElse(0, leaf_idx);
  os << " }\n";
  return os.str();
}

// ------------------------------------------------------------ TreeSHAP ----
// Path-dependent TreeSHAP (Lundberg et al.): polynomial-time exact Shapley values for one tree.
namespace {
struct PathElem { int feature; double zero_fraction, one_fraction, pweight; };

void ExtendPath(PathElem* path, int depth, double zf, double of, int feature) {
  path[depth] = {feature, zf, of, depth == 0 ? 1.0 : 0.0};
  for (int i = depth - 1; i >= 0; --i) {
    path[i + 1].pweight += of * path[i].pweight * (i + 1) / static_cast<double>(depth + 1);
    path[i].pweight = zf * path[i].pweight * (depth - i) / static_cast<double>(depth + 1);
  }
}
void UnwindPath(PathElem* path, int depth, int idx) {
  const double of = path[idx].one_fraction, zf = path[idx].zero_fraction;
  double next = path[depth].pweight;
  for (int i = depth - 1; i >= 0; --i) {
    if (of != 0) { double t = path[i].pweight; path[i].pweight = next * (depth + 1) / static_cast<double>((i + 1) * of); next = t - path[i].pweight * zf * (depth - i) / static_cast<double>(depth + 1); }
    else path[i].pweight = path[i].pweight * (depth + 1) / static_cast<double>(zf * (depth - i));
  }
  for (int i = idx; i < depth; ++i) { path[i].feature = path[i + 1].feature; path[i].zero_fraction = path[i + 1].zero_fraction; path[i].one_fraction = path[i + 1].one_fraction; }
}
double UnwoundSum(const PathElem* path, int depth, int idx) {
  const double of = path[idx].one_fraction, zf = path[idx].zero_fraction;
  double next = path[depth].pweight, total = 0;
  for (int i = depth - 1; i >= 0; --i) {
    if (of != 0) { double t = next * (depth + 1) / static_cast<double>((i + 1) * of); total += t; next = path[i].pweight - t * zf * ((depth - i) / static_cast<double>(depth + 1)); }
    else total += (path[i].pweight / zf) / ((depth - i) / static_cast<double>(depth + 1));
  }
  return total;
}
}  // namespace

double Tree::ExpectedValue() const {
  if (num_leaves == 1) return leaf_value[0];
  const double total = internal_count[0];
  double e = 0;
  for (int i = 0; i < num_leaves; ++i) e += (leaf_count[i] / total) * leaf_value[i];
  return e;
}

void Tree::PredictContrib(const double* row, int num_features, double* out) const {
  out[num_features] += ExpectedValue();
  if (num_leaves <= 1) return;
  const int maxd = MaxDepth() + 2;
  std::vector<PathElem> buf(static_cast<size_t>(maxd) * (maxd + 1) / 2 + maxd + 4);
  std::function<void(int, int, PathElem*, double, double, int)> rec = [&](int node, int depth, PathElem* parent_path, double pzf, double pof, int pfeat) {
    PathElem* path = parent_path + depth;
    if (depth > 0) std::copy(parent_path, parent_path + depth, path);
    ExtendPath(path, depth, pzf, pof, pfeat);
    if (node < 0) {
      for (int i = 1; i <= depth; ++i) {
        const double w = UnwoundSum(path, depth, i);
        out[path[i].feature] += w * (path[i].one_fraction - path[i].zero_fraction) * leaf_value[~node];
      }
      return;
    }
    const int hot = Decide(row[split_feature[node]], node);
    const int cold = hot == left_child[node] ? right_child[node] : left_child[node];
    auto cnt = [&](int n) { return static_cast<double>(n >= 0 ? internal_count[n] : leaf_count[~n]); };
    const double w = cnt(node);
    const double hzf = cnt(hot) / w, czf = cnt(cold) / w;
    double izf = 1, iof = 1;
    int pidx = 0;
    for (; pidx <= depth; ++pidx) if (path[pidx].feature == split_feature[node]) break;
    int d = depth;
    if (pidx != depth + 1) { izf = path[pidx].zero_fraction; iof = path[pidx].one_fraction; UnwindPath(path, d, pidx); d -= 1; }
    rec(hot, d + 1, path, hzf * izf, iof, split_feature[node]);
    rec(cold, d + 1, path, czf * izf, 0.0, split_feature[node]);
  };
  rec(0, 0, buf.data(), 1.0, 1.0, -1);
}

}  // namespace fb
