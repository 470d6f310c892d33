// Split gain / leaf output math and candidate evaluation, written once for the host learner
// and the device kernels so that the two cannot drift apart.
//
// Parity (semantics): include/Falcata/tree_split_math.h:L33-89 (leaf output and gain),
// src/treelearner/feature_histogram.hpp:L167-210, L393-440, L816-1041 (scan directions by
// missing type, constraints, tie rules), src/treelearner/split_info.hpp:L138-166 (ordering).
//
// Every double operation goes through FB_MUL/FB_ADD/... so that neither compiler contracts
// a*b+c into an FMA: with integer (quantized) histograms the host and the device then produce
// bit-identical gains, which is what the cross-device equality tests rely on.
#pragma once
#include "fb/common.h"

#if defined(__CUDA_ARCH__)
#define FB_MUL(a, b) __dmul_rn((a), (b))
#define FB_ADD(a, b) __dadd_rn((a), (b))
#define FB_SUB(a, b) __dadd_rn((a), -(b))
#define FB_DIV(a, b) __ddiv_rn((a), (b))
#else
#define FB_MUL(a, b) ((a) * (b))
#define FB_ADD(a, b) ((a) + (b))
#define FB_SUB(a, b) ((a) - (b))
#define FB_DIV(a, b) ((a) / (b))
#endif

namespace fb {

struct SplitParams {
  double lambda_l1, lambda_l2, max_delta_step, path_smooth;
  double min_sum_hessian_in_leaf, min_gain_to_split;
  int min_data_in_leaf;
  int max_depth;
  // categorical
  int max_cat_threshold, max_cat_to_onehot, min_data_per_group;
  double cat_l2, cat_smooth;
  int extra_trees;
  double monotone_penalty;   // splits on monotone-constrained features near the root are discouraged: their gain is scaled by MonotonePenaltyFactor(depth)
  double cegb_split;   // cost-effective boosting: cegb_tradeoff * cegb_penalty_split, charged per row of the leaf against every split gain
  int use_mc;   // some feature carries a monotone constraint: leaf outputs are clamped to the leaf's [min, max] range
};

// Fixed-size record of the best split of one leaf (or one (leaf, feature) task). POD: it is
// written by device kernels, copied between ranks and read by the host.
struct SplitRecord {
  double gain;            // gain above the leaf's own (already minus min_gain_shift); <= 0 / -inf: none
  int feature;            // inner feature index, -1 when no split
  int threshold;          // bin index: feature bin <= threshold goes left (numerical)
  int default_left;
  int is_categorical;
  double left_g, left_h, right_g, right_h;   // real-valued sums (scaled back when quantized)
  double left_out, right_out;
  int64_t left_gi, left_hi;                  // integer sums under quantized training
  int left_cnt, right_cnt;                   // estimated at find time; exact after partition
  int monotone;
  int num_cat_bins;                          // categorical: number of bins in cat_bins (<= 8 words bitset)
  uint32_t cat_bitset[8];                    // categorical: bins that go left
};

FB_HD inline void InitSplitRecord(SplitRecord* r) {
  r->gain = -1.0 / 0.0; r->feature = -1; r->threshold = 0; r->default_left = 1; r->is_categorical = 0;
  r->left_g = r->left_h = r->right_g = r->right_h = 0; r->left_out = r->right_out = 0;
  r->left_gi = r->left_hi = 0; r->left_cnt = r->right_cnt = 0; r->monotone = 0; r->num_cat_bins = 0;
  for (int i = 0; i < 8; ++i) r->cat_bitset[i] = 0;
}

// a is better than b: larger gain; on equal gain the lower feature index, then lower threshold.
FB_HD inline bool SplitBetter(double gain_a, int feat_a, int thr_a, double gain_b, int feat_b, int thr_b) {
  if (feat_a < 0) return false;
  if (feat_b < 0) return true;
  if (gain_a != gain_b) return gain_a > gain_b;
  if (feat_a != feat_b) return feat_a < feat_b;
  return thr_a < thr_b;
}

FB_HD inline double ThresholdL1(double s, double l1) {
  double r = fabs(s) - l1;
  if (r < 0.0) r = 0.0;
  return s >= 0.0 ? r : -r;
}

FB_HD inline double LeafOutputRaw(double g, double h, const SplitParams& p) {
  double num = p.lambda_l1 > 0.0 ? ThresholdL1(g, p.lambda_l1) : g;
  double out = -FB_DIV(num, FB_ADD(h, p.lambda_l2));
  if (p.max_delta_step > 0.0 && fabs(out) > p.max_delta_step) out = out >= 0.0 ? p.max_delta_step : -p.max_delta_step;
  return out;
}

FB_HD inline double LeafOutput(double g, double h, const SplitParams& p, int num_data, double parent_output) {
  double out = LeafOutputRaw(g, h, p);
  if (p.path_smooth > 0.0) {
    double w = FB_DIV(static_cast<double>(num_data), p.path_smooth);
    out = FB_ADD(FB_DIV(FB_MUL(out, w), FB_ADD(w, 1.0)), FB_DIV(parent_output, FB_ADD(w, 1.0)));
  }
  return out;
}

FB_HD inline double LeafGainGivenOutput(double g, double h, const SplitParams& p, double out) {
  double gg = p.lambda_l1 > 0.0 ? ThresholdL1(g, p.lambda_l1) : g;
  return -FB_ADD(FB_MUL(FB_MUL(2.0, gg), out), FB_MUL(FB_MUL(FB_ADD(h, p.lambda_l2), out), out));
}

FB_HD inline double LeafGain(double g, double h, const SplitParams& p, int num_data, double parent_output) {
  if (p.max_delta_step <= 0.0 && p.path_smooth <= 0.0) {
    double gg = p.lambda_l1 > 0.0 ? ThresholdL1(g, p.lambda_l1) : g;
    return FB_DIV(FB_MUL(gg, gg), FB_ADD(h, p.lambda_l2));
  }
  return LeafGainGivenOutput(g, h, p, LeafOutput(g, h, p, num_data, parent_output));
}

FB_HD inline double ClampOutput(double out, double lo, double hi) { return out < lo ? lo : (out > hi ? hi : out); }

// Gain of a (left, right) pair; returns false when a monotone constraint is violated.
// With use_mc the outputs are clamped to the leaf's range [min_c, max_c] (inherited from monotone splits above,
// "basic" method) and the gain is evaluated at the clamped outputs.
FB_HD inline bool SplitGain(double lg, double lh, double rg, double rh, const SplitParams& p, int lcnt, int rcnt,
                            double parent_output, int monotone, double min_c, double max_c, double* gain, double* lout, double* rout) {
  // the leaf outputs enter the gain only with max_delta_step / path_smooth and the monotone constraints; otherwise they
  // are left unset here (0) and the caller computes them once, for the winning candidate, with the same LeafOutput call
  const bool plain = p.max_delta_step <= 0.0 && p.path_smooth <= 0.0 && p.use_mc == 0;
  if (plain && monotone == 0) { *lout = 0.0; *rout = 0.0; }
  else {
    *lout = LeafOutput(lg, lh, p, lcnt, parent_output);
    *rout = LeafOutput(rg, rh, p, rcnt, parent_output);
    if (p.use_mc != 0) { *lout = ClampOutput(*lout, min_c, max_c); *rout = ClampOutput(*rout, min_c, max_c); }
    if ((monotone > 0 && *lout > *rout) || (monotone < 0 && *lout < *rout)) { *gain = 0.0; return false; }
  }
  if (plain) {
    *gain = FB_ADD(LeafGain(lg, lh, p, lcnt, parent_output), LeafGain(rg, rh, p, rcnt, parent_output));
  } else {
    *gain = FB_ADD(LeafGainGivenOutput(lg, lh, p, *lout), LeafGainGivenOutput(rg, rh, p, *rout));
  }
  return true;
}

// Per-leaf constants of the threshold search.
struct LeafScanInfo {
  double sum_g, sum_h;        // real-valued totals (sum_h without epsilon)
  int64_t sum_gi, sum_hi;     // integer totals (quantized)
  int num_data;
  double parent_output;
  double min_gain_shift;      // LeafGain(parent) + min_gain_to_split
  double cnt_factor;          // num_data / sum_h
  double g_scale, h_scale;    // quantized: real = int * scale; else 1
  double min_c, max_c;        // monotone range of the leaf's output (-inf, +inf when unconstrained)
  double mono_factor;         // factor on the gain of splits on monotone-constrained features at this leaf's depth (1: no penalty)
};

// Gain factor of a monotone split at `depth` (root = 0) for monotone_penalty p: 0 up to depth p - 1 (in effect
// forbidden), then rising towards 1 with depth. Parity: src/treelearner/monotone_constraints.hpp
// (ComputeMonotoneSplitGainPenalty).
FB_HD inline double MonotonePenaltyFactor(int depth, double p) {
  if (p <= 0.0) return 1.0;
  if (p >= depth + 1.0) return kEpsilon;
  double pow2 = 1.0;
  if (p <= 1.0) { for (int i = 0; i < depth; ++i) pow2 *= 2.0; return 1.0 - p / pow2 + kEpsilon; }
  // 1 - 2^(p - 1 - depth): the exponent is negative here
  const double e = p - 1.0 - depth;
#if defined(__CUDA_ARCH__)
  return 1.0 - exp2(e) + kEpsilon;
#else
  return 1.0 - std::exp2(e) + kEpsilon;
#endif
}

// Output of a child of leaf L: the regularised output, clamped to the leaf's monotone range when constraints are on.
FB_HD inline double ChildOutput(double g, double h, const SplitParams& p, int num_data, const LeafScanInfo& L) {
  const double out = LeafOutput(g, h, p, num_data, L.parent_output);
  return p.use_mc != 0 ? ClampOutput(out, L.min_c, L.max_c) : out;
}

// Rounded row-count estimate of one bin from its hessian mass.
FB_HD inline int BinCountEstimate(double h, double cnt_factor) { return static_cast<int>(FB_ADD(FB_MUL(h, cnt_factor), 0.5)); }

// Evaluate the candidate "bins on the LEFT side sum to (lg, lh, lcnt)". Returns the gain above
// min_gain_shift, or -inf when a constraint fails.
FB_HD inline double EvalCandidate(double lg, double lh, int lcnt, const LeafScanInfo& L, const SplitParams& p, int monotone,
                                  double* lout, double* rout) {
  const double ninf = -1.0 / 0.0;
  const int rcnt = L.num_data - lcnt;
  const double rg = FB_SUB(L.sum_g, lg), rh = FB_SUB(L.sum_h, lh);
  if (lcnt < p.min_data_in_leaf || rcnt < p.min_data_in_leaf) return ninf;
  if (lh < p.min_sum_hessian_in_leaf || rh < p.min_sum_hessian_in_leaf) return ninf;
  double gain;
  if (!SplitGain(lg, FB_ADD(lh, kEpsilon), rg, FB_ADD(rh, kEpsilon), p, lcnt, rcnt, L.parent_output, monotone, L.min_c, L.max_c, &gain, lout, rout)) return ninf;
  if (!(gain > L.min_gain_shift)) return ninf;
  const double above = FB_SUB(gain, L.min_gain_shift);
  return (monotone != 0 && L.mono_factor != 1.0) ? FB_MUL(above, L.mono_factor) : above;
}

// Leaf-wise (best-first) order key. Along the path from the root, keep the gains that are smaller than every later
// gain (a staircase of suffix minima, increasing): best-first growth pops node u before node v when u's staircase is
// lexicographically larger (a missing element counts as +inf, so a bottleneck node precedes its subtree). Only the
// first four steps are kept; equal truncated keys are treated as ties. The key of a node follows from its parent's
// key and its own best gain g: drop the trailing steps larger than g, then append g.
FB_HD inline void LeafwiseChildKey(const double* parent_key, double g, double* key) {
  const double inf = 1.0 / 0.0;
  int n = 0;
  for (int i = 0; i < 4; ++i) { key[i] = parent_key[i]; if (parent_key[i] != inf) n = i + 1; }
  while (n > 0 && key[n - 1] > g) { key[n - 1] = inf; --n; }
  if (n < 4) key[n] = g;
}
// a sorts strictly before b
FB_HD inline bool LeafwiseKeyBefore(const double* a, const double* b) {
  for (int i = 0; i < 4; ++i) { if (a[i] != b[i]) return a[i] > b[i]; }
  return false;
}

// extra_trees: the one threshold (0 .. nb-2) that a (tree, leaf, feature) evaluates. A counter-based draw, so
// the host learner, the device kernel and any rank count pick the same threshold.
FB_HD inline int ExtraTreesThreshold(uint32_t seed, int tree_index, int leaf, int real_feature, int nb) {
  if (nb <= 2) return -1;
  const uint32_t r = Philox4x32_10(static_cast<uint32_t>(tree_index), static_cast<uint32_t>(leaf), static_cast<uint32_t>(real_feature), 0xE7E7u, seed, 0x7EE5u).v[0];
  return static_cast<int>(r % static_cast<uint32_t>(nb - 1));
}

// Scan order of the numerical threshold search. For a feature with `nb` bins:
//   pass 0 (reverse): t = last .. 0, missing values (zero bin / NaN bin) counted on the LEFT, default_left = 1
//   pass 1 (forward): t = 0 .. last, missing values counted on the RIGHT, default_left = 0 (only when the
//                     feature has a missing type and more than 2 bins)
// Within a feature the first scanned candidate wins ties; `ScanRank` orders candidates accordingly.
FB_HD inline int ScanRank(int pass, int t, int nb) { return pass == 0 ? (nb - 1 - t) : (nb + t); }

}  // namespace fb
