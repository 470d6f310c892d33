// K3 + K4 (K4q): threshold search on the owned feature slice, with the larger child's histogram
// formed on the fly as parent - smaller and written back in place (no separate subtraction pass).
// Parity: src/treelearner/cuda/cuda_best_split_finder.cu:L417-970 (per task prefix scan, gain,
// min_data / min_hessian, missing-value directions), L3185-3285 (per-leaf argmax with the CPU's
// tie order), cuda_histogram_constructor.cu:L2641-3107 (subtract / fix kernels that are folded in).
// The candidate math is fb/split_math.h, shared with the host learner: with integer histograms the
// two produce bit-identical gains.
#include "controller.cuh"

namespace fb {

namespace {

constexpr int kFindThreads = 256;
constexpr int kWarpsPerBlock = kFindThreads / 32;

struct Acc {   // prefix accumulator of one lane
  long long gi, hi; double gd, hd; int c;
};

// Where the bins of one (child, feature) come from.
//  one rank  : child slot (smaller child: constructed there; larger child: still the parent) and,
//              for the larger child, the sibling's slot to subtract.
//  many ranks: the smaller child's bins are the sum over source ranks of this rank's staging slots
//              (fixed rank order, so the full-precision path is deterministic); the larger child is
//              parent minus that sum. Either way the result is written back to the child's slot.
struct BinSrc {
  const void* child; const void* other; bool larger;
  const void* stage; int world; long long rank_stride;   // stage: source rank 0's slot for this (task, feature)
};

template <bool QUANT>
__device__ inline void LoadBin(const BinSrc& s, int j, long long* gi, long long* hi, double* gd, double* hd, hist_q_t* raw_q, double2* raw_d) {
  if (QUANT) {
    hist_q_t v;
    if (s.world > 1) {
      hist_q_t sum = 0;
      for (int r = 0; r < s.world; ++r) sum += __ldcg(static_cast<const hist_q_t*>(s.stage) + r * s.rank_stride + j);
      v = s.larger ? static_cast<const hist_q_t*>(s.child)[j] - sum : sum;
    } else {
      v = static_cast<const hist_q_t*>(s.child)[j];
      if (s.larger) v -= static_cast<const hist_q_t*>(s.other)[j];
    }
    *raw_q = v; *gi = HistQGrad(v); *hi = HistQHess(v);
  } else {
    double2 v;
    if (s.world > 1) {
      double2 sum = make_double2(0.0, 0.0);
      for (int r = 0; r < s.world; ++r) { const double2 t = __ldcg(static_cast<const double2*>(s.stage) + r * s.rank_stride + j); sum.x += t.x; sum.y += t.y; }
      if (s.larger) { v = static_cast<const double2*>(s.child)[j]; v.x -= sum.x; v.y -= sum.y; } else v = sum;
    } else {
      v = static_cast<const double2*>(s.child)[j];
      if (s.larger) { const double2 o = static_cast<const double2*>(s.other)[j]; v.x -= o.x; v.y -= o.y; }
    }
    *raw_d = v; *gd = v.x; *hd = v.y;
  }
}

// Exact row count of a child over all ranks: every rank's partition published its local left count.
__device__ inline int ChildGlobalCount(const FindArgs& a, const FindChild& ch, int local_value) {
  if (a.wait.world <= 1 || ch.split < 0) return local_value;
  int lsum = 0;
  for (int r = 0; r < a.wait.world; ++r) lsum += __ldcg(a.counts + static_cast<size_t>(r) * a.counts_stride + ch.split);
  return ch.is_left ? lsum : ch.parent_global - lsum;
}

// Categorical search of one (child, feature) by one warp. The bins are staged in shared memory (and
// written back where the child's histogram is formed on the fly); the sort by g / (h + cat_smooth) is a
// rank count over all lanes (stable: ties keep bin order); the two directional scans run on lane 0 in
// the host learner's order, operation for operation, so both produce the same record.
// Parity: src/treelearner/cuda/cuda_best_split_finder.cu (categorical kernels), feature_histogram.hpp:L278-520.
constexpr int kCatMaxBins = 256;
struct CatScratch { double g[kCatMaxBins], h[kCatMaxBins]; long long gi[kCatMaxBins], hi[kCatMaxBins]; unsigned char order[kCatMaxBins]; };

template <bool QUANT>
__device__ void ScanCategoricalWarp(const FindArgs& a, const BinSrc& src, char* child, bool write_back, const FeatureMeta& m, const LeafInfo& leaf, int f, int fi,
                                    int lane, int warp) {
  extern __shared__ __align__(16) unsigned char find_smem[];
  CatScratch& S = reinterpret_cast<CatScratch*>(find_smem)[warp];
  const int nb = m.num_bin;
  const int nstored = m.bundled ? nb - 1 : nb;
  const int mfb = m.bundled ? m.most_freq_bin : -1;
  const double g_scale = QUANT ? static_cast<double>(a.scales[0]) : 1.0, h_scale = QUANT ? static_cast<double>(a.scales[1]) : 1.0;
  for (int b = lane; b < nb; b += 32) {
    if (b == mfb) continue;
    const int j = (mfb >= 0 && b > mfb) ? b - 1 : b;
    long long gi = 0, hi = 0; double gd = 0, hd = 0; hist_q_t rq; double2 rd;
    LoadBin<QUANT>(src, j, &gi, &hi, &gd, &hd, &rq, &rd);
    if (write_back) { if (QUANT) reinterpret_cast<hist_q_t*>(child)[j] = rq; else reinterpret_cast<double2*>(child)[j] = rd; }
    S.gi[b] = gi; S.hi[b] = hi;
    S.g[b] = QUANT ? FB_MUL(static_cast<double>(gi), g_scale) : gd; S.h[b] = QUANT ? FB_MUL(static_cast<double>(hi), h_scale) : hd;
  }
  (void)nstored;
  __syncwarp();
  LeafScanInfo L;
  L.sum_g = leaf.sum_g; L.sum_h = leaf.sum_h; L.sum_gi = leaf.sum_gi; L.sum_hi = leaf.sum_hi; L.num_data = leaf.num_data_global;
  L.parent_output = leaf.output; L.g_scale = g_scale; L.h_scale = h_scale; L.min_c = leaf.min_c; L.max_c = leaf.max_c;
  L.mono_factor = MonotonePenaltyFactor(leaf.depth, a.params.monotone_penalty);
  L.cnt_factor = FB_DIV(static_cast<double>(L.num_data), L.sum_h);
  if (a.params.max_delta_step <= 0.0 && a.params.path_smooth <= 0.0)
    L.min_gain_shift = FB_ADD(LeafGain(L.sum_g, FB_ADD(L.sum_h, 2 * kEpsilon), a.params, L.num_data, leaf.output), a.params.min_gain_to_split);
  else
    L.min_gain_shift = FB_ADD(LeafGainGivenOutput(L.sum_g, FB_ADD(L.sum_h, 2 * kEpsilon), a.params, leaf.output), a.params.min_gain_to_split);
  if (mfb >= 0 && lane == 0) {
    // the un-stored most-frequent bin: leaf total minus the stored bins, summed in bin order like the host
    double og = 0, oh = 0; long long ogi = 0, ohi = 0;
    for (int b = 0; b < nb; ++b) if (b != mfb) { og = FB_ADD(og, S.g[b]); oh = FB_ADD(oh, S.h[b]); ogi += S.gi[b]; ohi += S.hi[b]; }
    if (QUANT) { S.gi[mfb] = L.sum_gi - ogi; S.hi[mfb] = L.sum_hi - ohi; S.g[mfb] = FB_MUL(static_cast<double>(S.gi[mfb]), g_scale); S.h[mfb] = FB_MUL(static_cast<double>(S.hi[mfb]), h_scale); }
    else { S.gi[mfb] = S.hi[mfb] = 0; S.g[mfb] = FB_SUB(L.sum_g, og); S.h[mfb] = FB_SUB(L.sum_h, oh); }
  }
  __syncwarp();
  SplitParams p = a.params; p.lambda_l2 = FB_ADD(p.lambda_l2, a.params.cat_l2);
  const bool onehot = nb <= a.params.max_cat_to_onehot;
  int used = 0;
  if (!onehot) {
    // eligible categories in bin order, then their stable rank by ratio
    // (eligibility and the count of earlier eligible bins are cheap enough to recompute per lane)
    for (int b = 1 + lane; b < nb; b += 32) {
      const bool ok = static_cast<double>(BinCountEstimate(S.h[b], L.cnt_factor)) >= a.params.cat_smooth;
      if (!ok) continue;
      const double rb = FB_DIV(S.g[b], FB_ADD(S.h[b], a.params.cat_smooth));
      int rank = 0;
      for (int o = 1; o < nb; ++o) {
        if (o == b) continue;
        if (!(static_cast<double>(BinCountEstimate(S.h[o], L.cnt_factor)) >= a.params.cat_smooth)) continue;
        const double ro = FB_DIV(S.g[o], FB_ADD(S.h[o], a.params.cat_smooth));
        if (ro < rb || (!(rb < ro) && o < b)) ++rank;   // stable: equal (or unordered) ratios keep bin order
      }
      S.order[rank] = static_cast<unsigned char>(b);
    }
    int cnt = 0;
    for (int b = 1 + lane; b < nb; b += 32) cnt += static_cast<double>(BinCountEstimate(S.h[b], L.cnt_factor)) >= a.params.cat_smooth ? 1 : 0;
    for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
    used = cnt;
  }
  __syncwarp();
  if (lane != 0) return;
  CandLite c; c.gain = -1.0 / 0.0; c.feature = -1; c.threshold = 0; c.default_left = 0; c.left_cnt = 0; c.left_gi = c.left_hi = 0; c.left_g = c.left_h = 0;
  c.is_categorical = 1; c.num_cat_bins = 0; for (int w = 0; w < 8; ++w) c.cat_bitset[w] = 0;
  double best_gain = -1.0 / 0.0; int best_dir = -1, best_k = -1;
  if (onehot) {
    for (int b = 1; b < nb; ++b) {
      double lo, ro;
      const int lc = BinCountEstimate(S.h[b], L.cnt_factor);
      const double gain = EvalCandidate(S.g[b], S.h[b], lc, L, p, 0, &lo, &ro);
      if (gain > best_gain) { best_gain = gain; best_k = b; c.left_g = S.g[b]; c.left_h = S.h[b]; c.left_gi = S.gi[b]; c.left_hi = S.hi[b]; c.left_cnt = lc; }
    }
    if (best_k >= 0) { c.cat_bitset[best_k >> 5] |= 1u << (best_k & 31); c.num_cat_bins = 1; }
  } else {
    const int max_num = min(a.params.max_cat_threshold, (used + 1) / 2);
    for (int dir = 0; dir < 2; ++dir) {
      double lg = 0, lh = 0; long long lgi = 0, lhi = 0; int lc = 0, grp = 0;
      for (int k = 0; k < used && k < max_num; ++k) {
        const int b = dir == 0 ? S.order[k] : S.order[used - 1 - k];
        lg = FB_ADD(lg, S.g[b]); lh = FB_ADD(lh, S.h[b]); lgi += S.gi[b]; lhi += S.hi[b];
        const int cb = BinCountEstimate(S.h[b], L.cnt_factor); lc += cb; grp += cb;
        if (grp < a.params.min_data_per_group) continue;
        grp = 0;
        double lo, ro;
        const double gain = EvalCandidate(lg, lh, lc, L, p, 0, &lo, &ro);
        if (gain > best_gain) { best_gain = gain; best_dir = dir; best_k = k; c.left_g = lg; c.left_h = lh; c.left_gi = lgi; c.left_hi = lhi; c.left_cnt = lc; }
      }
    }
    if (best_k >= 0) {
      for (int k = 0; k <= best_k; ++k) { const int b = best_dir == 0 ? S.order[k] : S.order[used - 1 - k]; c.cat_bitset[b >> 5] |= 1u << (b & 31); }
      c.num_cat_bins = best_k + 1;
    }
  }
  if (best_k >= 0 && best_gain != -1.0 / 0.0) { c.gain = FB_MUL(best_gain, static_cast<double>(m.penalty)); c.feature = f; }
  a.cand[static_cast<size_t>(blockIdx.x) * a.num_features + fi] = c;
}

// The search of one (child, feature) by one warp; warps of a block work on different features of the same child and
// leave independently (only warp-level synchronisation inside).
template <bool QUANT>
__device__ void FindSplitsWarp(const FindArgs& a) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int fi = blockIdx.y * kWarpsPerBlock + warp;
  if (fi >= a.num_features + a.num_sub_features) return;
  const bool search = fi < a.num_features;
  const int f = search ? a.features[fi] : a.sub_features[fi - a.num_features];
  const FindChild ch = a.children[blockIdx.x];
  if (!search && !ch.is_larger && a.wait.world <= 1) return;
  const FeatureMeta m = a.meta[f];
  LeafInfo leaf = a.leaves[ch.leaf];
  leaf.num_data_global = ChildGlobalCount(a, ch, leaf.num_data_global);
  if (a.local_vote) {
    // voting, local pass: this rank's rows only
    const VoteLocalSum ls = a.vote_sums[blockIdx.x];
    leaf.sum_gi = ls.gi; leaf.sum_hi = ls.hi; leaf.sum_g = ls.g; leaf.sum_h = ls.h; leaf.num_data_global = leaf.count;
  }
  const bool vote_global = a.voted != nullptr;
  const int nb = m.num_bin;
  const int nstored = m.bundled ? nb - 1 : nb;
  const long long base = a.bin_local[m.hist_offset];
  const size_t esz = QUANT ? sizeof(hist_q_t) : sizeof(double2);
  char* child = static_cast<char*>(a.pool) + (static_cast<long long>(ch.slot) * a.slot_stride + base) * esz;
  const char* other = static_cast<const char*>(a.pool) + (static_cast<long long>(ch.other_slot) * a.slot_stride + base) * esz;
  const bool larger = ch.is_larger != 0 && !vote_global;   // voting: every child's slices are staged afresh
  const int world = a.wait.world;
  const bool write_back = (larger || world > 1) && !vote_global;
  BinSrc src; src.child = child; src.other = other; src.larger = larger; src.world = world;
  src.rank_stride = static_cast<long long>(a.stage_cap) * a.slot_stride;
  const int stage_task = vote_global ? static_cast<int>(blockIdx.x) : ch.task;
  src.stage = world > 1 ? static_cast<const char*>(a.stage) + (static_cast<long long>(stage_task) * a.slot_stride + base) * esz : nullptr;
  if (vote_global && (!search || a.voted[static_cast<size_t>(blockIdx.x) * a.voted_stride + f] == 0)) {
    if (search && lane == 0) {
      CandLite c; c.gain = -1.0 / 0.0; c.feature = -1; c.threshold = 0; c.default_left = 1; c.left_cnt = 0; c.left_gi = c.left_hi = 0; c.left_g = c.left_h = 0;
      c.is_categorical = 0; c.num_cat_bins = 0; for (int w = 0; w < 8; ++w) c.cat_bitset[w] = 0;
      a.cand[static_cast<size_t>(blockIdx.x) * a.num_features + fi] = c;
    }
    return;
  }

  const bool node_masked = search && a.node_mask != nullptr && a.node_mask[static_cast<size_t>(blockIdx.x) * a.node_mask_stride + f] == 0;
  if (node_masked && lane == 0) {
    CandLite c; c.gain = -1.0 / 0.0; c.feature = -1; c.threshold = 0; c.default_left = 1; c.left_cnt = 0; c.left_gi = c.left_hi = 0; c.left_g = c.left_h = 0;
    c.is_categorical = 0; c.num_cat_bins = 0; for (int w = 0; w < 8; ++w) c.cat_bitset[w] = 0;
    a.cand[static_cast<size_t>(blockIdx.x) * a.num_features + fi] = c;
  }
  if (search && !node_masked && m.bin_type != 0) {
    ScanCategoricalWarp<QUANT>(a, src, child, write_back, m, leaf, f, fi, lane, warp);
    return;
  }
  if (!search || node_masked) {
    // materialisation only (feature not sampled for this tree)
    if (write_back) for (int j = lane; j < nstored; j += 32) {
      long long gi, hi; double gd, hd; hist_q_t rq; double2 rd;
      LoadBin<QUANT>(src, j, &gi, &hi, &gd, &hd, &rq, &rd);
      if (QUANT) reinterpret_cast<hist_q_t*>(child)[j] = rq; else reinterpret_cast<double2*>(child)[j] = rd;
    }
    return;
  }

  LeafScanInfo L;
  L.sum_g = leaf.sum_g; L.sum_h = leaf.sum_h; L.sum_gi = leaf.sum_gi; L.sum_hi = leaf.sum_hi; L.num_data = leaf.num_data_global;
  L.parent_output = leaf.output; L.g_scale = QUANT ? static_cast<double>(a.scales[0]) : 1.0; L.h_scale = QUANT ? static_cast<double>(a.scales[1]) : 1.0; L.min_c = leaf.min_c; L.max_c = leaf.max_c;
  L.mono_factor = MonotonePenaltyFactor(leaf.depth, a.params.monotone_penalty);
  L.cnt_factor = FB_DIV(static_cast<double>(L.num_data), L.sum_h);
  if (a.params.max_delta_step <= 0.0 && a.params.path_smooth <= 0.0)
    L.min_gain_shift = FB_ADD(LeafGain(L.sum_g, FB_ADD(L.sum_h, 2 * kEpsilon), a.params, L.num_data, leaf.output), a.params.min_gain_to_split);
  else
    L.min_gain_shift = FB_ADD(LeafGainGivenOutput(L.sum_g, FB_ADD(L.sum_h, 2 * kEpsilon), a.params, leaf.output), a.params.min_gain_to_split);

  const bool two_pass = m.missing_type != 0 && nb > 2;
  const int skip = two_pass ? (m.missing_type == 1 ? m.default_bin : nb - 1) : -1;
  const int mfb = m.bundled ? m.most_freq_bin : -1;

  // pre-pass: the un-stored most-frequent bin of a bundled feature = leaf total - sum of stored bins
  long long mfb_gi = 0, mfb_hi = 0; double mfb_gd = 0, mfb_hd = 0;
  if (m.bundled) {
    long long sgi = 0, shi = 0; double sgd = 0, shd = 0;
    for (int j = lane; j < nstored; j += 32) {
      long long gi = 0, hi = 0; double gd = 0, hd = 0; hist_q_t rq; double2 rd;
      LoadBin<QUANT>(src, j, &gi, &hi, &gd, &hd, &rq, &rd);
      sgi += gi; shi += hi; sgd += gd; shd += hd;
    }
    for (int o = 16; o > 0; o >>= 1) {
      sgi += __shfl_xor_sync(0xffffffffu, sgi, o); shi += __shfl_xor_sync(0xffffffffu, shi, o);
      sgd += __shfl_xor_sync(0xffffffffu, sgd, o); shd += __shfl_xor_sync(0xffffffffu, shd, o);
    }
    mfb_gi = L.sum_gi - sgi; mfb_hi = L.sum_hi - shi; mfb_gd = L.sum_g - sgd; mfb_hd = L.sum_h - shd;
  }
  // mass of the missing-value bin (kept out of the prefix, added on the left in pass 0)
  long long Mgi = 0, Mhi = 0; double Mgd = 0, Mhd = 0; int Mc = 0;
  if (skip >= 0) {
    if (skip == mfb) { Mgi = mfb_gi; Mhi = mfb_hi; Mgd = mfb_gd; Mhd = mfb_hd; }
    else { hist_q_t rq; double2 rd; LoadBin<QUANT>(src, (mfb >= 0 && skip > mfb) ? skip - 1 : skip, &Mgi, &Mhi, &Mgd, &Mhd, &rq, &rd); }
    const double hreal = QUANT ? FB_MUL(static_cast<double>(Mhi), L.h_scale) : Mhd;
    Mc = BinCountEstimate(hreal, L.cnt_factor);
  }

  double best_gain = -1.0 / 0.0; int best_rank = 1 << 30, best_t = 0, best_pass = 0, best_lc = 0;
  long long best_lgi = 0, best_lhi = 0; double best_lg = 0, best_lh = 0;
  const int rand_t = a.params.extra_trees ? ExtraTreesThreshold(a.extra_seed, a.tree_index, ch.leaf, m.real_index, nb) : -1;
  Acc carry; carry.gi = carry.hi = 0; carry.gd = carry.hd = 0; carry.c = 0;
  for (int b0 = 0; b0 < nb; b0 += 32) {
    const int b = b0 + lane;
    long long gi = 0, hi = 0; double gd = 0, hd = 0; int c = 0;
    if (b < nb) {
      if (b == mfb) { gi = mfb_gi; hi = mfb_hi; gd = mfb_gd; hd = mfb_hd; }
      else {
        const int j = (mfb >= 0 && b > mfb) ? b - 1 : b;
        hist_q_t rq; double2 rd;
        LoadBin<QUANT>(src, j, &gi, &hi, &gd, &hd, &rq, &rd);
        if (write_back) { if (QUANT) reinterpret_cast<hist_q_t*>(child)[j] = rq; else reinterpret_cast<double2*>(child)[j] = rd; }
      }
      if (b == skip) { gi = hi = 0; gd = hd = 0; }
      else { const double hreal = QUANT ? FB_MUL(static_cast<double>(hi), L.h_scale) : hd; c = BinCountEstimate(hreal, L.cnt_factor); }
    }
    // inclusive warp scan
    for (int o = 1; o < 32; o <<= 1) {
      const long long tg = __shfl_up_sync(0xffffffffu, gi, o), th = __shfl_up_sync(0xffffffffu, hi, o);
      const double dg = __shfl_up_sync(0xffffffffu, gd, o), dh = __shfl_up_sync(0xffffffffu, hd, o);
      const int tc = __shfl_up_sync(0xffffffffu, c, o);
      if (lane >= o) { gi += tg; hi += th; gd += dg; hd += dh; c += tc; }
    }
    gi += carry.gi; hi += carry.hi; gd += carry.gd; hd += carry.hd; c += carry.c;
    if (b <= nb - 2 && (rand_t < 0 || b == rand_t)) {
      for (int pass = 0; pass < (two_pass ? 2 : 1); ++pass) {
        if (b == skip && pass == 1 && m.missing_type == 1) continue;
        long long lgi = gi, lhi = hi; int lc = c; double lg, lh;
        const bool addm = pass == 0 && skip >= 0;
        if (addm) { lgi += Mgi; lhi += Mhi; lc += Mc; }
        if (QUANT) { lg = FB_MUL(static_cast<double>(lgi), L.g_scale); lh = FB_MUL(static_cast<double>(lhi), L.h_scale); }
        else { lg = gd + (addm ? Mgd : 0.0); lh = hd + (addm ? Mhd : 0.0); }
        double lo, ro;
        const double gain = EvalCandidate(lg, lh, lc, L, a.params, m.monotone, &lo, &ro);
        if (gain == -1.0 / 0.0) continue;
        const int rank = ScanRank(pass, b, nb);
        if (gain > best_gain || (gain == best_gain && rank < best_rank)) {
          best_gain = gain; best_rank = rank; best_t = b; best_pass = pass; best_lc = lc; best_lgi = lgi; best_lhi = lhi; best_lg = lg; best_lh = lh;
        }
      }
    }
    carry.gi = __shfl_sync(0xffffffffu, gi, 31); carry.hi = __shfl_sync(0xffffffffu, hi, 31);
    carry.gd = __shfl_sync(0xffffffffu, gd, 31); carry.hd = __shfl_sync(0xffffffffu, hd, 31); carry.c = __shfl_sync(0xffffffffu, c, 31);
  }
  // warp argmax: larger gain, then lower scan rank
  for (int o = 16; o > 0; o >>= 1) {
    const double og = __shfl_xor_sync(0xffffffffu, best_gain, o); const int orank = __shfl_xor_sync(0xffffffffu, best_rank, o);
    const int ot = __shfl_xor_sync(0xffffffffu, best_t, o), op = __shfl_xor_sync(0xffffffffu, best_pass, o), olc = __shfl_xor_sync(0xffffffffu, best_lc, o);
    const long long ogi = __shfl_xor_sync(0xffffffffu, best_lgi, o), ohi = __shfl_xor_sync(0xffffffffu, best_lhi, o);
    const double olg = __shfl_xor_sync(0xffffffffu, best_lg, o), olh = __shfl_xor_sync(0xffffffffu, best_lh, o);
    if (og > best_gain || (og == best_gain && orank < best_rank)) {
      best_gain = og; best_rank = orank; best_t = ot; best_pass = op; best_lc = olc; best_lgi = ogi; best_lhi = ohi; best_lg = olg; best_lh = olh;
    }
  }
  if (lane == 0) {
    CandLite c;
    const bool ok = best_gain != -1.0 / 0.0;
    c.gain = ok ? FB_MUL(best_gain, static_cast<double>(m.penalty)) : best_gain;
    c.feature = ok ? f : -1; c.threshold = best_t; c.default_left = best_pass == 0 ? 1 : 0; c.left_cnt = best_lc;
    c.left_gi = best_lgi; c.left_hi = best_lhi; c.left_g = best_lg; c.left_h = best_lh;
    c.is_categorical = 0; c.num_cat_bins = 0; for (int w = 0; w < 8; ++w) c.cat_bitset[w] = 0;
    a.cand[static_cast<size_t>(blockIdx.x) * a.num_features + fi] = c;
  }
}

// Per-leaf argmax over the searched features of one child -> SplitRecord (the CPU's tie order: higher gain, then
// lower real feature index, then lower threshold). Multi-rank: the record is this rank's best over the features it
// owns; it is stored into every rank's slot array. Call with all T threads of a block.
struct ReduceShared { SplitRecord rec; double gain[kFindThreads]; int feat[kFindThreads], thr[kFindThreads], idx[kFindThreads]; };

template <int T>
__device__ inline void ReduceChildBody(const FindArgs& a, int child, ReduceShared& R) {
  const bool gather = a.wait_best.world > 1;   // data-parallel and feature-parallel both all-gather the rank-local best
  const FindChild ch = a.children[child];
  LeafInfo leaf = a.leaves[ch.leaf];
  leaf.num_data_global = ChildGlobalCount(a, ch, leaf.num_data_global);
  double bg = -1.0 / 0.0; int bf = -1, bt = 0, bi = -1;
  // a level that ended the tree was not searched: its candidate slots hold nothing meaningful, the record stays
  // empty and only the children's global row counts are settled here
  const bool searched = !(a.ctrl != nullptr && a.ctrl->skip_search);
  for (int k = threadIdx.x; searched && k < a.num_features; k += T) {
    const CandLite* cp = a.cand + static_cast<size_t>(child) * a.num_features + k;
    const double gain = LoadWords(&cp->gain); const int feature = LoadWords(&cp->feature), threshold = LoadWords(&cp->threshold);
    const int rf = feature >= 0 ? a.meta[feature].real_index : -1;
    if (SplitBetter(gain, rf, threshold, bg, bf, bt)) { bg = gain; bf = rf; bt = threshold; bi = k; }
  }
  R.gain[threadIdx.x] = bg; R.feat[threadIdx.x] = bf; R.thr[threadIdx.x] = bt; R.idx[threadIdx.x] = bi;
  __syncthreads();
  for (int o = T / 2; o > 0; o >>= 1) {
    if (threadIdx.x < o && SplitBetter(R.gain[threadIdx.x + o], R.feat[threadIdx.x + o], R.thr[threadIdx.x + o], R.gain[threadIdx.x], R.feat[threadIdx.x], R.thr[threadIdx.x])) {
      R.gain[threadIdx.x] = R.gain[threadIdx.x + o]; R.feat[threadIdx.x] = R.feat[threadIdx.x + o]; R.thr[threadIdx.x] = R.thr[threadIdx.x + o]; R.idx[threadIdx.x] = R.idx[threadIdx.x + o];
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    SplitRecord r; InitSplitRecord(&r);
    const bool depth_ok = a.params.max_depth <= 0 || leaf.depth < a.params.max_depth;
    const bool size_ok = leaf.num_data_global >= 2 * a.params.min_data_in_leaf;
    if (R.idx[0] >= 0 && depth_ok && size_ok) {
      const CandLite c = LoadWords(a.cand + static_cast<size_t>(child) * a.num_features + R.idx[0]);
      r.gain = c.gain; r.feature = c.feature; r.threshold = c.threshold; r.default_left = c.default_left;
      if (a.params.cegb_split > 0.0) r.gain -= a.params.cegb_split * static_cast<double>(leaf.num_data_global);
      r.left_g = c.left_g; r.left_h = c.left_h; r.right_g = FB_SUB(leaf.sum_g, c.left_g); r.right_h = FB_SUB(leaf.sum_h, c.left_h);
      r.left_gi = c.left_gi; r.left_hi = c.left_hi; r.left_cnt = c.left_cnt; r.right_cnt = leaf.num_data_global - c.left_cnt;
      r.monotone = c.is_categorical ? 0 : a.meta[c.feature].monotone;
      r.is_categorical = c.is_categorical; r.num_cat_bins = c.num_cat_bins; for (int w = 0; w < 8; ++w) r.cat_bitset[w] = c.cat_bitset[w];
      SplitParams p = a.params; if (c.is_categorical) p.lambda_l2 = FB_ADD(p.lambda_l2, a.params.cat_l2);
      r.left_out = LeafOutput(r.left_g, FB_ADD(r.left_h, kEpsilon), p, r.left_cnt, leaf.output);
      r.right_out = LeafOutput(r.right_g, FB_ADD(r.right_h, kEpsilon), p, r.right_cnt, leaf.output);
      if (p.use_mc != 0) { r.left_out = ClampOutput(r.left_out, leaf.min_c, leaf.max_c); r.right_out = ClampOutput(r.right_out, leaf.min_c, leaf.max_c); }
    }
    if (gather) { R.rec = r; a.leaves_rw[ch.leaf].num_data_global = leaf.num_data_global; }
    else a.best[ch.leaf] = r;
  }
  if (gather) {
    // all-gather of the rank-local best split: plain stores into every rank's slot array
    __syncthreads();
    const unsigned int* src = reinterpret_cast<const unsigned int*>(&R.rec);
    constexpr int kWords = sizeof(SplitRecord) / 4;
    for (int p = 0; p < a.wait_best.world; ++p) {
      unsigned int* dst = reinterpret_cast<unsigned int*>(a.peer_best[p] + ch.leaf);
      for (int w = threadIdx.x; w < kWords; w += T) dst[w] = src[w];
    }
  }
}

// Multi-rank: the best split of a leaf is the best of the ranks' records (each rank searched only the features it
// owns). Every rank runs this on the same records, so all ranks decide alike. One thread per child.
__device__ inline void GatherChild(const FindArgs& a, int child) {
  const FindChild ch = a.children[child];
  // compare on the records' first 16 bytes (gain, feature, threshold), then fetch only the winner whole
  SplitRecord best; InitSplitRecord(&best);
  int best_real = -1, best_rank = -1;
  for (int r = 0; r < a.wait_best.world; ++r) {
    const SplitRecord* rp = a.gathered + static_cast<size_t>(r) * a.gathered_stride + ch.leaf;
    const double gain = LoadWords(&rp->gain);
    const int feature = LoadWords(&rp->feature), threshold = LoadWords(&rp->threshold);
    const int real = feature >= 0 ? a.meta[feature].real_index : -1;
    if (SplitBetter(gain, real, threshold, best.gain, best_real, best.threshold)) { best.gain = gain; best.threshold = threshold; best_real = real; best_rank = r; }
  }
  if (best_rank >= 0) best = LoadWords(a.gathered + static_cast<size_t>(best_rank) * a.gathered_stride + ch.leaf);
  a.best[ch.leaf] = best;
}

template <bool QUANT>
__global__ void __launch_bounds__(kFindThreads) FindSplitsKernel(FindArgs a, CtrlArgs ca) {
  __shared__ int s_last;
  __shared__ union TailShared { ReduceShared r; CtrlShared c; } S;
  const int nchildren = a.ctrl != nullptr ? a.ctrl->num_children : a.num_children;
  if (nchildren <= 0) {
    // A level past the end of the tree (levels are enqueued ahead): nothing to search, but the NEXT level's record must
    // still be written, or that level would run on the stale record its ring half holds from two levels ago.
    if (a.fused_tail && a.run_controller && blockIdx.x == 0 && blockIdx.y == 0) ControllerBody<kFindThreads>(ca, S.c);
    return;
  }
  if (static_cast<int>(blockIdx.x) >= nchildren) return;
  // multi-rank: the owned slices are complete once every rank's construct has raised its flag. The wait also
  // orders the peers' child counts (stored by their partition, before their construct) ahead of the per-leaf
  // argmax that follows, so it is taken even when the search itself is skipped.
  if (a.wait.world > 1) FabricWaitAll(a.wait);
  // skip_search: the tree is complete, nothing was constructed for these children
  if (!(a.ctrl != nullptr && a.ctrl->skip_search)) FindSplitsWarp<QUANT>(a);
  if (!a.fused_tail) return;

  // ---- fused tail, step 1: the last block of this child reduces the child's candidates ----
  __syncthreads();   // every warp's candidate is written
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int prev = atomicAdd(a.child_done + blockIdx.x, 1u);
    s_last = (prev + 1 == gridDim.y) ? 1 : 0;
    if (s_last) a.child_done[blockIdx.x] = 0;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  ReduceChildBody<kFindThreads>(a, blockIdx.x, S.r);
  // ---- step 2: the last reducer of the level takes over ----
  const bool gather = a.wait_best.world > 1;
  __syncthreads();
  if (threadIdx.x == 0) {
    if (gather) __threadfence_system(); else __threadfence();   // this block's record (peer stores included) is published before it is counted
    const unsigned int prev = atomicAdd(a.level_done, 1u);
    s_last = (prev + 1 == static_cast<unsigned int>(nchildren)) ? 1 : 0;
    if (s_last) *a.level_done = 0;
  }
  __syncthreads();
  if (!s_last) return;
  if (gather) {
    // every child's record of this rank is on its way: raise "best published" on every peer, wait (bounded) for
    // theirs, then take the argmax over ranks for every child
    if (threadIdx.x == 0) { __threadfence_system(); for (int r = 0; r < a.sig.world; ++r) StoreFlagAfterFence(a.sig.peer_flag[r], a.sig.epoch); }
    FabricWaitAll(a.wait_best);
    for (int c = threadIdx.x; c < nchildren; c += kFindThreads) GatherChild(a, c);
  }
  __threadfence();
  __syncthreads();
  if (a.run_controller) ControllerBody<kFindThreads>(ca, S.c);
}

__global__ void __launch_bounds__(128) ReduceBestKernel(FindArgs a) {
  const bool gather = a.wait_best.world > 1;
  if (static_cast<int>(blockIdx.x) >= (a.ctrl != nullptr ? a.ctrl->num_children : a.num_children)) { if (gather) FabricSignalDone(a.sig, gridDim.x); return; }
  __shared__ ReduceShared R;
  ReduceChildBody<128>(a, blockIdx.x, R);
  if (gather) FabricSignalDone(a.sig, gridDim.x, true);
}

__global__ void GatherBestKernel(FindArgs a) {
  if (static_cast<int>(blockIdx.x) >= (a.ctrl != nullptr ? a.ctrl->num_children : a.num_children)) return;
  FabricWaitAll(a.wait_best);
  if (threadIdx.x != 0) return;
  GatherChild(a, blockIdx.x);
}

}  // namespace

void LaunchGatherBest(const FindArgs& a, cudaStream_t s) {
  if (a.num_children <= 0 || a.wait_best.world <= 1) return;
  GatherBestKernel<<<a.num_children, 32, 0, s>>>(a);
  FB_LAUNCHED(); FB_KERNEL_CHECK();
}

void LaunchFindSplits(const FindArgs& a, cudaStream_t s, const CtrlArgs* tail_ctrl) {
  if (a.num_children <= 0) return;
  const int nf = a.num_features + a.num_sub_features;
  if (nf <= 0 && !a.fused_tail) return;
  if (a.fused_tail && a.run_controller && (tail_ctrl == nullptr || tail_ctrl->max_leaves > kCtrlMaxLeaves)) Log::Fatal("The fused level controller handles up to %d leaves", kCtrlMaxLeaves);
  dim3 grid(a.num_children, std::max(1, (nf + kWarpsPerBlock - 1) / kWarpsPerBlock));
  // categorical features stage their bins in shared memory, one scratch per warp
  const size_t sm = a.has_categorical ? sizeof(CatScratch) * kWarpsPerBlock : 0;
  static bool attr = false;
  if (sm > 16 * 1024 && !attr) {   // together with the tail's static shared memory the default limit is passed early
    FB_CUDA(cudaFuncSetAttribute(FindSplitsKernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sm)));
    FB_CUDA(cudaFuncSetAttribute(FindSplitsKernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sm)));
    attr = true;
  }
  const CtrlArgs ca = tail_ctrl != nullptr ? *tail_ctrl : CtrlArgs();
  if (a.quant) FindSplitsKernel<true><<<grid, kFindThreads, sm, s>>>(a, ca); else FindSplitsKernel<false><<<grid, kFindThreads, sm, s>>>(a, ca);
  FB_LAUNCHED(); FB_KERNEL_CHECK();
}

void LaunchReduceBest(const FindArgs& a, cudaStream_t s) {
  if (a.num_children <= 0) return;
  ReduceBestKernel<<<a.num_children, 128, 0, s>>>(a);
  FB_LAUNCHED(); FB_KERNEL_CHECK();
}

}  // namespace fb
