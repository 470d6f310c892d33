// Device engine: one boosting iteration and the level loop of one tree.
//
// Per level (all splitting leaves at once): partition flags -> scan + child/leaf/task setup ->
// scatter -> construct (smaller children; the epilogue adds each bin into the slot of the rank that
// owns its feature) -> find on the owned slice (+ in-place larger = parent - smaller) -> per-leaf
// argmax (multi-rank: stored into every peer, then an argmax over the ranks' records) -> ONE
// read-back of the leaf records and best splits, on which the host applies the gain-ranked leaf
// budget. Exact child counts come back with that read-back: no second synchronisation per level.
//
// Multi-rank ordering (all inside kernels, no NCCL): construct's last block raises "construct done"
// on every peer; the split search waits for all ranks' flags; its last block raises "best published";
// the gather waits for those. Every wait is bounded and reports through the status word.
#include "engine.h"

#include <numeric>

namespace fb {

namespace {

// One split of the device's record applied to the host tree (numerical threshold or categorical set).
int ApplySplit(Tree* tree, const Dataset* ds, int leaf, const SplitRecord& b) {
  const FeatureMeta& m = ds->feature_meta[b.feature];
  const BinMapper& bm = *ds->mappers[m.real_index];
  if (!b.is_categorical)
    return tree->Split(leaf, b.feature, m.real_index, static_cast<uint32_t>(b.threshold), bm.BinToValue(b.threshold), b.left_out, b.right_out,
                       b.left_cnt, b.right_cnt, b.left_h, b.right_h, static_cast<float>(b.gain), m.missing_type, b.default_left != 0);
  std::vector<uint32_t> inner(b.cat_bitset, b.cat_bitset + 8);
  while (inner.size() > 1 && inner.back() == 0) inner.pop_back();
  std::vector<uint32_t> real;
  for (int bin = 0; bin < m.num_bin; ++bin) if ((b.cat_bitset[bin >> 5] >> (bin & 31)) & 1) {
    const int cat = bm.bin_2_categorical[bin]; if (cat < 0) continue;
    if (static_cast<int>(real.size()) <= (cat >> 5)) real.resize((cat >> 5) + 1, 0);
    real[cat >> 5] |= (1u << (cat & 31));
  }
  if (real.empty()) real.push_back(0);
  return tree->SplitCategorical(leaf, b.feature, m.real_index, inner.data(), static_cast<int>(inner.size()), real.data(), static_cast<int>(real.size()),
                                b.left_out, b.right_out, b.left_cnt, b.right_cnt, b.left_h, b.right_h, static_cast<float>(b.gain), m.missing_type);
}

}  // namespace

void CudaEngine::TrainOneIter(const float* custom_grad, const float* custom_hess, int iter, double shrinkage, const std::vector<double>& init_scores,
                              std::vector<std::unique_ptr<Tree>>* out, bool* all_constant) {
  const float* grad = grad_.get(); const float* hess = hess_.get();
  const bool goss = cfg_.data_sample_strategy == "goss" && iter >= static_cast<int>(1.0 / cfg_.learning_rate);
  bool bagging = !goss && cfg_.data_sample_strategy != "goss" && bag_freq_ > 0 &&
                 (cfg_.bagging_fraction < 1.0 || cfg_.pos_bagging_fraction < 1.0 || cfg_.neg_bagging_fraction < 1.0);
  if (bagging && (iter % bag_freq_ == 0 || bag_count_ < 0)) DrawBag(iter / bag_freq_);
  bag_active_ = bagging;
  const uint8_t* mask = bag_mask_ptr();
  root_count_ = bagging ? bag_count_ : n_; root_global_ = bagging ? bag_global_ : train_->global_num_data;
  clock_.Begin(st_grad_, stream_);
  if (custom_grad != nullptr) {
    grad = custom_grad; hess = custom_hess;
    FB_CUDA(cudaStreamSynchronize(0));   // custom gradients were produced on the caller's (default) stream
    if (goss) {
      // one-side sampling rescales gradients in place: work on the engine's own copy
      FB_CUDA(cudaMemcpyAsync(grad_.get(), custom_grad, sizeof(float) * static_cast<size_t>(n_) * K_, cudaMemcpyDeviceToDevice, stream_));
      FB_CUDA(cudaMemcpyAsync(hess_.get(), custom_hess, sizeof(float) * static_cast<size_t>(n_) * K_, cudaMemcpyDeviceToDevice, stream_));
      grad = grad_.get(); hess = hess_.get();
    } else LaunchAbsMax(grad, hess, n_, K_, maxbuf_.get(), stream_, mask);
  } else {
    if (obj_ == nullptr) Log::Fatal("No objective function provided and no custom gradients given");
    if (host_gradients_) {
      const size_t total = static_cast<size_t>(n_) * K_;
      std::vector<float> hs(total); std::vector<double> sc(total); std::vector<float> hg(total), hh(total);
      FB_CUDA(cudaMemcpyAsync(hs.data(), score_.get(), sizeof(float) * total, cudaMemcpyDeviceToHost, stream_));
      FB_CUDA(cudaStreamSynchronize(stream_));
      for (size_t i = 0; i < total; ++i) sc[i] = hs[i];
      obj_->GetGradients(sc.data(), hg.data(), hh.data());
      FB_CUDA(cudaMemcpyAsync(grad_.get(), hg.data(), sizeof(float) * total, cudaMemcpyHostToDevice, stream_));
      FB_CUDA(cudaMemcpyAsync(hess_.get(), hh.data(), sizeof(float) * total, cudaMemcpyHostToDevice, stream_));
      FB_CUDA(cudaStreamSynchronize(stream_));
      LaunchAbsMax(grad, hess, n_, K_, maxbuf_.get(), stream_, mask);
    } else {
      if (objd_.kind == kObjXendcg) objd_.p1 = static_cast<double>(xendcg_round_++);   // the round index keys this round's random draws
      LaunchObjectiveGradients(objd_, score_.get(), dd_->label.get(), dd_->weight.size() ? dd_->weight.get() : nullptr,
                               dd_->query_boundaries.size() ? dd_->query_boundaries.get() : nullptr, dd_->num_queries, label_gain_.get(),
                               static_cast<int>(label_gain_.size()), n_, grad_.get(), hess_.get(), maxbuf_.get(), stream_);
    }
    if (bagging && quant_) LaunchAbsMax(grad, hess, n_, K_, maxbuf_.get(), stream_, mask);   // the scale comes from the bag's rows only
  }
  if (goss) {
    DrawGoss(iter);
    bagging = true; bag_active_ = true; mask = bag_mask_ptr();
    root_count_ = bag_count_; root_global_ = bag_global_;
    LaunchAbsMax(grad, hess, n_, K_, maxbuf_.get(), stream_, mask);
  }
  // quantization scales must be the same on every rank: max over ranks of the per-class maxima
  if (data_parallel() && quant_) fabric_->AllReduce(kFabricMaxF32, maxbuf_.get(), global_max_.get(), 2 * K_, stream_);
  clock_.End(stream_);
  bool any_split = false;
  round_grad_ = grad; round_hess_ = hess;
  for (int k = 0; k < K_; ++k) {
    std::unique_ptr<Tree> tree;
    const bool need = obj_ == nullptr || obj_->ClassNeedTrain(k);
    if (need && train_->num_features > 0) {
      cur_grad_ = grad + static_cast<size_t>(k) * n_; cur_hess_ = hess + static_cast<size_t>(k) * n_;
      cur_shrinkage_ = shrinkage; cur_score_ = score_.get() + static_cast<size_t>(k) * n_; score_done_ = false;
      fast_score_ok_ = !leafwise_ && !bagging && !(quant_ && cfg_.quant_train_renew_leaf) && !(obj_ != nullptr && obj_->IsRenewTreeOutput());
      tree.reset(TrainTree(k, iter * K_ + k));
    } else tree.reset(new Tree(2));
    if (tree->num_leaves > 1) {
      any_split = true;
      if (quant_ && cfg_.quant_train_renew_leaf) RenewLeavesFromTrueGradients(tree.get());
      else if (obj_ != nullptr && obj_->IsRenewTreeOutput()) RenewLeavesByObjective(tree.get(), k);
      tree->Shrink(shrinkage);
      // training rows through the final partition; validation rows by traversal
      clock_.Begin(st_score_, stream_);
      if (!bagging && !score_done_) {
        leaf_value_.Upload(tree->leaf_value.data(), tree->num_leaves, stream_);
        LaunchAddLeafOutputs(leaves_.get(), leaf_value_.get(), tree->num_leaves, idx_[0].get(), idx_[1].get(), score_.get() + static_cast<size_t>(k) * n_, stream_);
      }
      clock_.End(stream_);
      if (!valid_.empty() || bagging) {
        DevTree dt; UploadTreeForTraversal(*tree, train_, &dt);
        // out-of-bag rows are in no leaf window: with bagging the training scores take the traversal too
        if (bagging) LaunchAddTreeBinned(dt, dd_->rows.get(), dd_->row_stride, n_, 1.f, score_.get() + static_cast<size_t>(k) * n_, stream_);
        for (auto& vs : valid_) LaunchAddTreeBinned(dt, vs.dd->rows.get(), vs.dd->row_stride, vs.ds->num_data, 1.f, vs.score.get() + static_cast<size_t>(k) * vs.ds->num_data, stream_);
      }
      FB_CUDA(cudaStreamSynchronize(stream_));   // leaf_value upload source and traversal staging are host memory
      if (std::fabs(init_scores[k]) > kEpsilon) tree->AddBias(init_scores[k]);
    } else {
      double outv = 0.0;
      if (iter == 0) { outv = (!need && obj_ != nullptr) ? obj_->BoostFromScore(k) : init_scores[k]; if (!need) AddConstantToScores(outv, k); }
      tree->AsConstantTree(outv);
    }
    out->push_back(std::move(tree));
  }
  clock_.Resolve();
  *all_constant = !any_split;
}

Tree* CudaEngine::TrainTree(int class_id, int tree_index) {
  const int NL = grow_leaves_;   // leaf capacity of the device tree (= num_leaves unless leaf-wise growth over-grows)
  col_sampler_.ResetByTree(tree_index);
  // features searched on this rank this tree (owned, sampled, numerical) and the rest of the owned ones
  std::vector<int> feats, subs;
  for (int f : owned_features_) { if (col_sampler_.used_by_tree()[f]) feats.push_back(f); else subs.push_back(f); }
  features_.Upload(feats, stream_); sub_features_.Upload(subs, stream_);
  const int NF = static_cast<int>(feats.size()), NS = static_cast<int>(subs.size());
  std::vector<int> feats_all, subs_all;   // voting: the local pass searches every sampled feature, owned or not
  if (voting_) {
    for (int f = 0; f < train_->num_features; ++f) { if (col_sampler_.used_by_tree()[f]) feats_all.push_back(f); else subs_all.push_back(f); }
    features_all_.Upload(feats_all, stream_); sub_features_all_.Upload(subs_all, stream_);
  }

  clock_.Begin(st_quant_, stream_);
  // The pool is cleared BEFORE this tree's first cross-rank exchange: a peer can only start adding
  // into this rank's slots after it has seen this rank's contribution to that exchange.
  FB_CUDA(cudaMemsetAsync(pool_base_, 0, pool_bytes_, stream_));
  const bool fixed_gate = quant_ && cfg_.quant == QuantMode::FixedPoint && plan_.robust_scale && cfg_.quant_bins_resolved <= 256 && cfg_.num_class <= 1;
  const bool fixed_ef = quant_ && cfg_.quant == QuantMode::FixedPoint && plan_.quant_ef;
  if (fixed_gate || fixed_ef) {
    // fixed point with its extras: (gate) log-magnitude histogram over all ranks' rows -> possibly a scale anchored below
    // an outlier cluster, outliers saturating; (feedback) last round's rounding residuals added before rounding
    const float* mx = data_parallel() ? global_max_.get() + 2 * class_id : maxbuf_.get() + 2 * class_id;
    if (qmax_.size() == 0) { qmax_.Alloc(2); qclamp_.Alloc(1); mag_hist_.Alloc(kQuantMagBuckets); }
    if (fixed_gate) {
      LaunchGradMagHist(cur_grad_, n_, mx, bag_mask_ptr(), mag_hist_.get(), stream_);
      if (data_parallel())   // the small all-reduce takes 128 counters at a time
        for (int off = 0; off < kQuantMagBuckets; off += 128) fabric_->AllReduce(kFabricSumI64, mag_hist_.get() + off, mag_hist_.get() + off, 128, stream_);
    }
    LaunchRobustScale(mag_hist_.get(), static_cast<long long>(root_global_), mx, cfg_.quant_bins_resolved, fixed_gate, qmax_.get(), qclamp_.get(), stream_);
    int8_t* residual = nullptr;
    if (fixed_ef) {
      const size_t per_class = 2 * static_cast<size_t>(n_);
      if (ef_residual_.size() != per_class * K_) { ef_residual_.Alloc(per_class * K_); ef_residual_.Zero(stream_); }
      residual = ef_residual_.get() + per_class * class_id;
    }
    LaunchQuantizeFeedback(cur_grad_, cur_hess_, n_, qmax_.get(), qclamp_.get(), cfg_.quant_bins_resolved, residual, const_cast<uint8_t*>(gh_base_), gh_stride_, scales_.get(),
                           root_sums_i_.get(), stream_, bag_mask_ptr());
    if (data_parallel()) fabric_->AllReduce(kFabricSumI64, root_sums_i_.get(), root_sums_i_.get(), 2, stream_);
  } else if (quant_) {
    LaunchQuantize(cur_grad_, cur_hess_, n_, maxbuf_.get() + 2 * class_id, data_parallel() ? global_max_.get() + 2 * class_id : nullptr, cfg_.quant_bins_resolved,
                   cfg_.quant == QuantMode::Stochastic, static_cast<uint32_t>(cfg_.seed), static_cast<uint32_t>(tree_index),
                   static_cast<uint64_t>(train_->global_row_offset), const_cast<uint8_t*>(gh_base_), gh_stride_, scales_.get(), root_sums_i_.get(), stream_, bag_mask_ptr());
    if (data_parallel()) fabric_->AllReduce(kFabricSumI64, root_sums_i_.get(), root_sums_i_.get(), 2, stream_);
  } else {
    LaunchInterleave(cur_grad_, cur_hess_, n_, gh2_.get(), partial_.get(), static_cast<int>(partial_.size() / 2), root_sums_d_.get(), stream_, bag_mask_ptr());
    if (data_parallel()) fabric_->AllReduce(kFabricSumF64, root_sums_d_.get(), root_sums_d_.get(), 2, stream_);
  }
  const bool bagged = bag_active_;
  {
    // root leaf record, level-record ring, frontier, the root's construct task and search descriptor: one small kernel
    TreeInitArgs ti;
    ti.leaves = leaves_.get(); ti.sums_i = root_sums_i_.get(); ti.sums_d = root_sums_d_.get(); ti.scales = scales_.get(); ti.quant = quant_ ? 1 : 0;
    ti.n_local = root_count_; ti.n_global = root_global_; ti.sp = sp_;
    ti.ctrl = use_ctrl_ ? ctrl_.get() : nullptr; ti.frontier = use_ctrl_ ? frontier_.get() : nullptr;
    ti.root_task = hist_tasks_.get(); ti.root_child = root_child_.get();
    const int rpb0 = ChooseRowsPerBlock(root_count_);
    ti.root_blocks = std::max(1, (root_count_ + rpb0 - 1) / rpb0);
    LaunchInitTree(ti, stream_);
  }
  if (bagged) FB_CUDA(cudaMemcpyAsync(idx_[0].get(), bag_idx_.get(), sizeof(int) * static_cast<size_t>(root_count_), cudaMemcpyDeviceToDevice, stream_));
  else LaunchInitIndices(idx_[0].get(), n_, stream_);
  clock_.End(stream_);

  // ---- common launch descriptors ----
  HistArgs ha = HistArgs();
  ha.rows = dd_->rows.get(); ha.row_stride = dd_->row_stride; ha.num_groups = dd_->num_groups; ha.gh_base = gh_base_; ha.gh_stride = gh_stride_;
  ha.idx[0] = idx_[0].get(); ha.idx[1] = idx_[1].get(); ha.tasks = hist_tasks_.get(); ha.parts = parts_.get(); ha.num_parts = static_cast<int>(h_parts_.size());
  ha.max_part_bins = max_part_bins_; ha.group_bin_start = dd_->group_bin_start.get(); ha.sub_rows = sub_rows_;
  const bool dp = data_parallel();
  const bool rs = dp && !voting_;   // construct fused with the reduce-scatter (plain data-parallel)
  ha.dest.bin_owner = bin_owner_.get(); ha.dest.bin_local = voting_ ? bin_identity_.get() : bin_local_.get(); ha.dest.num_ranks = rs ? world_ : 1; ha.dest.rank = rank_;
  ha.dest.owner_only = feature_parallel_ ? 1 : 0;
  for (int r = 0; r < kMaxRanks; ++r) { ha.dest.pool[r] = nullptr; ha.dest.slot_stride[r] = 0; }
  for (int r = 0; r < kMaxRanks; ++r) ha.dest.peer_stage[r] = nullptr;
  if (rs) {
    for (int r = 0; r < world_; ++r) { ha.dest.pool[r] = fabric_->Ptr<char>(r, off_pool_); ha.dest.slot_stride[r] = slot_strides_[r]; ha.dest.peer_stage[r] = fabric_->Ptr<char>(r, off_stage_); }
    ha.dest.stage_local = stage_local_.get(); ha.dest.task_done = task_done_.get(); ha.dest.stage_cap = NL;
  } else { ha.dest.pool[0] = pool_base_; ha.dest.slot_stride[0] = voting_ ? train_->num_total_bin : slot_stride_; }
  ha.num_total_bin = train_->num_total_bin; ha.lane_mode = lane_mode_; ha.lane_bins = lane_bins_; ha.lane_red = lane_red_ ? 1 : 0;
  ha.bulk_root = plan_.bulk_root ? 1 : 0; ha.status = hist_status_.get();
  // K9: when this tree samples few columns, construct from a dense per-tree copy of just those groups
  // (feature-parallel: just the sampled groups this rank owns)
  int first_group = 0;
  if (plan_.compact_view && lane_mode_ != 0 && dd_->cols.size() > 0) {
    std::vector<char> want(train_->num_groups, 0);
    for (int f = 0; f < train_->num_features; ++f) if (col_sampler_.used_by_tree()[f]) {
      const int g = train_->feature_meta[f].group;
      if (!feature_parallel_ || h_bin_owner_[train_->group_bin_start[g]] == rank_) want[g] = 1;
    }
    std::vector<int> glist, gstart, gcount;
    for (int g = 0; g < train_->num_groups; ++g) if (want[g]) { glist.push_back(g); gstart.push_back(train_->group_bin_start[g]); gcount.push_back(train_->group_num_bin[g]); }
    // groups of at most 16 bins are also packed two per byte (B4): the view then pays off even with every group listed
    const bool p4 = plan_.pack4 && train_->max_group_bin <= 16;
    if (!glist.empty() && (p4 || 2 * glist.size() <= static_cast<size_t>(train_->num_groups))) {
      const int nlist = static_cast<int>(glist.size());
      const int cstride = p4 ? ((nlist + 1) / 2 + 15) / 16 * 16 : (nlist + 15) / 16 * 16;
      if (glist != compact_list_ || p4 != compact_p4_) {   // the view depends on the list only: trees that sample the same groups reuse it
        compact_groups_.Upload(glist, stream_); compact_start_.Upload(gstart, stream_); compact_count_.Upload(gcount, stream_);
        if (compact_rows_.size() < static_cast<size_t>(n_) * cstride) compact_rows_.Alloc(static_cast<size_t>(n_) * cstride);
        LaunchCompactGather(dd_->cols.get(), n_, n_, compact_groups_.get(), nlist, compact_rows_.get(), cstride, stream_, p4);
        FB_CUDA(cudaStreamSynchronize(stream_));   // the host lists above go out of scope
        compact_list_ = glist; compact_p4_ = p4;
      }
      ha.rows = compact_rows_.get(); ha.row_stride = cstride; ha.num_groups = nlist; ha.pack4 = p4 ? 1 : 0;
      ha.group_bin_start = compact_start_.get(); ha.group_bin_count = compact_count_.get();
      first_group = glist[0];
    }
  }
  ha.sig.world = rs ? world_ : 1;
  FindArgs fa = FindArgs();
  fa.features = features_.get(); fa.num_features = NF; fa.sub_features = sub_features_.get(); fa.num_sub_features = NS; fa.meta = dd_->feature_meta.get();
  fa.bin_local = bin_local_.get(); fa.pool = pool_base_; fa.slot_stride = slot_stride_; fa.leaves = leaves_.get(); fa.scales = scales_.get(); fa.params = sp_;
  fa.cand = cand_.get(); fa.best = best_.get(); fa.quant = quant_ ? 1 : 0;
  fa.tree_index = tree_index; fa.extra_seed = static_cast<unsigned int>(cfg_.extra_seed);
  fa.has_categorical = 0; for (int f : feats) if (train_->feature_meta[f].bin_type != 0) fa.has_categorical = 1;
  // data-parallel: construct-done flags + staged slices + counts; both multi-rank modes all-gather the best records
  fa.wait.world = dp ? world_ : 1; fa.wait_best.world = world_; fa.sig.world = world_; fa.leaves_rw = leaves_.get();
  if (world_ > 1) {
    const FabricView v = fabric_->View();
    fa.sig.done_counter = fabric_->done_counter(1);
    for (int r = 0; r < world_; ++r) {
      fa.sig.peer_flag[r] = fabric_->Ptr<unsigned int>(r, flag_best_) + rank_;
      fa.peer_best[r] = fabric_->Ptr<SplitRecord>(r, off_best_) + static_cast<size_t>(rank_) * NL;
    }
    fa.wait_best.flags = fabric_->Local<unsigned int>(flag_best_); fa.wait_best.max_spins = v.max_spins; fa.wait_best.status = v.status;
    fa.gathered = fabric_->Local<SplitRecord>(off_best_); fa.gathered_stride = NL;
    if (dp) {
      ha.sig.done_counter = fabric_->done_counter(0);
      for (int r = 0; r < world_; ++r) ha.sig.peer_flag[r] = fabric_->Ptr<unsigned int>(r, flag_hist_) + rank_;
      if (voting_) { fa.voted = voted_.get(); fa.voted_stride = train_->num_features; }
      fa.wait.flags = fabric_->Local<unsigned int>(flag_hist_); fa.wait.max_spins = v.max_spins; fa.wait.status = v.status;
      fa.counts = fabric_->Local<int>(off_counts_); fa.counts_stride = NL;
      fa.stage = fabric_->Local<char>(off_stage_); fa.stage_cap = NL;
    }
  }
  NodeMaskArgs nm = NodeMaskArgs();
  if (node_mask_on_) {
    std::vector<int> pool;
    for (int f = 0; f < train_->num_features; ++f) if (col_sampler_.used_by_tree()[f]) pool.push_back(f);
    mask_pool_.Upload(pool, stream_);
    if (num_sets_ > 0) path_bits_.Zero(stream_);
    nm.leaves = leaves_.get(); nm.meta = dd_->feature_meta.get(); nm.num_inner = train_->num_features;
    nm.pool = mask_pool_.get(); nm.pool_size = static_cast<int>(pool.size());
    nm.fraction = col_sampler_.bynode_fraction(); nm.seed = static_cast<unsigned int>(col_sampler_.seed()); nm.tree_index = tree_index;
    nm.path_bits = num_sets_ > 0 ? path_bits_.get() : nullptr; nm.set_bits = num_sets_ > 0 ? set_bits_.get() : nullptr; nm.num_sets = num_sets_; nm.words = path_words_;
    nm.mask = node_mask_.get();
    fa.node_mask = node_mask_.get(); fa.node_mask_stride = train_->num_features;
  }
  VoteArgs va = VoteArgs(); FindArgs fl = fa;
  if (voting_) {
    const FabricView v = fabric_->View();
    va.world = world_; va.rank = rank_; va.top_k = std::max(1, cfg_.top_k); va.quant = quant_ ? 1 : 0; va.meta = dd_->feature_meta.get();
    va.num_inner_features = train_->num_features; va.local_pool = pool_base_; va.local_stride = train_->num_total_bin; va.g0_begin = train_->group_bin_start[first_group]; va.g0_bins = train_->group_num_bin[first_group];
    va.sums = vote_sums_.get(); va.scales = scales_.get(); va.cand_local = cand_local_.get(); va.num_searched = static_cast<int>(feats_all.size());
    va.votes_all = fabric_->Local<int>(off_votes_); va.child_cap = NL; va.voted = voted_.get();
    va.bin_owner = bin_owner_.get(); va.bin_local = bin_local_.get(); va.stage_cap = NL;
    va.vote_sig.world = world_; va.vote_sig.done_counter = fabric_->done_counter(3);
    va.hist_sig.world = world_; va.hist_sig.done_counter = fabric_->done_counter(0);
    for (int r = 0; r < world_; ++r) {
      va.peer_votes[r] = fabric_->Ptr<int>(r, off_votes_) + static_cast<size_t>(rank_) * NL * va.top_k;
      va.peer_stage[r] = fabric_->Ptr<char>(r, off_stage_); va.slot_stride[r] = slot_strides_[r];
      va.vote_sig.peer_flag[r] = fabric_->Ptr<unsigned int>(r, flag_vote_) + rank_;
      va.hist_sig.peer_flag[r] = fabric_->Ptr<unsigned int>(r, flag_hist_) + rank_;
    }
    va.vote_wait.world = world_; va.vote_wait.flags = fabric_->Local<unsigned int>(flag_vote_); va.vote_wait.max_spins = v.max_spins; va.vote_wait.status = v.status;
    // the local pass: every sampled feature on this rank's own histograms, thresholds scaled down to a rank's share
    fl.features = features_all_.get(); fl.num_features = static_cast<int>(feats_all.size()); fl.sub_features = sub_features_all_.get(); fl.num_sub_features = static_cast<int>(subs_all.size());
    fl.bin_local = bin_identity_.get(); fl.pool = pool_base_; fl.slot_stride = train_->num_total_bin; fl.cand = cand_local_.get();
    fl.params.min_data_in_leaf = std::max(1, sp_.min_data_in_leaf / world_); fl.params.min_sum_hessian_in_leaf = sp_.min_sum_hessian_in_leaf / world_;
    fl.wait.world = 1; fl.wait_best.world = 1; fl.sig.world = 1; fl.voted = nullptr; fl.local_vote = 1; fl.vote_sums = vote_sums_.get();
    fl.has_categorical = 0; for (int f : feats_all) if (train_->feature_meta[f].bin_type != 0) fl.has_categorical = 1;
  }
  // Device-controlled growth keeps two level records: the kernels of level k read ring[k & 1] while the controller
  // (the tail of level k's search) writes level k + 1's record into the other half, so a block that starts late
  // never sees the next level's sizes.
  const bool fused_tail = use_ctrl_ && plan_.fused_tail;
  CtrlArgs ca = CtrlArgs();
  fa.fused_tail = fused_tail ? 1 : 0; fa.run_controller = fused_tail ? 1 : 0; fa.child_done = child_done_.get(); fa.level_done = level_done_.get();
  fl.fused_tail = 0; fl.run_controller = 0;
  auto construct_and_find = [&]() {
    if (rs) { ha.sig.epoch = fabric_->NextEpoch(); fa.wait.epoch = ha.sig.epoch; }
    clock_.Begin(st_hist_, stream_);
    if (quant_) LaunchHistConstructQuant(ha, stream_); else LaunchHistConstructFloat(ha, stream_);
    if (voting_) {
      // local search, vote (all-gather), restricted reduce-scatter of the voted features
      va.children = fa.children; va.num_children = fa.num_children; va.ctrl = fa.ctrl;
      fl.children = fa.children; fl.num_children = fa.num_children; fl.ctrl = fa.ctrl;
      LaunchVoteLocalSums(va, stream_);
      LaunchFindSplits(fl, stream_);
      va.vote_sig.epoch = fabric_->NextEpoch(); va.vote_wait.epoch = va.vote_sig.epoch;
      LaunchVoteTopK(va, stream_);
      va.hist_sig.epoch = fabric_->NextEpoch(); fa.wait.epoch = va.hist_sig.epoch;
      LaunchVoteTallyPush(va, stream_);
    }
    clock_.End(stream_);
    if (world_ > 1) { fa.sig.epoch = fabric_->NextEpoch(); fa.wait_best.epoch = fa.sig.epoch; }
    clock_.Begin(st_find_, stream_);
    if (node_mask_on_) { nm.children = fa.children; nm.num_children = fa.num_children; nm.ctrl = fa.ctrl; LaunchNodeMask(nm, stream_); }
    if (fused_tail) LaunchFindSplits(fa, stream_, &ca);   // search + per-leaf argmax + cross-rank argmax + level controller
    else { LaunchFindSplits(fa, stream_); LaunchReduceBest(fa, stream_); LaunchGatherBest(fa, stream_); }
    clock_.End(stream_);
  };

  char* hb = h_level_blob_.get(); char* db = level_blob_.get();
  std::unique_ptr<Tree> tree(new Tree(NL));

  // ---- root ----
  {
    // the root's task and search descriptor were written by the tree-init kernel
    ha.rows_per_block = ChooseRowsPerBlock(root_count_);
    ha.num_tasks = 1; ha.total_blocks = std::max(1, (root_count_ + ha.rows_per_block - 1) / ha.rows_per_block); ha.identity_root = bagged ? 0 : 1;
    fa.children = root_child_.get(); fa.num_children = 1;
  }
  const int rpb = ChooseRowsPerBlock(std::max(1, n_ / 2));
  const int max_splits = NL / 2 + 1;
  if (use_ctrl_) {
    ca.cur = ctrl_.get(); ca.nxt = fused_tail ? ctrl_.get() + 1 : ctrl_.get(); ca.frontier = frontier_.get(); ca.journal = journal_.get(); ca.leaves = leaves_.get(); ca.best = best_.get(); ca.meta = dd_->feature_meta.get();
    ca.splits = reinterpret_cast<PartSplit*>(db); ca.child_init = reinterpret_cast<ChildInit*>(db + sizeof(PartSplit) * NL);
    ca.children = reinterpret_cast<FindChild*>(db + (sizeof(PartSplit) + sizeof(ChildInit)) * NL);
    ca.leafwise_budget = leafwise_ ? cfg_.num_leaves - 1 : 0; ca.eval_key = leafwise_ ? eval_key_.get() : nullptr;
    ca.max_leaves = NL; ca.rows_per_block = rpb; ca.bin_owner = feature_parallel_ ? bin_owner_.get() : nullptr;
  }
  // cuda_plan=hist_tc:on: the root histogram on the tensor cores where the instance applies (one rank, rows in order,
  // 32-byte rows of the resident matrix, 8-bit quantized values)
  const bool tc_root = plan_.hist_tc && quant_ && world_ == 1 && !bagged && ha.rows == dd_->rows.get() && dd_->row_stride == 32 && dd_->num_groups <= 32 &&
                       train_->max_group_bin <= 64 && gh_stride_ == 4 && cfg_.quant_bins_resolved <= 127;
  if (plan_.hist_tc && !tc_root && !tc_fallback_logged_) {
    tc_fallback_logged_ = true;
    Log::Warning("cuda_plan=hist_tc:on does not cover this run (needs one rank, no bagging, quantized gradients of at most 127 levels, at most 32 groups of at most 64 bins in 32-byte rows); the lane kernel builds the root histogram");
  }
  if (tc_root) { ha.lane_mode = 3; ha.tc_row_count = root_count_; ha.rows_per_block = HistTcRowsPerBlock(root_count_, num_sms_); ha.total_blocks = (root_count_ + ha.rows_per_block - 1) / ha.rows_per_block; }
  construct_and_find();   // root level (with the fused tail its last block already decides level 1)
  if (tc_root) ha.lane_mode = lane_mode_;
  if (use_ctrl_) {
    // ---- device-controlled growth: levels are enqueued ahead; the host reads one small record per batch ----
    FB_CUDA(cudaMemcpyAsync(h_root_.get(), leaves_.get(), sizeof(LeafInfo), cudaMemcpyDeviceToHost, stream_));   // the root record, before any split rewrites leaf 0
    PartArgs pa = PartArgs();
    pa.rows = dd_->rows.get(); pa.row_stride = dd_->row_stride; pa.idx[0] = idx_[0].get(); pa.idx[1] = idx_[1].get();
    pa.cols = dd_->cols.size() ? dd_->cols.get() : nullptr; pa.col_stride = n_;
    pa.splits = ca.splits; pa.num_splits = max_splits; pa.total_chunks = n_ / kPartChunk + max_splits; pa.bits = bits_.get(); pa.chunk_left = chunk_left_.get();
    pa.split_left_total = split_left_total_.get(); pa.leaves = leaves_.get(); pa.child_init = ca.child_init; pa.hist_tasks = hist_tasks_.get(); pa.rows_per_block = rpb;
    pa.world = dp ? world_ : 1;
    pa.fused_scan = (plan_.fused_scan && !feature_parallel_) ? 1 : 0; pa.split_done = split_done_.get();
    if (dp) for (int r = 0; r < world_; ++r) pa.peer_counts[r] = fabric_->Ptr<int>(r, off_counts_) + static_cast<size_t>(rank_) * NL;
    if (feature_parallel_) SetupBitmapBroadcast(&pa);
    ha.identity_root = 0; ha.rows_per_block = rpb; ha.num_tasks = max_splits; ha.total_blocks = n_ / rpb + max_splits;
    fa.children = ca.children; fa.num_children = 2 * max_splits;
    int level = 0;   // index of the last level enqueued (0 = root)
    auto enqueue_level = [&]() {
      ++level;
      // this level's record: fused tail -> the ring half the previous level's tail wrote; otherwise the one record, updated in place
      LevelCtrl* lc = fused_tail ? ctrl_.get() + (level & 1) : ctrl_.get();
      if (!fused_tail) LaunchLevelController(ca, stream_);
      else { ca.cur = lc; ca.nxt = ctrl_.get() + ((level + 1) & 1); }
      pa.ctrl = lc; ha.ctrl = lc; fa.ctrl = lc;
      if (num_sets_ > 0) LaunchPathBits(lc, journal_.get(), dd_->feature_meta.get(), path_bits_.get(), path_words_, max_splits, stream_);
      if (feature_parallel_) { pa.bc_sig.epoch = fabric_->NextEpoch(); pa.bc_wait.epoch = pa.bc_sig.epoch; }
      clock_.Begin(st_part_, stream_);
      LaunchPartitionFlags(pa, stream_); LaunchPartitionScanSetup(pa, stream_); LaunchPartitionScatter(pa, stream_);
      clock_.End(stream_);
      construct_and_find();
    };
    // the record that describes the tree after the last enqueued level: fused tail -> written by that level's tail into the other ring half
    auto final_ctrl = [&]() -> LevelCtrl* { return fused_tail ? ctrl_.get() + ((level + 1) & 1) : ctrl_.get(); };
    int enqueued = 0; bool records_ready = false;
    LevelCtrl hc;
    for (;;) {
      // leaf-wise trees vary in depth from tree to tree: enqueue a few levels past the last tree's depth (a level after
      // the tree is complete is a handful of empty launches) rather than pay a host round trip per extra level
      const int batch = enqueued == 0 ? std::max(1, levels_hint_ + (leafwise_ ? 3 : 0)) : (leafwise_ ? 4 : 1);
      for (int k = 0; k < batch; ++k) enqueue_level();
      const bool first = enqueued == 0;
      enqueued += batch;
      if (first && fast_score_ok_) {
        // the usual case: this batch completes the tree. The score update and the tree's records ride behind it, so
        // the host waits once per tree and the GPU already has the update while the host rebuilds the tree.
        clock_.Begin(st_score_, stream_);
        LaunchAddLeafOutputsFromRecords(leaves_.get(), final_ctrl(), cur_shrinkage_, NL, idx_[0].get(), idx_[1].get(), cur_score_, stream_, fused_tail);
        clock_.End(stream_);
      }
      clock_.Begin(st_sync_, stream_);
      FB_CUDA(cudaMemcpyAsync(h_ctrl_.get(), final_ctrl(), sizeof(LevelCtrl), cudaMemcpyDeviceToHost, stream_));
      if (first) { journal_.Download(h_journal_.get(), NL, stream_); leaves_.Download(h_leaves_.get(), NL, stream_); hist_status_.Download(h_hist_status_.get(), 1, stream_); }
      clock_.End(stream_);
      if (world_ > 1) { const int st = fabric_->CheckStatus(stream_); if (st != 0) Log::Fatal("A cross-rank wait gave up (device status %d): a peer rank did not reach the same step", st); }
      else FB_CUDA(cudaStreamSynchronize(stream_));
      hc = *h_ctrl_.get();
      if (first && *h_hist_status_.get() != 0) Log::Fatal("A bounded wait inside the construct kernel gave up (device status %u)", *h_hist_status_.get());
      // with the fused tail the record is one decision ahead of the partition: splits it counts may still be pending
      const bool complete = (hc.done || hc.num_leaves >= NL || hc.frontier_count == 0) && (!fused_tail || hc.num_splits == 0);
      if (first && complete) records_ready = true;   // the journal and leaf records fetched with this batch are final
      if (first && complete && fast_score_ok_ && hc.num_leaves > 1) score_done_ = true;   // the device-side update applied itself
      if (complete) break;
      if (enqueued > 4 * NL) Log::Fatal("The device level loop did not finish the tree within %d levels", enqueued);
    }
    levels_hint_ = std::max(1, hc.pad0);
    if (world_ > 1 && DebugFlags::Get().canary) {
      const int broken = fabric_->CheckCanaries(stream_);
      if (broken >= 0) Log::Fatal("FALCATA_DEBUG=canary: the guard behind region %d of the symmetric heap was overwritten during tree %d (rank %d)", broken, tree_index, rank_);
    }
    if (DebugFlags::Get().diag)
      Log::Info("[diag] tree %d: %d leaves, %d journal records, %d levels run on the device, %d enqueued by the host, %lld kernel launches so far", tree_index, hc.num_leaves,
                hc.journal_count, hc.pad0, enqueued, static_cast<long long>(LaunchCounter().load()));
    if (!records_ready) {
      // the tree needed more levels than the first batch: fetch its records now
      journal_.Download(h_journal_.get(), hc.journal_count, stream_);
      leaves_.Download(h_leaves_.get(), hc.num_leaves, stream_);
      FB_CUDA(cudaStreamSynchronize(stream_));
    }
    if (leafwise_ && hc.journal_count > 0) { FinalizeLeafwise(hc, tree.get()); return tree.release(); }
    if (hc.journal_count == 0) { const LeafInfo& R = *h_root_.get(); tree->leaf_value[0] = R.output; tree->leaf_count[0] = R.num_data_global; tree->leaf_weight[0] = R.sum_h; return tree.release(); }
    { const LeafInfo& R = *h_root_.get(); tree->leaf_value[0] = R.output; tree->leaf_count[0] = R.num_data_global; tree->leaf_weight[0] = R.sum_h; }
    for (int j = 0; j < hc.journal_count; ++j) {
      const SplitJournal& sj = h_journal_[j];
      const SplitRecord& b = sj.rec;
      const int right = ApplySplit(tree.get(), train_, sj.leaf, b);
      tree->internal_count[tree->num_leaves - 2] = sj.parent_global;
      if (right != sj.right_leaf) Log::Fatal("Device journal out of order (split %d)", j);
    }
    for (int l = 0; l < tree->num_leaves; ++l) tree->leaf_count[l] = h_leaves_[l].num_data_global;
    return tree.release();
  }
  ReadBackLevel(1);
  {
    const LeafInfo& R = h_leaves_[0];
    HostLeaf& hl = host_leaves_[0];
    hl.begin = 0; hl.count = root_count_; hl.buffer = 0; hl.depth = 0; hl.slot = 0; hl.best = h_best_[0]; hl.valid = true;
    tree->leaf_value[0] = R.output; tree->leaf_count[0] = R.num_data_global; tree->leaf_weight[0] = R.sum_h;
  }
  int next_slot = 1;
  std::vector<int> frontier = {0};
  ha.identity_root = 0;
  // one level: the listed leaves are split by their `best` records in the order given; next_out = the children
  auto apply_level = [&](const std::vector<int>& cand, std::vector<int>* next_out) {
    const int S = static_cast<int>(cand.size());
    PartSplit* ps = reinterpret_cast<PartSplit*>(hb);
    ChildInit* ci = reinterpret_cast<ChildInit*>(hb + sizeof(PartSplit) * S);
    FindChild* fc = reinterpret_cast<FindChild*>(hb + (sizeof(PartSplit) + sizeof(ChildInit)) * S);
    long long total_rows = 0; for (int l : cand) total_rows += host_leaves_[l].count;
    ha.rows_per_block = ChooseRowsPerBlock(total_rows);
    int chunk_cursor = 0, block_cursor = 0;
    std::vector<int>& next = *next_out; next.clear();
    for (int s = 0; s < S; ++s) {
      const int l = cand[s];
      HostLeaf& P = host_leaves_[l];
      const SplitRecord& b = P.best;
      const FeatureMeta& m = train_->feature_meta[b.feature];
      const LeafInfo& PL = h_leaves_[l];
      const int right = ApplySplit(tree.get(), train_, l, b);
      tree->internal_count[tree->num_leaves - 2] = PL.num_data_global;
      PartSplit& q = ps[s];
      memset(&q, 0, sizeof(q));
      q.leaf = l; q.right_leaf = right; q.begin = P.begin; q.count = P.count; q.buffer = P.buffer; q.group = m.group; q.bundled = m.bundled; q.group_offset = m.group_offset;
      q.num_bin = m.num_bin; q.most_freq_bin = m.most_freq_bin; q.threshold = b.threshold; q.default_left = b.default_left; q.missing_type = m.missing_type;
      q.default_bin = m.default_bin; q.is_categorical = b.is_categorical; for (int w = 0; w < 8; ++w) q.cat_bitset[w] = b.cat_bitset[w];
      q.chunk_begin = chunk_cursor; q.num_chunks = (P.count + kPartChunk - 1) / kPartChunk; chunk_cursor += q.num_chunks;
      q.owner = feature_parallel_ ? h_bin_owner_[m.hist_offset] : 0;
      ChildInit& c = ci[s];
      memset(&c, 0, sizeof(c));
      c.smaller_is_left = b.left_cnt <= b.right_cnt ? 1 : 0;
      const int fresh = next_slot++;
      c.left_slot = c.smaller_is_left ? fresh : P.slot; c.right_slot = c.smaller_is_left ? P.slot : fresh;
      c.left_g = b.left_g; c.left_h = b.left_h; c.right_g = b.right_g; c.right_h = b.right_h; c.left_out = b.left_out; c.right_out = b.right_out;
      c.left_gi = b.left_gi; c.left_hi = b.left_hi; c.monotone = b.monotone;
      c.right_gi = PL.sum_gi - b.left_gi; c.right_hi = PL.sum_hi - b.left_hi;
      c.hist_block_begin = block_cursor; c.hist_num_blocks = std::max(1, (P.count + ha.rows_per_block - 1) / ha.rows_per_block); block_cursor += c.hist_num_blocks;
      FindChild& fl = fc[2 * s]; FindChild& fr = fc[2 * s + 1];
      fl.leaf = l; fl.slot = c.left_slot; fl.other_slot = c.right_slot; fl.is_larger = c.smaller_is_left ? 0 : 1; fl.split = s; fl.is_left = 1; fl.parent_global = PL.num_data_global; fl.task = s;
      fr.leaf = right; fr.slot = c.right_slot; fr.other_slot = c.left_slot; fr.is_larger = c.smaller_is_left ? 1 : 0; fr.split = s; fr.is_left = 0; fr.parent_global = PL.num_data_global; fr.task = s;
      host_leaves_[right].slot = c.right_slot; P.slot = c.left_slot;
      next.push_back(l); next.push_back(right);
    }
    const size_t blob_bytes = (sizeof(PartSplit) + sizeof(ChildInit) + 2 * sizeof(FindChild)) * S;
    FB_CUDA(cudaMemcpyAsync(db, hb, blob_bytes, cudaMemcpyHostToDevice, stream_));
    PartArgs pa = PartArgs();
    pa.rows = dd_->rows.get(); pa.row_stride = dd_->row_stride; pa.idx[0] = idx_[0].get(); pa.idx[1] = idx_[1].get();
    pa.cols = dd_->cols.size() ? dd_->cols.get() : nullptr; pa.col_stride = n_;
    pa.splits = reinterpret_cast<const PartSplit*>(db); pa.num_splits = S; pa.total_chunks = chunk_cursor; pa.bits = bits_.get(); pa.chunk_left = chunk_left_.get();
    pa.split_left_total = split_left_total_.get(); pa.leaves = leaves_.get(); pa.child_init = reinterpret_cast<const ChildInit*>(db + sizeof(PartSplit) * S);
    pa.hist_tasks = hist_tasks_.get(); pa.rows_per_block = ha.rows_per_block;
    pa.world = dp ? world_ : 1;
    if (dp) for (int r = 0; r < world_; ++r) pa.peer_counts[r] = fabric_->Ptr<int>(r, off_counts_) + static_cast<size_t>(rank_) * NL;
    if (feature_parallel_) { SetupBitmapBroadcast(&pa); pa.bc_sig.epoch = fabric_->NextEpoch(); pa.bc_wait.epoch = pa.bc_sig.epoch; }
    clock_.Begin(st_part_, stream_);
    LaunchPartitionFlags(pa, stream_); LaunchPartitionScanSetup(pa, stream_); LaunchPartitionScatter(pa, stream_);
    clock_.End(stream_);
    ha.num_tasks = S; ha.total_blocks = std::max(1, block_cursor);
    fa.children = reinterpret_cast<const FindChild*>(db + (sizeof(PartSplit) + sizeof(ChildInit)) * S); fa.num_children = 2 * S;
    construct_and_find();
    ReadBackLevel(tree->num_leaves);
    for (int l : next) {
      const LeafInfo& R = h_leaves_[l];
      HostLeaf& hl = host_leaves_[l];
      hl.begin = R.begin; hl.count = R.count; hl.buffer = R.buffer; hl.depth = R.depth; hl.best = h_best_[l]; hl.valid = true;
      tree->leaf_count[l] = R.num_data_global;
    }
  };
  if (!forced_.empty()) {
    // Forced splits first, breadth first and a level at a time, in the order the host learner's queue visits them (so
    // the leaves get the same numbers); the other leaves wait. A forced split that is not admissible is dropped with
    // its subtree and the leaf keeps the split it found itself.
    std::vector<std::pair<int, int>> queue = {{0, 0}};   // (leaf, forced node)
    while (!queue.empty() && tree->num_leaves < NL) {
      std::vector<int> cand; std::vector<int> node_of;
      for (const auto& e : queue) {
        if (static_cast<int>(cand.size()) >= NL - tree->num_leaves) break;
        const ForcedSplitNode& fn = forced_[e.second];
        if (fn.feature < 0 || fn.feature >= train_->num_total_features) continue;
        const int inner = train_->used_feature_map[fn.feature];
        if (inner < 0 || train_->feature_meta[inner].bin_type != static_cast<int>(BinType::Numerical)) {
          Log::Warning("Forced split on feature %d is ignored (constant or categorical feature)", fn.feature);
          continue;
        }
        const int nb = train_->feature_meta[inner].num_bin;
        const int bin = std::min(static_cast<int>(train_->mappers[fn.feature]->ValueToBin(fn.threshold)), nb - 2);
        SplitRecord r;
        if (!ForcedRecord(e.first, inner, bin, &r) || !(r.gain > 0.0)) {
          Log::Warning("Forced split on feature %d is ignored: it does not improve the leaf", fn.feature);
          continue;
        }
        host_leaves_[e.first].best = r;
        cand.push_back(e.first); node_of.push_back(e.second);
      }
      if (cand.empty()) break;
      std::vector<int> next;
      apply_level(cand, &next);
      queue.clear();
      for (size_t s = 0; s < cand.size(); ++s) {
        const ForcedSplitNode& fn = forced_[node_of[s]];
        if (fn.left >= 0) queue.push_back({next[2 * s], fn.left});
        if (fn.right >= 0) queue.push_back({next[2 * s + 1], fn.right});
      }
    }
    frontier.resize(tree->num_leaves); std::iota(frontier.begin(), frontier.end(), 0);   // everything grows on from here
  }
  while (tree->num_leaves < NL && !frontier.empty()) {
    std::vector<int> cand;
    for (int l : frontier) if (host_leaves_[l].best.feature >= 0 && host_leaves_[l].best.gain > 0.0) cand.push_back(l);
    if (cand.empty()) break;
    const int budget = NL - tree->num_leaves;
    if (static_cast<int>(cand.size()) > budget) {
      std::stable_sort(cand.begin(), cand.end(), [&](int a, int b) {
        if (host_leaves_[a].best.gain != host_leaves_[b].best.gain) return host_leaves_[a].best.gain > host_leaves_[b].best.gain;
        return a < b; });
      cand.resize(budget);
    }
    std::sort(cand.begin(), cand.end());   // a level's splits are always applied in ascending leaf order
    std::vector<int> next;
    apply_level(cand, &next);
    frontier.swap(next);
  }
  return tree.release();
}

// Feature-parallel: the partition's bit words and chunk counts live in the symmetric heap; the owner of a
// split's feature writes them into every rank.
void CudaEngine::SetupBitmapBroadcast(PartArgs* pa) {
  const FabricView v = fabric_->View();
  pa->bc_world = world_; pa->bc_rank = rank_;
  pa->bits = fabric_->Local<unsigned int>(off_bits_); pa->chunk_left = fabric_->Local<int>(off_chunk_left_);
  for (int r = 0; r < world_; ++r) {
    pa->peer_bits[r] = fabric_->Ptr<unsigned int>(r, off_bits_); pa->peer_chunk_left[r] = fabric_->Ptr<int>(r, off_chunk_left_);
    pa->bc_sig.peer_flag[r] = fabric_->Ptr<unsigned int>(r, flag_part_) + rank_;
  }
  pa->bc_sig.world = world_; pa->bc_sig.done_counter = fabric_->done_counter(2);
  pa->bc_wait.world = world_; pa->bc_wait.flags = fabric_->Local<unsigned int>(flag_part_); pa->bc_wait.max_spins = v.max_spins; pa->bc_wait.status = v.status;
}

// K6r: leaf values recomputed from the unquantized gradients of the rows that ended up in each leaf.
// Parity: src/treelearner/cuda/cuda_single_gpu_tree_learner.cu:L20-79 (renew from true gradients), gradient_discretizer.cpp (RenewIntGradTreeOutput).
void CudaEngine::RenewLeavesFromTrueGradients(Tree* tree) {
  const int nl = tree->num_leaves, slices = LeafGradSumSlices();
  if (renew_partial_.size() < static_cast<size_t>(2) * nl * slices) { renew_partial_.Alloc(static_cast<size_t>(2) * cfg_.num_leaves * slices); h_renew_partial_.Alloc(static_cast<size_t>(2) * cfg_.num_leaves * slices); }
  LaunchLeafGradSums(leaves_.get(), nl, idx_[0].get(), idx_[1].get(), cur_grad_, cur_hess_, renew_partial_.get(), stream_);
  renew_partial_.Download(h_renew_partial_.get(), static_cast<size_t>(2) * nl * slices, stream_);
  FB_CUDA(cudaStreamSynchronize(stream_));
  std::vector<double> sums(2 * static_cast<size_t>(nl), 0.0);
  for (int l = 0; l < nl; ++l) for (int s = 0; s < slices; ++s) { sums[2 * l] += h_renew_partial_[2 * (l * slices + s)]; sums[2 * l + 1] += h_renew_partial_[2 * (l * slices + s) + 1]; }
  if (data_parallel()) Network::SumDouble(sums.data(), static_cast<int64_t>(sums.size()));
  for (int l = 0; l < nl; ++l) tree->SetLeafOutput(l, LeafOutputRaw(sums[2 * l], sums[2 * l + 1] + kEpsilon, sp_));
}

// Objectives whose leaf value is a statistic of the residuals (L1: median, quantile: the alpha-quantile): the
// leaf windows and the scores come back to the host and the objective's own renewal runs there.
void DeviceRenewPercentile(const LeafInfo* leaves_dev, const LeafInfo* leaves_host, int num_leaves, const int* idx0, const int* idx1, const float* score,
                           const float* label, int n, double alpha, DevBuf<double>* keys_in, DevBuf<double>* keys_out, DevBuf<int>* offsets, DevBuf<double>* out_dev,
                           DevBuf<char>* temp, double* out_host, cudaStream_t s);

void CudaEngine::RenewLeavesByObjective(Tree* tree, int class_id) {
  const int nl = tree->num_leaves;
  leaves_.Download(h_leaves_.get(), nl, stream_);
  const int kind = obj_->DeviceKind();
  if ((kind == kObjL1 || kind == kObjQuantile) && dd_->weight.size() == 0 && !cfg_.reg_sqrt && getenv("FALCATA_RENEW_ON_HOST") == nullptr) {
    // unweighted L1 / quantile: per-leaf percentile of the residuals by a segmented sort on the device
    FB_CUDA(cudaStreamSynchronize(stream_));   // the leaf records are on the host now
    std::vector<double> outs(nl, 0.0), have(nl, 0.0);
    DeviceRenewPercentile(leaves_.get(), h_leaves_.get(), nl, idx_[0].get(), idx_[1].get(), score_.get() + static_cast<size_t>(class_id) * n_, dd_->label.get(), n_,
                          kind == kObjL1 ? 0.5 : obj_->DeviceParam(0), &renew_in_, &renew_out_, &renew_off_, &renew_res_, &renew_temp_, outs.data(), stream_);
    for (int l = 0; l < nl; ++l) have[l] = h_leaves_[l].count > 0 ? 1.0 : 0.0;
    for (int l = 0; l < nl; ++l) if (have[l] == 0.0) outs[l] = 0.0;
    if (data_parallel()) { Network::SumDouble(outs.data(), nl); Network::SumDouble(have.data(), nl); }   // ranks' statistics are averaged
    for (int l = 0; l < nl; ++l) if (have[l] > 0) tree->SetLeafOutput(l, outs[l] / have[l]);
    return;
  }
  std::vector<int> h_idx0(n_), h_idx1(n_); std::vector<float> h_score(n_);
  FB_CUDA(cudaMemcpyAsync(h_idx0.data(), idx_[0].get(), sizeof(int) * n_, cudaMemcpyDeviceToHost, stream_));
  FB_CUDA(cudaMemcpyAsync(h_idx1.data(), idx_[1].get(), sizeof(int) * n_, cudaMemcpyDeviceToHost, stream_));
  FB_CUDA(cudaMemcpyAsync(h_score.data(), score_.get() + static_cast<size_t>(class_id) * n_, sizeof(float) * n_, cudaMemcpyDeviceToHost, stream_));
  FB_CUDA(cudaStreamSynchronize(stream_));
  std::vector<double> sc(h_score.begin(), h_score.end());
  std::vector<double> outs(nl, 0.0), have(nl, 0.0);
  for (int l = 0; l < nl; ++l) {
    const LeafInfo& L = h_leaves_[l];
    if (L.count <= 0) continue;
    const int* w = (L.buffer ? h_idx1.data() : h_idx0.data()) + L.begin;
    outs[l] = obj_->RenewTreeOutput(tree->leaf_value[l], sc.data(), w, L.count); have[l] = 1.0;
  }
  if (data_parallel()) { Network::SumDouble(outs.data(), nl); Network::SumDouble(have.data(), nl); }   // ranks' statistics are averaged
  for (int l = 0; l < nl; ++l) if (have[l] > 0) tree->SetLeafOutput(l, outs[l] / have[l]);
}

// Gradient-based one-side sampling for this iteration (works on grad_/hess_, which hold this iteration's gradients).
void CudaEngine::DrawGoss(int iter) {
  if (bag_mask_.size() == 0) {
    bag_mask_.Alloc(std::max(1, n_)); bag_idx_.Alloc(std::max(1, n_)); bag_chunk_.Alloc(n_ / 1024 + 2); bag_count_dev_.Alloc(1); h_bag_count_.Alloc(1);
  }
  if (goss_mag_.size() == 0) { goss_mag_.Alloc(std::max(1, n_)); goss_sorted_.Alloc(std::max(1, n_)); goss_temp_.Alloc(GossSortTempBytes(n_) + 16); }
  GossArgs a;
  a.n = n_; a.num_class = K_; a.grad = grad_.get(); a.hess = hess_.get();
  a.top_k = std::max(1, std::min(n_, static_cast<int>(cfg_.top_rate * n_)));
  const int other_k = static_cast<int>(cfg_.other_rate * n_);
  a.prob = n_ > a.top_k ? static_cast<double>(other_k) / static_cast<double>(n_ - a.top_k) : 0.0;
  a.multiply = static_cast<float>(n_ - a.top_k) / static_cast<float>(std::max(1, other_k));
  a.iter = static_cast<uint32_t>(iter); a.seed = static_cast<uint32_t>(cfg_.bagging_seed); a.global_row_offset = static_cast<unsigned long long>(train_->global_row_offset);
  a.mag = goss_mag_.get(); a.sorted = goss_sorted_.get(); a.sort_temp = goss_temp_.get(); a.sort_temp_bytes = goss_temp_.size();
  a.mask = bag_mask_.get(); a.bag_idx = bag_idx_.get(); a.chunk_count = bag_chunk_.get(); a.bag_count = bag_count_dev_.get();
  LaunchGoss(a, stream_);
  bag_count_dev_.Download(h_bag_count_.get(), 1, stream_);
  FB_CUDA(cudaStreamSynchronize(stream_));
  bag_count_ = *h_bag_count_.get();
  int64_t g = bag_count_;
  if (data_parallel()) Network::SumInt64(&g, 1);
  bag_global_ = g;
}

// A new bag: flags by global row id, compaction of the in-bag rows, and the (global) bag size.
void CudaEngine::DrawBag(int round) {
  if (bag_mask_.size() == 0) {
    bag_mask_.Alloc(std::max(1, n_)); bag_idx_.Alloc(std::max(1, n_)); bag_chunk_.Alloc(n_ / 1024 + 2); bag_count_dev_.Alloc(1); h_bag_count_.Alloc(1);
  }
  BagArgs a;
  a.n = n_; a.global_row_offset = static_cast<unsigned long long>(train_->global_row_offset); a.round = static_cast<uint32_t>(round);
  a.seed = static_cast<uint32_t>(bag_seed_);
  a.fraction = cfg_.bagging_fraction; a.pos_fraction = cfg_.pos_bagging_fraction; a.neg_fraction = cfg_.neg_bagging_fraction;
  a.balanced = (cfg_.pos_bagging_fraction < 1.0 || cfg_.neg_bagging_fraction < 1.0) ? 1 : 0;
  a.label = dd_->label.get();
  a.by_query = (cfg_.bagging_by_query && dd_->num_queries > 0) ? 1 : 0;
  a.query_boundaries = dd_->query_boundaries.size() ? dd_->query_boundaries.get() : nullptr; a.num_queries = dd_->num_queries; a.global_query_offset = 0;
  a.mask = bag_mask_.get(); a.bag_idx = bag_idx_.get(); a.chunk_count = bag_chunk_.get(); a.bag_count = bag_count_dev_.get();
  LaunchBagging(a, stream_);
  bag_count_dev_.Download(h_bag_count_.get(), 1, stream_);
  FB_CUDA(cudaStreamSynchronize(stream_));
  bag_count_ = *h_bag_count_.get();
  int64_t g = bag_count_;
  if (data_parallel()) Network::SumInt64(&g, 1);
  bag_global_ = g;
}

void CudaEngine::ReadBackLevel(int num_leaves) {
  clock_.Begin(st_sync_, stream_);
  leaves_.Download(h_leaves_.get(), num_leaves, stream_);
  best_.Download(h_best_.get(), num_leaves, stream_);
  clock_.End(stream_);
  if (world_ > 1) {
    const int st = fabric_->CheckStatus(stream_);   // synchronises the stream
    if (st != 0) Log::Fatal("A cross-rank wait gave up (device status %d): a peer rank did not reach the same step", st);
  } else {
    FB_CUDA(cudaStreamSynchronize(stream_));
  }
}

// Exact leaf-wise tree from an over-grown device tree. The journal lists every split the device applied (in level
// order), h_leaves_ holds the final device leaves. The controller splits every node that best-first growth with the
// leaf budget would split (and some more), so replaying best-first growth on the host over the device's splits
// (largest gain among the current leaves, the order of the host leaf-wise learner) gives the exact tree; nodes the
// device did not split count as unsplittable, which only matters when the growth cap was reached. The device
// leaves tile the rows by position; after their rows are gathered into index buffer 0 a pruned subtree is the
// contiguous range it covered when it was split, and these ranges replace the device leaf records, so the score
// update and the leaf renewal see the final tree.
// Parity: src/treelearner/cuda/cuda_single_gpu_tree_learner.cpp:L2524-3067 (selective grow-then-prune with a host heap simulation).
void CudaEngine::FinalizeLeafwise(const LevelCtrl& hc, Tree* tree) {
  struct Node { int parent = -1, left = -1, right = -1, journal = -1, dev_leaf = 0; bool is_left = true; };
  const int J = hc.journal_count, LD = hc.num_leaves;
  const SplitJournal* jr = h_journal_.get();
  const LeafInfo* dl = h_leaves_.get();
  std::vector<Node> nodes; nodes.reserve(2 * static_cast<size_t>(J) + 1);
  std::vector<int> cur(LD, -1);
  nodes.emplace_back(); cur[0] = 0;
  for (int j = 0; j < J; ++j) {
    const SplitJournal& s = jr[j];
    if (s.leaf >= LD || s.right_leaf >= LD || cur[s.leaf] < 0) Log::Fatal("Device journal is inconsistent (split %d)", j);
    const int v = cur[s.leaf];
    nodes[v].journal = j;
    Node l, r; l.parent = r.parent = v; l.dev_leaf = s.leaf; r.dev_leaf = s.right_leaf; l.is_left = true; r.is_left = false;
    nodes[v].left = static_cast<int>(nodes.size()); nodes.push_back(l); cur[s.leaf] = nodes[v].left;
    nodes[v].right = static_cast<int>(nodes.size()); nodes.push_back(r); cur[s.right_leaf] = nodes[v].right;
  }
  const LeafInfo& R = *h_root_.get();
  tree->leaf_value[0] = R.output; tree->leaf_count[0] = R.num_data_global; tree->leaf_weight[0] = R.sum_h;
  std::vector<int> node_of_leaf(cfg_.num_leaves, -1); node_of_leaf[0] = 0;
  while (tree->num_leaves < cfg_.num_leaves) {
    int best = -1; double best_gain = 0.0;
    for (int t = 0; t < tree->num_leaves; ++t) {
      const Node& n = nodes[node_of_leaf[t]];
      if (n.journal < 0) continue;
      const double g = jr[n.journal].rec.gain;
      if (best < 0 || g > best_gain) { best = t; best_gain = g; }
    }
    if (best < 0) break;
    const Node n = nodes[node_of_leaf[best]];
    const SplitJournal& s = jr[n.journal];
    const int right = ApplySplit(tree, train_, best, s.rec);
    tree->internal_count[tree->num_leaves - 2] = s.parent_global;
    node_of_leaf[best] = n.left; node_of_leaf[right] = n.right;
  }
  // every device leaf's rows into index buffer 0 (the device still holds the device-leaf records here), so that a
  // pruned subtree's rows are the contiguous range its leaves cover
  LaunchCollapseLeafWindows(leaves_.get(), LD, idx_[0].get(), idx_[1].get(), stream_);
  // leaf records of the final tree
  std::vector<LeafInfo> fin(tree->num_leaves);
  for (int t = 0; t < tree->num_leaves; ++t) {
    const Node& n = nodes[node_of_leaf[t]];
    LeafInfo L;
    if (n.journal < 0) L = dl[n.dev_leaf];
    else {
      // split on the device, pruned here: the window and totals the node had when it was split
      const SplitJournal& s = jr[n.journal];
      L = dl[n.dev_leaf];
      L.begin = s.begin; L.count = s.count; L.buffer = s.buffer; L.depth = s.depth; L.num_data_global = s.parent_global;
      L.sum_g = FB_ADD(s.rec.left_g, s.rec.right_g); L.sum_h = FB_ADD(s.rec.left_h, s.rec.right_h);
      const SplitJournal& ps = jr[nodes[n.parent].journal];
      L.output = n.is_left ? ps.rec.left_out : ps.rec.right_out;
      if (n.is_left) { L.sum_gi = ps.rec.left_gi; L.sum_hi = ps.rec.left_hi; }
    }
    L.buffer = 0;
    fin[t] = L;
    tree->leaf_count[t] = L.num_data_global;
  }
  for (int t = 0; t < tree->num_leaves; ++t) h_leaves_.get()[t] = fin[t];
  FB_CUDA(cudaMemcpyAsync(leaves_.get(), h_leaves_.get(), sizeof(LeafInfo) * tree->num_leaves, cudaMemcpyHostToDevice, stream_));
}

}  // namespace fb
