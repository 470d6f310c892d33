// Device engine: construction, buffers, score bookkeeping, validation sets, metrics.
#include "engine.h"

#include <nvtx3/nvToolsExt.h>

#include <exception>
#include <sstream>
#include <thread>

namespace fb {

// ------------------------------------------------------------ StageClock ----
StageClock::~StageClock() { for (auto& p : pool) { cudaEventDestroy(p.first); cudaEventDestroy(p.second); } }
int StageClock::Stage(const char* name) { names.push_back(name); total_ms.push_back(0.0); calls.push_back(0); return static_cast<int>(names.size()) - 1; }
void StageClock::Begin(int stage, cudaStream_t s) {
  if (nvtx) { nvtxRangePushA(names[stage].c_str()); nvtx_open = true; }   // host-side range around the stage's launches (FALCATA_NVTX=1)
  if (!enabled) return;
  if (next >= pool.size()) { cudaEvent_t a, b; FB_CUDA(cudaEventCreate(&a)); FB_CUDA(cudaEventCreate(&b)); pool.emplace_back(a, b); }
  FB_CUDA(cudaEventRecord(pool[next].first, s));
  pending.emplace_back(stage, static_cast<int>(next));
  open_ = static_cast<int>(next); ++next;
}
void StageClock::End(cudaStream_t s) { if (nvtx_open) { nvtxRangePop(); nvtx_open = false; } if (!enabled || open_ < 0) return; FB_CUDA(cudaEventRecord(pool[open_].second, s)); open_ = -1; }
void StageClock::Resolve() {
  if (!enabled) return;
  static const bool dump = getenv("FALCATA_STAGE_DUMP") != nullptr;
  for (auto& pr : pending) {
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, pool[pr.second].first, pool[pr.second].second) == cudaSuccess) { total_ms[pr.first] += ms; calls[pr.first] += 1; if (dump) fprintf(stderr, "[stage] %s %.1f us\n", names[pr.first].c_str(), ms * 1000.f); }
  }
  pending.clear(); next = 0;
}
std::string StageClock::Report() const {
  std::ostringstream os;
  for (size_t i = 0; i < names.size(); ++i) os << names[i] << ": " << total_ms[i] << " ms in " << calls[i] << " spans\n";
  return os.str();
}

// --------------------------------------------------------------- engine ----
DeviceEngine* CreateDeviceEngine(const Config& cfg, const Dataset* train, const ObjectiveFunction* obj, int num_tree_per_iter) {
  return new CudaEngine(cfg, train, obj, num_tree_per_iter);
}

CudaEngine::CudaEngine(const Config& cfg, const Dataset* train, const ObjectiveFunction* obj, int K)
    : cfg_(cfg), plan_(Plan::FromString(cfg.cuda_plan)), train_(train), obj_(obj), K_(K) {
  if (!CudaAvailable()) Log::Fatal("device_type=cuda needs a CUDA device");
  // single attributes: the full property query reads every field of the device and takes milliseconds
  int dev = 0, cc_major = 0, cc_minor = 0; FB_CUDA(cudaGetDevice(&dev));
  FB_CUDA(cudaDeviceGetAttribute(&cc_major, cudaDevAttrComputeCapabilityMajor, dev)); FB_CUDA(cudaDeviceGetAttribute(&cc_minor, cudaDevAttrComputeCapabilityMinor, dev));
  FB_CUDA(cudaDeviceGetAttribute(&num_sms_, cudaDevAttrMultiProcessorCount, dev));
  if (cc_major < 10) Log::Warning("This build targets sm_100a; device %d is compute %d.%d", dev, cc_major, cc_minor);
  if (Fabric::Get().active() && cfg.tree_learner != "serial") {
    if (cfg.tree_learner != "data" && cfg.tree_learner != "feature" && cfg.tree_learner != "voting") Log::Fatal("Unknown tree_learner %s", cfg.tree_learner.c_str());
    voting_ = cfg.tree_learner == "voting";
    fabric_ = &Fabric::Get(); world_ = fabric_->world(); rank_ = fabric_->rank();
    feature_parallel_ = cfg.tree_learner == "feature";   // every rank holds all rows; features are split between the ranks
    if (!Network::active()) Log::Fatal("Multi-GPU training needs the host collectives as well (falcata_b200.parallel.init())");
  } else if (Network::active() && cfg.tree_learner != "serial") {
    Log::Fatal("Multi-GPU training needs the device fabric (call falcata_b200.parallel.init() before creating the Booster)");
  }
  { ScopedTimer t("Engine::EnsureDeviceDataset"); EnsureDeviceDataset(const_cast<Dataset*>(train)); }
  dd_ = train->device; n_ = train->num_data;
  FB_CUDA(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking));
  // labels, weights and query boundaries go up on a helper thread (a copy from pageable memory keeps its caller busy
  // for the whole transfer) while this thread allocates and clears the training state; joined before the first use
  cudaStream_t meta_stream = nullptr; FB_CUDA(cudaStreamCreateWithFlags(&meta_stream, cudaStreamNonBlocking));
  std::exception_ptr meta_error;
  std::thread meta_upload([&, dev]() {
    try { FB_CUDA(cudaSetDevice(dev)); ScopedTimer t("Engine::SyncDeviceMetadata"); SyncDeviceMetadata(train, meta_stream); }
    catch (...) { meta_error = std::current_exception(); }
  });
  struct JoinMeta { std::thread& t; ~JoinMeta() { if (t.joinable()) t.join(); } } join_meta{meta_upload};
  ScopedTimer t_rest("Engine::AllocAndSetup");
  quant_ = cfg.quant != QuantMode::None;
  sp_.lambda_l1 = cfg.lambda_l1; sp_.lambda_l2 = cfg.lambda_l2; sp_.max_delta_step = cfg.max_delta_step; sp_.path_smooth = cfg.path_smooth;
  sp_.min_sum_hessian_in_leaf = cfg.min_sum_hessian_in_leaf; sp_.min_gain_to_split = cfg.min_gain_to_split; sp_.min_data_in_leaf = cfg.min_data_in_leaf;
  sp_.max_depth = cfg.max_depth; sp_.max_cat_threshold = cfg.max_cat_threshold; sp_.max_cat_to_onehot = cfg.max_cat_to_onehot;
  sp_.min_data_per_group = cfg.min_data_per_group; sp_.cat_l2 = cfg.cat_l2; sp_.cat_smooth = cfg.cat_smooth; sp_.extra_trees = cfg.extra_trees ? 1 : 0;
  sp_.cegb_split = cfg.cegb_tradeoff * cfg.cegb_penalty_split;
  sp_.monotone_penalty = cfg.monotone_penalty;
  sp_.use_mc = 0; for (const auto& m : train->feature_meta) if (m.monotone != 0) sp_.use_mc = 1;
  col_sampler_.Init(cfg, train);
  clock_.enabled = getenv("FALCATA_STAGE_TIMING") != nullptr;
  clock_.nvtx = getenv("FALCATA_NVTX") != nullptr;
  st_grad_ = clock_.Stage("gradients"); st_quant_ = clock_.Stage("quantize+root"); st_hist_ = clock_.Stage("histogram");
  st_find_ = clock_.Stage("find-split"); st_part_ = clock_.Stage("partition"); st_score_ = clock_.Stage("score-update"); st_sync_ = clock_.Stage("level-readback");

  // objective descriptor
  objd_.kind = obj ? obj->DeviceKind() : kObjCustom; objd_.num_class = cfg.num_class; objd_.p0 = objd_.p1 = objd_.p2 = 0; objd_.max_docs = 0;
  if (obj != nullptr) {
    if (objd_.kind < 0) {
      // no gradient kernel for this objective: the scores go to the host every round, the objective's own code
      // computes the gradients there and they come back for the device learner
      Log::Warning("Objective %s has no device gradient kernel: gradients are computed on the host every round", obj->GetName());
      host_gradients_ = true;
    }
    if (objd_.kind >= 0 && getenv("FALCATA_HOST_GRADIENTS") != nullptr) host_gradients_ = true;   // A/B switch: the objective's host code instead of the gradient kernel
    objd_.p0 = obj->DeviceParam(0); objd_.p1 = obj->DeviceParam(1); objd_.p2 = obj->DeviceParam(2);
    if (objd_.kind == kObjLambdarank) {
      const auto& qb = train->metadata.query_boundaries;
      for (size_t q = 0; q + 1 < qb.size(); ++q) max_docs_ = std::max(max_docs_, qb[q + 1] - qb[q]);
      objd_.max_docs = max_docs_;
      label_gain_.Upload(cfg.label_gain_vec, stream_);
    }
  }
  const size_t total = static_cast<size_t>(n_) * K_;
  score_.Alloc(total); score_.Zero(stream_);
  if (!train->metadata.init_score.empty()) {
    std::vector<float> f(train->metadata.init_score.begin(), train->metadata.init_score.end());
    if (f.size() != total) Log::Fatal("init_score size does not match num_data * num_class");
    score_.Upload(f, stream_);
  }
  grad_.Alloc(total); hess_.Alloc(total); maxbuf_.Alloc(2 * K_); scales_.Alloc(2); root_sums_i_.Alloc(2); root_sums_d_.Alloc(2);
  partial_.Alloc(2 * (static_cast<size_t>(n_) / 256 + 2));
  if (quant_) {
    ResolveQuantBins();
    if (plan_.gh_in_row && K_ == 1) { gh_base_ = dd_->rows.get() + dd_->gh_offset; gh_stride_ = dd_->row_stride; }
    else { gh_sep_.Alloc(n_); gh_base_ = reinterpret_cast<const uint8_t*>(gh_sep_.get()); gh_stride_ = 4; }
    hist_elem_ = sizeof(hist_q_t);
  } else {
    gh2_.Alloc(n_); gh_base_ = reinterpret_cast<const uint8_t*>(gh2_.get()); gh_stride_ = 8; hist_elem_ = sizeof(double2);
  }
  {
    const int qb = std::max(2, cfg_.quant_bins_resolved);
    sub_rows_ = quant_ ? std::max(1, std::min(65535 / qb, 32767 / std::max(1, qb / 2))) : (1 << 30);
    lane_mode_ = 0; lane_bins_ = 64;
    // lane construct: 16-, 64- or 256-bin tiles; beyond 64 bins (and for fp32 gradients) only in the reduction form,
    // whose tiles are shared by several warps
    lane_red_ = quant_ ? plan_.hist_lane_red : plan_.hist_float_red;
    if ((plan_.hist_lane || plan_.hist_lane_atomic) && train->max_group_bin <= 256 && (!quant_ || train->max_group_bin <= 64 || lane_red_)) {
      lane_mode_ = plan_.hist_lane_atomic ? 2 : 1;
      lane_bins_ = train->max_group_bin <= 16 ? 16 : (train->max_group_bin <= 64 ? 64 : 256);
    }
    if (plan_.col_major_part) EnsureColumnMajor(dd_, stream_);
  }
  idx_[0].Alloc(n_); idx_[1].Alloc(n_);
  forced_ = LoadForcedSplitsFile(cfg.forcedsplits_filename);
  if (!forced_.empty() && world_ > 1) Log::Fatal("Forced splits on the device are single-GPU (a multi-GPU booster trains them on the host learner)");
  leafwise_ = cfg.grow_policy == "leaf" && plan_.device_controller && cfg.num_leaves <= 512 && !voting_ && forced_.empty();
  if (cfg.grow_policy == "leaf" && !leafwise_)
    Log::Warning("grow_policy=leaf on the device needs the level controller, num_leaves <= 512 and tree_learner serial, data or feature; growing level-wise with a gain-ranked leaf budget");
  // leaf-wise: the device may grow past the budget (nodes that looked good enough when they were split); the cap bounds every buffer
  grow_leaves_ = leafwise_ ? std::min(1024, 4 * cfg.num_leaves) : cfg.num_leaves;
  const int NL = grow_leaves_;
  if (leafwise_) eval_key_.Alloc(4 * (2 * static_cast<size_t>(NL) + 2));
  leaves_.Alloc(NL); best_.Alloc(NL); h_leaves_.Alloc(NL); h_best_.Alloc(NL); leaf_value_.Alloc(NL);
  host_leaves_.resize(NL);
  use_ctrl_ = plan_.device_controller && NL <= 1024;
  if (!forced_.empty()) use_ctrl_ = false;   // forced splits: the host decides every level
  if (use_ctrl_) {
    ctrl_.Alloc(2); frontier_.Alloc(NL + 2); journal_.Alloc(NL); h_ctrl_.Alloc(1); h_journal_.Alloc(NL); h_root_.Alloc(1);
    levels_hint_ = 1; while ((1 << levels_hint_) < NL) ++levels_hint_;
  }
  node_mask_on_ = col_sampler_.by_node();
  if (node_mask_on_) {
    if (!use_ctrl_) Log::Fatal("feature_fraction_bynode / interaction_constraints on the device need the device level controller (num_leaves <= 1024)");
    if (cfg.tree_learner == "voting" && world_ > 1) Log::Fatal("feature_fraction_bynode / interaction_constraints are not built for the device voting learner");
    node_mask_.Alloc(static_cast<size_t>(2 * (NL / 2 + 1)) * std::max(1, train->num_features));
    const auto& sets = col_sampler_.interaction_sets();
    num_sets_ = static_cast<int>(sets.size());
    if (num_sets_ > 0) {
      path_words_ = (train->num_total_features + 31) / 32;
      std::vector<unsigned int> bits(static_cast<size_t>(num_sets_) * path_words_, 0u);
      for (int s = 0; s < num_sets_; ++s) for (int rf : sets[s]) if (rf >= 0 && rf < train->num_total_features) bits[static_cast<size_t>(s) * path_words_ + (rf >> 5)] |= 1u << (rf & 31);
      set_bits_.Upload(bits, stream_);
      path_bits_.Alloc(static_cast<size_t>(NL) * path_words_);
    }
  }
  BuildPartitions();
  SetupOwnership();
  if (feature_parallel_) {
    // histograms stay local (own features only); the heap carries the best-split slots and the partition bitmap
    fabric_->Reset();
    off_best_ = fabric_->Alloc(static_cast<size_t>(world_) * NL * sizeof(SplitRecord));
    const size_t max_chunks_fp = static_cast<size_t>(n_) / kPartChunk + NL + 1;
    off_bits_ = fabric_->Alloc(max_chunks_fp * (kPartChunk / 32) * sizeof(unsigned int));
    off_chunk_left_ = fabric_->Alloc(max_chunks_fp * sizeof(int));
    flag_best_ = fabric_->NewFlagSlot(); flag_part_ = fabric_->NewFlagSlot();
    pool_bytes_ = static_cast<size_t>(NL) * slot_stride_ * hist_elem_;
    pool_.Alloc(pool_bytes_);
    pool_base_ = pool_.get();
  } else if (voting_) {
    // local pool with all features (identity bin map); the heap carries vote slots, the staging slots of the
    // voted features, the row counts and the best-split slots
    long long max_stride = 0; for (int r = 0; r < world_; ++r) max_stride = std::max(max_stride, slot_strides_[r]);
    fabric_->Reset();
    off_stage_ = fabric_->Alloc(static_cast<size_t>(world_) * NL * max_stride * hist_elem_);
    off_counts_ = fabric_->Alloc(static_cast<size_t>(world_) * NL * sizeof(int));
    off_best_ = fabric_->Alloc(static_cast<size_t>(world_) * NL * sizeof(SplitRecord));
    off_votes_ = fabric_->Alloc(static_cast<size_t>(world_) * NL * std::max(1, cfg.top_k) * sizeof(int));
    flag_hist_ = fabric_->NewFlagSlot(); flag_best_ = fabric_->NewFlagSlot(); flag_vote_ = fabric_->NewFlagSlot();
    pool_bytes_ = static_cast<size_t>(NL) * train->num_total_bin * hist_elem_;
    pool_.Alloc(pool_bytes_); pool_base_ = pool_.get();
    std::vector<int> ident(train->num_total_bin); for (int b = 0; b < train->num_total_bin; ++b) ident[b] = b;
    bin_identity_.Upload(ident, stream_);
    const size_t F = std::max(1, train->num_features);
    cand_local_.Alloc(static_cast<size_t>(NL) * F); cand_local_.Zero(stream_); vote_sums_.Alloc(NL); voted_.Alloc(static_cast<size_t>(NL) * F);
    features_all_.Alloc(F); sub_features_all_.Alloc(F);
    global_max_.Alloc(2 * K_);
  } else if (world_ > 1) {
    // same carving order on every rank: offsets name the same object everywhere
    long long max_stride = 0; for (int r = 0; r < world_; ++r) max_stride = std::max(max_stride, slot_strides_[r]);
    fabric_->Reset();
    pool_bytes_ = static_cast<size_t>(NL) * max_stride * hist_elem_;
    off_pool_ = fabric_->Alloc(pool_bytes_);
    off_stage_ = fabric_->Alloc(static_cast<size_t>(world_) * NL * max_stride * hist_elem_);
    stage_local_.Alloc(static_cast<size_t>(NL) * train->num_total_bin * hist_elem_); stage_local_.Zero(stream_);
    task_done_.Alloc(NL); task_done_.Zero(stream_);
    off_counts_ = fabric_->Alloc(static_cast<size_t>(world_) * NL * sizeof(int));
    off_best_ = fabric_->Alloc(static_cast<size_t>(world_) * NL * sizeof(SplitRecord));
    flag_hist_ = fabric_->NewFlagSlot(); flag_best_ = fabric_->NewFlagSlot();
    pool_base_ = fabric_->Local<char>(off_pool_);
    global_max_.Alloc(2 * K_);
  } else {
    pool_bytes_ = static_cast<size_t>(NL) * slot_stride_ * hist_elem_;
    pool_.Alloc(pool_bytes_);
    pool_base_ = pool_.get();
  }
  cand_.Alloc(static_cast<size_t>(NL) * std::max<size_t>(1, owned_features_.size())); cand_.Zero(stream_);
  root_child_.Alloc(1); child_done_.Alloc(2 * static_cast<size_t>(NL) + 2); child_done_.Zero(stream_); level_done_.Alloc(1); level_done_.Zero(stream_);
  split_done_.Alloc(NL + 1); split_done_.Zero(stream_);
  hist_tasks_.Alloc(NL); hist_status_.Alloc(1); hist_status_.Zero(stream_); h_hist_status_.Alloc(1); *h_hist_status_.get() = 0;
  const size_t max_chunks = static_cast<size_t>(n_) / kPartChunk + NL + 1;
  bits_.Alloc(max_chunks * (kPartChunk / 32)); chunk_left_.Alloc(max_chunks); split_left_total_.Alloc(NL);
  const size_t blob = static_cast<size_t>(NL) * (sizeof(PartSplit) + sizeof(ChildInit) + 2 * sizeof(FindChild)) + 256;
  level_blob_.Alloc(blob); h_level_blob_.Alloc(blob);
  features_.Alloc(std::max(1, train->num_features)); sub_features_.Alloc(std::max(1, train->num_features));
  FB_CUDA(cudaStreamSynchronize(stream_));
  meta_upload.join();
  cudaStreamDestroy(meta_stream);
  if (meta_error) std::rethrow_exception(meta_error);
  Log::Info("CUDA engine: %d rows x %d groups (%d bins, %d partitions), row stride %d B, %s histograms, plan: %s", n_, dd_->num_groups,
            train->num_total_bin, static_cast<int>(h_parts_.size()), dd_->row_stride, quant_ ? "integer" : "fp64", plan_.ToString().c_str());
  if (DebugFlags::Get().diag)
    Log::Info("[diag] construct: lane mode %d (%d-bin tiles, %s adds), %d rows per block at %d rows, quant_bins %d, sub-rows %d, %d SMs; growth %s, %d trees per round, ranks %d",
              lane_mode_, lane_bins_, lane_red_ ? "reduction" : "load-add-store", ChooseRowsPerBlock(n_), n_, cfg_.quant_bins_resolved, sub_rows_, num_sms_,
              leafwise_ ? "leaf-wise (over-grow + best-first replay)" : "level", K_, world_);
}

// The record of splitting `leaf` on (inner_feature, bin): what the search kernel reports for that one candidate (both
// missing-value directions where the feature has them; the better one wins), evaluated on the host from the leaf's
// histogram in the pool. False when the split is not admissible (a child too small, no gain above the leaf's own).
bool CudaEngine::ForcedRecord(int leaf, int f, int t, SplitRecord* out) {
  const FeatureMeta& m = train_->feature_meta[f];
  const int nb = m.num_bin, nstored = m.bundled ? nb - 1 : nb;
  if (m.bin_type != static_cast<int>(BinType::Numerical) || nb < 2 || t < 0 || t > nb - 2) return false;
  const LeafInfo& PL = h_leaves_[leaf];
  const size_t esz = quant_ ? sizeof(hist_q_t) : sizeof(double2);
  const char* src = pool_base_ + (static_cast<long long>(host_leaves_[leaf].slot) * slot_stride_ + m.hist_offset) * esz;
  std::vector<char> raw(static_cast<size_t>(nstored) * esz);
  FB_CUDA(cudaMemcpyAsync(raw.data(), src, raw.size(), cudaMemcpyDeviceToHost, stream_));
  float sc[2] = {1.f, 1.f};
  if (quant_) FB_CUDA(cudaMemcpyAsync(sc, scales_.get(), sizeof(sc), cudaMemcpyDeviceToHost, stream_));
  FB_CUDA(cudaStreamSynchronize(stream_));
  std::vector<long long> gi(nb, 0), hi(nb, 0); std::vector<double> gd(nb, 0.0), hd(nb, 0.0);
  long long sgi = 0, shi = 0; double sgd = 0, shd = 0;
  for (int b = 0; b < nb; ++b) {
    if (m.bundled && b == m.most_freq_bin) continue;
    const int j = (m.bundled && b > m.most_freq_bin) ? b - 1 : b;
    if (quant_) { const hist_q_t v = reinterpret_cast<const hist_q_t*>(raw.data())[j]; gi[b] = HistQGrad(v); hi[b] = HistQHess(v); sgi += gi[b]; shi += hi[b]; }
    else { const double2 v = reinterpret_cast<const double2*>(raw.data())[j]; gd[b] = v.x; hd[b] = v.y; sgd += v.x; shd += v.y; }
  }
  if (m.bundled) { const int q = m.most_freq_bin; gi[q] = PL.sum_gi - sgi; hi[q] = PL.sum_hi - shi; gd[q] = PL.sum_g - sgd; hd[q] = PL.sum_h - shd; }
  LeafScanInfo L;
  L.sum_g = PL.sum_g; L.sum_h = PL.sum_h; L.sum_gi = PL.sum_gi; L.sum_hi = PL.sum_hi; L.num_data = PL.num_data_global;
  L.parent_output = PL.output; L.g_scale = quant_ ? static_cast<double>(sc[0]) : 1.0; L.h_scale = quant_ ? static_cast<double>(sc[1]) : 1.0; L.min_c = PL.min_c; L.max_c = PL.max_c;
  L.mono_factor = MonotonePenaltyFactor(PL.depth, sp_.monotone_penalty);
  L.cnt_factor = FB_DIV(static_cast<double>(L.num_data), L.sum_h);
  if (sp_.max_delta_step <= 0.0 && sp_.path_smooth <= 0.0) L.min_gain_shift = FB_ADD(LeafGain(L.sum_g, FB_ADD(L.sum_h, 2 * kEpsilon), sp_, L.num_data, PL.output), sp_.min_gain_to_split);
  else L.min_gain_shift = FB_ADD(LeafGainGivenOutput(L.sum_g, FB_ADD(L.sum_h, 2 * kEpsilon), sp_, PL.output), sp_.min_gain_to_split);
  const bool two_pass = m.missing_type != 0 && nb > 2;
  const int skip = two_pass ? (m.missing_type == 1 ? m.default_bin : nb - 1) : -1;
  auto bin_h = [&](int b) { return quant_ ? FB_MUL(static_cast<double>(hi[b]), L.h_scale) : hd[b]; };
  long long Mgi = 0, Mhi = 0; double Mgd = 0, Mhd = 0; int Mc = 0;
  if (skip >= 0) { Mgi = gi[skip]; Mhi = hi[skip]; Mgd = gd[skip]; Mhd = hd[skip]; Mc = BinCountEstimate(bin_h(skip), L.cnt_factor); }
  long long pgi = 0, phi = 0; double pgd = 0, phd = 0; int pc = 0;
  for (int b = 0; b <= t; ++b) if (b != skip) { pgi += gi[b]; phi += hi[b]; pgd += gd[b]; phd += hd[b]; pc += BinCountEstimate(bin_h(b), L.cnt_factor); }
  double best_gain = -std::numeric_limits<double>::infinity(); int best_rank = 1 << 30, best_pass = 0, best_lc = 0;
  long long best_lgi = 0, best_lhi = 0; double best_lg = 0, best_lh = 0;
  for (int pass = 0; pass < (two_pass ? 2 : 1); ++pass) {
    if (t == skip && pass == 1 && m.missing_type == 1) continue;
    long long lgi = pgi, lhi = phi; int lc = pc; double lg, lh;
    const bool addm = pass == 0 && skip >= 0;
    if (addm) { lgi += Mgi; lhi += Mhi; lc += Mc; }
    if (quant_) { lg = FB_MUL(static_cast<double>(lgi), L.g_scale); lh = FB_MUL(static_cast<double>(lhi), L.h_scale); }
    else { lg = pgd + (addm ? Mgd : 0.0); lh = phd + (addm ? Mhd : 0.0); }
    double lo, ro;
    const double gain = EvalCandidate(lg, lh, lc, L, sp_, m.monotone, &lo, &ro);
    if (gain == -std::numeric_limits<double>::infinity()) continue;
    const int rank = ScanRank(pass, t, nb);
    if (gain > best_gain || (gain == best_gain && rank < best_rank)) { best_gain = gain; best_rank = rank; best_pass = pass; best_lc = lc; best_lgi = lgi; best_lhi = lhi; best_lg = lg; best_lh = lh; }
  }
  if (best_gain == -std::numeric_limits<double>::infinity()) return false;
  if (sp_.max_depth > 0 && PL.depth >= sp_.max_depth) return false;
  if (PL.num_data_global < 2 * sp_.min_data_in_leaf) return false;
  SplitRecord r; InitSplitRecord(&r);
  r.gain = FB_MUL(best_gain, static_cast<double>(m.penalty)); r.feature = f; r.threshold = t; r.default_left = best_pass == 0 ? 1 : 0;
  if (sp_.cegb_split > 0.0) r.gain -= sp_.cegb_split * static_cast<double>(PL.num_data_global);
  r.left_g = best_lg; r.left_h = best_lh; r.right_g = FB_SUB(PL.sum_g, best_lg); r.right_h = FB_SUB(PL.sum_h, best_lh);
  r.left_gi = best_lgi; r.left_hi = best_lhi; r.left_cnt = best_lc; r.right_cnt = PL.num_data_global - best_lc; r.monotone = m.monotone;
  r.left_out = LeafOutput(r.left_g, FB_ADD(r.left_h, kEpsilon), sp_, r.left_cnt, PL.output);
  r.right_out = LeafOutput(r.right_g, FB_ADD(r.right_h, kEpsilon), sp_, r.right_cnt, PL.output);
  if (sp_.use_mc != 0) { r.left_out = ClampOutput(r.left_out, PL.min_c, PL.max_c); r.right_out = ClampOutput(r.right_out, PL.min_c, PL.max_c); }
  *out = r;
  return true;
}

CudaEngine::~CudaEngine() { if (stream_) cudaStreamDestroy(stream_); }

// Feature partitions of the construct kernel: runs of groups, starting on a 4-group boundary (the
// kernel loads 4 group bytes per item), whose bins fit the shared-memory tile.
void CudaEngine::BuildPartitions() {
  const int kMaxBins = 6144;
  h_parts_.clear();
  const int G = train_->num_groups;
  int g = 0;
  while (g < G) {
    HistPartition p; p.group_begin = g; p.bin_begin = train_->group_bin_start[g]; p.bin_count = 0;
    int e = g;
    while (e < G) {
      int e4 = std::min(G, e + 4); int add = 0;
      for (int k = e; k < e4; ++k) add += train_->group_num_bin[k];
      if (p.bin_count + add > kMaxBins && e > g) break;
      p.bin_count += add; e = e4;
    }
    p.group_end = e; h_parts_.push_back(p); g = e;
  }
  max_part_bins_ = 0; for (auto& p : h_parts_) max_part_bins_ = std::max(max_part_bins_, p.bin_count);
  parts_.Upload(h_parts_, stream_);
}

// Which rank owns which histogram bins. One rank: identity. (The multi-rank map is installed by the fabric.)
void CudaEngine::SetupOwnership() {
  const int nb = train_->num_total_bin;
  std::vector<unsigned char> owner(nb, 0); std::vector<int> local(nb);
  owned_features_.clear();
  if (world_ <= 1) {
    for (int b = 0; b < nb; ++b) local[b] = b;
    slot_stride_ = nb; slot_strides_[0] = nb;
    for (int f = 0; f < train_->num_features; ++f) owned_features_.push_back(f);
  } else {
    // feature groups go to ranks greedily by bin count (largest first, least-loaded rank, ties to the
    // lower rank): the same deterministic map on every rank. A group is never split between ranks.
    const int G = train_->num_groups;
    std::vector<int> order(G); for (int g = 0; g < G; ++g) order[g] = g;
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return train_->group_num_bin[a] > train_->group_num_bin[b]; });
    std::vector<long long> load(world_, 0); std::vector<int> gowner(G, 0);
    for (int g : order) { int best = 0; for (int r = 1; r < world_; ++r) if (load[r] < load[best]) best = r; gowner[g] = best; load[best] += train_->group_num_bin[g]; }
    std::vector<int> cursor(world_, 0);
    for (int g = 0; g < G; ++g) {
      const int r = gowner[g], s = train_->group_bin_start[g];
      for (int b = 0; b < train_->group_num_bin[g]; ++b) { owner[s + b] = static_cast<unsigned char>(r); local[s + b] = cursor[r] + b; }
      cursor[r] += train_->group_num_bin[g];
    }
    for (int r = 0; r < world_; ++r) slot_strides_[r] = std::max(1, cursor[r]);
    slot_stride_ = slot_strides_[rank_];
    for (int f = 0; f < train_->num_features; ++f) if (gowner[train_->feature_meta[f].group] == rank_) owned_features_.push_back(f);
  }
  bin_owner_.Upload(owner, stream_); bin_local_.Upload(local, stream_);
  h_bin_owner_ = owner;
}

// Gradient levels actually used. The global histograms keep 32-bit halves per bin, so rows x levels must stay below
// 2^31 over ALL ranks' rows; a default count that breaks this is lowered, an explicit one is refused. A default
// stochastic count (4) is raised where leaves get small on large data, where 4 levels fit rounding noise: to 64 with a
// constant hessian, else 16; not for multiclass and not for binary labels beyond 50:1, where rare large gradients pin the
// scale. Every rank takes the same decision (global row count, label counts summed over the ranks).
// Parity: src/treelearner/cuda/cuda_single_gpu_tree_learner.cpp:L93-193.
void CudaEngine::ResolveQuantBins() {
  int qb = cfg_.quant_bins_resolved;
  const unsigned long long rows = static_cast<unsigned long long>(std::max<long long>(1, train_->global_num_data));
  if (rows * static_cast<unsigned long long>(qb) >= (1ULL << 31)) {
    const int max_bins = static_cast<int>((1ULL << 31) / rows) - 1;
    if (cfg_.quant_bins_from_auto && max_bins >= 2) {
      Log::Warning("The default quant_bins=%d exceeds the 32-bit histogram range for %llu rows; using quant_bins=%d (set quant_bins to override)", qb, rows, max_bins);
      qb = max_bins;
    } else {
      Log::Fatal("quant_bins=%d is too large for %llu rows: a bin's sum can exceed the 32-bit histogram range. Use quant_bins <= %d for this data set", qb, rows, std::max(0, max_bins));
    }
  }
  if (cfg_.quant == QuantMode::Stochastic && cfg_.quant_bins_from_auto) {
    const long long depth_cap = (cfg_.max_depth > 0 && cfg_.max_depth < 31) ? (1LL << cfg_.max_depth) : std::numeric_limits<long long>::max();
    const long long leaves = std::min<long long>(cfg_.num_leaves, depth_cap);
    const long long rows_per_leaf = static_cast<long long>(rows) / std::max<long long>(1, leaves);
    bool extreme = false;
    if (cfg_.objective == "binary") {
      double cnt[2] = {0.0, static_cast<double>(train_->metadata.label.size())};
      for (float y : train_->metadata.label) cnt[0] += y > 0 ? 1.0 : 0.0;
      if (world_ > 1 && !feature_parallel_) Network::SumDouble(cnt, 2);
      const double minority = std::min(cnt[0], cnt[1] - cnt[0]);
      extreme = minority <= 0.0 || (cnt[1] - minority) >= 50.0 * minority;
    }
    if (rows >= 100000ULL && rows_per_leaf < 4096 && !extreme && K_ == 1) {
      const int target = (obj_ != nullptr && obj_->IsConstantHessian()) ? 64 : 16;
      const int raised = static_cast<int>(std::min<unsigned long long>(target, (1ULL << 31) / rows - 1));
      if (raised > qb) {
        Log::Info("Stochastic quant_bins raised from the default %d to %d: about %lld rows per leaf is too few for %d levels (set quant_bins to override)", qb, raised, rows_per_leaf, qb);
        qb = raised;
      }
    }
  }
  cfg_.quant_bins_resolved = qb;
}

int CudaEngine::ChooseRowsPerBlock(long long total_rows) const {
  if (lane_mode_ != 0) {
    // the lane kernel runs one block per SM with a fixed cost per block (tile clear, pipeline fill, merge of
    // the warps' tiles): aim at about four waves (measured best at 11M and 1.4M rows), in units of 384 rows,
    // within what the 16-bit lanes of the packed cells allow per warp tile
    const int unit = LaneRowsUnit(lane_red_, sub_rows_, lane_bins_, !quant_);   // rows of one stage across the block's warps
    long long rpb = (total_rows / (4LL * num_sms_) + unit - 1) / unit * unit;
    if (!quant_) {
      // fp32: every block clears and merges whole tiles of float pairs and nothing can overflow, so fewer, longer blocks:
      // about two waves over all 32-group parts
      const long long parts = (train_->num_groups + 31) / 32;
      const long long row_blocks = std::max<long long>(1, 2LL * num_sms_ / parts);
      rpb = (total_rows / row_blocks + unit - 1) / unit * unit;
      return static_cast<int>(std::max<long long>(rpb, 8LL * unit));
    }
    rpb = std::min<long long>(std::max<long long>(rpb, 3LL * unit), 13LL * unit);
    rpb = std::min<long long>(rpb, static_cast<long long>(LaneTiles(lane_red_, sub_rows_, lane_bins_, !quant_)) * (sub_rows_ / 32 * 32));
    return static_cast<int>(rpb);
  }
  long long target = total_rows / (static_cast<long long>(num_sms_) * 6) + 1;
  long long rpb = 512; while (rpb < target && rpb < 8192) rpb <<= 1;
  return static_cast<int>(std::max<long long>(rpb, 32));
}

void CudaEngine::AddConstantToScores(double v, int k) {
  LaunchAddConstant(score_.get() + static_cast<size_t>(k) * n_, n_, static_cast<float>(v), stream_);
  for (auto& vs : valid_) LaunchAddConstant(vs.score.get() + static_cast<size_t>(k) * vs.ds->num_data, vs.ds->num_data, static_cast<float>(v), stream_);
}

void CudaEngine::UploadGradients(const float* host_grad, const float* host_hess, const float** dev_grad, const float** dev_hess) {
  const size_t total = static_cast<size_t>(n_) * K_;
  fixed_grad_.Alloc(total); fixed_hess_.Alloc(total);
  FB_CUDA(cudaMemcpyAsync(fixed_grad_.get(), host_grad, sizeof(float) * total, cudaMemcpyHostToDevice, stream_));
  FB_CUDA(cudaMemcpyAsync(fixed_hess_.get(), host_hess, sizeof(float) * total, cudaMemcpyHostToDevice, stream_));
  FB_CUDA(cudaStreamSynchronize(stream_));
  *dev_grad = fixed_grad_.get(); *dev_hess = fixed_hess_.get();
}

void CudaEngine::DownloadGradients(int class_id, float* host_grad, float* host_hess) {
  if (round_grad_ == nullptr || class_id < 0 || class_id >= K_) Log::Fatal("No gradients of class %d to copy: no round has been trained yet", class_id);
  FB_CUDA(cudaMemcpyAsync(host_grad, round_grad_ + static_cast<size_t>(class_id) * n_, sizeof(float) * n_, cudaMemcpyDeviceToHost, stream_));
  FB_CUDA(cudaMemcpyAsync(host_hess, round_hess_ + static_cast<size_t>(class_id) * n_, sizeof(float) * n_, cudaMemcpyDeviceToHost, stream_));
  FB_CUDA(cudaStreamSynchronize(stream_));
}

void CudaEngine::AddRowValuesToScores(int data_idx, int class_id, const float* host_values) {
  if (data_idx < 0 || data_idx > static_cast<int>(valid_.size()) || class_id < 0 || class_id >= K_) Log::Fatal("AddRowValuesToScores: data set %d / class %d does not exist", data_idx, class_id);
  const int rows = data_idx == 0 ? n_ : valid_[data_idx - 1].ds->num_data;
  float* score = (data_idx == 0 ? score_.get() : valid_[data_idx - 1].score.get()) + static_cast<size_t>(class_id) * rows;
  if (rows <= 0) return;
  row_values_.Alloc(static_cast<size_t>(rows));
  FB_CUDA(cudaMemcpyAsync(row_values_.get(), host_values, sizeof(float) * rows, cudaMemcpyHostToDevice, stream_));
  LaunchAddVector(score, row_values_.get(), rows, stream_);
  FB_CUDA(cudaStreamSynchronize(stream_));   // the source is the caller's host buffer
}

void CudaEngine::ScaleScores(double a, const std::vector<double>& b) {
  for (int k = 0; k < K_; ++k) {
    const float bk = k < static_cast<int>(b.size()) ? static_cast<float>(b[k]) : 0.f;
    LaunchScaleAdd(score_.get() + static_cast<size_t>(k) * n_, n_, static_cast<float>(a), bk, stream_);
    for (auto& vs : valid_) LaunchScaleAdd(vs.score.get() + static_cast<size_t>(k) * vs.ds->num_data, vs.ds->num_data, static_cast<float>(a), bk, stream_);
  }
}

void CudaEngine::AddValid(const Dataset* valid) {
  EnsureDeviceDataset(const_cast<Dataset*>(valid));
  SyncDeviceMetadata(valid, stream_);
  valid_.emplace_back();
  ValidSet& vs = valid_.back();
  vs.ds = valid; vs.dd = valid->device;
  const size_t total = static_cast<size_t>(valid->num_data) * K_;
  vs.score.Alloc(total); vs.score.Zero(stream_);
  if (!valid->metadata.init_score.empty()) { std::vector<float> f(valid->metadata.init_score.begin(), valid->metadata.init_score.end()); vs.score.Upload(f, stream_); }
  FB_CUDA(cudaStreamSynchronize(stream_));
}

void CudaEngine::UploadTreeForTraversal(const Tree& tree, const Dataset* ds, DevTree* out) {
  const int ni = std::max(1, tree.num_leaves - 1), nl = tree.num_leaves;
  std::vector<int> ints(static_cast<size_t>(ni) * 19 /* 11 per-node arrays + 8 words of categorical bins per node */, 0); std::vector<float> fl(nl); std::vector<signed char> dec(ni, 0);
  int* left = ints.data(); int* right = left + ni; int* sf = right + ni; int* sg = sf + ni; int* tb = sg + ni; int* db = tb + ni; int* nanb = db + ni;
  int* bun = nanb + ni; int* goff = bun + ni; int* mfb = goff + ni; int* nbin = mfb + ni;
  for (int s = 0; s < tree.num_leaves - 1; ++s) {
    const int f = tree.split_feature_inner[s]; const FeatureMeta& m = ds->feature_meta[f];
    left[s] = tree.left_child[s]; right[s] = tree.right_child[s]; sf[s] = f; sg[s] = m.group; tb[s] = static_cast<int>(tree.threshold_in_bin[s]);
    db[s] = m.default_bin; nanb[s] = m.num_bin - 1; bun[s] = m.bundled; goff[s] = m.group_offset; mfb[s] = m.most_freq_bin; nbin[s] = m.num_bin; dec[s] = tree.decision_type[s];
    if (tree.decision_type[s] & kCategoricalMask) {
      const int ci = static_cast<int>(tree.threshold_in_bin[s]);
      const int lo = tree.cat_boundaries_inner[ci], nw = std::min(8, tree.cat_boundaries_inner[ci + 1] - lo);
      for (int w = 0; w < nw; ++w) ints[static_cast<size_t>(ni) * 11 + static_cast<size_t>(s) * 8 + w] = static_cast<int>(tree.cat_threshold_inner[lo + w]);
    }
  }
  for (int l = 0; l < nl; ++l) fl[l] = static_cast<float>(tree.leaf_value[l]);
  FB_CUDA(cudaStreamSynchronize(stream_));   // staging buffers are reused: the previous traversal must be done
  tree_ints_.Upload(ints, stream_); tree_floats_.Upload(fl, stream_); tree_dec_.Upload(dec, stream_);
  FB_CUDA(cudaStreamSynchronize(stream_));   // host vectors go out of scope
  const int* d = tree_ints_.get();
  out->num_leaves = nl; out->left = d; out->right = d + ni; out->split_feature = d + 2 * ni; out->split_group = d + 3 * ni; out->threshold_bin = d + 4 * ni;
  out->default_bin = d + 5 * ni; out->nan_bin = d + 6 * ni; out->bundled = d + 7 * ni; out->group_offset = d + 8 * ni; out->most_freq_bin = d + 9 * ni; out->num_bin = d + 10 * ni;
  out->cat_bits = reinterpret_cast<const unsigned int*>(d + 11 * ni);
  out->threshold = nullptr; out->decision = tree_dec_.get(); out->leaf_value = tree_floats_.get();
}

void CudaEngine::AddTreeToScores(const Tree& tree, int k, double scale, int which) {
  DevTree dt; UploadTreeForTraversal(tree, train_, &dt);
  if (which != 2) LaunchAddTreeBinned(dt, dd_->rows.get(), dd_->row_stride, n_, static_cast<float>(scale), score_.get() + static_cast<size_t>(k) * n_, stream_);
  if (which != 1) for (auto& vs : valid_) LaunchAddTreeBinned(dt, vs.dd->rows.get(), vs.dd->row_stride, vs.ds->num_data, static_cast<float>(scale), vs.score.get() + static_cast<size_t>(k) * vs.ds->num_data, stream_);
  FB_CUDA(cudaStreamSynchronize(stream_));
}

void CudaEngine::CopyScoresToHost(int data_idx, double* out) {
  const float* src = data_idx == 0 ? score_.get() : valid_[data_idx - 1].score.get();
  const size_t total = static_cast<size_t>(data_idx == 0 ? n_ : valid_[data_idx - 1].ds->num_data) * K_;
  std::vector<float> tmp(total);
  FB_CUDA(cudaMemcpyAsync(tmp.data(), src, total * sizeof(float), cudaMemcpyDeviceToHost, stream_));
  FB_CUDA(cudaStreamSynchronize(stream_));
  for (size_t i = 0; i < total; ++i) out[i] = tmp[i];
}

std::vector<double> CudaEngine::EvalMetric(int data_idx, const std::string& name, bool* supported) {
  *supported = false;
  int kind = -1;
  if (name == "l2") kind = kMetL2; else if (name == "rmse") kind = kMetRMSE; else if (name == "l1") kind = kMetL1;
  else if (name == "binary_logloss") kind = kMetBinaryLogloss; else if (name == "binary_error") kind = kMetBinaryError;
  else if (name == "multi_logloss") kind = kMetMultiLogloss; else if (name == "multi_error" && cfg_.multi_error_top_k == 1) kind = kMetMultiError;
  if (name == "auc" || name == "ndcg") {
    const Dataset* ds = data_idx == 0 ? train_ : valid_[data_idx - 1].ds;
    DeviceDataset* dd = data_idx == 0 ? dd_ : valid_[data_idx - 1].dd;
    const float* score = data_idx == 0 ? score_.get() : valid_[data_idx - 1].score.get();
    if (dd->label.size() == 0 || ds->num_data == 0) return {};
    if (name == "auc") {
      // rows sharded over ranks: the exact AUC needs every (positive, negative) pair, so the host metric gathers the scores
      if (data_parallel() || K_ != 1) return {};
      double r[3];
      DeviceAuc(score, dd->label.get(), dd->weight.size() ? dd->weight.get() : nullptr, ds->num_data, r, stream_);
      *supported = true;
      return {r[0]};
    }
    if (dd->num_queries <= 0 || !ds->metadata.query_weights.empty() || cfg_.eval_at_vec.empty()) return {};
    int max_docs = 0; const auto& qb = ds->metadata.query_boundaries;
    for (size_t q = 0; q + 1 < qb.size(); ++q) max_docs = std::max(max_docs, qb[q + 1] - qb[q]);
    if (metric_gain_.size() == 0) metric_gain_.Upload(cfg_.label_gain_vec, stream_);
    std::vector<double> sums(cfg_.eval_at_vec.size() + 1, 0.0);
    if (!DeviceNdcgSums(score, dd->label.get(), dd->query_boundaries.get(), dd->num_queries, max_docs, metric_gain_.get(), static_cast<int>(metric_gain_.size()),
                        cfg_.eval_at_vec, sums.data(), stream_)) return {};
    sums[cfg_.eval_at_vec.size()] = dd->num_queries;
    if (data_parallel()) Network::SumDouble(sums.data(), static_cast<int64_t>(sums.size()));   // queries are sharded whole: per-query values add up
    std::vector<double> out(cfg_.eval_at_vec.size());
    for (size_t j = 0; j < out.size(); ++j) out[j] = sums[j] / sums[cfg_.eval_at_vec.size()];
    *supported = true;
    return out;
  }
  if (kind < 0) return {};
  if ((kind == kMetL2 || kind == kMetRMSE || kind == kMetL1) && cfg_.reg_sqrt) return {};
  if ((kind == kMetL2 || kind == kMetRMSE || kind == kMetL1) && K_ > 1) return {};   // several regression targets: the host metric averages over targets
  const Dataset* ds = data_idx == 0 ? train_ : valid_[data_idx - 1].ds;
  DeviceDataset* dd = data_idx == 0 ? dd_ : valid_[data_idx - 1].dd;
  const float* score = data_idx == 0 ? score_.get() : valid_[data_idx - 1].score.get();
  if (dd->label.size() == 0) return {};
  const int n = ds->num_data;
  if (partial_.size() < 2 * (static_cast<size_t>(n) / 256 + 2)) partial_.Alloc(2 * (static_cast<size_t>(n) / 256 + 2));
  LaunchPointwiseMetric(kind == kMetRMSE ? kMetL2 : kind, objd_.kind, objd_.kind == kObjBinary || objd_.kind == kObjMulticlassOVA ? objd_.p0 : 1.0, score, dd->label.get(),
                        dd->weight.size() ? dd->weight.get() : nullptr, n, K_, partial_.get(), static_cast<int>(partial_.size() / 2), root_sums_d_.get(), stream_);
  double h[2];
  FB_CUDA(cudaMemcpyAsync(h, root_sums_d_.get(), sizeof(h), cudaMemcpyDeviceToHost, stream_));
  FB_CUDA(cudaStreamSynchronize(stream_));
  if (!feature_parallel_) Network::SumDouble(h, 2);   // rows sharded over ranks: (weighted loss, weight) sums add up; replicated rows: already complete
  *supported = true;
  double v = h[1] > 0 ? h[0] / h[1] : 0.0;
  if (kind == kMetRMSE) v = std::sqrt(v);
  return {v};
}

}  // namespace fb
