// Device training engine: owns the scores, gradients, index buffers, histogram pool and level
// descriptors of one rank, and drives the level loop.
// Parity: src/treelearner/cuda/cuda_single_gpu_tree_learner.cpp (Train L3245-3506, level-batched
// prefix L1804-1937, EnqueueLevelBestSplitSearch L1129-1285, ApplyLevelBatched L1480-1716),
// src/boosting/cuda/cuda_score_updater.cpp, src/boosting/cuda/nccl_gbdt.cpp (per-rank component).
#pragma once
#include <memory>
#include <vector>

#include "fb/gbdt.h"
#include "kernels.cuh"

namespace fb {

void EnsureDeviceDataset(Dataset* ds);
void SyncDeviceMetadata(const Dataset* ds, cudaStream_t s);
void EnsureColumnMajor(DeviceDataset* dd, cudaStream_t s);
class Fabric;   // symmetric heap + peer pointers of the multi-rank path (fabric.h)

struct StageClock {
  // CUDA-event stage timing without host synchronisation inside a tree: events are recorded on the
  // stream and resolved once per tree.
  std::vector<std::pair<cudaEvent_t, cudaEvent_t>> pool;
  std::vector<std::pair<int, int>> pending;   // (stage, pool index)
  std::vector<double> total_ms; std::vector<int64_t> calls; std::vector<std::string> names;
  size_t next = 0; bool enabled = false; bool nvtx = false, nvtx_open = false;   // nvtx: NVTX ranges named after the stages, for timeline tools
  int Stage(const char* name);
  void Begin(int stage, cudaStream_t s);
  void End(cudaStream_t s);
  void Resolve();
  std::string Report() const;
  ~StageClock();
 private:
  int open_ = -1;
};

class CudaEngine : public DeviceEngine {
 public:
  CudaEngine(const Config& cfg, const Dataset* train, const ObjectiveFunction* obj, int num_tree_per_iter);
  ~CudaEngine() override;
  void AddValid(const Dataset* valid) override;
  void AddConstantToScores(double v, int class_id) override;
  void ScaleScores(double a, const std::vector<double>& b) override;
  void DownloadGradients(int class_id, float* host_grad, float* host_hess) override;
  void AddRowValuesToScores(int data_idx, int class_id, const float* host_values) override;
  void UploadGradients(const float* host_grad, const float* host_hess, const float** dev_grad, const float** dev_hess) override;
  void TrainOneIter(const float* custom_grad, const float* custom_hess, int iter, double shrinkage, const std::vector<double>& init_scores,
                    std::vector<std::unique_ptr<Tree>>* out, bool* all_constant) override;
  std::vector<double> EvalMetric(int data_idx, const std::string& metric_name, bool* supported) override;
  void CopyScoresToHost(int data_idx, double* out) override;
  void AddTreeToScores(const Tree& tree, int class_id, double scale, int which = 0) override;
  void* TrainScorePtr() override { return score_.get(); }
  int64_t GpuLaunches() const override { return LaunchCounter().load(); }
  std::string StageReport() const override { return clock_.Report(); }
  void SetBagging(double fraction, int freq, int seed) override { bag_fraction_ = fraction; bag_freq_ = freq; bag_seed_ = seed; }

 private:
  struct HostLeaf { int begin = 0, count = 0, buffer = 0, depth = 0, slot = 0; SplitRecord best; bool valid = false; };
  struct ValidSet { const Dataset* ds; DeviceDataset* dd; DevBuf<float> score; };

  Tree* TrainTree(int class_id, int tree_index);
  void BuildPartitions();
  void SetupOwnership();
  void RunRootHistogram();
  void ReadBackLevel(int num_leaves);
  // forced splits (forcedsplits_filename): the tree is grown under the host's control and the forced nodes' records are
  // evaluated on the host from the leaf's histogram (a few hundred bytes from the pool) with the shared split math
  DevBuf<float> fixed_grad_, fixed_hess_;   // gradients uploaded once and reused every round (random forests)
  std::vector<ForcedSplitNode> forced_;
  bool ForcedRecord(int leaf, int inner_feature, int bin, SplitRecord* out);
  void DrawBag(int round);
  void DrawGoss(int iter);
  void RenewLeavesFromTrueGradients(Tree* tree);
  void RenewLeavesByObjective(Tree* tree, int class_id);
  void SetupBitmapBroadcast(PartArgs* pa);
  const uint8_t* bag_mask_ptr() const { return bag_active_ ? bag_mask_.get() : nullptr; }
  void UploadTreeForTraversal(const Tree& tree, const Dataset* ds, DevTree* out);
  int ChooseRowsPerBlock(long long total_rows) const;
  void ResolveQuantBins();

  Config cfg_; Plan plan_;
  const Dataset* train_; DeviceDataset* dd_; const ObjectiveFunction* obj_;
  int K_ = 1, n_ = 0;
  bool quant_ = false;
  bool host_gradients_ = false;   // the objective has no device kernel: gradients come from its host code each round
  cudaStream_t stream_ = nullptr;
  int num_sms_ = 148;
  SplitParams sp_;
  ObjDesc objd_;
  ColSampler col_sampler_;
  StageClock clock_;
  int st_grad_, st_quant_, st_hist_, st_find_, st_part_, st_score_, st_sync_;

  DevBuf<float> score_, grad_, hess_, maxbuf_, scales_;
  DevBuf<long long> root_sums_i_;
  DevBuf<double> root_sums_d_, partial_, label_gain_, metric_gain_;
  DevBuf<int32_t> gh_sep_;
  DevBuf<float2> gh2_;
  const uint8_t* gh_base_ = nullptr; int gh_stride_ = 0;
  DevBuf<int> idx_[2];
  DevBuf<LeafInfo> leaves_;
  DevBuf<SplitRecord> best_;
  DevBuf<CandLite> cand_;
  DevBuf<char> pool_;              // single rank: owned here; multi-rank: the pool lives in the symmetric heap
  char* pool_base_ = nullptr; size_t pool_bytes_ = 0;
  // ---- multi-rank state (world_ > 1) ----
  Fabric* fabric_ = nullptr; int rank_ = 0, world_ = 1;
  bool feature_parallel_ = false;                      // tree_learner=feature: rows replicated, features split
  bool data_parallel() const { return world_ > 1 && !feature_parallel_; }
  // tree_learner=voting: rows sharded, histograms local, only the voted features' bins are exchanged
  bool voting_ = false;
  size_t off_votes_ = 0, flag_vote_ = 0;
  DevBuf<int> bin_identity_, features_all_, sub_features_all_; DevBuf<CandLite> cand_local_; DevBuf<VoteLocalSum> vote_sums_; DevBuf<unsigned char> voted_;
  size_t off_bits_ = 0, off_chunk_left_ = 0, flag_part_ = 0; std::vector<unsigned char> h_bin_owner_;
  long long slot_strides_[kMaxRanks] = {0};
  size_t off_pool_ = 0, off_counts_ = 0, off_best_ = 0, flag_hist_ = 0, flag_best_ = 0;
  DevBuf<float> global_max_;
  size_t off_stage_ = 0; DevBuf<char> stage_local_; DevBuf<unsigned int> task_done_;
  long long slot_stride_ = 0;      // bins per pool slot on this rank
  size_t hist_elem_ = 8;
  DevBuf<HistPartition> parts_; std::vector<HistPartition> h_parts_; int max_part_bins_ = 0;
  DevBuf<unsigned char> bin_owner_; DevBuf<int> bin_local_;
  std::vector<int> owned_features_;
  DevBuf<char> level_blob_; PinnedBuf<char> h_level_blob_;
  DevBuf<HistTask> hist_tasks_; DevBuf<unsigned int> hist_status_; PinnedBuf<unsigned int> h_hist_status_;
  DevBuf<unsigned int> bits_; DevBuf<int> chunk_left_, split_left_total_;
  DevBuf<int> features_, sub_features_;
  // exact leaf-wise growth (grow_policy=leaf): the device grows up to grow_leaves_ leaves, the host keeps the best num_leaves
  bool leafwise_ = false; int grow_leaves_ = 0;
  DevBuf<double> renew_in_, renew_out_, renew_res_; DevBuf<int> renew_off_; DevBuf<char> renew_temp_;   // percentile leaf renewal on the device
  DevBuf<float> qmax_; DevBuf<int> qclamp_; DevBuf<unsigned long long> mag_hist_; DevBuf<int8_t> ef_residual_;   // fixed-point quantization: robust scale and error feedback
  unsigned int xendcg_round_ = 0;   // rank_xendcg: rounds of gradients computed so far (keys the per-round random draws, like the host objective's counter)
  bool tc_fallback_logged_ = false;
  bool lane_red_ = true;   // reduction form of the lane construct (integer: plan hist_lane_red, fp32: plan hist_float_red)
  DevBuf<double> eval_key_;
  void FinalizeLeafwise(const LevelCtrl& hc, Tree* tree);
  // per-node feature masks (feature_fraction_bynode, interaction constraints)
  bool node_mask_on_ = false; int path_words_ = 0, num_sets_ = 0;
  DevBuf<unsigned char> node_mask_; DevBuf<unsigned int> path_bits_, set_bits_; DevBuf<int> mask_pool_;
  DevBuf<double> leaf_value_, renew_partial_; PinnedBuf<double> h_renew_partial_;
  PinnedBuf<LeafInfo> h_leaves_; PinnedBuf<SplitRecord> h_best_;
  std::vector<HostLeaf> host_leaves_;
  std::vector<ValidSet> valid_;
  // traversal staging
  DevBuf<int> tree_ints_; DevBuf<float> tree_floats_; DevBuf<signed char> tree_dec_;
  const float* cur_grad_ = nullptr; const float* cur_hess_ = nullptr;
  const float* round_grad_ = nullptr; const float* round_hess_ = nullptr;   // this round's gradients of all class trees ([class][row], device)
  DevBuf<float> row_values_;
  int lane_mode_ = 0, lane_bins_ = 64, sub_rows_ = 1 << 30;
  // compact per-tree view of the sampled feature groups
  DevBuf<uint8_t> compact_rows_; DevBuf<int> compact_groups_, compact_start_, compact_count_;
  std::vector<int> compact_list_; bool compact_p4_ = false;
  // device controller state
  bool use_ctrl_ = false; int levels_hint_ = 8;
  // score update enqueued from the device's leaf records, before the per-tree read-back
  bool fast_score_ok_ = false, score_done_ = false; double cur_shrinkage_ = 1.0; float* cur_score_ = nullptr;
  DevBuf<LevelCtrl> ctrl_; DevBuf<int> frontier_; DevBuf<SplitJournal> journal_;   // ctrl_: two level records (a ring, see TrainTree)
  DevBuf<FindChild> root_child_;                                   // the root's search descriptor
  DevBuf<unsigned int> child_done_, level_done_, split_done_;     // arrival counters of the fused kernels (zero between launches)
  PinnedBuf<LevelCtrl> h_ctrl_; PinnedBuf<SplitJournal> h_journal_; PinnedBuf<LeafInfo> h_root_;
  // bagging (device-drawn; -1 = no bag drawn)
  double bag_fraction_ = 1.0; int bag_freq_ = 0, bag_seed_ = 0;
  bool bag_active_ = false; int bag_count_ = -1, root_count_ = 0; long long bag_global_ = 0, root_global_ = 0;
  DevBuf<float> goss_mag_, goss_sorted_; DevBuf<char> goss_temp_;
  DevBuf<uint8_t> bag_mask_; DevBuf<int> bag_idx_, bag_chunk_, bag_count_dev_; PinnedBuf<int> h_bag_count_;
  int max_docs_ = 0;
};

}  // namespace fb
