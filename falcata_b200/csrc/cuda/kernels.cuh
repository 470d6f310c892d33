// Launcher declarations of every device kernel of the training and prediction paths.
// One launcher per kernel (or fused kernel); the engine and the kernel-level test API call these.
#pragma once
#include "device_common.cuh"
#include <vector>

#include "fabric.h"
#include "fb/learner.h"

namespace fb {

// -------------------------------------------------------- level controller ----
// Device-resident state of the level loop. With the device controller the host enqueues the kernels
// of several levels ahead with upper-bound grids; every kernel reads how much work the level really
// has from this record, which the controller kernel rewrites between levels.
struct LevelCtrl {
  int num_leaves, next_slot, done, level;
  int num_splits, num_children, total_chunks, total_blocks;
  int frontier_count, journal_count, pad0;
  int num_eval, pad1;   // leaf-wise growth: evaluated nodes recorded so far (eval_key)
  int skip_search;   // 1: this level used up the leaf budget - its children can never split, so their construct and search are skipped
};
// One applied split, in application order: enough for the host to rebuild the tree after the last level.
struct SplitJournal { int leaf, right_leaf, parent_global, pad; int begin, count, buffer, depth; /* the parent's window and depth */ SplitRecord rec; };
struct ChildInit;

// ------------------------------------------------------------- objective ----
struct ObjDesc {
  int kind;          // ObjKind
  int num_class;
  double p0, p1, p2; // binary: sigmoid, neg weight, pos weight; lambdarank: sigmoid, norm, truncation; others: their one parameter
  int max_docs;      // lambdarank: largest query
};

void LaunchObjectiveGradients(const ObjDesc& d, const float* score, const float* label, const float* weight, const int* qb, int num_queries,
                              const double* label_gain, int num_gain, int n, float* grad, float* hess, float* maxbuf, cudaStream_t s);
// `mask` (one byte per row, 0 = out of bag; nullptr = all rows) limits the maxima and root sums to the bag.
void LaunchAbsMax(const float* grad, const float* hess, int n, int num_class, float* maxbuf, cudaStream_t s, const uint8_t* mask = nullptr);
void LaunchQuantize(const float* grad, const float* hess, int n, const float* maxbuf, const float* global_max, int bins, bool stochastic, uint32_t seed,
                    uint32_t iter_key, uint64_t global_row_offset, uint8_t* gh_base, int gh_stride, float* scales_out, long long* root_sums, cudaStream_t s, const uint8_t* mask = nullptr);
// fixed-point extras: log-magnitude histogram of the gradients (kQuantMagBuckets counters), the gate that may re-anchor
// the scale below an outlier cluster (qmax: top-level gradient magnitude and hessian maximum; clamp: saturation level or
// 0), and the quantizer with saturation and int8 error feedback (`residual`: 2 bytes per row, may be null)
void LaunchGradMagHist(const float* grad, int n, const float* max2, const uint8_t* mask, unsigned long long* hist, cudaStream_t s);
void LaunchRobustScale(const unsigned long long* hist, long long num_rows, const float* max2, int bins, bool use_gate, float* qmax, int* clamp, cudaStream_t s);
void LaunchQuantizeFeedback(const float* grad, const float* hess, int n, const float* qmax, const int* clamp, int bins, int8_t* residual, uint8_t* gh_base, int gh_stride,
                            float* scales_out, long long* root_sums, cudaStream_t s, const uint8_t* mask = nullptr);
void LaunchInterleave(const float* grad, const float* hess, int n, float2* gh2, double* partial, int partial_capacity, double* root_sums_d, cudaStream_t s,
                      const uint8_t* mask = nullptr);

// ------------------------------------------------------------- histogram ----
// Where a histogram bin lives: owner rank and index inside that rank's slot. With one rank the
// map is the identity. Peer pools are device pointers mapped into this process (CUDA IPC).
struct HistDest {
  void* pool[8];            // pool base per rank (this rank's own pointer at [rank])
  long long slot_stride[8]; // bins per slot of each rank's pool
  const unsigned char* bin_owner;  // [num_total_bin]
  const int* bin_local;            // [num_total_bin]
  int num_ranks, rank;
  int owner_only;                  // feature-parallel: every rank sees all rows; only bins of owned features are kept (no exchange)
  // num_ranks > 1: blocks add into a LOCAL staging histogram of their task; the last block of a
  // task to finish stores the finished slices into the owner ranks' per-source staging slots
  // (plain coalesced stores over NVLink) while other tasks' tiles are still being constructed.
  void* stage_local;               // [stage_cap][num_total_bin] bins, zero between uses
  unsigned int* task_done;         // [stage_cap] blocks finished per task
  void* peer_stage[8];             // base of every rank's staging area: [source rank][stage_cap][slot_stride(owner)]
  int stage_cap;
};

struct HistArgs {
  const uint8_t* rows; int row_stride; int num_groups;
  const uint8_t* gh_base; int gh_stride;
  const int* idx[2];
  const HistTask* tasks; int num_tasks; int total_blocks;
  const HistPartition* parts; int num_parts; int max_part_bins;
  const int* group_bin_start;
  int bulk_root;                // 1: root level (rows in order, 32-byte rows) staged by bulk asynchronous copies with mbarrier completion
  unsigned int* status;         // device status word (nullable): a bounded wait that gives up records kStatusWaitTimeout here
  int pack4;                    // 1 (compact view of groups with at most 16 bins): two groups per byte, low nibble first
  const int* group_bin_count;   // non-null (compact view): bins per listed group; null: groups are consecutive in the bin space
  int rows_per_block; int sub_rows;
  int identity_root;        // 1: task rows are 0..count-1 (no index load)
  int num_total_bin;
  int lane_share;           // lane kernel: warps per tile (set by the launcher)
  int lane_red;             // lane kernel: shared-memory reduction adds instead of load-add-store with forwarding
  int lane_mode;            // 0: flat items + shared atomics; 1: lane-per-group warp-private tiles (no atomics); 2: lane-per-group, one shared tile + atomics;
                            // 3: one-hot tcgen05 MMA (root level, 32-byte rows; falls back to mode 1 outside its coverage)
  int tc_row_count;         // mode 3: rows of the task as the host knows them (extent of the TMA tensor maps)
  int lane_bins;            // lane modes: bins per group tile (16 or 64)
  HistDest dest;
  FabricSignal sig;         // world > 1: the last block raises this rank's "construct done" flag on every peer
  const LevelCtrl* ctrl;    // non-null: num_tasks / total_blocks come from the device controller
};
void LaunchHistConstructQuant(const HistArgs& a, cudaStream_t s);
int LaneTiles(bool red, int sub_rows, int nb, bool flt);      // tiles of a lane-construct block: each takes at most `sub_rows` rows before its 16-bit lanes could overflow
int LaneRowsUnit(bool red, int sub_rows, int nb, bool flt);   // rows per stage of a lane-construct block (warps x 32): rows_per_block is chosen in these units
// K9: per-tree compact view. out[row][j] = cols[groups[j]][row] for the listed (sampled) feature groups: a dense
// row-major matrix with only the columns this tree can split on, read from the column-major copy (coalesced
// along rows) and written in 32-byte row pieces through a shared-memory transpose tile.
void LaunchCompactGather(const uint8_t* cols, long long col_stride, int n, const int* groups, int num_groups, uint8_t* out, int out_stride, cudaStream_t s,
                         bool pack4 = false);   // pack4: out[row][j / 2] holds listed groups j (low nibble) and j + 1 (high nibble)
void LaunchHistConstructFloat(const HistArgs& a, cudaStream_t s);
// tcgen05 one-hot instance (same arguments, same result); returns false, having launched nothing, when the shape is outside
// what it covers (see hist_tc_kernel.cu). rows_per_block must come from HistTcRowsPerBlock (whole 32-row steps).
bool LaunchHistConstructQuantTC(const HistArgs& a, cudaStream_t s);
int HistTcRowsPerBlock(long long count, int num_sms);

// ------------------------------------------------------------ split find ----
struct FindChild { int leaf; int slot; int other_slot; int is_larger; int split; int is_left; int parent_global; int task; };   // task: construct task of this pair's smaller child   // larger: bins = pool[slot] - pool[other_slot], written back to pool[slot]

struct CandLite {      // best threshold of one (child, feature)
  double gain; int feature; int threshold; int default_left; int left_cnt;
  long long left_gi, left_hi; double left_g, left_h;
  int is_categorical, num_cat_bins; uint32_t cat_bitset[8];   // categorical: the bins that go left
};

struct FindArgs {
  const FindChild* children; int num_children;
  const int* features; int num_features;          // inner feature indices searched on this rank (owned and sampled)
  const int* sub_features; int num_sub_features;  // owned features that are not sampled: larger-child subtraction only
  const FeatureMeta* meta;
  const int* bin_local;                           // histogram slot index -> index inside this rank's pool slot
  void* pool; long long slot_stride;
  const LeafInfo* leaves;
  const float* scales;                            // quantized: (g_scale, h_scale) of this tree
  SplitParams params;
  CandLite* cand;                                 // [num_children x num_features]
  SplitRecord* best;                              // [leaf]
  int quant;
  int tree_index; unsigned int extra_seed;        // extra_trees: key of the per-(tree, leaf, feature) threshold draw
  int has_categorical;                            // some searched feature is categorical: the kernel gets its shared scratch
  const unsigned char* node_mask; int node_mask_stride;   // non-null: [child][inner feature], 0 = not searched at this node
  // ---- voting-parallel (see VoteArgs) ----
  int local_vote;                                 // 1: local pass - leaf totals and count are this rank's (vote_sums, LeafInfo.count)
  const struct VoteLocalSum* vote_sums;           // [child] local totals of the child's histogram
  const unsigned char* voted; int voted_stride;   // non-null: global pass - search only voted (child, feature) pairs; bins are the
                                                  // sums of the ranks' staged slices of child blockIdx.x; nothing is written back
  // ---- multi-rank (world > 1) ----
  FabricWait wait;                                // construct-done flags of all ranks (the reduce-scatter is complete when they are up)
  const void* stage; int stage_cap;               // this rank's staging area [source rank][stage_cap][slot_stride] written by the ranks' constructs
  const int* counts; int counts_stride;           // [rank][split] local left counts published by every rank's partition
  LeafInfo* leaves_rw;                            // exact global row counts are written back here
  SplitRecord* peer_best[kMaxRanks];              // address of best_slots[this rank][0] inside every rank's heap
  const SplitRecord* gathered; int gathered_stride;   // local [rank][leaf] records written by the peers
  FabricSignal sig;                               // "rank-local best splits published" signal
  FabricWait wait_best;
  const LevelCtrl* ctrl;                          // non-null: num_children comes from the device controller
  // ---- fused tail (fused_tail != 0): the last block of every child reduces that child's candidates to its best split
  // (multi-rank: and stores it into every peer); the last of those blocks waits for the peers' records, takes the
  // argmax over ranks for every child and then runs the level controller. A level then costs one launch from finished
  // histograms to the next level's descriptors.
  int fused_tail;
  unsigned int* child_done;                       // [children] blocks finished per child (zero between launches)
  unsigned int* level_done;                       // [1] children reduced (zero between launches)
  int run_controller;                             // 0: the tail stops after the per-leaf records (host-driven growth)
};
struct CtrlArgs;

// Device-side level controller: applies the gain-ranked leaf budget to the frontier's best splits
// and writes the next level's descriptors, the journal and the new frontier.
struct CtrlArgs {
  const LevelCtrl* cur; LevelCtrl* nxt;   // level record read / written (the same object for the stand-alone launch; the two
                                          // halves of a ring when the controller runs as the search kernel's tail)
  int* frontier; SplitJournal* journal;
  LeafInfo* leaves; const SplitRecord* best; const FeatureMeta* meta;
  PartSplit* splits; ChildInit* child_init; FindChild* children;
  int max_leaves; int rows_per_block;
  const unsigned char* bin_owner;   // feature-parallel: owner rank of every histogram bin (null otherwise)
  // Exact leaf-wise growth (grow_policy=leaf). A frontier leaf is split while fewer than B evaluated nodes sort
  // strictly before it in best-first order (LeafwiseChildKey): that never misses a node that best-first growth
  // with a budget of B splits would split, because a node's rank only gets worse as more nodes are evaluated.
  // The tree is grown past the budget where needed (max_leaves is the growth cap) and the host keeps the
  // best-first tree.
  int leafwise_budget;              // B = num_leaves - 1; 0: level growth with a gain-ranked budget
  double* eval_key;                 // [evaluated nodes][4] order keys
};
void LaunchLevelController(const CtrlArgs& a, cudaStream_t s);
// Per-tree start state written on the device: root leaf record (from the gradient sums), both halves of the
// level-record ring, the frontier, the root's construct task and search descriptor.
struct TreeInitArgs {
  LeafInfo* leaves; const long long* sums_i; const double* sums_d; const float* scales; int quant; int n_local; long long n_global; SplitParams sp;
  LevelCtrl* ctrl; int* frontier;   // null without the device controller
  HistTask* root_task; FindChild* root_child; int root_blocks;
};
void LaunchInitTree(const TreeInitArgs& a, cudaStream_t s);

// Per-node feature masks (feature_fraction_bynode, interaction constraints): mask[child][inner feature] = 1 when
// the child's split search may use the feature.
struct NodeMaskArgs {
  const FindChild* children; int num_children; const LevelCtrl* ctrl;
  const LeafInfo* leaves; const FeatureMeta* meta;
  int num_inner;                               // row length of the mask
  const int* pool; int pool_size;              // inner features sampled for this tree, ascending
  double fraction; unsigned int seed; int tree_index;   // per-node sample: round(fraction * allowed) features, >= 1
  const unsigned int* path_bits;               // [leaf][words] real features split on above the leaf
  const unsigned int* set_bits; int num_sets; int words;   // interaction sets as bitsets over real features
  unsigned char* mask;
};
void LaunchNodeMask(const NodeMaskArgs& a, cudaStream_t s);
void LaunchPathBits(const LevelCtrl* ctrl, const SplitJournal* journal, const FeatureMeta* meta, unsigned int* path_bits, int words, int max_splits, cudaStream_t s);

// ----------------------------------------------------------------- voting ----
// Voting-parallel (PV-Tree) on the device, rows sharded over ranks. Histograms stay LOCAL (all features,
// one pool slot per leaf); per level and child:
//   1. VoteLocalSums   local totals of the child (bins of feature group 0)
//   2. FindSplits      local pass: best local gain of every sampled feature
//   3. VoteTopK        the rank's top_k features by local gain, stored into EVERY rank's vote slots (all-gather
//                      by peer stores) + flag
//   4. VoteTallyPush   waits for all ranks' votes, counts them, keeps the 2*top_k most voted features, and stores
//                      ONLY their local bins into the owner rank's staging slot (restricted reduce-scatter) + flag
//   5. FindSplits      global pass on the owned, voted features (bins = sum of the ranks' slices), then the usual
//                      per-leaf argmax and all-gather of the best record.
struct VoteLocalSum { long long gi, hi; double g, h; };
struct VoteArgs {
  const FindChild* children; int num_children; const LevelCtrl* ctrl;
  int world, rank, top_k, quant;
  const FeatureMeta* meta; int num_inner_features;
  const void* local_pool; long long local_stride; int g0_begin, g0_bins;   // local histogram pool; bin range of one constructed feature group
  VoteLocalSum* sums; const float* scales;                       // [child]; quantized: (g_scale, h_scale) of this tree
  const CandLite* cand_local; int num_searched;                  // [child][num_searched] local candidates
  int* peer_votes[kMaxRanks]; const int* votes_all; int child_cap;   // votes: [source rank][child_cap][top_k] inner feature ids (-1: none)
  FabricSignal vote_sig; FabricWait vote_wait;
  unsigned char* voted;                                          // [child_cap][num_inner_features]
  const unsigned char* bin_owner; const int* bin_local; void* peer_stage[kMaxRanks]; long long slot_stride[kMaxRanks]; int stage_cap;
  FabricSignal hist_sig;
};
void LaunchVoteLocalSums(const VoteArgs& a, cudaStream_t s);
void LaunchVoteTopK(const VoteArgs& a, cudaStream_t s);
void LaunchVoteTallyPush(const VoteArgs& a, cudaStream_t s);
void LaunchFindSplits(const FindArgs& a, cudaStream_t s, const CtrlArgs* tail_ctrl = nullptr);   // per (child, feature) search + in-place larger-child subtraction; fused tail when a.fused_tail
void LaunchReduceBest(const FindArgs& a, cudaStream_t s);      // per child argmax over features -> SplitRecord (world > 1: stored into every peer)
void LaunchGatherBest(const FindArgs& a, cudaStream_t s);      // world > 1: argmax over the ranks' records

// ------------------------------------------------------------- partition ----
constexpr int kPartChunk = 2048;
struct ChildInit {     // host-decided child bookkeeping of one split
  int left_slot, right_slot;       // histogram slots of the children
  int smaller_is_left;
  double left_g, left_h, right_g, right_h, left_out, right_out;
  long long left_gi, left_hi, right_gi, right_hi;
  int hist_block_begin, hist_num_blocks;
  int monotone, pad_;              // constraint of the split feature: tightens the children's output ranges
  double pkey[4];                  // leaf-wise growth: order key of the split node (the children's parent key)
};
struct PartArgs {
  const uint8_t* rows; int row_stride;
  const uint8_t* cols; long long col_stride;   // column-major copy (null: read the byte from the row)
  int* idx[2];
  const PartSplit* splits; int num_splits; int total_chunks;
  unsigned int* bits;        // kPartChunk/32 words per chunk
  int* chunk_left;           // lefts per chunk, then exclusive offsets
  int* split_left_total;     // [num_splits]
  LeafInfo* leaves;
  const ChildInit* child_init;
  HistTask* hist_tasks;      // one per split: the smaller child
  int rows_per_block;
  int world; int* peer_counts[kMaxRanks];   // world > 1: address of counts[this rank][0] inside every rank's heap
  const LevelCtrl* ctrl;     // non-null: num_splits / total_chunks come from the device controller
  int fused_scan;            // 1: the last chunk block of each split runs the scan + set-up step (every split has >= 1 chunk)
  unsigned int* split_done;  // [splits] chunk blocks finished per split (zero between launches)
  // ---- feature-parallel bitmap broadcast (bc_world > 1) ----
  // Every rank holds all rows but only the histograms of the features it owns. The rank that owns a
  // split's feature computes the go-left bit words of the leaf's rows and stores them, with the chunk
  // counts, into EVERY rank's buffers over NVLink (N/8 bytes per level); the other ranks skip the
  // column read and scatter from the received bitmap.
  int bc_world, bc_rank;
  unsigned int* peer_bits[kMaxRanks]; int* peer_chunk_left[kMaxRanks];
  FabricSignal bc_sig; FabricWait bc_wait;
};
void LaunchPartitionFlags(const PartArgs& a, cudaStream_t s);
void LaunchPartitionScanSetup(const PartArgs& a, cudaStream_t s);
void LaunchPartitionScatter(const PartArgs& a, cudaStream_t s);
void LaunchInitIndices(int* idx, int n, cudaStream_t s);

// ---------------------------------------------------------- rank metrics ----
// AUC: out = [auc, sum of positive weights, sum of negative weights] (radix sort + tie-group reduction on the device).
void DeviceAuc(const float* score, const float* label, const float* weight, int n, double out[3], cudaStream_t s);
// NDCG: out[j] = sum over queries of ndcg@ks[j]; false when a query is longer than the kernel's shared tile.
bool DeviceNdcgSums(const float* score, const float* label, const int* query_boundaries, int num_queries, int max_docs, const double* gains, int num_gains,
                    const std::vector<int>& ks, double* out, cudaStream_t s);

// ---------------------------------------------------------------- bagging ----
// Row sampling on the device: a row is in the bag iff a Philox number keyed on (bagging seed, bagging
// round, GLOBAL row id) is below its fraction, so the bag does not depend on how rows are sharded and is
// the one the host learner draws. Outputs: a byte mask, the ascending list of in-bag rows, their count.
struct BagArgs {
  int n; unsigned long long global_row_offset; uint32_t round, seed;
  double fraction, pos_fraction, neg_fraction; int balanced;    // balanced: fraction by label sign
  const float* label;
  const int* query_boundaries; int num_queries; int by_query;   // by_query: one draw per query, keyed on the global query id
  unsigned long long global_query_offset;
  uint8_t* mask; int* bag_idx; int* chunk_count; int* bag_count;
};
void LaunchBagging(const BagArgs& a, cudaStream_t s);
// Gradient-based one-side sampling on the device: |g*h| per row (summed over classes), the top_k-th largest value by
// a radix sort, rows at or above it kept, the others kept with probability `prob` (Philox on the global row id) and
// their gradients scaled by `multiply`; then the same scan + scatter as bagging.
struct GossArgs {
  int n, num_class; float* grad; float* hess;   // [num_class][n], scaled in place for the sampled small-gradient rows
  int top_k; double prob; float multiply; uint32_t iter, seed; unsigned long long global_row_offset;
  float* mag; float* sorted; void* sort_temp; size_t sort_temp_bytes;
  uint8_t* mask; int* bag_idx; int* chunk_count; int* bag_count;
};
size_t GossSortTempBytes(int n);
void LaunchGoss(const GossArgs& a, cudaStream_t s);

// ----------------------------------------------------------------- score ----
void LaunchCollapseLeafWindows(const LeafInfo* leaves, int num_leaves, int* idx0, const int* idx1, cudaStream_t s);
void LaunchAddLeafOutputs(const LeafInfo* leaves, const double* leaf_value, int num_leaves, const int* idx0, const int* idx1, float* score, cudaStream_t s);
// decided_ahead: `ctrl` comes from the fused search tail, which decides the NEXT level's splits: complete only with none pending
void LaunchAddLeafOutputsFromRecords(const LeafInfo* leaves, const LevelCtrl* ctrl, double shrinkage, int max_leaves, const int* idx0, const int* idx1, float* score,
                                     cudaStream_t s, bool decided_ahead = false);
void LaunchAddConstant(float* score, int n, float v, cudaStream_t s);
void LaunchScaleAdd(float* score, int n, float a, float b, cudaStream_t s);
void LaunchAddVector(float* score, const float* values, int n, cudaStream_t s);
// per-leaf (sum g, sum h) of float gradients over the leaf windows: partial[2 * (leaf * slices + slice) + {0,1}]
int LeafGradSumSlices();
void LaunchLeafGradSums(const LeafInfo* leaves, int num_leaves, const int* idx0, const int* idx1, const float* grad, const float* hess, double* partial, cudaStream_t s);

// Device form of one tree for traversal.
struct DevTree {
  int num_leaves;
  const int* left; const int* right; const int* split_feature; const int* split_group;
  const float* threshold; const int* threshold_bin; const signed char* decision; const float* leaf_value;
  const int* default_bin; const int* nan_bin; const int* bundled; const int* group_offset; const int* most_freq_bin; const int* num_bin;
  const unsigned int* cat_bits;   // [internal nodes][8]: bins that go left at a categorical node (decision bit 0)
};
// score[i] += scale * tree(row i) on binned rows (validation sets, out-of-bag rows, rollback)
void LaunchAddTreeBinned(const DevTree& t, const uint8_t* rows, int row_stride, int n, float scale, float* score, cudaStream_t s);

// Packed forest for raw-feature prediction: nodes of all trees in one array.
// flags: bit0 default_left, bits1-2 missing type, bit3 leaf (threshold = value), bit4 categorical (threshold holds,
// as an int, the offset of the node's category bitset in the forest's word array; bits 8.. = number of words)
struct ForestNode { float threshold; int feature; int left; int right; int flags; };
template <typename T>
void LaunchPredictRaw(const ForestNode* nodes, const unsigned int* cat_words, const int* tree_root, int num_trees, int num_class, const T* data, int nrow, int ncol, bool row_major,
                      float* out /* [num_class x nrow] */, bool average, cudaStream_t s);
void LaunchConvertOutput(int obj_kind, double sigmoid, float* out, int nrow, int num_class, cudaStream_t s);

// --------------------------------------------------------------- metrics ----
void LaunchPointwiseMetric(int metric_kind, int obj_kind, double sigmoid, const float* score, const float* label, const float* weight, int n, int num_class,
                           double* partial, int partial_capacity, double* out2, cudaStream_t s);

}  // namespace fb
