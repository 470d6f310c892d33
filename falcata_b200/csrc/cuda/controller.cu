// K8: device-side level controller. One block decides, between two levels, which frontier leaves
// split (all of them, or the highest gains when the leaf budget binds; ties: lower leaf id), numbers
// the new leaves, and writes everything the next level's kernels need: partition descriptors, child
// bookkeeping, the smaller children's construct allotments, the search children, the journal entry of
// every split and the new frontier. The host never looks at a level: it enqueues the kernels of
// several levels ahead and reads the journal once per tree.
// Parity: src/treelearner/cuda/cuda_hybrid_graph.cu:L220-631 (device controller of the graph loop),
// cuda_single_gpu_tree_learner.cpp:L1355-1478 (CollectSplittableLeaves / ArbitrateLevelBudget),
// L1718-1775 (FinishLevelBookkeeping). The selection rule is the one of the host-driven loop and of
// the host learner's `level` policy, so all three grow identical trees.
#include "kernels.cuh"

namespace fb {

namespace {

constexpr int kCtrlThreads = 256;
constexpr int kCtrlMaxLeaves = 1024;

__global__ void InitLevelCtrlKernel(LevelCtrl* c, int* frontier) {
  c->num_leaves = 1; c->next_slot = 1; c->done = 0; c->level = 0; c->num_splits = 0; c->num_children = 1; c->total_chunks = 0; c->total_blocks = 0;
  c->frontier_count = 1; c->journal_count = 0; c->pad0 = 0; c->skip_search = 0; c->num_eval = 0; c->pad1 = 0;
  frontier[0] = 0;
}

__global__ void __launch_bounds__(kCtrlThreads) LevelControllerKernel(CtrlArgs a) {
  __shared__ int s_leaf[kCtrlMaxLeaves];      // candidate leaves, later the chosen leaves in ascending order
  __shared__ double s_gain[kCtrlMaxLeaves / 2];   // gains as doubles for exact comparison (frontier <= max_leaves, candidates <= max_leaves / 2 + ...)
  __shared__ int s_order[kCtrlMaxLeaves];
  __shared__ int s_chunks[kCtrlMaxLeaves / 2 + 1], s_blocks[kCtrlMaxLeaves / 2 + 1];
  __shared__ double s_first[2 * kCtrlMaxLeaves + 2];   // leaf-wise growth: first order-key step of every evaluated node
  __shared__ int s_ncand, s_nkeep;
  LevelCtrl* c = a.ctrl;
  const int nfront = c->done ? 0 : c->frontier_count;
  if (threadIdx.x == 0) { s_ncand = 0; s_nkeep = 0; }
  __syncthreads();
  // 1. candidates: frontier leaves with a usable split
  for (int i = threadIdx.x; i < nfront; i += kCtrlThreads) {
    const int l = a.frontier[i];
    const SplitRecord& b = a.best[l];
    if (b.feature >= 0 && b.gain > 0.0) { const int p = atomicAdd(&s_ncand, 1); s_leaf[p] = l; }
  }
  __syncthreads();
  const int ncand = s_ncand;
  const int budget = a.max_leaves - c->num_leaves;
  if (a.leafwise_budget > 0) {
    // 2'. leaf-wise: record the order keys of the newly evaluated nodes, then keep the candidates with fewer than
    //     leafwise_budget evaluated nodes strictly before them; if the growth cap binds, the best of those by rank
    const int base_eval = c->num_eval;
    for (int i = threadIdx.x; i < ncand; i += kCtrlThreads) {
      const int li = s_leaf[i];
      LeafwiseChildKey(a.leaves[li].pkey, a.best[li].gain, a.eval_key + static_cast<size_t>(base_eval + i) * 4);
    }
    __syncthreads();
    const int total = base_eval + ncand;
    // first key step of every evaluated node in shared memory: it decides nearly every comparison
    for (int j = threadIdx.x; j < total; j += kCtrlThreads) s_first[j] = a.eval_key[static_cast<size_t>(j) * 4];
    __syncthreads();
    {
      // one warp per candidate, the lanes stride over the evaluated nodes
      const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
      for (int i = warp; i < ncand; i += kCtrlThreads / 32) {
        double ki[4]; for (int k = 0; k < 4; ++k) ki[k] = a.eval_key[static_cast<size_t>(base_eval + i) * 4 + k];
        int cnt = 0;
        for (int j = lane; j < total; j += 32) {
          const double pj = s_first[j];
          bool before = pj > ki[0];
          if (pj == ki[0]) before = LeafwiseKeyBefore(a.eval_key + static_cast<size_t>(j) * 4, ki);
          cnt += before ? 1 : 0;
        }
        for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
        if (lane == 0) s_order[i] = cnt < a.leafwise_budget ? cnt : 0x7fffffff;
      }
    }
    __syncthreads();
    unsigned int keep_bits = 0;   // this thread's decisions, one bit per stride step (written back after all ranks were read)
    for (int i = threadIdx.x, step = 0; i < ncand; i += kCtrlThreads, ++step) {
      const int ri = s_order[i];
      bool keep = ri != 0x7fffffff;
      if (keep) { int better = 0; for (int j = 0; j < ncand; ++j) better += (s_order[j] < ri) || (s_order[j] == ri && s_leaf[j] < s_leaf[i]); keep = better < budget; }
      if (keep) keep_bits |= 1u << step;
    }
    __syncthreads();
    for (int i = threadIdx.x, step = 0; i < ncand; i += kCtrlThreads, ++step) s_order[i] = (keep_bits >> step) & 1u;
    if (threadIdx.x == 0) c->num_eval = total;
  } else {
  // 2. rank by (gain desc, leaf asc) when the budget binds; 3. order the kept ones by leaf id
  for (int i = threadIdx.x; i < ncand; i += kCtrlThreads) {
    const int li = s_leaf[i]; const double gi = a.best[li].gain;
    bool keep = true;
    if (ncand > budget) {
      int better = 0;
      for (int j = 0; j < ncand; ++j) { const int lj = s_leaf[j]; const double gj = a.best[lj].gain; better += (gj > gi) || (gj == gi && lj < li); }
      keep = better < budget;
    }
    s_order[i] = keep ? 1 : 0;
  }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < ncand; i += kCtrlThreads) {
    if (!s_order[i]) continue;
    const int li = s_leaf[i];
    int pos = 0;
    for (int j = 0; j < ncand; ++j) pos += (s_order[j] && s_leaf[j] < li);
    // chosen leaves go to the upper half of a scratch view: write after everyone has read
    reinterpret_cast<int*>(s_gain)[pos] = li;
    atomicAdd(&s_nkeep, 1);
  }
  __syncthreads();
  const int S = s_nkeep;
  int* chosen = reinterpret_cast<int*>(s_gain);
  // 4. local allotments (chunks of the partition, blocks of the construct) and their prefixes
  for (int s = threadIdx.x; s < S; s += kCtrlThreads) {
    const int cnt = a.leaves[chosen[s]].count;
    s_chunks[s] = (cnt + kPartChunk - 1) / kPartChunk;
    s_blocks[s] = max(1, (cnt + a.rows_per_block - 1) / a.rows_per_block);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int ac = 0, ab = 0;
    for (int s = 0; s < S; ++s) { const int t = s_chunks[s]; s_chunks[s] = ac; ac += t; const int u = s_blocks[s]; s_blocks[s] = ab; ab += u; }
    s_chunks[S] = ac; s_blocks[S] = ab;
  }
  __syncthreads();
  // 5. descriptors
  const int base_leaf = c->num_leaves, base_slot = c->next_slot, base_journal = c->journal_count;
  for (int s = threadIdx.x; s < S; s += kCtrlThreads) {
    const int l = chosen[s];
    const int right = base_leaf + s;
    const LeafInfo P = a.leaves[l];
    const SplitRecord b = a.best[l];
    const FeatureMeta m = a.meta[b.feature];
    PartSplit q;
    q.leaf = l; q.right_leaf = right; q.begin = P.begin; q.count = P.count; q.buffer = P.buffer; q.group = m.group; q.bundled = m.bundled; q.group_offset = m.group_offset;
    q.num_bin = m.num_bin; q.most_freq_bin = m.most_freq_bin; q.threshold = b.threshold; q.default_left = b.default_left; q.missing_type = m.missing_type;
    q.default_bin = m.default_bin; q.is_categorical = b.is_categorical; for (int w = 0; w < 8; ++w) q.cat_bitset[w] = b.cat_bitset[w];
    q.chunk_begin = s_chunks[s]; q.num_chunks = s_chunks[s + 1] - s_chunks[s]; q.pad_[0] = q.pad_[1] = 0;
    q.owner = a.bin_owner != nullptr ? a.bin_owner[m.hist_offset] : 0;
    a.splits[s] = q;
    ChildInit ci;
    ci.smaller_is_left = b.left_cnt <= b.right_cnt ? 1 : 0;
    const int fresh = base_slot + s;
    ci.left_slot = ci.smaller_is_left ? fresh : P.hist_slot; ci.right_slot = ci.smaller_is_left ? P.hist_slot : fresh;
    ci.left_g = b.left_g; ci.left_h = b.left_h; ci.right_g = b.right_g; ci.right_h = b.right_h; ci.left_out = b.left_out; ci.right_out = b.right_out;
    ci.left_gi = b.left_gi; ci.left_hi = b.left_hi; ci.right_gi = P.sum_gi - b.left_gi; ci.right_hi = P.sum_hi - b.left_hi;
    ci.hist_block_begin = s_blocks[s]; ci.hist_num_blocks = s_blocks[s + 1] - s_blocks[s];
    ci.monotone = b.monotone; ci.pad_ = 0; LeafwiseChildKey(P.pkey, b.gain, ci.pkey);
    a.child_init[s] = ci;
    FindChild fl, fr;
    fl.leaf = l; fl.slot = ci.left_slot; fl.other_slot = ci.right_slot; fl.is_larger = ci.smaller_is_left ? 0 : 1; fl.split = s; fl.is_left = 1; fl.parent_global = P.num_data_global; fl.task = s;
    fr.leaf = right; fr.slot = ci.right_slot; fr.other_slot = ci.left_slot; fr.is_larger = ci.smaller_is_left ? 1 : 0; fr.split = s; fr.is_left = 0; fr.parent_global = P.num_data_global; fr.task = s;
    a.children[2 * s] = fl; a.children[2 * s + 1] = fr;
    SplitJournal j; j.leaf = l; j.right_leaf = right; j.parent_global = P.num_data_global; j.pad = 0; j.rec = b;
    j.begin = P.begin; j.count = P.count; j.buffer = P.buffer; j.depth = P.depth;
    a.journal[base_journal + s] = j;
  }
  __syncthreads();
  // 6. new frontier (children in split order) and the level record
  for (int s = threadIdx.x; s < S; s += kCtrlThreads) { a.frontier[2 * s] = chosen[s]; a.frontier[2 * s + 1] = base_leaf + s; }
  if (threadIdx.x == 0) {
    c->num_leaves = base_leaf + S; c->next_slot = base_slot + S; c->journal_count = base_journal + S; c->level += 1;
    // A level that uses up the leaf budget ends the tree: its children are partitioned (the score update and the
    // leaf counts need their windows) but neither constructed nor searched.
    const bool last = base_leaf + S >= a.max_leaves;
    c->num_splits = S; c->num_children = 2 * S; c->total_chunks = s_chunks[S]; c->total_blocks = last ? 0 : s_blocks[S];
    c->skip_search = last ? 1 : 0;
    c->frontier_count = last ? 0 : 2 * S;
    if (S == 0) c->done = 1; else c->pad0 = c->level;   // pad0: last level that applied a split
  }
}

}  // namespace

void LaunchInitLevelCtrl(LevelCtrl* ctrl, int* frontier, cudaStream_t s) {
  InitLevelCtrlKernel<<<1, 1, 0, s>>>(ctrl, frontier);
  FB_LAUNCHED(); FB_KERNEL_CHECK();
}

void LaunchLevelController(const CtrlArgs& a, cudaStream_t s) {
  if (a.max_leaves > kCtrlMaxLeaves) Log::Fatal("The device controller handles up to %d leaves", kCtrlMaxLeaves);
  LevelControllerKernel<<<1, kCtrlThreads, 0, s>>>(a);
  FB_LAUNCHED(); FB_KERNEL_CHECK();
}

}  // namespace fb
