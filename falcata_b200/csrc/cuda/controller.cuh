// K8: the level controller as a device function, shared by its own kernel and by the fused tail of the
// split search (the last block of the search grid runs it, so a level needs no controller launch).
// One block decides, between two levels, which frontier leaves split (all of them, or the highest gains
// when the leaf budget binds; ties: lower leaf id), numbers the new leaves, and writes everything the next
// level's kernels need: partition descriptors, child bookkeeping, the smaller children's construct
// allotments, the search children, the journal entry of every split and the new frontier.
// Parity: src/treelearner/cuda/cuda_hybrid_graph.cu:L220-631 (device controller of the graph loop),
// cuda_single_gpu_tree_learner.cpp:L1355-1478 (CollectSplittableLeaves / ArbitrateLevelBudget),
// L1718-1775 (FinishLevelBookkeeping). The selection rule is the one of the host-driven loop and of
// the host learner's `level` policy, so all three grow identical trees.
#pragma once
#include "kernels.cuh"

namespace fb {

constexpr int kCtrlMaxLeaves = 1024;

// Shared-memory working set of the controller (the caller provides it: a kernel's static shared memory).
struct CtrlShared {
  int leaf[kCtrlMaxLeaves];            // candidate leaves, later the chosen leaves in ascending order
  double gain[kCtrlMaxLeaves / 2];     // scratch view: the chosen leaves as ints
  int order[kCtrlMaxLeaves];
  int chunks[kCtrlMaxLeaves / 2 + 1], blocks[kCtrlMaxLeaves / 2 + 1];
  double first[2 * kCtrlMaxLeaves + 2];   // leaf-wise growth: first order-key step of every evaluated node
  int ncand, nkeep;
};

// A record that another block of the SAME launch may have written a moment ago: read through L2, in 8-byte pieces
// where the type allows it (the loads of one record are independent and issue back to back).
template <typename T>
__device__ inline T LoadWords(const T* p) {
  static_assert(sizeof(T) % 4 == 0, "word-sized records only");
  T v;
  if constexpr (sizeof(T) % 8 == 0 && alignof(T) >= 8) {
    const unsigned long long* s = reinterpret_cast<const unsigned long long*>(p);
    unsigned long long* d = reinterpret_cast<unsigned long long*>(&v);
#pragma unroll
    for (int w = 0; w < static_cast<int>(sizeof(T) / 8); ++w) d[w] = __ldcg(s + w);
  } else {
    const unsigned int* s = reinterpret_cast<const unsigned int*>(p);
    unsigned int* d = reinterpret_cast<unsigned int*>(&v);
#pragma unroll
    for (int w = 0; w < static_cast<int>(sizeof(T) / 4); ++w) d[w] = __ldcg(s + w);
  }
  return v;
}

// Call with all T threads of one block. Reads the level record `a.cur`, writes the next level's into `a.nxt`.
template <int T>
__device__ inline void ControllerBody(const CtrlArgs& a, CtrlShared& S) {
  int num_eval_out = LoadWords(&a.cur->num_eval);
  // the level record is read whole before anything is written: `cur` and `nxt` may be the same object
  const LevelCtrl c0 = LoadWords(a.cur);
  LevelCtrl* c = a.nxt;
  const int nfront = c0.done ? 0 : c0.frontier_count;
  if (threadIdx.x == 0) { S.ncand = 0; S.nkeep = 0; }
  __syncthreads();
  // 1. candidates: frontier leaves with a usable split
  for (int i = threadIdx.x; i < nfront; i += T) {
    const int l = a.frontier[i];
    const SplitRecord b = LoadWords(a.best + l);
    if (b.feature >= 0 && b.gain > 0.0) { const int p = atomicAdd(&S.ncand, 1); S.leaf[p] = l; }
  }
  __syncthreads();
  const int ncand = S.ncand;
  const int budget = a.max_leaves - c0.num_leaves;
  if (a.leafwise_budget > 0) {
    // 2'. leaf-wise: record the order keys of the newly evaluated nodes, then keep the candidates with fewer than
    //     leafwise_budget evaluated nodes strictly before them; if the growth cap binds, the best of those by rank
    const int base_eval = c0.num_eval;
    for (int i = threadIdx.x; i < ncand; i += T) {
      const int li = S.leaf[i];
      LeafwiseChildKey(LoadWords(a.leaves + li).pkey, LoadWords(a.best + li).gain, a.eval_key + static_cast<size_t>(base_eval + i) * 4);
    }
    __syncthreads();
    const int total = base_eval + ncand;
    // first key step of every evaluated node in shared memory: it decides nearly every comparison
    for (int j = threadIdx.x; j < total; j += T) S.first[j] = a.eval_key[static_cast<size_t>(j) * 4];
    __syncthreads();
    {
      // one warp per candidate, the lanes stride over the evaluated nodes
      const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
      for (int i = warp; i < ncand; i += T / 32) {
        double ki[4]; for (int k = 0; k < 4; ++k) ki[k] = a.eval_key[static_cast<size_t>(base_eval + i) * 4 + k];
        int cnt = 0;
        for (int j = lane; j < total; j += 32) {
          const double pj = S.first[j];
          bool before = pj > ki[0];
          if (pj == ki[0]) before = LeafwiseKeyBefore(a.eval_key + static_cast<size_t>(j) * 4, ki);
          cnt += before ? 1 : 0;
        }
        for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
        if (lane == 0) S.order[i] = cnt < a.leafwise_budget ? cnt : 0x7fffffff;
      }
    }
    __syncthreads();
    unsigned int keep_bits = 0;   // this thread's decisions, one bit per stride step (written back after all ranks were read)
    for (int i = threadIdx.x, step = 0; i < ncand; i += T, ++step) {
      const int ri = S.order[i];
      bool keep = ri != 0x7fffffff;
      if (keep) { int better = 0; for (int j = 0; j < ncand; ++j) better += (S.order[j] < ri) || (S.order[j] == ri && S.leaf[j] < S.leaf[i]); keep = better < budget; }
      if (keep) keep_bits |= 1u << step;
    }
    __syncthreads();
    for (int i = threadIdx.x, step = 0; i < ncand; i += T, ++step) S.order[i] = (keep_bits >> step) & 1u;
    num_eval_out = total;
  } else {
  // 2. rank by (gain desc, leaf asc) when the budget binds; 3. order the kept ones by leaf id
  for (int i = threadIdx.x; i < ncand; i += T) {
    const int li = S.leaf[i]; const double gi = LoadWords(&a.best[li].gain);
    bool keep = true;
    if (ncand > budget) {
      int better = 0;
      for (int j = 0; j < ncand; ++j) { const int lj = S.leaf[j]; const double gj = LoadWords(&a.best[lj].gain); better += (gj > gi) || (gj == gi && lj < li); }
      keep = better < budget;
    }
    S.order[i] = keep ? 1 : 0;
  }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < ncand; i += T) {
    if (!S.order[i]) continue;
    const int li = S.leaf[i];
    int pos = 0;
    for (int j = 0; j < ncand; ++j) pos += (S.order[j] && S.leaf[j] < li);
    // chosen leaves go to the upper half of a scratch view: write after everyone has read
    reinterpret_cast<int*>(S.gain)[pos] = li;
    atomicAdd(&S.nkeep, 1);
  }
  __syncthreads();
  const int NS = S.nkeep;
  int* chosen = reinterpret_cast<int*>(S.gain);
  // 4. local allotments (chunks of the partition, blocks of the construct) and their prefixes
  for (int s = threadIdx.x; s < NS; s += T) {
    const int cnt = LoadWords(&a.leaves[chosen[s]].count);
    S.chunks[s] = max(1, (cnt + kPartChunk - 1) / kPartChunk);   // at least one: the chunk block of a split also sets up its children
    S.blocks[s] = max(1, (cnt + a.rows_per_block - 1) / a.rows_per_block);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int ac = 0, ab = 0;
    for (int s = 0; s < NS; ++s) { const int t = S.chunks[s]; S.chunks[s] = ac; ac += t; const int u = S.blocks[s]; S.blocks[s] = ab; ab += u; }
    S.chunks[NS] = ac; S.blocks[NS] = ab;
  }
  __syncthreads();
  // 5. descriptors
  const int base_leaf = c0.num_leaves, base_slot = c0.next_slot, base_journal = c0.journal_count;
  for (int s = threadIdx.x; s < NS; s += T) {
    const int l = chosen[s];
    const int right = base_leaf + s;
    const LeafInfo P = LoadWords(a.leaves + l);
    const SplitRecord b = LoadWords(a.best + l);
    const FeatureMeta m = a.meta[b.feature];
    PartSplit q;
    q.leaf = l; q.right_leaf = right; q.begin = P.begin; q.count = P.count; q.buffer = P.buffer; q.group = m.group; q.bundled = m.bundled; q.group_offset = m.group_offset;
    q.num_bin = m.num_bin; q.most_freq_bin = m.most_freq_bin; q.threshold = b.threshold; q.default_left = b.default_left; q.missing_type = m.missing_type;
    q.default_bin = m.default_bin; q.is_categorical = b.is_categorical; for (int w = 0; w < 8; ++w) q.cat_bitset[w] = b.cat_bitset[w];
    q.chunk_begin = S.chunks[s]; q.num_chunks = S.chunks[s + 1] - S.chunks[s]; q.pad_[0] = q.pad_[1] = 0;
    q.owner = a.bin_owner != nullptr ? a.bin_owner[m.hist_offset] : 0;
    a.splits[s] = q;
    ChildInit ci;
    ci.smaller_is_left = b.left_cnt <= b.right_cnt ? 1 : 0;
    const int fresh = base_slot + s;
    ci.left_slot = ci.smaller_is_left ? fresh : P.hist_slot; ci.right_slot = ci.smaller_is_left ? P.hist_slot : fresh;
    ci.left_g = b.left_g; ci.left_h = b.left_h; ci.right_g = b.right_g; ci.right_h = b.right_h; ci.left_out = b.left_out; ci.right_out = b.right_out;
    ci.left_gi = b.left_gi; ci.left_hi = b.left_hi; ci.right_gi = P.sum_gi - b.left_gi; ci.right_hi = P.sum_hi - b.left_hi;
    ci.hist_block_begin = S.blocks[s]; ci.hist_num_blocks = S.blocks[s + 1] - S.blocks[s];
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
  for (int s = threadIdx.x; s < NS; s += T) { a.frontier[2 * s] = chosen[s]; a.frontier[2 * s + 1] = base_leaf + s; }
  if (threadIdx.x == 0) {
    LevelCtrl o = c0;
    o.num_leaves = base_leaf + NS; o.next_slot = base_slot + NS; o.journal_count = base_journal + NS; o.level = c0.level + 1; o.num_eval = num_eval_out;
    // A level that uses up the leaf budget ends the tree: its children are partitioned (the score update and the
    // leaf counts need their windows) but neither constructed nor searched.
    const bool last = base_leaf + NS >= a.max_leaves;
    o.num_splits = NS; o.num_children = 2 * NS; o.total_chunks = S.chunks[NS]; o.total_blocks = last ? 0 : S.blocks[NS];
    o.skip_search = last ? 1 : 0;
    o.frontier_count = last ? 0 : 2 * NS;
    if (NS == 0) o.done = 1; else o.pad0 = o.level;   // pad0: last level that applied a split
    *c = o;
  }
}

}  // namespace fb
