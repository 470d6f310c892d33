// K5: level-batched stable row partition. Three launches per level for ALL splitting leaves:
//   flags   : per 2048-row chunk, go-left ballot words + left count
//   scan    : per split, exclusive scan of its chunks' counts; child windows, leaf records and the
//             construct task of the smaller child are written here (no host round trip). With
//             `fused_scan` this step runs inside the flags launch, in the last chunk block of each split.
//   scatter : popc-ranked stable scatter into the other index buffer (ping-pong, no copy back)
// Parity: src/treelearner/cuda/cuda_data_partition.cu:L1380-1433 (ballot bit vectors, flat grid),
// L1479 (per-split scan), L1562-1617 (stable scatter), L1681-1840 (tree-structure bookkeeping),
// L1921 (copy back — removed here by the ping-pong buffers).
#include "kernels.cuh"

namespace fb {

namespace {

constexpr int kPartThreads = 256;
constexpr int kRowsPerThread = kPartChunk / kPartThreads;   // 8
constexpr int kWordsPerChunk = kPartChunk / 32;             // 64

__device__ inline int FindSplitOfChunk(const PartSplit* splits, int num_splits, int chunk) {
  int lo = 0, hi = num_splits - 1;
  while (lo < hi) { const int m = (lo + hi + 1) >> 1; if (splits[m].chunk_begin <= chunk) lo = m; else hi = m - 1; }
  return lo;
}

__device__ inline bool GoLeft(const PartSplit& sp, int gb) {
  int fb = gb;
  if (sp.bundled) {
    const int rel = gb - sp.group_offset;
    fb = (rel < 0 || rel >= sp.num_bin - 1) ? sp.most_freq_bin : (rel >= sp.most_freq_bin ? rel + 1 : rel);
  }
  if (sp.is_categorical) return (sp.cat_bitset[(fb >> 5) & 7] >> (fb & 31)) & 1;
  if ((sp.missing_type == 1 && fb == sp.default_bin) || (sp.missing_type == 2 && fb == sp.num_bin - 1)) return sp.default_left != 0;
  return fb <= sp.threshold;
}

// Per split: exclusive scan of its chunks' left counts, then the children's windows, leaf records and the smaller
// child's construct task (no host round trip). Call with all threads of one block.
__device__ inline void ScanSetupBody(const PartArgs& a, int si, int* s_scan, int* s_carry_p) {
  int& s_carry = *s_carry_p;
  const PartSplit sp = a.splits[si];
  if (threadIdx.x == 0) s_carry = 0;
  __syncthreads();
  for (int c0 = 0; c0 < sp.num_chunks; c0 += kPartThreads) {
    const int c = c0 + threadIdx.x;
    const int v = c < sp.num_chunks ? __ldcg(a.chunk_left + sp.chunk_begin + c) : 0;   // written by other blocks of this launch when fused
    s_scan[threadIdx.x] = v;
    __syncthreads();
    for (int o = 1; o < kPartThreads; o <<= 1) {
      const int t = threadIdx.x >= o ? s_scan[threadIdx.x - o] : 0;
      __syncthreads();
      s_scan[threadIdx.x] += t;
      __syncthreads();
    }
    if (c < sp.num_chunks) a.chunk_left[sp.chunk_begin + c] = s_carry + s_scan[threadIdx.x] - v;   // exclusive offset
    __syncthreads();
    if (threadIdx.x == kPartThreads - 1) s_carry += s_scan[threadIdx.x];
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    const int nl = s_carry, nr = sp.count - nl;
    a.split_left_total[si] = nl;
    // multi-rank: every rank learns every rank's left count (summed by the split search, which runs
    // after the construct-done flags; this store is ordered before them by the stream)
    if (a.world > 1) { for (int r = 0; r < a.world; ++r) a.peer_counts[r][si] = nl; __threadfence_system(); }
    const ChildInit ci = a.child_init[si];
    const LeafInfo parent = a.leaves[sp.leaf];
    LeafInfo L = parent, R = parent;
    L.count = nl; R.begin = parent.begin + nl; R.count = nr;
    L.buffer = R.buffer = sp.buffer ^ 1;
    L.depth = R.depth = parent.depth + 1;
    L.hist_slot = ci.left_slot; R.hist_slot = ci.right_slot;
    L.sum_g = ci.left_g; L.sum_h = ci.left_h; L.sum_gi = ci.left_gi; L.sum_hi = ci.left_hi; L.output = ci.left_out;
    R.sum_g = ci.right_g; R.sum_h = ci.right_h; R.sum_gi = ci.right_gi; R.sum_hi = ci.right_hi; R.output = ci.right_out;
    for (int k = 0; k < 4; ++k) L.pkey[k] = R.pkey[k] = ci.pkey[k];
    if (ci.monotone != 0) {   // "basic" monotone method: the children's ranges meet at the mid point of their outputs
      const double mid = (ci.left_out + ci.right_out) / 2.0;
      if (ci.monotone > 0) { L.max_c = fmin(L.max_c, mid); R.min_c = fmax(R.min_c, mid); }
      else { L.min_c = fmax(L.min_c, mid); R.max_c = fmin(R.max_c, mid); }
    }
    L.num_data_global = nl; R.num_data_global = nr;   // single rank: exact; multi-rank: summed over ranks by the exchange that follows
    a.leaves[sp.leaf] = L; a.leaves[sp.right_leaf] = R;
    HistTask t;
    const LeafInfo& S = ci.smaller_is_left ? L : R;
    t.slot = S.hist_slot; t.begin = S.begin; t.count = S.count; t.buffer = S.buffer; t.block_begin = ci.hist_block_begin; t.num_blocks = ci.hist_num_blocks; t.pad0 = t.pad1 = 0;
    a.hist_tasks[si] = t;
  }
}

__global__ void __launch_bounds__(kPartThreads) PartitionScanSetupKernel(PartArgs a) {
  const int si = blockIdx.x;
  if (si >= (a.ctrl != nullptr ? a.ctrl->num_splits : a.num_splits)) return;
  // feature-parallel: the bitmaps of this level come from the owners of the split features
  if (a.bc_world > 1) FabricWaitAll(a.bc_wait);
  __shared__ int s_scan[kPartThreads];
  __shared__ int s_carry;
  ScanSetupBody(a, si, s_scan, &s_carry);
}

// (The register cap keeps eight blocks per SM for the latency-bound chunk pass; the rarely taken scan step of the
// last block per split may spill.)
__global__ void __launch_bounds__(kPartThreads, 8) PartitionFlagsKernel(PartArgs a) {
  const int chunk = blockIdx.x;
  const int nsplits = a.ctrl != nullptr ? a.ctrl->num_splits : a.num_splits;
  const bool bc = a.bc_world > 1;
  if (chunk >= (a.ctrl != nullptr ? a.ctrl->total_chunks : a.total_chunks)) { if (bc) FabricSignalDone(a.bc_sig, gridDim.x); return; }
  const int si = FindSplitOfChunk(a.splits, nsplits, chunk);
  const PartSplit sp = a.splits[si];
  const int local_chunk = chunk - sp.chunk_begin;
  // feature-parallel: only the owner of the split feature reads the column; it writes every rank's bitmap
  if (local_chunk >= sp.num_chunks || (bc && sp.owner != a.bc_rank)) { if (bc) FabricSignalDone(a.bc_sig, gridDim.x); return; }
  const int* idx = a.idx[sp.buffer] + sp.begin;
  const int pos0 = local_chunk * kPartChunk;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int cnt = 0;
  // three separate unrolled passes keep eight independent row-id loads, then eight independent bin loads, in
  // flight per thread (the kernel is bound by the latency of this dependent pair, not by bandwidth)
  int rowv[kRowsPerThread]; int binv[kRowsPerThread];
#pragma unroll
  for (int k = 0; k < kRowsPerThread; ++k) {
    const int pos = pos0 + k * kPartThreads + threadIdx.x;
    rowv[k] = pos < sp.count ? idx[pos] : -1;
  }
#pragma unroll
  for (int k = 0; k < kRowsPerThread; ++k) {
    const int row = rowv[k];
    binv[k] = row < 0 ? 0 : (a.cols != nullptr ? a.cols[static_cast<size_t>(sp.group) * a.col_stride + row] : a.rows[static_cast<size_t>(row) * a.row_stride + sp.group]);
  }
#pragma unroll
  for (int k = 0; k < kRowsPerThread; ++k) {
    const bool left = rowv[k] >= 0 && GoLeft(sp, binv[k]);
    const unsigned int word = __ballot_sync(0xffffffffu, left);
    if (lane == 0) {
      const size_t wi = static_cast<size_t>(chunk) * kWordsPerChunk + k * (kPartThreads / 32) + warp;
      if (bc) { for (int r = 0; r < a.bc_world; ++r) a.peer_bits[r][wi] = word; } else a.bits[wi] = word;
      cnt += __popc(word);
    }
  }
  __shared__ int s_cnt[kPartThreads / 32];
  if (lane == 0) s_cnt[warp] = cnt;
  __syncthreads();
  if (threadIdx.x == 0) {
    int t = 0; for (int w = 0; w < kPartThreads / 32; ++w) t += s_cnt[w];
    if (bc) { for (int r = 0; r < a.bc_world; ++r) a.peer_chunk_left[r][chunk] = t; } else a.chunk_left[chunk] = t;
  }
  if (bc) FabricSignalDone(a.bc_sig, gridDim.x, true);
  if (!a.fused_scan) return;
  // fused scan + set-up: the last chunk block of a split finds all of the split's counts written and closes the split
  __shared__ int s_last;
  __shared__ int s_scan[kPartThreads];
  __shared__ int s_carry;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int prev = atomicAdd(a.split_done + si, 1u);
    s_last = (prev + 1 == static_cast<unsigned int>(sp.num_chunks)) ? 1 : 0;
    if (s_last) a.split_done[si] = 0;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  ScanSetupBody(a, si, s_scan, &s_carry);
}


__global__ void __launch_bounds__(kPartThreads) PartitionScatterKernel(PartArgs a) {
  const int chunk = blockIdx.x;
  const int nsplits = a.ctrl != nullptr ? a.ctrl->num_splits : a.num_splits;
  if (chunk >= (a.ctrl != nullptr ? a.ctrl->total_chunks : a.total_chunks)) return;
  const int si = FindSplitOfChunk(a.splits, nsplits, chunk);
  const PartSplit sp = a.splits[si];
  const int local_chunk = chunk - sp.chunk_begin;
  if (local_chunk >= sp.num_chunks) return;
  const int* src = a.idx[sp.buffer] + sp.begin;
  int* dst = a.idx[sp.buffer ^ 1] + sp.begin;
  const int total_left = a.split_left_total[si];
  const int left_before = a.chunk_left[chunk];
  const int pos0 = local_chunk * kPartChunk;
  const int right_before = pos0 - left_before;
  __shared__ unsigned int s_bits[kWordsPerChunk];
  __shared__ int s_pref[kWordsPerChunk];
  if (threadIdx.x < kWordsPerChunk) s_bits[threadIdx.x] = a.bits[static_cast<size_t>(chunk) * kWordsPerChunk + threadIdx.x];
  __syncthreads();
  if (threadIdx.x < 32) {
    // exclusive prefix of the 64 word counts by one warp: two words per lane, then a shuffle scan of the lane sums
    const int l = threadIdx.x;
    const int c0 = __popc(s_bits[2 * l]), c1 = __popc(s_bits[2 * l + 1]);
    int incl = c0 + c1;
    for (int o = 1; o < 32; o <<= 1) { const int y = __shfl_up_sync(0xffffffffu, incl, o); if (l >= o) incl += y; }
    const int excl = incl - (c0 + c1);
    s_pref[2 * l] = excl; s_pref[2 * l + 1] = excl + c0;
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int k = 0; k < kRowsPerThread; ++k) {
    const int in_chunk = k * kPartThreads + threadIdx.x;
    const int pos = pos0 + in_chunk;
    if (pos >= sp.count) continue;
    const int w = k * (kPartThreads / 32) + warp;
    const unsigned int word = s_bits[w];
    const int lefts_before_me = s_pref[w] + __popc(word & ((1u << lane) - 1u));
    const int row = src[pos];
    if ((word >> lane) & 1u) dst[left_before + lefts_before_me] = row;
    else dst[total_left + right_before + (in_chunk - lefts_before_me)] = row;
  }
}

__global__ void InitIndicesKernel(int* idx, int n) { const int i = blockIdx.x * blockDim.x + threadIdx.x; if (i < n) idx[i] = i; }

}  // namespace

void LaunchPartitionFlags(const PartArgs& a, cudaStream_t s) {
  if (a.total_chunks <= 0) return;
  PartitionFlagsKernel<<<a.total_chunks, kPartThreads, 0, s>>>(a);
  FB_LAUNCHED(); FB_KERNEL_CHECK();
}
void LaunchPartitionScanSetup(const PartArgs& a, cudaStream_t s) {
  if (a.num_splits <= 0 || a.fused_scan) return;   // fused: the flags kernel's last block per split did it
  PartitionScanSetupKernel<<<a.num_splits, kPartThreads, 0, s>>>(a);
  FB_LAUNCHED(); FB_KERNEL_CHECK();
}
void LaunchPartitionScatter(const PartArgs& a, cudaStream_t s) {
  if (a.total_chunks <= 0) return;
  PartitionScatterKernel<<<a.total_chunks, kPartThreads, 0, s>>>(a);
  FB_LAUNCHED(); FB_KERNEL_CHECK();
}
void LaunchInitIndices(int* idx, int n, cudaStream_t s) {
  if (n <= 0) return;
  InitIndicesKernel<<<(n + 255) / 256, 256, 0, s>>>(idx, n);
  FB_LAUNCHED(); FB_KERNEL_CHECK();
}

}  // namespace fb
