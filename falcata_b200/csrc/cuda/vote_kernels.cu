// K15: voting-parallel training on the device (PV-Tree). The vote is an all-gather done with plain
// stores into every peer's slot array; the reduce-scatter that follows moves only the bins of the voted
// features, straight from the local histogram pool into the owner ranks' staging slots. No NCCL call.
// Parity: src/treelearner/voting_parallel_tree_learner.cpp:L152-182 (local top-k, global vote),
// L365-397 (reduce of the voted features only, search on the reduced bins).
#include "kernels.cuh"

namespace fb {

namespace {

constexpr int kVoteThreads = 128;
constexpr int kVoteMaxFeatures = 8192;

__device__ inline int NumChildren(const VoteArgs& a) { return a.ctrl != nullptr ? a.ctrl->num_children : a.num_children; }

// Local totals of a child: every row falls into exactly one bin of a feature group, so the sum of one
// constructed group's bins is the leaf total. The larger child's bins are still parent - smaller at this point.
__global__ void VoteLocalSumsKernel(VoteArgs a) {
  if (static_cast<int>(blockIdx.x) >= NumChildren(a)) return;
  const FindChild ch = a.children[blockIdx.x];
  const int lane = threadIdx.x;
  long long gi = 0, hi = 0; double gd = 0, hd = 0;
  for (int j = lane; j < a.g0_bins; j += 32) {
    if (a.quant) {
      hist_q_t v = static_cast<const hist_q_t*>(a.local_pool)[static_cast<long long>(ch.slot) * a.local_stride + a.g0_begin + j];
      if (ch.is_larger) v -= static_cast<const hist_q_t*>(a.local_pool)[static_cast<long long>(ch.other_slot) * a.local_stride + a.g0_begin + j];
      gi += HistQGrad(v); hi += HistQHess(v);
    } else {
      double2 v = static_cast<const double2*>(a.local_pool)[static_cast<long long>(ch.slot) * a.local_stride + a.g0_begin + j];
      if (ch.is_larger) { const double2 o = static_cast<const double2*>(a.local_pool)[static_cast<long long>(ch.other_slot) * a.local_stride + a.g0_begin + j]; v.x -= o.x; v.y -= o.y; }
      gd += v.x; hd += v.y;
    }
  }
  for (int o = 16; o > 0; o >>= 1) {
    gi += __shfl_xor_sync(0xffffffffu, gi, o); hi += __shfl_xor_sync(0xffffffffu, hi, o);
    gd += __shfl_xor_sync(0xffffffffu, gd, o); hd += __shfl_xor_sync(0xffffffffu, hd, o);
  }
  if (lane == 0) {
    VoteLocalSum s; s.gi = gi; s.hi = hi; s.g = gd; s.h = hd;
    if (a.quant) { s.g = FB_MUL(static_cast<double>(gi), static_cast<double>(a.scales[0])); s.h = FB_MUL(static_cast<double>(hi), static_cast<double>(a.scales[1])); }
    a.sums[blockIdx.x] = s;
  }
}

// Block argmax helper: larger key first, then the lower index.
template <typename K>
__device__ inline void BlockArgBest(K key, int idx, K* s_key, int* s_idx, K* out_key, int* out_idx) {
  s_key[threadIdx.x] = key; s_idx[threadIdx.x] = idx;
  __syncthreads();
  for (int o = blockDim.x / 2; o > 0; o >>= 1) {
    if (threadIdx.x < o) {
      const K k2 = s_key[threadIdx.x + o]; const int i2 = s_idx[threadIdx.x + o];
      const K k1 = s_key[threadIdx.x]; const int i1 = s_idx[threadIdx.x];
      const bool take = i2 >= 0 && (i1 < 0 || k2 > k1 || (k2 == k1 && i2 < i1));
      if (take) { s_key[threadIdx.x] = k2; s_idx[threadIdx.x] = i2; }
    }
    __syncthreads();
  }
  *out_key = s_key[0]; *out_idx = s_idx[0];
  __syncthreads();
}

// The rank's top_k features of one child by local gain (ties: the earlier searched feature), stored into
// the vote slots of every rank.
__global__ void __launch_bounds__(kVoteThreads) VoteTopKKernel(VoteArgs a) {
  if (static_cast<int>(blockIdx.x) >= NumChildren(a)) { FabricSignalDone(a.vote_sig, gridDim.x); return; }
  __shared__ unsigned char s_taken[kVoteMaxFeatures];
  __shared__ double s_key[kVoteThreads]; __shared__ int s_idx[kVoteThreads];
  __shared__ int s_votes[64];
  const int F = a.num_searched;
  for (int i = threadIdx.x; i < F; i += kVoteThreads) s_taken[i] = 0;
  __syncthreads();
  const CandLite* cand = a.cand_local + static_cast<size_t>(blockIdx.x) * F;
  for (int r = 0; r < a.top_k; ++r) {
    double bk = 0; int bi = -1;
    for (int i = threadIdx.x; i < F; i += kVoteThreads) {
      if (s_taken[i] || cand[i].feature < 0) continue;
      const double g = cand[i].gain;
      if (bi < 0 || g > bk) { bk = g; bi = i; }
    }
    double wk; int wi;
    BlockArgBest<double>(bk, bi, s_key, s_idx, &wk, &wi);
    if (threadIdx.x == 0) { s_votes[r] = wi >= 0 ? cand[wi].feature : -1; if (wi >= 0) s_taken[wi] = 1; }
    __syncthreads();
  }
  for (int p = 0; p < a.world; ++p)
    for (int r = threadIdx.x; r < a.top_k; r += kVoteThreads) a.peer_votes[p][static_cast<size_t>(blockIdx.x) * a.top_k + r] = s_votes[r];
  FabricSignalDone(a.vote_sig, gridDim.x, true);
}

// Vote count, choice of the 2*top_k most voted features (ties: the lower feature), and the restricted
// reduce-scatter: only the chosen features' local bins go to their owners' staging slots.
__global__ void __launch_bounds__(kVoteThreads) VoteTallyPushKernel(VoteArgs a) {
  if (static_cast<int>(blockIdx.x) >= NumChildren(a)) { FabricSignalDone(a.hist_sig, gridDim.x); return; }
  FabricWaitAll(a.vote_wait);
  __shared__ int s_cnt[kVoteMaxFeatures];
  __shared__ int s_key[kVoteThreads]; __shared__ int s_idx[kVoteThreads];
  __shared__ int s_sel[128];
  __shared__ int s_nsel;
  const int F = a.num_inner_features;
  const int child = blockIdx.x;
  for (int i = threadIdx.x; i < F; i += kVoteThreads) { s_cnt[i] = 0; a.voted[static_cast<size_t>(child) * F + i] = 0; }
  if (threadIdx.x == 0) s_nsel = 0;
  __syncthreads();
  for (int e = threadIdx.x; e < a.world * a.top_k; e += kVoteThreads) {
    const int r = e / a.top_k, k = e % a.top_k;
    const int f = __ldcg(a.votes_all + (static_cast<size_t>(r) * a.child_cap + child) * a.top_k + k);
    if (f >= 0 && f < F) atomicAdd(&s_cnt[f], 1);
  }
  __syncthreads();
  const int want = min(2 * a.top_k, F);
  for (int r = 0; r < want; ++r) {
    int bk = 0, bi = -1;
    for (int i = threadIdx.x; i < F; i += kVoteThreads) {
      const int c = s_cnt[i];
      if (c <= 0) continue;
      if (bi < 0 || c > bk) { bk = c; bi = i; }
    }
    int wk, wi;
    BlockArgBest<int>(bk, bi, s_key, s_idx, &wk, &wi);
    if (wi < 0) break;   // uniform: every thread sees the same result
    if (threadIdx.x == 0) { s_sel[s_nsel++] = wi; s_cnt[wi] = 0; a.voted[static_cast<size_t>(child) * F + wi] = 1; }
    __syncthreads();
  }
  __syncthreads();
  const FindChild ch = a.children[child];
  const int nsel = s_nsel;
  for (int q = 0; q < nsel; ++q) {
    const FeatureMeta m = a.meta[s_sel[q]];
    const int nstored = m.bundled ? m.num_bin - 1 : m.num_bin;
    const int owner = a.bin_owner[m.hist_offset];
    const long long dst0 = (static_cast<long long>(a.rank) * a.stage_cap + child) * a.slot_stride[owner] + a.bin_local[m.hist_offset];
    const long long src0 = static_cast<long long>(ch.slot) * a.local_stride + m.hist_offset;
    for (int b = threadIdx.x; b < nstored; b += kVoteThreads) {
      if (a.quant) static_cast<hist_q_t*>(a.peer_stage[owner])[dst0 + b] = static_cast<const hist_q_t*>(a.local_pool)[src0 + b];
      else static_cast<double2*>(a.peer_stage[owner])[dst0 + b] = static_cast<const double2*>(a.local_pool)[src0 + b];
    }
  }
  FabricSignalDone(a.hist_sig, gridDim.x, true);
}

}  // namespace

void LaunchVoteLocalSums(const VoteArgs& a, cudaStream_t s) {
  if (a.num_children <= 0) return;
  VoteLocalSumsKernel<<<a.num_children, 32, 0, s>>>(a); FB_LAUNCHED(); FB_KERNEL_CHECK();
}
void LaunchVoteTopK(const VoteArgs& a, cudaStream_t s) {
  if (a.num_children <= 0) return;
  if (a.num_searched > kVoteMaxFeatures || a.num_inner_features > kVoteMaxFeatures) Log::Fatal("Voting on the device covers up to %d features", kVoteMaxFeatures);
  if (a.top_k > 64) Log::Fatal("Voting on the device covers top_k up to 64");
  VoteTopKKernel<<<a.num_children, kVoteThreads, 0, s>>>(a); FB_LAUNCHED(); FB_KERNEL_CHECK();
}
void LaunchVoteTallyPush(const VoteArgs& a, cudaStream_t s) {
  if (a.num_children <= 0) return;
  VoteTallyPushKernel<<<a.num_children, kVoteThreads, 0, s>>>(a); FB_LAUNCHED(); FB_KERNEL_CHECK();
}

}  // namespace fb
