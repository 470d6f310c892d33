// Per-node feature masks on the device: feature_fraction_bynode and interaction constraints.
// One block per child of the level writes mask[child][inner feature] (1 = the split search may use it); the
// split-search kernel skips the rest. The draw is the host learner's (ColSampler::SampleByNode): the k smallest
// Philox keys (key, feature) among the features still allowed, keyed on (seed, tree, leaf id + 1000003 * depth).
// Parity: src/treelearner/col_sampler.hpp (GetByNode: interaction sets that contain the whole branch, then the
// per-node sample inside them).
#include "kernels.cuh"

namespace fb {

namespace {

constexpr int kMaskThreads = 256;

__global__ void __launch_bounds__(kMaskThreads) NodeMaskKernel(NodeMaskArgs a) {
  extern __shared__ unsigned int s_dyn[];
  unsigned int* s_key = s_dyn;                                  // [pool_size] Philox key of every pool feature
  unsigned char* s_ok = reinterpret_cast<unsigned char*>(s_dyn + a.pool_size);   // [pool_size] allowed by the interaction sets
  unsigned char* s_set = s_ok + a.pool_size;                    // [num_sets] the set applies to this node
  __shared__ int s_count;
  const int nchildren = a.ctrl != nullptr ? a.ctrl->num_children : a.num_children;
  if (static_cast<int>(blockIdx.x) >= nchildren) return;
  if (a.ctrl != nullptr && a.ctrl->skip_search) return;
  const FindChild ch = a.children[blockIdx.x];
  const int depth = a.leaves[ch.leaf].depth;
  unsigned char* row = a.mask + static_cast<size_t>(blockIdx.x) * a.num_inner;
  for (int f = threadIdx.x; f < a.num_inner; f += kMaskThreads) row[f] = 0;
  if (threadIdx.x == 0) s_count = 0;
  // interaction sets that hold every feature of the path
  const unsigned int* path = a.path_bits != nullptr ? a.path_bits + static_cast<size_t>(ch.leaf) * a.words : nullptr;
  for (int s = threadIdx.x; s < a.num_sets; s += kMaskThreads) {
    const unsigned int* set = a.set_bits + static_cast<size_t>(s) * a.words;
    bool applies = true;
    for (int w = 0; w < a.words; ++w) if ((path[w] & ~set[w]) != 0u) { applies = false; break; }
    s_set[s] = applies ? 1 : 0;
  }
  __syncthreads();
  const unsigned int node_key = static_cast<unsigned int>(ch.leaf + 1000003 * depth) + 1u;
  for (int i = threadIdx.x; i < a.pool_size; i += kMaskThreads) {
    const int f = a.pool[i];
    bool ok = true;
    if (a.num_sets > 0) {
      ok = false;
      const int rf = a.meta[f].real_index;
      if ((rf >> 5) < a.words) for (int s = 0; s < a.num_sets && !ok; ++s)
        if (s_set[s] && ((a.set_bits[static_cast<size_t>(s) * a.words + (rf >> 5)] >> (rf & 31)) & 1u)) ok = true;
    }
    s_ok[i] = ok ? 1 : 0;
    s_key[i] = Philox4x32_10(static_cast<unsigned int>(f), static_cast<unsigned int>(a.tree_index), node_key, 0x51ED27u, a.seed, 0xC0FFEEu).v[0];
    if (ok) atomicAdd(&s_count, 1);
  }
  __syncthreads();
  const int allowed = s_count;
  if (allowed == 0) return;
  int k = allowed;
  if (a.fraction < 1.0) {
    k = static_cast<int>(floor(a.fraction * static_cast<double>(allowed) + 0.5));
    k = max(1, min(k, allowed));
  }
  for (int i = threadIdx.x; i < a.pool_size; i += kMaskThreads) {
    if (!s_ok[i]) continue;
    bool in = true;
    if (k < allowed) {
      // rank of (key, feature) among the allowed pool entries; the pool lists features in ascending order
      const unsigned int key = s_key[i];
      int rank = 0;
      for (int j = 0; j < a.pool_size; ++j) rank += (s_ok[j] && (s_key[j] < key || (s_key[j] == key && j < i))) ? 1 : 0;
      in = rank < k;
    }
    if (in) row[a.pool[i]] = 1;
  }
}

// children of a split inherit the parent's path plus the split feature (real index)
__global__ void PathBitsKernel(const LevelCtrl* ctrl, const SplitJournal* journal, const FeatureMeta* meta, unsigned int* path_bits, int words, int max_splits) {
  const int s = blockIdx.x;
  if (s >= ctrl->num_splits || s >= max_splits) return;
  const SplitJournal j = journal[ctrl->journal_count - ctrl->num_splits + s];
  const int rf = meta[j.rec.feature].real_index;
  unsigned int* pl = path_bits + static_cast<size_t>(j.leaf) * words;
  unsigned int* pr = path_bits + static_cast<size_t>(j.right_leaf) * words;
  for (int w = threadIdx.x; w < words; w += blockDim.x) {
    const unsigned int v = pl[w] | ((w == (rf >> 5)) ? (1u << (rf & 31)) : 0u);
    pl[w] = v; pr[w] = v;
  }
}

}  // namespace

size_t NodeMaskSharedBytes(const NodeMaskArgs& a) {
  return sizeof(unsigned int) * static_cast<size_t>(a.pool_size) + static_cast<size_t>(a.pool_size) + static_cast<size_t>(a.num_sets) + 16;
}

void LaunchNodeMask(const NodeMaskArgs& a, cudaStream_t s) {
  if (a.num_children <= 0 || a.pool_size <= 0) return;
  const size_t sm = NodeMaskSharedBytes(a);
  static size_t attr = 48 * 1024;
  if (sm > attr) { FB_CUDA(cudaFuncSetAttribute(NodeMaskKernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sm))); attr = sm; }
  NodeMaskKernel<<<a.num_children, kMaskThreads, sm, s>>>(a); FB_LAUNCHED(); FB_KERNEL_CHECK();
}

void LaunchPathBits(const LevelCtrl* ctrl, const SplitJournal* journal, const FeatureMeta* meta, unsigned int* path_bits, int words, int max_splits, cudaStream_t s) {
  if (max_splits <= 0 || words <= 0) return;
  PathBitsKernel<<<max_splits, 64, 0, s>>>(ctrl, journal, meta, path_bits, words, max_splits); FB_LAUNCHED(); FB_KERNEL_CHECK();
}

}  // namespace fb
