// K8 launchers: the stand-alone level controller (used when the search kernel's fused tail is off) and the
// per-tree initialisation of the device-side growth state.
#include "controller.cuh"

namespace fb {

namespace {

constexpr int kCtrlThreads = 256;

__global__ void __launch_bounds__(kCtrlThreads) LevelControllerKernel(CtrlArgs a) {
  __shared__ CtrlShared S;
  ControllerBody<kCtrlThreads>(a, S);
}

// One thread sets up everything a tree starts from, from the device-side gradient sums (no host round trip
// between quantization and the root histogram): the root leaf record, the level record of the root level,
// the frontier, the root's construct task and its search descriptor.
__global__ void InitTreeKernel(TreeInitArgs a) {
  LeafInfo L;
  L.begin = 0; L.count = a.n_local; L.buffer = 0; L.depth = 0; L.hist_slot = 0; L.num_data_global = static_cast<int>(a.n_global);
  if (a.quant) {
    L.sum_gi = a.sums_i[0]; L.sum_hi = a.sums_i[1];
    L.sum_g = FB_MUL(static_cast<double>(L.sum_gi), static_cast<double>(a.scales[0])); L.sum_h = FB_MUL(static_cast<double>(L.sum_hi), static_cast<double>(a.scales[1]));
  } else { L.sum_gi = L.sum_hi = 0; L.sum_g = a.sums_d[0]; L.sum_h = a.sums_d[1]; }
  L.output = LeafOutput(L.sum_g, FB_ADD(L.sum_h, 2 * kEpsilon), a.sp, L.num_data_global, 0.0);
  L.min_c = -1.0 / 0.0; L.max_c = 1.0 / 0.0; for (int k = 0; k < 4; ++k) L.pkey[k] = 1.0 / 0.0;
  a.leaves[0] = L;
  if (a.ctrl != nullptr) {
    LevelCtrl c;
    c.num_leaves = 1; c.next_slot = 1; c.done = 0; c.level = 0; c.num_splits = 0; c.num_children = 1; c.total_chunks = 0; c.total_blocks = 0;
    c.frontier_count = 1; c.journal_count = 0; c.pad0 = 0; c.skip_search = 0; c.num_eval = 0; c.pad1 = 0;
    a.ctrl[0] = c; a.ctrl[1] = c;
    a.frontier[0] = 0;
  }
  HistTask t; t.slot = 0; t.begin = 0; t.count = a.n_local; t.buffer = 0; t.block_begin = 0; t.num_blocks = a.root_blocks; t.pad0 = t.pad1 = 0;
  a.root_task[0] = t;
  FindChild fc; fc.leaf = 0; fc.slot = 0; fc.other_slot = 0; fc.is_larger = 0; fc.split = -1; fc.is_left = 1; fc.parent_global = 0; fc.task = 0;
  a.root_child[0] = fc;
}

}  // namespace

void LaunchInitTree(const TreeInitArgs& a, cudaStream_t s) {
  InitTreeKernel<<<1, 1, 0, s>>>(a);
  FB_LAUNCHED(); FB_KERNEL_CHECK();
}

void LaunchLevelController(const CtrlArgs& a, cudaStream_t s) {
  if (a.max_leaves > kCtrlMaxLeaves) Log::Fatal("The device controller handles up to %d leaves", kCtrlMaxLeaves);
  LevelControllerKernel<<<1, kCtrlThreads, 0, s>>>(a);
  FB_LAUNCHED(); FB_KERNEL_CHECK();
}

}  // namespace fb
