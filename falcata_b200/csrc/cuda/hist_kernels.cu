// K1q / K1: level-batched histogram construction with shared-memory atomics, and its fusion with
// the cross-rank reduce-scatter (K1q-RS): the epilogue adds every non-zero bin of the block's tile
// straight into the slot of the rank that OWNS the bin's feature — a local `red.add.u64`, or the
// same instruction on a peer pointer over NVLink. No staging buffer, no NCCL call.
//
// Parity: src/treelearner/cuda/cuda_histogram_constructor.cu:L1602-1910 (quantized dense construct:
// packed int32 (g16|h16) shared-memory atomics, rows per block capped so the 16-bit lanes cannot
// overflow, level-batched launch), L530-832 (full-precision construct), and the staging kernels
// around ncclAllReduce that this fusion removes (cuda_single_gpu_tree_learner.cu:L584-708).
//
// Work mapping: a block owns (task = one leaf's row window chunk, partition = a run of feature
// groups whose bins fit the shared tile). Items are (row, 4-group word) pairs laid out flat over the
// block's threads, so a warp reads whole 32-byte sectors of consecutive rows and its lanes hit
// different features' bins (no same-address serialisation inside a row).
#include "kernels.cuh"

#include <cuda_pipeline.h>

namespace fb {

namespace {

constexpr int kHistThreads = 256;

__device__ inline int FindTask(const HistTask* tasks, int num_tasks, int block) {
  int lo = 0, hi = num_tasks - 1;
  while (lo < hi) { const int m = (lo + hi + 1) >> 1; if (tasks[m].block_begin <= block) lo = m; else hi = m - 1; }
  return lo;
}

__device__ inline void FlushBinQuant(const HistDest& d, int slot, int global_bin, long long g, long long h) {
  const int owner = d.bin_owner[global_bin];
  hist_q_t* p = static_cast<hist_q_t*>(d.pool[owner]) + static_cast<long long>(slot) * d.slot_stride[owner] + d.bin_local[global_bin];
  const hist_q_t v = HistQPack(g, h);
  if (owner == d.rank) atomicAdd(p, v);
  else atomicAdd_system(p, v);     // red.add.u64 on the peer's memory: the reduce-scatter, bin by bin
}

template <bool TWO_PHASE>
__global__ void __launch_bounds__(kHistThreads) HistQuantKernel(HistArgs a) {
  extern __shared__ int smem_i[];
  const HistPartition part = a.parts[blockIdx.y];
  int* s_packed = smem_i;                                        // [bin_count] (g16|h16)
  int* s_wide = s_packed + part.bin_count;                       // TWO_PHASE: [2 * bin_count] int32 g, int32 h
  int* s_gstart = TWO_PHASE ? s_wide + 2 * part.bin_count : s_packed + part.bin_count;   // [groups in partition]
  const int ti = FindTask(a.tasks, a.num_tasks, blockIdx.x);
  const HistTask task = a.tasks[ti];
  const int chunk = blockIdx.x - task.block_begin;
  const long long row0 = static_cast<long long>(chunk) * a.rows_per_block;
  if (chunk >= task.num_blocks || row0 >= task.count) { if (a.sig.world > 1) FabricSignalDone(a.sig, gridDim.x * gridDim.y); return; }
  const int nrows = static_cast<int>(min(static_cast<long long>(a.rows_per_block), task.count - row0));
  const int ngroups = part.group_end - part.group_begin;
  const int G4 = (ngroups + 3) >> 2;
  for (int b = threadIdx.x; b < part.bin_count * (TWO_PHASE ? 3 : 1); b += kHistThreads) s_packed[b] = 0;
  for (int g = threadIdx.x; g < ngroups; g += kHistThreads) s_gstart[g] = a.group_bin_start[part.group_begin + g] - part.bin_begin;
  __syncthreads();
  const int* idx = a.idx[task.buffer] + task.begin + row0;
  const int step_r = kHistThreads / G4, step_w = kHistThreads % G4;
  for (int sub0 = 0; sub0 < nrows; sub0 += a.sub_rows) {
    const int sub_n = min(a.sub_rows, nrows - sub0);
    int r = threadIdx.x / G4, w = threadIdx.x % G4;
    while (r < sub_n) {
      const int row = a.identity_root ? static_cast<int>(task.begin + row0 + sub0 + r) : idx[sub0 + r];
      const uint8_t* rp = a.rows + static_cast<size_t>(row) * a.row_stride;
      const unsigned int word = *reinterpret_cast<const unsigned int*>(rp + part.group_begin + 4 * w);
      const int gh = *reinterpret_cast<const int*>(a.gh_base + static_cast<size_t>(row) * a.gh_stride);
      const int g0 = 4 * w;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if (g0 + k < ngroups) atomicAdd(&s_packed[s_gstart[g0 + k] + ((word >> (8 * k)) & 0xFF)], gh);
      }
      r += step_r; w += step_w;
      if (w >= G4) { w -= G4; ++r; }
    }
    if (TWO_PHASE) {
      __syncthreads();
      for (int b = threadIdx.x; b < part.bin_count; b += kHistThreads) {
        const int v = s_packed[b];
        if (v != 0) { const int h = v & 0xFFFF; s_wide[2 * b] += (v - h) >> 16; s_wide[2 * b + 1] += h; s_packed[b] = 0; }
      }
      __syncthreads();
    }
  }
  if (!TWO_PHASE) __syncthreads();
  for (int b = threadIdx.x; b < part.bin_count; b += kHistThreads) {
    long long g, h;
    if (TWO_PHASE) { g = s_wide[2 * b]; h = s_wide[2 * b + 1]; }
    else { const int v = s_packed[b]; h = v & 0xFFFF; g = (v - static_cast<int>(h)) >> 16; }
    if (g != 0 || h != 0) FlushBinQuant(a.dest, task.slot, part.bin_begin + b, g, h);
  }
  if (a.sig.world > 1) FabricSignalDone(a.sig, gridDim.x * gridDim.y);
}

// Lane-per-group instance, fed by an asynchronous gather pipeline.
//
// Two measurements on B200 shaped this kernel. (1) With plain loads a block keeps only a few KB of
// row data in flight; the construct then waits on DRAM latency, far from HBM bandwidth. Here every
// thread copies one row's 32 bytes (and its gradient word) global->shared with cp.async, several
// stages ahead, so each SM has tens of KB in flight without holding registers. (2) Shared-memory
// atomics into a [group][bin] tile suffer bank conflicts between the lanes' random bins. Here lane l
// of a warp owns feature group (32*blockIdx.y + l) and the tile is laid out [bin][32 lanes]: the 32
// lanes of an instruction always touch 32 different banks. With PRIVATE tiles (one per warp) the
// update is a plain load-add-store, no atomics at all, because no other thread touches a lane's column.
constexpr int kLaneWarps = kHistThreads / 32;
constexpr int kPipeStages = 4;
template <int NB, bool PRIVATE>
__global__ void __launch_bounds__(kHistThreads) HistQuantLaneKernel(HistArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int kTile = NB * 32;
  constexpr int kTiles = PRIVATE ? kLaneWarps : 1;
  int* tiles = reinterpret_cast<int*>(smem_raw);
  unsigned char* stage_rows = smem_raw + sizeof(int) * kTiles * kTile;                    // [stages][256 rows][32 B]
  int* stage_gh = reinterpret_cast<int*>(stage_rows + kPipeStages * kHistThreads * 32);   // [stages][256]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ti = FindTask(a.tasks, a.num_tasks, blockIdx.x);
  const HistTask task = a.tasks[ti];
  const int chunk = blockIdx.x - task.block_begin;
  const long long row0 = static_cast<long long>(chunk) * a.rows_per_block;
  if (chunk >= task.num_blocks || row0 >= task.count) { if (a.sig.world > 1) FabricSignalDone(a.sig, gridDim.x * gridDim.y); return; }
  const int nrows = static_cast<int>(min(static_cast<long long>(a.rows_per_block), task.count - row0));
  const int g0 = blockIdx.y * 32;
  const int ng = min(32, a.num_groups - g0);
  const int copy16 = min(2, (a.row_stride - g0) / 16);          // 16-byte pieces of this part inside the row
  for (int i = threadIdx.x; i < kTiles * kTile; i += kHistThreads) tiles[i] = 0;
  int* tile = tiles + (PRIVATE ? warp * kTile : 0);
  const int* idx = a.idx[task.buffer] + task.begin + row0;
  const int nstage = (nrows + kHistThreads - 1) / kHistThreads;
  auto row_of = [&](int r) -> int { return a.identity_root ? static_cast<int>(task.begin + row0 + r) : idx[r]; };
  auto issue = [&](int s, int row) {
    if (s < nstage && s * kHistThreads + static_cast<int>(threadIdx.x) < nrows) {
      const int slot = s % kPipeStages;
      const unsigned char* src = a.rows + static_cast<size_t>(row) * a.row_stride + g0;
      unsigned char* dst = stage_rows + (static_cast<size_t>(slot) * kHistThreads + threadIdx.x) * 32;
      __pipeline_memcpy_async(dst, src, 16);
      if (copy16 > 1) __pipeline_memcpy_async(dst + 16, src + 16, 16);
      __pipeline_memcpy_async(stage_gh + slot * kHistThreads + threadIdx.x, a.gh_base + static_cast<size_t>(row) * a.gh_stride, 4);
    }
    __pipeline_commit();
  };
  // prologue: stages 0 .. S-2 in flight, and the row index of the next stage already loaded
  int next_row = 0;
  for (int s = 0; s < kPipeStages - 1; ++s) {
    const int r = s * kHistThreads + threadIdx.x;
    issue(s, (s < nstage && r < nrows) ? row_of(r) : 0);
  }
  { const int r = (kPipeStages - 1) * kHistThreads + threadIdx.x; next_row = (kPipeStages - 1 < nstage && r < nrows) ? row_of(r) : 0; }
  __syncthreads();
  const bool active = lane < ng;
  for (int s = 0; s < nstage; ++s) {
    issue(s + kPipeStages - 1, next_row);
    { const int r = (s + kPipeStages) * kHistThreads + threadIdx.x; next_row = (s + kPipeStages < nstage && r < nrows) ? row_of(r) : 0; }
    __pipeline_wait_prior(kPipeStages - 1);
    __syncthreads();
    const int slot = s % kPipeStages;
    const int base = s * kHistThreads + warp * 32;
    const int cnt = min(32, nrows - base);
    if (cnt > 0) {
      const unsigned char* sr = stage_rows + (static_cast<size_t>(slot) * kHistThreads + warp * 32) * 32 + lane;
      const int ghv = stage_gh[slot * kHistThreads + warp * 32 + lane];
      if (cnt == 32 && PRIVATE) {
        // four rows per step: the four tile loads are issued together and equal addresses are
        // forwarded in registers, so the dependent shared-memory chain is paid once per four rows
#pragma unroll 2
        for (int j = 0; j < 32; j += 4) {
          const int a0 = sr[j * 32] * 32 + lane, a1 = sr[(j + 1) * 32] * 32 + lane, a2 = sr[(j + 2) * 32] * 32 + lane, a3 = sr[(j + 3) * 32] * 32 + lane;
          const int g0v = __shfl_sync(0xffffffffu, ghv, j), g1v = __shfl_sync(0xffffffffu, ghv, j + 1);
          const int g2v = __shfl_sync(0xffffffffu, ghv, j + 2), g3v = __shfl_sync(0xffffffffu, ghv, j + 3);
          if (active) {
            int v0 = tile[a0], v1 = tile[a1], v2 = tile[a2], v3 = tile[a3];
            v0 += g0v;
            v1 = (a1 == a0) ? v0 : v1; v1 += g1v;
            v2 = (a2 == a1) ? v1 : ((a2 == a0) ? v0 : v2); v2 += g2v;
            v3 = (a3 == a2) ? v2 : ((a3 == a1) ? v1 : ((a3 == a0) ? v0 : v3)); v3 += g3v;
            tile[a0] = v0; tile[a1] = v1; tile[a2] = v2; tile[a3] = v3;   // program order: the last store to an address holds its full sum
          }
        }
      } else if (cnt == 32) {
#pragma unroll 8
        for (int j = 0; j < 32; ++j) {
          const int b = sr[j * 32];
          const int g = __shfl_sync(0xffffffffu, ghv, j);
          if (active) atomicAdd(&tile[b * 32 + lane], g);
        }
      } else {
        for (int j = 0; j < cnt; ++j) {
          const int b = sr[j * 32];
          const int g = __shfl_sync(0xffffffffu, ghv, j);
          if (active) { if (PRIVATE) tile[b * 32 + lane] += g; else atomicAdd(&tile[b * 32 + lane], g); }
        }
      }
    }
    __syncthreads();
  }
  for (int cell = threadIdx.x; cell < kTile; cell += kHistThreads) {
    const int l = cell & 31, b = cell >> 5;
    if (l >= ng) continue;
    const int g = g0 + l;
    const int gstart = a.group_bin_start[g];
    const int gbins = (g + 1 < a.num_groups ? a.group_bin_start[g + 1] : a.num_total_bin) - gstart;
    if (b >= gbins) continue;
    long long sg = 0, sh = 0;
    for (int w = 0; w < kTiles; ++w) { const int v = tiles[w * kTile + cell]; const int h = v & 0xFFFF; sg += (v - h) >> 16; sh += h; }
    if (sg != 0 || sh != 0) FlushBinQuant(a.dest, task.slot, gstart + b, sg, sh);
  }
  if (a.sig.world > 1) FabricSignalDone(a.sig, gridDim.x * gridDim.y);
}


__global__ void __launch_bounds__(kHistThreads) HistFloatKernel(HistArgs a) {
  extern __shared__ float smem_f[];
  const HistPartition part = a.parts[blockIdx.y];
  float* s_hist = smem_f;                                               // [2 * bin_count]
  int* s_gstart = reinterpret_cast<int*>(s_hist + 2 * part.bin_count);
  const int ti = FindTask(a.tasks, a.num_tasks, blockIdx.x);
  const HistTask task = a.tasks[ti];
  const int chunk = blockIdx.x - task.block_begin;
  const long long row0 = static_cast<long long>(chunk) * a.rows_per_block;
  if (chunk >= task.num_blocks || row0 >= task.count) { if (a.sig.world > 1) FabricSignalDone(a.sig, gridDim.x * gridDim.y); return; }
  const int nrows = static_cast<int>(min(static_cast<long long>(a.rows_per_block), task.count - row0));
  const int ngroups = part.group_end - part.group_begin;
  const int G4 = (ngroups + 3) >> 2;
  for (int b = threadIdx.x; b < 2 * part.bin_count; b += kHistThreads) s_hist[b] = 0.f;
  for (int g = threadIdx.x; g < ngroups; g += kHistThreads) s_gstart[g] = a.group_bin_start[part.group_begin + g] - part.bin_begin;
  __syncthreads();
  const int* idx = a.idx[task.buffer] + task.begin + row0;
  const int step_r = kHistThreads / G4, step_w = kHistThreads % G4;
  int r = threadIdx.x / G4, w = threadIdx.x % G4;
  while (r < nrows) {
    const int row = a.identity_root ? static_cast<int>(task.begin + row0 + r) : idx[r];
    const uint8_t* rp = a.rows + static_cast<size_t>(row) * a.row_stride;
    const unsigned int word = *reinterpret_cast<const unsigned int*>(rp + part.group_begin + 4 * w);
    const float2 gh = *reinterpret_cast<const float2*>(a.gh_base + static_cast<size_t>(row) * a.gh_stride);
    const int g0 = 4 * w;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      if (g0 + k < ngroups) {
        const int b = s_gstart[g0 + k] + ((word >> (8 * k)) & 0xFF);
        atomicAdd(&s_hist[2 * b], gh.x); atomicAdd(&s_hist[2 * b + 1], gh.y);
      }
    }
    r += step_r; w += step_w;
    if (w >= G4) { w -= G4; ++r; }
  }
  __syncthreads();
  const HistDest& d = a.dest;
  for (int b = threadIdx.x; b < part.bin_count; b += kHistThreads) {
    const float g = s_hist[2 * b], h = s_hist[2 * b + 1];
    if (g == 0.f && h == 0.f) continue;
    const int gb = part.bin_begin + b, owner = d.bin_owner[gb];
    double* p = static_cast<double*>(d.pool[owner]) + 2 * (static_cast<long long>(task.slot) * d.slot_stride[owner] + d.bin_local[gb]);
    if (owner == d.rank) { atomicAdd(p, static_cast<double>(g)); atomicAdd(p + 1, static_cast<double>(h)); }
    else { atomicAdd_system(p, static_cast<double>(g)); atomicAdd_system(p + 1, static_cast<double>(h)); }
  }
  if (a.sig.world > 1) FabricSignalDone(a.sig, gridDim.x * gridDim.y);
}

}  // namespace

void LaunchHistConstructQuant(const HistArgs& a, cudaStream_t s) {
  if (a.total_blocks <= 0 || a.num_tasks <= 0) return;
  if (a.lane_mode != 0) {
    const bool priv = a.lane_mode == 1;
    const int cap = priv ? kLaneWarps * a.sub_rows : a.sub_rows;
    if (a.rows_per_block > cap) Log::Fatal("lane histogram: %d rows per block would overflow the 16-bit lanes (cap %d)", a.rows_per_block, cap);
    dim3 grid(a.total_blocks, (a.num_groups + 31) / 32);
    const size_t sm = static_cast<size_t>(a.lane_bins) * 32 * 4 * (priv ? kLaneWarps : 1) + static_cast<size_t>(kPipeStages) * kHistThreads * (32 + 4);
#define FB_LANE(NB, P)                                                                                                             \
    {                                                                                                                              \
      static bool attr = false;                                                                                                    \
      if (!attr) { FB_CUDA(cudaFuncSetAttribute(HistQuantLaneKernel<NB, P>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)); attr = true; } \
      HistQuantLaneKernel<NB, P><<<grid, kHistThreads, sm, s>>>(a);                                                                \
    }
    if (a.lane_bins == 16) { if (priv) FB_LANE(16, true) else FB_LANE(16, false) }
    else if (a.lane_bins == 64) { if (priv) FB_LANE(64, true) else FB_LANE(64, false) }
    else Log::Fatal("lane histogram: unsupported tile of %d bins", a.lane_bins);
#undef FB_LANE
    FB_LAUNCHED(); FB_KERNEL_CHECK();
    return;
  }
  const bool two_phase = a.rows_per_block > a.sub_rows;
  int max_groups = 0;
  // shared bytes: packed (+ wide) + group starts; sized for the largest partition
  const size_t sm = static_cast<size_t>(a.max_part_bins) * (two_phase ? 12 : 4) + static_cast<size_t>(a.num_groups) * 4;
  (void)max_groups;
  dim3 grid(a.total_blocks, a.num_parts);
  if (two_phase) {
    static bool attr = false; if (!attr) { FB_CUDA(cudaFuncSetAttribute(HistQuantKernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)); attr = true; }
    HistQuantKernel<true><<<grid, kHistThreads, sm, s>>>(a);
  } else {
    static bool attr = false; if (!attr) { FB_CUDA(cudaFuncSetAttribute(HistQuantKernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)); attr = true; }
    HistQuantKernel<false><<<grid, kHistThreads, sm, s>>>(a);
  }
  FB_LAUNCHED(); FB_KERNEL_CHECK();
}

void LaunchHistConstructFloat(const HistArgs& a, cudaStream_t s) {
  if (a.total_blocks <= 0 || a.num_tasks <= 0) return;
  const size_t sm = static_cast<size_t>(a.max_part_bins) * 8 + static_cast<size_t>(a.num_groups) * 4;
  static bool attr = false; if (!attr) { FB_CUDA(cudaFuncSetAttribute(HistFloatKernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)); attr = true; }
  dim3 grid(a.total_blocks, a.num_parts);
  HistFloatKernel<<<grid, kHistThreads, sm, s>>>(a);
  FB_LAUNCHED(); FB_KERNEL_CHECK();
}

}  // namespace fb
