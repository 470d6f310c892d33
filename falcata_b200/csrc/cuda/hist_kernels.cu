// K1q / K1: level-batched histogram construction, and its fusion with the cross-rank reduce-scatter
// (K1q-RS). One rank: a block's non-zero bins are added into the leaf's pool slot with `red.add.u64`.
// Several ranks: blocks add into a local staging histogram of the task; the LAST block of a task
// (a per-task arrival counter) cuts the staged histogram by feature owner and writes each slice with
// plain stores into the owner's [source rank][task] staging slot over NVLink, then signals the owner's
// flag. The owner sums the R source slices in rank order when the split search loads a bin, so the
// reduction order, and with integer bins the result, does not depend on timing. No NCCL call.
//
// Parity: src/treelearner/cuda/cuda_histogram_constructor.cu:L1602-1910 (quantized dense construct:
// packed int32 (g16|h16) shared-memory atomics, rows per block capped so the 16-bit lanes cannot
// overflow, level-batched launch), L530-832 (full-precision construct), and the staging kernels
// around ncclAllReduce that this fusion removes (cuda_single_gpu_tree_learner.cu:L584-708).
//
// Work mapping of the atomic instances: a block owns (task = one leaf's row window chunk, partition =
// a run of feature groups whose bins fit the shared tile). Items are (row, 4-group word) pairs laid out
// flat over the block's threads, so a warp reads whole 32-byte sectors of consecutive rows and its
// lanes hit different features' bins (no same-address serialisation inside a row). The lane-per-group
// instance further down is the default for groups of at most 64 bins.
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

// One rank: the bin goes straight into the pool slot. Several ranks: into the LOCAL staging
// histogram of the task (L2 atomics); PushTaskIfLast ships the finished task to the owners.
// `single`: this block is the only one that adds to the task's cells (which were cleared beforehand): a plain store.
__device__ inline void FlushBinQuant(const HistDest& d, int slot, int task_index, int num_total_bin, int global_bin, long long g, long long h, bool single = false) {
  const hist_q_t v = HistQPack(g, h);
  if (d.owner_only && d.bin_owner[global_bin] != d.rank) return;
  hist_q_t* p = d.num_ranks > 1 ? static_cast<hist_q_t*>(d.stage_local) + static_cast<long long>(task_index) * num_total_bin + global_bin
                                : static_cast<hist_q_t*>(d.pool[0]) + static_cast<long long>(slot) * d.slot_stride[0] + d.bin_local[global_bin];
  if (single) *p = v; else atomicAdd(p, v);
}

// Reduce-scatter step, fused into the construct kernel. Called by every block that worked on task
// `ti` after its flush. The last of them finds the task's histogram complete in the local staging
// area and stores each feature slice into the staging slot [this rank][ti] of the rank that owns the
// feature: plain 8/16-byte stores to peer memory, contiguous per feature group, over NVLink, while
// other blocks are still constructing other leaves. Zeros are stored too, so the destination never
// needs clearing, and the local staging cells are reset for the next level.
template <bool QUANT>
__device__ inline bool PushTaskIfLast(const HistArgs& a, int ti, const HistTask& task) {
  const HistDest& d = a.dest;
  __shared__ int s_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const int row_blocks = max(1, (task.count + a.rows_per_block - 1) / a.rows_per_block);
    const unsigned int need = static_cast<unsigned int>(min(row_blocks, task.num_blocks)) * gridDim.y;
    const unsigned int prev = atomicAdd(d.task_done + ti, 1u);
    s_last = (prev + 1 == need) ? 1 : 0;
    if (s_last) d.task_done[ti] = 0;
  }
  __syncthreads();
  if (!s_last) return false;
  __threadfence();
  const int nb = a.num_total_bin;
  for (int b = threadIdx.x; b < nb; b += blockDim.x) {
    const int owner = d.bin_owner[b];
    const long long dst_index = (static_cast<long long>(d.rank) * d.stage_cap + ti) * d.slot_stride[owner] + d.bin_local[b];
    if (QUANT) {
      hist_q_t* src = static_cast<hist_q_t*>(d.stage_local) + static_cast<long long>(ti) * nb + b;
      const hist_q_t v = __ldcg(src);
      *src = 0;
      static_cast<hist_q_t*>(d.peer_stage[owner])[dst_index] = v;
    } else {
      double2* src = static_cast<double2*>(d.stage_local) + static_cast<long long>(ti) * nb + b;
      const double2 v = __ldcg(src);
      *src = make_double2(0.0, 0.0);
      static_cast<double2*>(d.peer_stage[owner])[dst_index] = v;
    }
  }
  __threadfence_system();   // every storing thread publishes its own peer stores before the block counts itself done
  return true;
}

template <bool TWO_PHASE>
__global__ void __launch_bounds__(kHistThreads) HistQuantKernel(HistArgs a) {
  extern __shared__ int smem_i[];
  const HistPartition part = a.parts[blockIdx.y];
  int* s_packed = smem_i;                                        // [bin_count] (g16|h16)
  int* s_wide = s_packed + part.bin_count;                       // TWO_PHASE: [2 * bin_count] int32 g, int32 h
  int* s_gstart = TWO_PHASE ? s_wide + 2 * part.bin_count : s_packed + part.bin_count;   // [groups in partition]
  const int num_tasks = a.ctrl != nullptr ? a.ctrl->num_splits : a.num_tasks;
  if (num_tasks <= 0 || static_cast<int>(blockIdx.x) >= (a.ctrl != nullptr ? a.ctrl->total_blocks : a.total_blocks)) { if (a.sig.world > 1) FabricSignalDone(a.sig, gridDim.x * gridDim.y); return; }
  const int ti = FindTask(a.tasks, num_tasks, blockIdx.x);
  const HistTask task = a.tasks[ti];
  const int chunk = blockIdx.x - task.block_begin;
  const long long row0 = static_cast<long long>(chunk) * a.rows_per_block;
  // a task always keeps its first block (even with no local rows): it closes the task's reduce-scatter
  const int row_blocks = max(1, (task.count + a.rows_per_block - 1) / a.rows_per_block);
  if (chunk >= task.num_blocks || chunk >= row_blocks) { if (a.sig.world > 1) FabricSignalDone(a.sig, gridDim.x * gridDim.y); return; }
  const int nrows = static_cast<int>(max(0LL, min(static_cast<long long>(a.rows_per_block), task.count - row0)));
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
    if (g != 0 || h != 0) FlushBinQuant(a.dest, task.slot, ti, a.num_total_bin, part.bin_begin + b, g, h);
  }
  const bool pushed = a.dest.num_ranks > 1 && PushTaskIfLast<true>(a, ti, task);
  if (a.sig.world > 1) FabricSignalDone(a.sig, gridDim.x * gridDim.y, pushed);
}

// Lane-per-group instance with warp-autonomous asynchronous pipelines.
//
// Measurements on B200 that shaped this kernel:
//  (1) with plain loads a block keeps only a few KB of row data in flight and the construct waits on
//      DRAM latency; with block-wide stages the warps wait for each other at barriers instead.
//      Here every WARP runs its own pipeline: per stage, lane l copies row l of the warp's next 32
//      rows (32 bytes of bins + the packed gradient word) global->shared with cp.async, kLaneStages - 1
//      stages ahead, and waits only for its own copies. No block barrier until the final merge.
//      Measured at 11M x 28: 12 warps x 8 stages 2.90 ms per round, 16 x 4 2.78, 20 x 2 2.72 - the update
//      chain wants more warps per scheduler more than it wants deeper prefetch.
//  (2) shared-memory atomics into a [group][bin] tile lose most of their rate to bank conflicts
//      between the lanes' random bins. Here lane l owns feature group (32*blockIdx.y + l) and each
//      warp has a private tile laid out [bin][32 lanes]: an instruction's 32 lanes always hit 32
//      different banks and the update is a plain load-add-store (nobody else touches a lane's column).
//  (3) the load-add-store chain is taken four rows at a time: four tile loads issue together and equal
//      addresses are forwarded in registers.
// ---- bulk asynchronous copies (TMA engine, non-tensor form) with mbarrier completion ----
__device__ inline uint32_t SmemAddr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ inline void MbarInit(uint64_t* bar, uint32_t count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(SmemAddr(bar)), "r"(count) : "memory"); }
__device__ inline void MbarExpectTx(uint64_t* bar, uint32_t bytes) { asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(SmemAddr(bar)), "r"(bytes) : "memory"); }
__device__ inline bool MbarTryWait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(SmemAddr(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// global -> this block's shared memory, `bytes` a multiple of 16, both addresses 16-byte aligned; completion is counted on `bar`
__device__ inline void BulkCopyG2S(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(SmemAddr(dst)), "l"(src), "r"(bytes), "r"(SmemAddr(bar)) : "memory");
}
// Bounded wait: false when the budget ran out (the caller records the status and winds down).
__device__ inline bool MbarWaitBounded(uint64_t* bar, uint32_t parity) {
  for (int i = 0; i < (1 << 16); ++i) if (MbarTryWait(bar, parity)) return true;
  return false;
}

// One staged block of up to 32 rows (32 bytes apart in shared memory) added into a warp's private tile
// [bin][32 lanes]: lane l owns the column of feature group l. Four rows per step: the four tile loads issue
// together, and cells that repeat inside the four are forwarded in registers so that every store holds its full sum.
// P4: two groups per byte (low nibble = even group).
template <bool P4>
__device__ __forceinline__ void ConsumeStage(int* __restrict__ tile, const unsigned char* __restrict__ stage_rows, const int* __restrict__ sg, int cnt, int lane, bool active, bool red = false) {
  const unsigned char* sr = stage_rows + (P4 ? (lane >> 1) : lane);
  const int nshift = (lane & 1) * 4;
  auto bin_of = [&](int j) -> int { const int b = sr[j * 32]; return P4 ? ((b >> nshift) & 15) : b; };
  if (red && cnt == 32) {
    // reduction form: one shared-memory add per row and lane, no value comes back, so nothing has to be forwarded
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
      const int4 g4 = *reinterpret_cast<const int4*>(sg + j);
      const int a0 = bin_of(j) * 32 + lane, a1 = bin_of(j + 1) * 32 + lane, a2 = bin_of(j + 2) * 32 + lane, a3 = bin_of(j + 3) * 32 + lane;
      if (active) { atomicAdd(tile + a0, g4.x); atomicAdd(tile + a1, g4.y); atomicAdd(tile + a2, g4.z); atomicAdd(tile + a3, g4.w); }
    }
  } else if (cnt == 32) {
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
      const int a0 = bin_of(j) * 32 + lane, a1 = bin_of(j + 1) * 32 + lane, a2 = bin_of(j + 2) * 32 + lane, a3 = bin_of(j + 3) * 32 + lane;
      const int4 g4 = *reinterpret_cast<const int4*>(sg + j);     // same address in every lane: one broadcast load
      if (active) {
        int v0 = tile[a0], v1 = tile[a1], v2 = tile[a2], v3 = tile[a3];
        v0 += g4.x;
        v1 = (a1 == a0) ? v0 : v1; v1 += g4.y;
        v2 = (a2 == a1) ? v1 : ((a2 == a0) ? v0 : v2); v2 += g4.z;
        v3 = (a3 == a2) ? v2 : ((a3 == a1) ? v1 : ((a3 == a0) ? v0 : v3)); v3 += g4.w;
        tile[a0] = v0; tile[a1] = v1; tile[a2] = v2; tile[a3] = v3;   // program order: the last store to an address holds its full sum
      }
    }
  } else {
    for (int j = 0; j < cnt; ++j) {
      const int b = bin_of(j); const int g = sg[j];
      if (active) { if (red) atomicAdd(tile + b * 32 + lane, g); else tile[b * 32 + lane] += g; }
    }
  }
}

// fp32 form of ConsumeStage: the tile holds a (gradient, hessian) float pair per cell, [NB][32] pairs; lane l adds the
// row's pair into column l. `red`: shared-memory reduction adds (tiles shared by several warps); otherwise the warp owns
// the tile and the update is a load-add-store, eight rows at a time with repeated cells forwarded in registers - the
// sums are then those of the rows in order, whatever the timing.
template <int NB, bool P4, bool RED>
__device__ __forceinline__ void ConsumeStageFloat(float2* __restrict__ tile, const unsigned char* __restrict__ stage_rows, const float2* __restrict__ sg, int cnt, int lane, bool active) {
  const unsigned char* sr = stage_rows + (P4 ? (lane >> 1) : lane);
  const int nshift = (lane & 1) * 4;
  auto bin_of = [&](int j) -> int { const int b = sr[j * 32]; return P4 ? ((b >> nshift) & 15) : b; };
  float2* col = tile + lane;
  if constexpr (RED) {
    // two planes, [gradient | hessian][NB][32] floats: the 32 lanes of an add hit 32 different banks
    float* tg = reinterpret_cast<float*>(tile) + lane; float* th = tg + NB * 32;
    if (cnt == 32) {
#pragma unroll
      for (int j = 0; j < 32; j += 2) {
        const float4 g2 = *reinterpret_cast<const float4*>(sg + j);   // two rows' pairs, the same address in every lane
        const int a0 = bin_of(j) * 32, a1 = bin_of(j + 1) * 32;
        if (active) { atomicAdd(tg + a0, g2.x); atomicAdd(th + a0, g2.y); atomicAdd(tg + a1, g2.z); atomicAdd(th + a1, g2.w); }
      }
    } else {
      for (int j = 0; j < cnt; ++j) {
        const float2 g = sg[j]; const int a0 = bin_of(j) * 32;
        if (active) { atomicAdd(tg + a0, g.x); atomicAdd(th + a0, g.y); }
      }
    }
  } else if (cnt == 32) {
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
      int ad[8]; float2 v[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) ad[k] = bin_of(j + k) * 32;
      if (active) {
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = col[ad[k]];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          // the latest earlier row of this group of eight that hit the same cell holds the cell's running sum
#pragma unroll
          for (int m = 0; m < k; ++m) if (ad[m] == ad[k]) v[k] = v[m];
          const float2 g = sg[j + k];
          v[k].x += g.x; v[k].y += g.y;
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) col[ad[k]] = v[k];   // program order: the last store to a cell holds its full sum
      }
    }
  } else {
    for (int j = 0; j < cnt; ++j) {
      const float2 g = sg[j]; const int a0 = bin_of(j) * 32;
      if (active) { float2 v = col[a0]; v.x += g.x; v.y += g.y; col[a0] = v; }
    }
  }
}

constexpr int kLaneMaxThreads = 1024;
// Block shape: `lane_warps` warps (the block size), every `lane_share` consecutive warps add into one tile. Sharing
// a tile needs the reduction form of the update (`lane_red`); with one warp per tile both forms are valid.
// FLT: fp32 gradients (a float2 per row) added into (gradient, hessian) float pairs, [NB][32] pairs per tile; otherwise
// packed int16|uint16 gradient words added into [NB][32] ints.
// MODE 0: integer; 1: fp32 load-add-store (pairs, a tile per warp, at most 16 warps); 2: fp32 reduction adds (planes).
template <int NB, int kLaneStages, int MODE>
__global__ void __launch_bounds__(MODE == 1 ? kLaneMaxThreads / 2 : kLaneMaxThreads, 1) HistQuantLaneKernel(HistArgs a) {
  constexpr bool FLT = MODE != 0;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int kTile = NB * 32 * (FLT ? 2 : 1);   // 4-byte cells of a tile
  constexpr int kGhWords = FLT ? 2 : 1;            // 4-byte words of a row's gradient record
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kLaneWarps = blockDim.x >> 5, kLaneThreads = blockDim.x;
  const int share = max(1, a.lane_share), ntiles = kLaneWarps / share;
  int* tiles = reinterpret_cast<int*>(smem_raw);                                                 // [tiles][planes][NB][32]
  unsigned char* rows_w = smem_raw + sizeof(int) * ntiles * kTile + static_cast<size_t>(warp) * kLaneStages * 32 * 32;   // [stages][32 rows][32 B]
  int* gh_w = reinterpret_cast<int*>(smem_raw + sizeof(int) * ntiles * kTile + static_cast<size_t>(kLaneWarps) * kLaneStages * 32 * 32) + warp * kLaneStages * 32 * kGhWords;
  uint64_t* bars_w = reinterpret_cast<uint64_t*>(smem_raw + sizeof(int) * ntiles * kTile + static_cast<size_t>(kLaneWarps) * kLaneStages * 32 * (32 + 4 * kGhWords)) + warp * kLaneStages;   // one "stage full" barrier per (warp, stage)
  const int num_tasks = a.ctrl != nullptr ? a.ctrl->num_splits : a.num_tasks;
  if (num_tasks <= 0 || static_cast<int>(blockIdx.x) >= (a.ctrl != nullptr ? a.ctrl->total_blocks : a.total_blocks)) { if (a.sig.world > 1) FabricSignalDone(a.sig, gridDim.x * gridDim.y); return; }
  const int ti = FindTask(a.tasks, num_tasks, blockIdx.x);
  const HistTask task = a.tasks[ti];
  const int chunk = blockIdx.x - task.block_begin;
  const long long row0 = static_cast<long long>(chunk) * a.rows_per_block;
  // a task always keeps its first block (even with no local rows): it closes the task's reduce-scatter
  const int row_blocks = max(1, (task.count + a.rows_per_block - 1) / a.rows_per_block);
  if (chunk >= task.num_blocks || chunk >= row_blocks) { if (a.sig.world > 1) FabricSignalDone(a.sig, gridDim.x * gridDim.y); return; }
  const int nrows = static_cast<int>(max(0LL, min(static_cast<long long>(a.rows_per_block), task.count - row0)));
  const int g0 = blockIdx.y * 32;
  const int ng = min(32, a.num_groups - g0);
  const int byte0 = a.pack4 ? g0 / 2 : g0;                       // first byte of this 32-group part inside the row
  const int copy16 = a.pack4 ? 1 : min(2, (a.row_stride - g0) / 16);   // 16-byte pieces of this part inside the row
  int* tile = tiles + (warp / share) * kTile;
  if (share == 1) {
    for (int i = lane; i < kTile; i += 32) tile[i] = 0;
    __syncwarp();
  } else {
    for (int i = threadIdx.x; i < ntiles * kTile; i += kLaneThreads) tiles[i] = 0;
    __syncthreads();   // no exit path lies between here and the merge barrier, so every thread of the block arrives
  }
  // this warp's slice of the block's rows, in stages of 32 rows
  const int per_warp = ((nrows + kLaneWarps - 1) / kLaneWarps + 31) / 32 * 32;
  const int wbeg = min(nrows, warp * per_warp), wend = min(nrows, wbeg + per_warp);
  const int nstage = (wend - wbeg + 31) / 32;
  const int* idx = a.idx[task.buffer] + task.begin + row0 + wbeg;
  const long long ident0 = task.begin + row0 + wbeg;
  auto load_row = [&](int s) -> int {   // row id that this lane copies in stage s (-1: none)
    const int r = s * 32 + lane;
    if (s >= nstage || wbeg + r >= wend) return -1;
    return a.identity_root ? static_cast<int>(ident0 + r) : idx[r];
  };
  // Root level with 32-byte rows: a stage's 32 rows are one contiguous kilobyte, so the lanes copy it as 64
  // consecutive 16-byte pieces (two fully coalesced requests per warp) instead of two half-used sectors per lane.
  const bool block_copy = a.identity_root != 0 && a.row_stride == 32 && g0 == 0 && copy16 == 2 && !a.pack4;
  auto issue = [&](int s, int row) {
    if (row >= 0) {
      const int slot = s % kLaneStages;
      if (block_copy && wbeg + s * 32 + 32 <= wend) {
        const unsigned char* src = a.rows + static_cast<size_t>(ident0 + static_cast<long long>(s) * 32) * 32 + lane * 16;
        unsigned char* dst = rows_w + slot * 32 * 32 + lane * 16;
        __pipeline_memcpy_async(dst, src, 16);
        __pipeline_memcpy_async(dst + 512, src + 512, 16);
      } else {
        const unsigned char* src = a.rows + static_cast<size_t>(row) * a.row_stride + byte0;
        unsigned char* dst = rows_w + (slot * 32 + lane) * 32;
        __pipeline_memcpy_async(dst, src, 16);
        if (copy16 > 1) __pipeline_memcpy_async(dst + 16, src + 16, 16);
      }
      __pipeline_memcpy_async(gh_w + (slot * 32 + lane) * kGhWords, a.gh_base + static_cast<size_t>(row) * a.gh_stride, 4 * kGhWords);
    }
    __pipeline_commit();
  };
  const bool active = lane < ng;
  const bool red = a.lane_red != 0 || share > 1;
  auto consume = [&](int slot, int cnt) {   // add the stage's rows into this warp's tile
    if constexpr (FLT) {
      if (a.pack4) ConsumeStageFloat<NB, true, MODE == 2>(reinterpret_cast<float2*>(tile), rows_w + slot * 32 * 32, reinterpret_cast<const float2*>(gh_w + slot * 32 * kGhWords), cnt, lane, active);
      else ConsumeStageFloat<NB, false, MODE == 2>(reinterpret_cast<float2*>(tile), rows_w + slot * 32 * 32, reinterpret_cast<const float2*>(gh_w + slot * 32 * kGhWords), cnt, lane, active);
    } else {
      if (a.pack4) ConsumeStage<true>(tile, rows_w + slot * 32 * 32, gh_w + slot * 32, cnt, lane, active, red);
      else ConsumeStage<false>(tile, rows_w + slot * 32 * 32, gh_w + slot * 32, cnt, lane, active, red);
    }
  };
  // Root level of a 32-byte-row data set: a stage's rows are one contiguous kilobyte and its gradient words 128
  // contiguous bytes, so ONE lane hands both to the TMA engine as bulk copies and everybody waits on the stage's
  // mbarrier - no per-lane copy instructions, no address arithmetic in the other 31 lanes.
  const bool bulk = a.bulk_root != 0 && block_copy && a.gh_stride == 4 * kGhWords && (ident0 & 31) == 0;
  if (bulk) {
    const int nfull = (wend - wbeg) / 32, tail = (wend - wbeg) - nfull * 32;
    if (lane == 0) { for (int st = 0; st < kLaneStages; ++st) MbarInit(bars_w + st, 1); asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
    __syncwarp();
    auto produce = [&](int s) {
      if (s < nfull && lane == 0) {
        const int slot = s % kLaneStages;
        MbarExpectTx(bars_w + slot, 32 * 32 + 32 * 4 * kGhWords);
        BulkCopyG2S(rows_w + slot * 32 * 32, a.rows + static_cast<size_t>(ident0 + static_cast<long long>(s) * 32) * 32, 32 * 32, bars_w + slot);
        BulkCopyG2S(gh_w + slot * 32 * kGhWords, a.gh_base + static_cast<size_t>(ident0 + static_cast<long long>(s) * 32) * 4 * kGhWords, 32 * 4 * kGhWords, bars_w + slot);
      }
    };
    for (int s = 0; s < kLaneStages - 1; ++s) produce(s);
    bool ok = true;
    int s = 0;
    for (; s < nfull; ++s) {
      produce(s + kLaneStages - 1);   // refills the slot consumed one iteration ago (all lanes passed that iteration's __syncwarp)
      ok = __all_sync(0xffffffffu, MbarWaitBounded(bars_w + s % kLaneStages, (s / kLaneStages) & 1) ? 1 : 0) != 0;   // one decision per warp
      if (!ok) break;
      consume(s % kLaneStages, 32);
      __syncwarp();
    }
    if (!ok) {
      // the wait gave up: report it, then give every copy still in flight a (bounded) chance to land before leaving
      if (lane == 0 && a.status != nullptr) atomicExch(a.status, static_cast<unsigned int>(kStatusWaitTimeout));
      for (int t = s; t < min(nfull, s + kLaneStages); ++t) MbarWaitBounded(bars_w + t % kLaneStages, (t / kLaneStages) & 1);
    } else if (tail > 0) {
      // the last, partial stage comes in with plain loads (a bulk copy could run past the end of the arrays)
      if (lane < tail) {
        const size_t row = static_cast<size_t>(ident0) + static_cast<size_t>(nfull) * 32 + lane;
        const uint4* src = reinterpret_cast<const uint4*>(a.rows + row * 32);
        uint4* dst = reinterpret_cast<uint4*>(rows_w + lane * 32);
        dst[0] = src[0]; dst[1] = src[1];
        for (int k = 0; k < kGhWords; ++k) gh_w[lane * kGhWords + k] = reinterpret_cast<const int*>(a.gh_base + row * 4 * kGhWords)[k];
      }
      __syncwarp();
      consume(0, tail);
      __syncwarp();
    }
  } else {
  for (int s = 0; s < kLaneStages - 1; ++s) issue(s, load_row(s));
  // row ids are fetched three stages before they are needed, so their latency is off the critical path
  int q0 = load_row(kLaneStages - 1), q1 = load_row(kLaneStages), q2 = load_row(kLaneStages + 1);
  for (int s = 0; s < nstage; ++s) {
    issue(s + kLaneStages - 1, q0);
    q0 = q1; q1 = q2; q2 = load_row(s + kLaneStages + 2);
    __pipeline_wait_prior(kLaneStages - 1);
    __syncwarp();
    consume(s % kLaneStages, min(32, wend - wbeg - s * 32));
    __syncwarp();   // every lane is done with this stage's buffer before it is refilled
  }
  }
  __syncthreads();
  const bool single_block = row_blocks == 1;   // blocks beyond the task's rows left above: nobody else adds to these cells
  for (int cell = threadIdx.x; cell < NB * 32; cell += kLaneThreads) {
    const int l = cell & 31, b = cell >> 5;
    if (l >= ng) continue;
    const int g = g0 + l;
    const int gstart = a.group_bin_start[g];
    const int gbins = a.group_bin_count != nullptr ? a.group_bin_count[g] : (g + 1 < a.num_groups ? a.group_bin_start[g + 1] : a.num_total_bin) - gstart;
    if (b >= gbins) continue;
    if constexpr (FLT) {
      // the tiles of a block are summed in tile order, in double; the blocks of a task meet in double-precision global
      // adds, and a task with a single block stores (its cells were cleared with the pool)
      double sg = 0.0, sh = 0.0;
      if constexpr (MODE == 2) {
        const float* ft = reinterpret_cast<const float*>(tiles);
        for (int w = 0; w < ntiles; ++w) { sg += static_cast<double>(ft[w * kTile + cell]); sh += static_cast<double>(ft[w * kTile + NB * 32 + cell]); }
      } else {
        const float2* ft = reinterpret_cast<const float2*>(tiles);
        for (int w = 0; w < ntiles; ++w) { const float2 v = ft[w * (kTile / 2) + cell]; sg += static_cast<double>(v.x); sh += static_cast<double>(v.y); }
      }
      if (sg != 0.0 || sh != 0.0) {
        const HistDest& d = a.dest;
        const int gb = gstart + b;
        double* p = d.num_ranks > 1 ? static_cast<double*>(d.stage_local) + 2 * (static_cast<long long>(ti) * a.num_total_bin + gb)
                                    : static_cast<double*>(d.pool[0]) + 2 * (static_cast<long long>(task.slot) * d.slot_stride[0] + d.bin_local[gb]);
        if (single_block) *reinterpret_cast<double2*>(p) = make_double2(sg, sh);
        else { atomicAdd(p, sg); atomicAdd(p + 1, sh); }
      }
    } else {
      long long sg = 0, sh = 0;
      for (int w = 0; w < ntiles; ++w) { const int v = tiles[w * kTile + cell]; const int h = v & 0xFFFF; sg += (v - h) >> 16; sh += h; }
      if (sg != 0 || sh != 0) FlushBinQuant(a.dest, task.slot, ti, a.num_total_bin, gstart + b, sg, sh, single_block);
    }
  }
  const bool pushed = a.dest.num_ranks > 1 && PushTaskIfLast<!FLT>(a, ti, task);
  if (a.sig.world > 1) FabricSignalDone(a.sig, gridDim.x * gridDim.y, pushed);
}

__global__ void __launch_bounds__(kHistThreads) HistFloatKernel(HistArgs a) {
  extern __shared__ float smem_f[];
  const HistPartition part = a.parts[blockIdx.y];
  float* s_hist = smem_f;                                               // [2 * bin_count]
  int* s_gstart = reinterpret_cast<int*>(s_hist + 2 * part.bin_count);
  const int num_tasks = a.ctrl != nullptr ? a.ctrl->num_splits : a.num_tasks;
  if (num_tasks <= 0 || static_cast<int>(blockIdx.x) >= (a.ctrl != nullptr ? a.ctrl->total_blocks : a.total_blocks)) { if (a.sig.world > 1) FabricSignalDone(a.sig, gridDim.x * gridDim.y); return; }
  const int ti = FindTask(a.tasks, num_tasks, blockIdx.x);
  const HistTask task = a.tasks[ti];
  const int chunk = blockIdx.x - task.block_begin;
  const long long row0 = static_cast<long long>(chunk) * a.rows_per_block;
  // a task always keeps its first block (even with no local rows): it closes the task's reduce-scatter
  const int row_blocks = max(1, (task.count + a.rows_per_block - 1) / a.rows_per_block);
  if (chunk >= task.num_blocks || chunk >= row_blocks) { if (a.sig.world > 1) FabricSignalDone(a.sig, gridDim.x * gridDim.y); return; }
  const int nrows = static_cast<int>(max(0LL, min(static_cast<long long>(a.rows_per_block), task.count - row0)));
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
    const int gb = part.bin_begin + b;
    double* p = d.num_ranks > 1 ? static_cast<double*>(d.stage_local) + 2 * (static_cast<long long>(ti) * a.num_total_bin + gb)
                                : static_cast<double*>(d.pool[0]) + 2 * (static_cast<long long>(task.slot) * d.slot_stride[0] + d.bin_local[gb]);
    atomicAdd(p, static_cast<double>(g)); atomicAdd(p + 1, static_cast<double>(h));
  }
  const bool pushed = d.num_ranks > 1 && PushTaskIfLast<false>(a, ti, task);
  if (a.sig.world > 1) FabricSignalDone(a.sig, gridDim.x * gridDim.y, pushed);
}

// Transpose tile of the compact view: 32 rows x 32 listed groups per block.
__global__ void __launch_bounds__(256) CompactGatherKernel(const uint8_t* __restrict__ cols, long long col_stride, int n, const int* __restrict__ groups,
                                                           int num_groups, uint8_t* __restrict__ out, int out_stride) {
  __shared__ uint8_t tile[32][33];
  const int row0 = blockIdx.x * 32, j0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;   // 32 x 8
  for (int jj = ty; jj < 32; jj += 8) {
    const int j = j0 + jj, row = row0 + tx;
    tile[jj][tx] = (j < num_groups && row < n) ? cols[static_cast<size_t>(groups[j]) * col_stride + row] : 0;
  }
  __syncthreads();
  for (int rr = ty; rr < 32; rr += 8) {
    const int row = row0 + rr, j = j0 + tx;
    if (row < n && j < out_stride) out[static_cast<size_t>(row) * out_stride + j] = tile[tx][rr];
  }
}

// 4-bit variant: 32 rows x 64 listed groups per block, two groups per output byte.
__global__ void __launch_bounds__(256) CompactGatherPack4Kernel(const uint8_t* __restrict__ cols, long long col_stride, int n, const int* __restrict__ groups,
                                                                int num_groups, uint8_t* __restrict__ out, int out_stride) {
  __shared__ uint8_t tile[64][33];
  const int row0 = blockIdx.x * 32, j0 = blockIdx.y * 64;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int jj = ty; jj < 64; jj += 8) {
    const int j = j0 + jj, row = row0 + tx;
    tile[jj][tx] = (j < num_groups && row < n) ? cols[static_cast<size_t>(groups[j]) * col_stride + row] : 0;
  }
  __syncthreads();
  for (int rr = ty; rr < 32; rr += 8) {
    const int row = row0 + rr, byte = j0 / 2 + tx;
    if (row < n && byte < out_stride) out[static_cast<size_t>(row) * out_stride + byte] = static_cast<uint8_t>((tile[2 * tx][rr] & 15) | (tile[2 * tx + 1][rr] << 4));
  }
}

}  // namespace

void LaunchCompactGather(const uint8_t* cols, long long col_stride, int n, const int* groups, int num_groups, uint8_t* out, int out_stride, cudaStream_t s, bool pack4) {
  if (n <= 0 || num_groups <= 0) return;
  if (pack4) {
    dim3 grid((n + 31) / 32, (2 * out_stride + 63) / 64);
    CompactGatherPack4Kernel<<<grid, 256, 0, s>>>(cols, col_stride, n, groups, num_groups, out, out_stride);
    FB_LAUNCHED(); FB_KERNEL_CHECK();
    return;
  }
  dim3 grid((n + 31) / 32, (out_stride + 31) / 32);
  CompactGatherKernel<<<grid, 256, 0, s>>>(cols, col_stride, n, groups, num_groups, out, out_stride);
  FB_LAUNCHED(); FB_KERNEL_CHECK();
}

// Block shape of the lane construct, measured on B200 at 11M x 28 and 1.4M x 28 rows (ms per boosting round, 64-bin
// integer tiles):
//   load-add-store form: 20 warps with a tile each              2.82 / 0.986
//   reduction form:      20 warps x 1 per tile 2.69 / 0.958;  32 x 2: 2.63 / 0.919;  32 x 4: 2.48 / 0.866;
//                        32 x 8 (4 tiles): 2.46 / 0.858;  32 x 32 (1 tile): 2.46 / 0.859;  3 or 4 stages: 1-2 % slower
// So: 32 warps on up to 4 tiles in the reduction form (fewer when the tiles are large: 256 bins, float planes), 20 warps
// otherwise. Many gradient levels leave a tile few rows before its 16-bit lanes could overflow (`sub_rows`): the block
// then keeps as many tiles as fit so that it still takes a few thousand rows.
// The environment overrides serve shape sweeps (FALCATA_LANE_WARPS: 4..32 warps per block, FALCATA_LANE_SHARE: warps per
// tile, a divisor of the warps; FALCATA_LANE_STAGES: 2..4).
struct LaneGeometry { int warps, share, stages; size_t smem; bool red; };
static LaneGeometry LaneShape(bool red, int sub_rows, int nb, bool flt) {
  LaneGeometry g;
  g.stages = 2;
  if (const char* e = std::getenv("FALCATA_LANE_STAGES")) g.stages = std::atoi(e);
  if (g.stages < 2 || g.stages > 4) Log::Fatal("FALCATA_LANE_STAGES must be 2, 3 or 4");
  const size_t tile_bytes = static_cast<size_t>(nb) * 32 * 4 * (flt ? 2 : 1);
  const size_t budget = 220 * 1024;
  // fp32 with 256-bin tiles: a tile per warp leaves room for three warps only, and one warp per scheduler cannot hide the
  // latency of its own dependent instructions (measured: 445 us against 326 us for a 1M x 100 root): reduction form
  if (flt && nb > 64) red = true;
  if (flt && !red) {
    // fp32, load-add-store: a tile per warp, as many warps as fit, and deeper staging since few warps are in flight
    if (std::getenv("FALCATA_LANE_STAGES") == nullptr) g.stages = 4;
    const size_t per_warp = tile_bytes + static_cast<size_t>(g.stages) * (32 * (32 + 8) + 8);
    g.warps = static_cast<int>(std::min<size_t>(16, budget / per_warp));
    if (const char* e = std::getenv("FALCATA_LANE_WARPS")) g.warps = std::min(g.warps, std::max(1, std::atoi(e)));
    if (g.warps < 1) Log::Fatal("lane histogram: a %d-bin fp32 tile does not fit in shared memory", nb);
    g.share = 1;
    g.smem = per_warp * g.warps;
    g.red = false;
    return g;
  }
  const bool wide = red && sub_rows >= 4096;
  g.warps = red ? 32 : 20;
  if (const char* e = std::getenv("FALCATA_LANE_WARPS")) g.warps = std::atoi(e);
  if (g.warps < 4 || g.warps > 32) Log::Fatal("FALCATA_LANE_WARPS must be within 4..32");
  const size_t stage_bytes = static_cast<size_t>(g.warps) * g.stages * (32 * (32 + (flt ? 8 : 4)) + 8);
  if (stage_bytes + tile_bytes > budget) Log::Fatal("lane histogram: a %d-bin tile does not fit beside the stages of %d warps", nb, g.warps);
  const int fit = static_cast<int>((budget - stage_bytes) / tile_bytes);
  int tiles = 1;
  if (!red) tiles = g.warps;   // the load-add-store form needs a tile per warp
  else for (int t = 1; t <= g.warps; ++t) if (g.warps % t == 0 && t <= fit && (!wide || t <= 4)) tiles = t;
  if (const char* e = std::getenv("FALCATA_LANE_SHARE")) { const int ss = std::atoi(e); if (red && ss >= 1 && g.warps % ss == 0) tiles = g.warps / ss; }
  if (tiles > fit) Log::Fatal("lane histogram: %d tiles of %d bins do not fit beside the stages of %d warps", tiles, nb, g.warps);
  g.share = g.warps / tiles;
  g.smem = stage_bytes + tile_bytes * tiles;
  g.red = red;
  return g;
}
int LaneRowsUnit(bool red, int sub_rows, int nb, bool flt) { return LaneShape(red, sub_rows, nb, flt).warps * 32; }
int LaneTiles(bool red, int sub_rows, int nb, bool flt) { const LaneGeometry g = LaneShape(red, sub_rows, nb, flt); return g.warps / g.share; }

template <int MODE>
static void LaunchLane(const HistArgs& a, cudaStream_t s, const LaneGeometry& g) {
  constexpr bool FLT = MODE != 0;
  const int ntiles = g.warps / g.share;
  if (!FLT) {
    const long long cap = static_cast<long long>(ntiles) * a.sub_rows;
    if (a.rows_per_block > cap) Log::Fatal("lane histogram: %d rows per block would overflow the 16-bit lanes (cap %lld)", a.rows_per_block, cap);
  }
  dim3 grid(a.total_blocks, (a.num_groups + 31) / 32);
  HistArgs b = a; b.lane_share = g.share;
#define FB_LANE(NB, ST)                                                                                                            \
  {                                                                                                                                \
    static bool attr = false;                                                                                                      \
    if (!attr) { FB_CUDA(cudaFuncSetAttribute(HistQuantLaneKernel<NB, ST, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024)); attr = true; } \
    HistQuantLaneKernel<NB, ST, MODE><<<grid, g.warps * 32, g.smem, s>>>(b);                                                       \
  }
#define FB_LANE_ST(NB) { if (g.stages == 2) FB_LANE(NB, 2) else if (g.stages == 3) FB_LANE(NB, 3) else FB_LANE(NB, 4) }
  if (a.lane_bins == 16) FB_LANE_ST(16)
  else if (a.lane_bins == 64) FB_LANE_ST(64)
  else if (a.lane_bins == 256) FB_LANE_ST(256)
  else Log::Fatal("lane histogram: unsupported tile of %d bins", a.lane_bins);
#undef FB_LANE_ST
#undef FB_LANE
  FB_LAUNCHED(); FB_KERNEL_CHECK();
}

void LaunchHistConstructQuant(const HistArgs& a, cudaStream_t s) {
  if (a.total_blocks <= 0 || a.num_tasks <= 0) return;
  if (a.lane_mode == 3) {
    if (LaunchHistConstructQuantTC(a, s)) return;
    Log::Fatal("tensor-core histogram: the shape is outside what the instance covers (root level, 32-byte rows, <= 32 groups of <= 64 bins, one rank)");
  }
  if (a.lane_mode != 0) { LaunchLane<0>(a, s, LaneShape(a.lane_red != 0, a.sub_rows, a.lane_bins, false)); return; }
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
  if (a.lane_mode != 0) {
    const LaneGeometry g = LaneShape(a.lane_red != 0, a.sub_rows, a.lane_bins, true);
    if (g.red) LaunchLane<2>(a, s, g); else LaunchLane<1>(a, s, g);
    return;
  }
  const size_t sm = static_cast<size_t>(a.max_part_bins) * 8 + static_cast<size_t>(a.num_groups) * 4;
  static bool attr = false; if (!attr) { FB_CUDA(cudaFuncSetAttribute(HistFloatKernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)); attr = true; }
  dim3 grid(a.total_blocks, a.num_parts);
  HistFloatKernel<<<grid, kHistThreads, sm, s>>>(a);
  FB_LAUNCHED(); FB_KERNEL_CHECK();
}

}  // namespace fb
