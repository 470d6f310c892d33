// K1q on the tensor cores: the root-level quantized histogram as a one-hot integer GEMM on tcgen05.
//
// For one feature group, hist[bin] = sum over rows of v(row) * [bin(row) == bin] is a contraction over rows. With
// bin = 8 * hi + lo (groups of at most 64 bins) the indicator factorises, [bin == 8 hi + lo] = [hi(row) == hi] *
// [lo(row) == lo], so for a set of 8 groups
//     D[(val, g, hi)][(g', lo)] = sum_rows A[(val, g, hi)][row] * B[row][(g', lo)]
//     A = v_val(row) * [hi_g(row) == hi]   (val = gradient or hessian word, signed 8-bit)   128 x K
//     B = [lo_g'(row) == lo]               (0 / 1)                                           K x 64
// holds every group's histogram on its block diagonal (g == g'): one `tcgen05.mma.kind::i8` of M = 128, N = 64,
// K = 32 rows per set and step, int32 accumulators in tensor memory. 1 / 8 of the outputs are used; in exchange a
// (row, group) costs 24 operand bytes instead of the 128 a plain one-hot over 64 bins x 2 values would.
//
// Per CTA (128 threads, a contiguous slice of the rows):
//   * one thread feeds a 4-stage ring of raw tiles (32 rows x 32 bin bytes, 32 gradient words) with tensor-map TMA
//     loads (`cp.async.bulk.tensor`, no multicast; rows past the end read as zero and contribute nothing);
//   * all threads turn a raw tile into the A / B operand tiles of the four 8-group sets (a thread = one row x one set,
//     a warp = 32 rows of one set): operands are MN-major (16 consecutive M or N bytes per row), so the two groups of
//     a byte pair become ONE 16-byte store per operand, v << (8 * hi) resp. 1 << (8 * lo) per half, and a warp's
//     stores are 512 contiguous bytes;
//   * one thread issues the four MMAs of the step and commits them to the "operand stage free" mbarrier (2 stages);
//   * after the last step the accumulators (4 sets x 64 columns x 128 lanes) are read back with `tcgen05.ld`, the
//     diagonal blocks are kept and added into the leaf's pool slot like every other construct instance does.
// Every wait is bounded; a wait that gives up records the status word, lets the copies in flight land (bounded),
// frees the tensor memory and leaves.
//
// Covers: root level (rows in order), 32-byte rows, at most 32 groups of at most 64 bins, |quantized values| <= 127,
// one rank. Parity: the reference's tensor-core prototype (benchmarks/tc_hist_prototype.cu: wmma / mma.sync one-hot
// kernels); this instance is the tcgen05 form of that experiment. Measured against the lane kernel it does not win
// (operand construction costs about as many instructions per (row, group) as the direct update and three times the
// shared-memory bytes), so the planner keeps it off; `cuda_plan=hist_tc:on` selects it.
#include <cuda.h>
#include <cudaTypedefs.h>

#include "kernels.cuh"

namespace fb {

namespace {

constexpr int kTcThreads = 128;
constexpr int kTcRows = 32;                        // rows per step = K of one kind::i8 MMA
constexpr int kTcSets = 4;                         // 8 groups per set
constexpr int kRawStages = 4, kOpStages = 2;
constexpr int kABytes = 128 * kTcRows, kBBytes = 64 * kTcRows;
constexpr int kSetBytes = kABytes + kBBytes;       // 6144
constexpr int kOpStageBytes = kTcSets * kSetBytes; // 24576
constexpr int kTmemCols = 256;                     // 4 sets x 64 accumulator columns
constexpr int kOffRawGh = kRawStages * kTcRows * 32;          // 4096
constexpr int kOffBars = kOffRawGh + kRawStages * kTcRows * 4;   // 4608
constexpr int kOffTmemSlot = kOffBars + 64;
constexpr int kOffOps = 5120;
constexpr int kTcSmemBytes = kOffOps + kOpStages * kOpStageBytes + 1024;   // + slack for the 1024-byte alignment of the base
constexpr uint32_t kStageTxBytes = kTcRows * 32 + kTcRows * 4;

__device__ inline uint32_t Smem32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ inline void BarInit(uint64_t* bar, uint32_t count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(Smem32(bar)), "r"(count) : "memory"); }
__device__ inline void BarExpectTx(uint64_t* bar, uint32_t bytes) { asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(Smem32(bar)), "r"(bytes) : "memory"); }
__device__ inline bool BarTryWait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(Smem32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// false when the budget ran out
__device__ inline bool BarWaitBounded(uint64_t* bar, uint32_t parity) {
  for (int i = 0; i < (1 << 20); ++i) if (BarTryWait(bar, parity)) return true;
  return false;
}
// tile of a 2-D tensor map (x = byte inside the row, y = row) -> shared memory; completion in bytes on `bar`
__device__ inline void TmaLoad2D(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(Smem32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(Smem32(bar)) : "memory");
}
// Shared-memory matrix descriptor of an MN-major operand without swizzle: 16 consecutive M (N) bytes per K row, K rows
// 16 bytes apart inside an 8-row core matrix; `lbo` = bytes between core matrices along K, `sbo` = along M (N).
__device__ inline uint64_t OperandDesc(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
  return static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4) | (static_cast<uint64_t>(lbo >> 4) << 16) | (static_cast<uint64_t>(sbo >> 4) << 32) | (1ull << 46);
}
// kind::i8, D = S32, A = B = signed 8-bit, both MN-major, N = 64, M = 128
constexpr uint32_t kInstrDesc = (2u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | (1u << 16) | ((64u >> 3) << 17) | ((128u >> 4) << 24);
__device__ inline void MmaI8(uint32_t d_tmem, uint64_t da, uint64_t db, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
               ::"r"(d_tmem), "l"(da), "l"(db), "r"(kInstrDesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ inline void MmaCommit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(Smem32(bar)) : "memory");
}
__device__ inline void TmemLoad8(uint32_t taddr, int (&v)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]) : "r"(taddr) : "memory");
}

__global__ void __launch_bounds__(kTcThreads) HistQuantTCKernel(HistArgs a, const __grid_constant__ CUtensorMap rows_map, const __grid_constant__ CUtensorMap gh_map) {
  extern __shared__ unsigned char tc_smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(tc_smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  unsigned char* raw_rows = smem;                                    // [kRawStages][32 rows][32 B]
  int* raw_gh = reinterpret_cast<int*>(smem + kOffRawGh);            // [kRawStages][32]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kOffBars);     // raw_full[4], op_free[2], done
  uint64_t* raw_full = bars; uint64_t* op_free = bars + kRawStages; uint64_t* done = bars + kRawStages + kOpStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kOffTmemSlot);
  unsigned char* ops = smem + kOffOps;                               // [kOpStages][kTcSets][A 4096 | B 2048]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const HistTask task = a.tasks[0];
  const long long row0 = static_cast<long long>(blockIdx.x) * a.rows_per_block;
  const int nrows = static_cast<int>(max(0LL, min(static_cast<long long>(a.rows_per_block), task.count - row0)));
  if (nrows <= 0) return;   // before any allocation: nothing to free
  const int nsteps = (nrows + kTcRows - 1) / kTcRows;

  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(Smem32(tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (threadIdx.x == 0) {
    for (int i = 0; i < kRawStages; ++i) BarInit(raw_full + i, 1);
    for (int i = 0; i < kOpStages; ++i) BarInit(op_free + i, 1);
    BarInit(done, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

  auto issue_raw = [&](int step) {   // thread 0 only
    const int rs = step % kRawStages;
    const int y = static_cast<int>(task.begin + row0) + step * kTcRows;
    BarExpectTx(raw_full + rs, kStageTxBytes);
    TmaLoad2D(raw_rows + rs * kTcRows * 32, &rows_map, 0, y, raw_full + rs);
    TmaLoad2D(raw_gh + rs * kTcRows, &gh_map, y, 0, raw_full + rs);
  };
  if (threadIdx.x == 0) for (int st = 0; st < min(nsteps, kRawStages); ++st) issue_raw(st);

  // this thread: row r = lane of the step, the 8 groups of set `set` = warp. One 8-byte read of the raw tile per thread;
  // a warp's 16-byte operand stores cover 32 consecutive rows of one column group: contiguous, free of bank conflicts.
  const int r = lane, set = warp;
  bool ok = true;
  int step = 0;
  for (; step < nsteps; ++step) {
    const int rs = step % kRawStages, os = step % kOpStages;
    ok = BarWaitBounded(raw_full + rs, (step / kRawStages) & 1);
    if (ok && step >= kOpStages) ok = BarWaitBounded(op_free + os, ((step / kOpStages) - 1) & 1);
    ok = __syncthreads_and(ok ? 1 : 0) != 0;   // one decision per block
    if (!ok) break;
    const int w = raw_gh[rs * kTcRows + r];
    const int hq = w & 0xFFFF, gq = (w - hq) >> 16;
    const unsigned long long g8 = static_cast<unsigned long long>(static_cast<unsigned char>(static_cast<signed char>(gq)));
    const unsigned long long h8 = static_cast<unsigned long long>(static_cast<unsigned char>(static_cast<signed char>(hq)));
    const unsigned long long bins8 = *reinterpret_cast<const unsigned long long*>(raw_rows + (rs * kTcRows + r) * 32 + 8 * set);
    unsigned char* stage = ops + os * kOpStageBytes;
    unsigned char* A = stage + set * kSetBytes; unsigned char* B = A + kABytes;
    const int koff = (r >> 3) * 128 + (r & 7) * 16;   // this row inside a 16-byte column group: K core matrices 128 B apart
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {   // byte pair jj of the set = groups 8 set + 2 jj, + 1 = one 16-byte column group
      const int G0 = 8 * set + 2 * jj;
      const int b0 = static_cast<int>((bins8 >> (16 * jj)) & 0xFF), b1 = static_cast<int>((bins8 >> (16 * jj + 8)) & 0xFF);
      const bool v0 = G0 < a.num_groups, v1 = G0 + 1 < a.num_groups;
      const int s0 = 8 * (b0 >> 3), s1 = 8 * (b1 >> 3), l0 = 8 * (b0 & 7), l1 = 8 * (b1 & 7);
      ulonglong2 ag, ah, bb;
      ag.x = v0 ? g8 << s0 : 0ull; ag.y = v1 ? g8 << s1 : 0ull;
      ah.x = v0 ? h8 << s0 : 0ull; ah.y = v1 ? h8 << s1 : 0ull;
      bb.x = 1ull << l0; bb.y = 1ull << l1;
      *reinterpret_cast<ulonglong2*>(A + (0 * 4 + jj) * 512 + koff) = ag;   // M rows (val 0, groups 2 jj, 2 jj + 1 of the set, hi 0..7)
      *reinterpret_cast<ulonglong2*>(A + (1 * 4 + jj) * 512 + koff) = ah;   // M rows (val 1, ...)
      *reinterpret_cast<ulonglong2*>(B + jj * 512 + koff) = bb;             // N columns (groups 2 jj, 2 jj + 1, lo 0..7)
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // operand stores -> visible to the tensor core's reads
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (threadIdx.x == 0) {
      if (step + kRawStages < nsteps) issue_raw(step + kRawStages);   // every thread is done with this raw stage
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
      for (int s = 0; s < kTcSets; ++s) {
        const uint32_t abase = Smem32(stage + s * kSetBytes);
        MmaI8(tmem_base + s * 64, OperandDesc(abase, 128, 512), OperandDesc(abase + kABytes, 128, 512), step > 0 ? 1u : 0u);
      }
      MmaCommit(op_free + os);
      if (step == nsteps - 1) MmaCommit(done);
    }
  }
  if (ok) ok = __syncthreads_and(BarWaitBounded(done, 0) ? 1 : 0) != 0;
  if (!ok) {
    // a wait gave up: report it, then give the raw copies still in flight a (bounded) chance to land before leaving
    if (threadIdx.x == 0 && a.status != nullptr) atomicExch(a.status, static_cast<unsigned int>(kStatusWaitTimeout));
    if (threadIdx.x == 0) for (int t = step; t < min(nsteps, step + kRawStages); ++t) BarWaitBounded(raw_full + t % kRawStages, (t / kRawStages) & 1);
  } else {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    // warp w reads its own 32 lanes: M rows 32 w .. 32 w + 31 = (val = w / 2, group-in-set 4 (w & 1) + lane / 8, hi = lane % 8)
    const int val = warp >> 1, gsub = lane >> 3, hi = lane & 7;
#pragma unroll
    for (int s = 0; s < kTcSets; ++s) {
      int keep[8];
#pragma unroll
      for (int gq2 = 0; gq2 < 4; ++gq2) {
        int v[8];
        const int gset = 4 * (warp & 1) + gq2;   // the diagonal block of this group: columns 8 gset .. 8 gset + 7
        TmemLoad8(tmem_base + (static_cast<uint32_t>(32 * warp) << 16) + s * 64 + gset * 8, v);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (gsub == gq2) { for (int k = 0; k < 8; ++k) keep[k] = v[k]; }
      }
      const int G = 8 * s + 4 * (warp & 1) + gsub;
      if (G < a.num_groups) {
        const int gstart = a.group_bin_start[G];
        const int gbins = (G + 1 < a.num_groups ? a.group_bin_start[G + 1] : a.num_total_bin) - gstart;
#pragma unroll
        for (int lo = 0; lo < 8; ++lo) {
          const int bin = 8 * hi + lo;
          if (bin < gbins && keep[lo] != 0) {
            const hist_q_t add = val == 0 ? HistQPack(keep[lo], 0) : HistQPack(0, keep[lo]);
            atomicAdd(static_cast<hist_q_t*>(a.dest.pool[0]) + static_cast<long long>(task.slot) * a.dest.slot_stride[0] + a.dest.bin_local[gstart + bin], add);
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
}

PFN_cuTensorMapEncodeTiled_v12000 EncodeFn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = []() -> PFN_cuTensorMapEncodeTiled_v12000 {
    void* p = nullptr; cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) return nullptr;
    return reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  }();
  return fn;
}

}  // namespace

int HistTcRowsPerBlock(long long count, int num_sms) {
  // two CTAs per SM (tensor memory: 2 x 256 of 512 columns), whole 32-row steps
  long long rpb = (count + 2LL * num_sms - 1) / (2LL * num_sms);
  rpb = (rpb + kTcRows - 1) / kTcRows * kTcRows;
  return static_cast<int>(std::max<long long>(rpb, 8 * kTcRows));
}

bool LaunchHistConstructQuantTC(const HistArgs& a, cudaStream_t s) {
  if (a.identity_root == 0 || a.row_stride != 32 || a.num_groups > 32 || a.pack4 != 0 || a.gh_stride != 4 || a.num_tasks != 1 || a.ctrl != nullptr ||
      a.dest.num_ranks > 1 || a.sig.world > 1 || a.dest.owner_only != 0 || a.group_bin_count != nullptr || a.lane_bins > 64 || a.rows_per_block % kTcRows != 0 ||
      a.total_blocks <= 0) {
    Log::Warning("tensor-core histogram: unsupported shape (identity %d stride %d groups %d pack4 %d gh_stride %d tasks %d ranks %d world %d lane_bins %d rpb %d blocks %d)", a.identity_root,
                 a.row_stride, a.num_groups, a.pack4, a.gh_stride, a.num_tasks, a.dest.num_ranks, a.sig.world, a.lane_bins, a.rows_per_block, a.total_blocks);
    return false;
  }
  PFN_cuTensorMapEncodeTiled_v12000 encode = EncodeFn();
  if (encode == nullptr) { Log::Warning("tensor-core histogram: the driver's tensor-map encoder is not available"); return false; }
  // the kernel reads the task's row count from device memory; the maps are sized from the launch bounds
  const unsigned long long nrows = static_cast<unsigned long long>(a.total_blocks) * a.rows_per_block;
  const unsigned long long count = a.tc_row_count > 0 ? static_cast<unsigned long long>(a.tc_row_count) : nrows;
  CUtensorMap rows_map, gh_map;
  {
    const cuuint64_t dims[2] = {32, count}; const cuuint64_t strides[1] = {32};
    const cuuint32_t box[2] = {32, kTcRows}; const cuuint32_t estr[2] = {1, 1};
    if (encode(&rows_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(a.rows), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
               CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) { Log::Warning("tensor-core histogram: the row tensor map was refused"); return false; }
  }
  {
    // the gradient words as a one-row 2-D tensor: x = row (out-of-range x reads as zero), y = 0
    const cuuint64_t dims[2] = {count, 1}; const cuuint64_t strides[1] = {(count * 4 + 15) / 16 * 16};
    const cuuint32_t box[2] = {kTcRows, 1}; const cuuint32_t estr[2] = {1, 1};
    const CUresult rc = encode(&gh_map, CU_TENSOR_MAP_DATA_TYPE_INT32, 2, const_cast<uint8_t*>(a.gh_base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                               CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) { Log::Warning("tensor-core histogram: the gradient tensor map was refused (driver code %d)", static_cast<int>(rc)); return false; }
  }
  static bool attr = false;
  if (!attr) { FB_CUDA(cudaFuncSetAttribute(HistQuantTCKernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kTcSmemBytes)); attr = true; }
  HistQuantTCKernel<<<a.total_blocks, kTcThreads, kTcSmemBytes, s>>>(a, rows_map, gh_map);
  FB_LAUNCHED(); FB_KERNEL_CHECK();
  return true;
}

}  // namespace fb
