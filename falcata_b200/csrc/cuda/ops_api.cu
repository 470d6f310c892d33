// Kernel-level C entry points: each runs ONE device kernel of the training path on caller-owned
// device buffers, so that the numerics tests can compare it with a plain PyTorch reference.
#include "kernels.cuh"

#include <vector>

using namespace fb;

namespace {
thread_local std::string g_ops_error;
std::vector<HistPartition> MakePartitions(const std::vector<int>& gstart, const std::vector<int>& gbins, int max_bins) {
  std::vector<HistPartition> parts; const int G = static_cast<int>(gbins.size()); int g = 0;
  while (g < G) {
    HistPartition p; p.group_begin = g; p.bin_begin = gstart[g]; p.bin_count = 0; int e = g;
    while (e < G) { int e4 = std::min(G, e + 4), add = 0; for (int k = e; k < e4; ++k) add += gbins[k]; if (p.bin_count + add > max_bins && e > g) break; p.bin_count += add; e = e4; }
    p.group_end = e; parts.push_back(p); g = e;
  }
  return parts;
}
}  // namespace

#define OPS_BEGIN() try {
#define OPS_END() } catch (std::exception& ex) { g_ops_error = ex.what(); return -1; } return 0;

namespace fb {
__global__ void BoundedWaitProbeKernel(const unsigned int* flag, unsigned int* status, unsigned int* seen, unsigned long long max_spins) {
  FabricWait w; w.world = 1; w.flags = flag; w.epoch = 1u; w.max_spins = max_spins; w.status = status;
  FabricWaitAll(w);                       // the production wait: bounded, reports through the status word
  if (threadIdx.x == 0) *seen = (*reinterpret_cast<const volatile unsigned int*>(flag) >= 1u) ? 1u : 0u;
}
}  // namespace fb

extern "C" {

const char* FB_OpsLastError() { return g_ops_error.c_str(); }

// Histogram of rows idx[0..count) (or rows 0..count-1 when idx is null).
// quant != 0: gh is int32 packed (g16|h16) per row, out is int64 [total_bins x 2] (grad, hess sums).
// quant == 0: gh is float2 per row, out is float64 [total_bins x 2].
int FB_OpHistogram(const uint8_t* rows, int row_stride, int num_groups, const void* gh, int gh_stride, const int* idx, int count,
                   const int* group_num_bin_host, int quant, int quant_bins, int rows_per_block, int max_part_bins, int lane_mode, void* out) {
  OPS_BEGIN();
  std::vector<int> gbins(group_num_bin_host, group_num_bin_host + num_groups), gstart(num_groups);
  int total = 0; for (int g = 0; g < num_groups; ++g) { gstart[g] = total; total += gbins[g]; }
  auto parts = MakePartitions(gstart, gbins, max_part_bins > 0 ? max_part_bins : 6144);
  int mpb = 0; for (auto& p : parts) mpb = std::max(mpb, p.bin_count);
  cudaStream_t s = 0;
  DevBuf<HistPartition> d_parts; d_parts.Upload(parts, s);
  DevBuf<int> d_gstart; d_gstart.Upload(gstart, s);
  std::vector<unsigned char> owner(total, 0); std::vector<int> local(total); for (int b = 0; b < total; ++b) local[b] = b;
  DevBuf<unsigned char> d_owner; d_owner.Upload(owner, s); DevBuf<int> d_local; d_local.Upload(local, s);
  HistTask t; t.slot = 0; t.begin = 0; t.count = count; t.buffer = 0; t.block_begin = 0; t.pad0 = t.pad1 = 0;
  if (rows_per_block <= 0) rows_per_block = 2048;
  t.num_blocks = (count + rows_per_block - 1) / rows_per_block;
  DevBuf<HistTask> d_task; d_task.Upload(&t, 1, s);
  DevBuf<char> pool; pool.Alloc(static_cast<size_t>(total) * (quant ? 8 : 16)); pool.Zero(s);
  HistArgs a = HistArgs();
  a.rows = rows; a.row_stride = row_stride; a.num_groups = num_groups; a.gh_base = static_cast<const uint8_t*>(gh); a.gh_stride = gh_stride;
  a.idx[0] = idx; a.idx[1] = idx; a.tasks = d_task.get(); a.num_tasks = 1; a.total_blocks = t.num_blocks; a.parts = d_parts.get(); a.num_parts = static_cast<int>(parts.size());
  a.max_part_bins = mpb; a.group_bin_start = d_gstart.get(); a.rows_per_block = rows_per_block;
  const int qb = std::max(2, quant_bins);
  a.sub_rows = quant ? std::max(1, std::min(65535 / qb, 32767 / std::max(1, qb / 2))) : (1 << 30);
  a.identity_root = idx == nullptr ? 1 : 0;
  a.num_total_bin = total; a.lane_mode = quant ? lane_mode : (lane_mode == 1 || lane_mode == 2 ? 1 : 0); a.lane_red = quant ? 1 : (lane_mode == 2 ? 1 : 0);   // fp32: lane_mode 1 load-add-store, 2 reduction adds
  a.bulk_root = getenv("FALCATA_NO_BULK_ROOT") == nullptr ? 1 : 0;   // the kernel itself decides where the bulk-copy pipeline applies
  int mgb = 0; for (int v : gbins) mgb = std::max(mgb, v);
  a.lane_bins = mgb <= 16 ? 16 : (mgb <= 64 ? 64 : 256);
  if (a.lane_mode != 0 && mgb > 256) Log::Fatal("lane histogram covers groups of at most 256 bins");
  if (a.lane_mode == 3 && mgb > 64) Log::Fatal("tensor-core histogram covers groups of at most 64 bins");
  if (a.lane_mode == 3) {
    if (quant_bins > 127) Log::Fatal("tensor-core histogram: quantized values must fit 8 bits");
    a.lane_bins = 64; a.tc_row_count = count;
    cudaDeviceProp prop; int dev = 0; FB_CUDA(cudaGetDevice(&dev)); FB_CUDA(cudaGetDeviceProperties(&prop, dev));
    a.rows_per_block = rows_per_block = HistTcRowsPerBlock(count, prop.multiProcessorCount);
    t.num_blocks = (count + rows_per_block - 1) / rows_per_block; a.total_blocks = t.num_blocks;
    d_task.Upload(&t, 1, s);
  }
  if (a.lane_mode == 1 && quant && rows_per_block > static_cast<long long>(LaneTiles(true, a.sub_rows, a.lane_bins, false)) * a.sub_rows) { a.rows_per_block = rows_per_block = LaneTiles(true, a.sub_rows, a.lane_bins, false) * a.sub_rows; }
  if (a.lane_mode == 2 && rows_per_block > a.sub_rows) { a.rows_per_block = rows_per_block = a.sub_rows; }
  if (a.lane_mode == 1 || a.lane_mode == 2) {
    t.num_blocks = (count + rows_per_block - 1) / rows_per_block; a.total_blocks = t.num_blocks;
    d_task.Upload(&t, 1, s);
  }
  for (int r = 0; r < 8; ++r) { a.dest.pool[r] = nullptr; a.dest.slot_stride[r] = 0; }
  a.dest.pool[0] = pool.get(); a.dest.slot_stride[0] = total; a.dest.bin_owner = d_owner.get(); a.dest.bin_local = d_local.get(); a.dest.num_ranks = 1; a.dest.rank = 0;
  if (quant) LaunchHistConstructQuant(a, s); else LaunchHistConstructFloat(a, s);
  FB_CUDA(cudaStreamSynchronize(s));
  if (quant) {
    std::vector<hist_q_t> h(total); FB_CUDA(cudaMemcpy(h.data(), pool.get(), total * 8, cudaMemcpyDeviceToHost));
    std::vector<long long> o(2 * static_cast<size_t>(total)); for (int b = 0; b < total; ++b) { o[2 * b] = HistQGrad(h[b]); o[2 * b + 1] = HistQHess(h[b]); }
    FB_CUDA(cudaMemcpy(out, o.data(), o.size() * 8, cudaMemcpyHostToDevice));
  } else FB_CUDA(cudaMemcpy(out, pool.get(), static_cast<size_t>(total) * 16, cudaMemcpyDeviceToDevice));
  OPS_END();
}

// Quantize float gradients into packed words; returns scales (2 floats) and integer sums (2 int64) on the device.
int FB_OpQuantize(const float* grad, const float* hess, int n, int bins, int stochastic, unsigned int seed, unsigned int iter_key, unsigned long long row_offset,
                  int* out_packed, float* out_scales, long long* out_sums) {
  OPS_BEGIN();
  cudaStream_t s = 0;
  DevBuf<float> maxbuf; maxbuf.Alloc(2);
  LaunchAbsMax(grad, hess, n, 1, maxbuf.get(), s);
  LaunchQuantize(grad, hess, n, maxbuf.get(), nullptr, bins, stochastic != 0, seed, iter_key, row_offset, reinterpret_cast<uint8_t*>(out_packed), 4, out_scales, out_sums, s);
  FB_CUDA(cudaStreamSynchronize(s));
  OPS_END();
}

// Stable partition of idx[0..count) by "bin(row, group) <= threshold"; writes the result to out_idx and the left count to *left_count (host).
int FB_OpPartition(const uint8_t* rows, int row_stride, const int* idx, int count, int group, int threshold, int default_left, int missing_type, int default_bin,
                   int num_bin, int* out_idx, int* left_count) {
  OPS_BEGIN();
  cudaStream_t s = 0;
  PartSplit sp; memset(&sp, 0, sizeof(sp));
  sp.leaf = 0; sp.right_leaf = 1; sp.begin = 0; sp.count = count; sp.buffer = 0; sp.group = group; sp.num_bin = num_bin; sp.threshold = threshold; sp.default_left = default_left;
  sp.missing_type = missing_type; sp.default_bin = default_bin; sp.chunk_begin = 0; sp.num_chunks = (count + kPartChunk - 1) / kPartChunk;
  ChildInit ci; memset(&ci, 0, sizeof(ci)); ci.left_slot = 0; ci.right_slot = 1; ci.smaller_is_left = 1; ci.hist_num_blocks = 1;
  LeafInfo leaf; memset(&leaf, 0, sizeof(leaf)); leaf.count = count;
  DevBuf<PartSplit> d_sp; d_sp.Upload(&sp, 1, s); DevBuf<ChildInit> d_ci; d_ci.Upload(&ci, 1, s);
  DevBuf<LeafInfo> d_leaves; d_leaves.Alloc(2); d_leaves.Upload(&leaf, 1, s); d_leaves.Alloc(2);
  DevBuf<LeafInfo> d_leaves2; d_leaves2.Alloc(2); FB_CUDA(cudaMemcpyAsync(d_leaves2.get(), d_leaves.get(), sizeof(LeafInfo), cudaMemcpyDeviceToDevice, s));
  DevBuf<unsigned int> bits; bits.Alloc(static_cast<size_t>(sp.num_chunks + 1) * (kPartChunk / 32));
  DevBuf<int> chunk_left; chunk_left.Alloc(sp.num_chunks + 1); DevBuf<int> left_total; left_total.Alloc(1); DevBuf<HistTask> tasks; tasks.Alloc(1);
  PartArgs a = PartArgs(); a.rows = rows; a.row_stride = row_stride; a.cols = nullptr; a.col_stride = 0; a.idx[0] = const_cast<int*>(idx); a.idx[1] = out_idx; a.splits = d_sp.get(); a.num_splits = 1; a.total_chunks = sp.num_chunks;
  a.bits = bits.get(); a.chunk_left = chunk_left.get(); a.split_left_total = left_total.get(); a.leaves = d_leaves2.get(); a.child_init = d_ci.get(); a.hist_tasks = tasks.get(); a.rows_per_block = 2048;
  LaunchPartitionFlags(a, s); LaunchPartitionScanSetup(a, s); LaunchPartitionScatter(a, s);
  FB_CUDA(cudaMemcpyAsync(left_count, left_total.get(), sizeof(int), cudaMemcpyDeviceToHost, s));
  FB_CUDA(cudaStreamSynchronize(s));
  OPS_END();
}

// Failure-detection probe: one block waits, with the given spin budget, for a flag that nothing sets.
// The wait must run out, record kStatusWaitTimeout in the status word and return: *out_status is that
// word, *out_flag_seen tells whether the wait (wrongly) reported the flag as set.
int FB_OpBoundedWaitProbe(long long max_spins, int* out_status, int* out_flag_seen) {
  OPS_BEGIN();
  cudaStream_t s = 0;
  DevBuf<unsigned int> words; words.Alloc(3); words.Zero(s);   // [0] flag (stays 0), [1] status, [2] seen
  BoundedWaitProbeKernel<<<1, 32, 0, s>>>(words.get(), words.get() + 1, words.get() + 2, static_cast<unsigned long long>(std::max(1LL, max_spins)));
  FB_LAUNCHED(); FB_KERNEL_CHECK();
  unsigned int h[3] = {0, 0, 0};
  FB_CUDA(cudaMemcpyAsync(h, words.get(), sizeof(h), cudaMemcpyDeviceToHost, s));
  FB_CUDA(cudaStreamSynchronize(s));
  *out_status = static_cast<int>(h[1]); *out_flag_seen = static_cast<int>(h[2]);
  OPS_END();
}

// Rows of [global_offset, global_offset + n) whose Philox draw (keyed on seed and the GLOBAL row id) falls below
// `fraction`, ascending, as local indices. The draw depends on nothing else, so any sharding of the rows and both
// variants (device kernel, host loop) select the same global rows. Used for the bin-construction sample.
int FB_OpBernoulliRowsDevice(int n, long long global_offset, unsigned int seed, double fraction, int* out_idx_device, int* out_count) {
  OPS_BEGIN();
  cudaStream_t s = 0;
  // scratch kept between calls: freeing device memory waits for every copy in flight on the device, and this draw
  // runs while the caller's matrix is still on its way to the GPU
  static thread_local DevBuf<uint8_t> mask; static thread_local DevBuf<int> chunk, cnt;
  mask.Alloc(std::max(1, n)); chunk.Alloc(n / 1024 + 2); cnt.Alloc(1);
  BagArgs a = BagArgs();
  a.n = n; a.global_row_offset = static_cast<unsigned long long>(global_offset); a.round = 0x5A3Du; a.seed = seed; a.fraction = fraction; a.pos_fraction = a.neg_fraction = 1.0;
  a.mask = mask.get(); a.bag_idx = out_idx_device; a.chunk_count = chunk.get(); a.bag_count = cnt.get();
  LaunchBagging(a, s);
  FB_CUDA(cudaMemcpyAsync(out_count, cnt.get(), sizeof(int), cudaMemcpyDeviceToHost, s));
  FB_CUDA(cudaStreamSynchronize(s));
  OPS_END();
}
int FB_OpBernoulliRowsHost(int n, long long global_offset, unsigned int seed, double fraction, int* out_idx, int* out_count) {
  OPS_BEGIN();
  // row blocks on the host cores: flags per block, block offsets in order, then the ascending fill
  const int kBlock = 1 << 16;
  const int nblocks = (n + kBlock - 1) / kBlock;
  std::vector<int> count(nblocks + 1, 0);
  std::vector<uint8_t> flag(static_cast<size_t>(std::max(1, n)));
#pragma omp parallel for schedule(static) num_threads(TeamThreads())
  for (int b = 0; b < nblocks; ++b) {
    int c = 0;
    for (int i = b * kBlock; i < std::min(n, (b + 1) * kBlock); ++i) {
      const float u = U01From24(Philox4x32_10(static_cast<uint32_t>(static_cast<unsigned long long>(global_offset) + static_cast<unsigned long long>(i)), 0x5A3Du, 0xBA660000u, 0u, seed, 0x9876u).v[0]);
      const bool in = static_cast<double>(u) < fraction;
      flag[i] = in ? 1 : 0; c += in ? 1 : 0;
    }
    count[b + 1] = c;
  }
  for (int b = 0; b < nblocks; ++b) count[b + 1] += count[b];
#pragma omp parallel for schedule(static) num_threads(TeamThreads())
  for (int b = 0; b < nblocks; ++b) {
    int w = count[b];
    for (int i = b * kBlock; i < std::min(n, (b + 1) * kBlock); ++i) if (flag[i]) out_idx[w++] = i;
  }
  *out_count = count[nblocks];
  OPS_END();
}

int FB_OpLaunchCount(long long* out) { *out = LaunchCounter().load(); return 0; }

}  // extern "C"
