// Allocation-free stable row partition: see fb/no_alloc.h for who needs it, the limits and the
// sharing rules. Same kernels as FB_OpPartition; only the home of the scratch memory differs.
#include "fb/no_alloc.h"

#include "kernels.cuh"

using namespace fb;

namespace {

constexpr int kMaxChunks = FB_NO_ALLOC_MAX_ROWS / kPartChunk;

struct NoAllocScratch {
  PartSplit split;
  ChildInit child;
  LeafInfo leaves[2];
  HistTask task;
  int left_total;
  int pad[3];
  int chunk_left[kMaxChunks + 1];
  unsigned int bits[(kMaxChunks + 1) * (kPartChunk / 32)];
};

// The scratch array is part of the library image: every device that loads the library gets its
// own copy, which stays until the process exits. In HOST code this name is only a handle for the
// runtime's symbol table, not a device address; the address is asked for once per device below.
static __device__ __align__(256) unsigned char g_no_alloc_scratch[sizeof(NoAllocScratch)];

// Descriptors travel as kernel parameters and are written into the scratch array by device code
// (device code can name the array directly), so no host-to-device copy is needed either.
__global__ void NoAllocSetupKernel(PartSplit sp, ChildInit ci, LeafInfo leaf) {
  NoAllocScratch* s = reinterpret_cast<NoAllocScratch*>(g_no_alloc_scratch);
  s->split = sp; s->child = ci; s->leaves[0] = leaf; s->leaves[1] = leaf; s->left_total = 0;
}

thread_local std::string g_no_alloc_error;
constexpr int kMaxDevices = 64;
void* g_scratch_addr[kMaxDevices] = {nullptr};

}  // namespace

extern "C" {

const char* FB_NoAllocLastError() { return g_no_alloc_error.c_str(); }

int FB_OpPartitionNoAlloc(const uint8_t* rows, int row_stride, const int* idx, int count, int group, int threshold, int default_left,
                          int missing_type, int default_bin, int num_bin, int* out_idx, int* left_count_device, void* stream) {
  try {
    if (count < 0 || count > FB_NO_ALLOC_MAX_ROWS)
      Log::Fatal("FB_OpPartitionNoAlloc handles at most %d rows per call (got %d): split the call or use FB_OpPartition", FB_NO_ALLOC_MAX_ROWS, count);
    if (row_stride <= 0 || group < 0 || group >= row_stride)
      Log::Fatal("FB_OpPartitionNoAlloc: feature group %d is outside a row of %d bytes", group, row_stride);
    if (left_count_device == nullptr || (count > 0 && (rows == nullptr || idx == nullptr || out_idx == nullptr)))
      Log::Fatal("FB_OpPartitionNoAlloc: a null buffer was passed (rows, idx, out_idx and left_count_device must be device pointers)");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int dev = 0;
    FB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) Log::Fatal("device ordinal %d is outside the supported range", dev);
    if (g_scratch_addr[dev] == nullptr) {
      // first call on this device: resolve the device address of the scratch array (no allocation). Two host
      // threads that both make a first call may both run the lookup; they store the same value, so the race is harmless.
      void* p = nullptr;
      const cudaError_t e = cudaGetSymbolAddress(&p, g_no_alloc_scratch);
      if (e != cudaSuccess || p == nullptr) Log::Fatal("cudaGetSymbolAddress failed for the scratch array: %s", cudaGetErrorString(e));
      g_scratch_addr[dev] = p;
    }
    NoAllocScratch* sc = static_cast<NoAllocScratch*>(g_scratch_addr[dev]);
    PartSplit sp; memset(&sp, 0, sizeof(sp));
    sp.leaf = 0; sp.right_leaf = 1; sp.begin = 0; sp.count = count; sp.buffer = 0; sp.group = group; sp.num_bin = num_bin; sp.threshold = threshold;
    sp.default_left = default_left; sp.missing_type = missing_type; sp.default_bin = default_bin; sp.chunk_begin = 0; sp.num_chunks = (count + kPartChunk - 1) / kPartChunk;
    ChildInit ci; memset(&ci, 0, sizeof(ci)); ci.left_slot = 0; ci.right_slot = 1; ci.smaller_is_left = 1; ci.hist_num_blocks = 1;
    LeafInfo leaf; memset(&leaf, 0, sizeof(leaf)); leaf.count = count;
    NoAllocSetupKernel<<<1, 1, 0, s>>>(sp, ci, leaf);
    FB_LAUNCHED(); FB_KERNEL_CHECK();
    PartArgs a = PartArgs();
    a.rows = rows; a.row_stride = row_stride; a.cols = nullptr; a.col_stride = 0; a.idx[0] = const_cast<int*>(idx); a.idx[1] = out_idx;
    a.splits = &sc->split; a.num_splits = 1; a.total_chunks = sp.num_chunks; a.bits = sc->bits; a.chunk_left = sc->chunk_left; a.split_left_total = &sc->left_total;
    a.leaves = sc->leaves; a.child_init = &sc->child; a.hist_tasks = &sc->task; a.rows_per_block = 2048; a.world = 1;
    LaunchPartitionFlags(a, s); LaunchPartitionScanSetup(a, s); LaunchPartitionScatter(a, s);
    FB_CUDA(cudaMemcpyAsync(left_count_device, &sc->left_total, sizeof(int), cudaMemcpyDeviceToDevice, s));
  } catch (std::exception& ex) { g_no_alloc_error = ex.what(); return -1; }
  return 0;
}

}  // extern "C"
