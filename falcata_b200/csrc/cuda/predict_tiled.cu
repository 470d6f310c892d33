// K7, tiled form: a block stages a tile of rows in shared memory once (feature-major, so that the lane that owns a
// row always reads its own bank) and walks it through the whole forest; the trees stream through shared memory in
// chunks of a few trees, double-buffered with asynchronous copies, as 8-byte nodes whose two children sit next to
// each other. Every thread owns one row and keeps eight tree walks in flight.
//
// Parity: python-package/falcata/basic.py:L5112-5163 (device predict route: raw score, converted score, leaf index),
// include/Falcata/tree.h:L361-439 (numerical decision with missing-value handling). Forests with categorical splits,
// more than 65534 used features, or trees above 4096 leaves take the general one-thread-per-row kernel.
#include <cuda_fp16.h>
#include <cuda_pipeline.h>

#include <algorithm>
#include <cstring>
#include <limits>
#include <vector>

#include "engine.h"

namespace fb {

namespace {

// value: threshold of an internal node, output of a leaf.
// meta:  bits 0-15 feature slot (0xFFFF: leaf), bits 16-28 index of the left child inside the tree (the right child
//        is the next node; for a leaf: the leaf's index), bit 29 default-left, bits 30-31 missing type.
struct PackedNode { float value; unsigned int meta; };
static_assert(sizeof(PackedNode) == 8, "8-byte nodes");

constexpr int kTileThreads = 256;          // rows of a tile = threads of a block
constexpr int kChunkBytes = 32 * 1024;     // one buffer of the tree ring
constexpr unsigned int kLeafSlot = 0xFFFFu;
constexpr int kWalks = 8;                  // tree walks a thread keeps in flight

struct ChunkDesc { long long offset; int bytes; int ntrees; int cls; int first_tree; };   // blob offset (16-byte aligned)

template <typename T> __device__ inline float ToF(T v) { return static_cast<float>(v); }
template <> __device__ inline float ToF<__half>(__half v) { return __half2float(v); }

// PLAIN: no node of the forest treats zero or NaN as missing; NaN inputs were replaced by 0 when the tile was staged
// (that is what such nodes do with them), so a step is one comparison.
template <bool PLAIN>
__device__ __forceinline__ bool GoLeft(float v, float thr, unsigned int meta) {
  if (PLAIN) return v <= thr;
  const unsigned int mt = meta >> 30;
  const bool nan = isnan(v);
  if (nan && mt != 2u) v = 0.f;
  const bool use_default = (mt == 1u && fabsf(v) <= 1e-35f) || (mt == 2u && nan);
  return use_default ? ((meta >> 29) & 1u) != 0u : v <= thr;
}

// LEAF: write the leaf index of every (row, tree) instead of summing outputs.
template <typename T, bool LEAF, bool PLAIN>
__global__ void __launch_bounds__(kTileThreads, 1)
PredictTiledKernel(const unsigned char* __restrict__ blob, const ChunkDesc* __restrict__ chunks, int num_chunks, const int* __restrict__ used, int num_used,
                   const T* __restrict__ data, int nrow, int ncol, int row_major, int num_class, int trees_total, float inv_avg, float* __restrict__ out,
                   int* __restrict__ out_leaf) {
  extern __shared__ __align__(16) unsigned char smem[];
  unsigned char* ring = smem;                                                   // [2][kChunkBytes]
  float* rows_s = reinterpret_cast<float*>(smem + 2 * kChunkBytes);             // [num_used][kTileThreads]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int num_tiles = (nrow + kTileThreads - 1) / kTileThreads;
  for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
    const int row0 = tile * kTileThreads;
    const int row = row0 + tid;
    __syncthreads();   // the previous tile's walks are over before its rows and ring buffers are overwritten
    // ---- stage the tile: rows_s[j][r] = value of used feature j in row row0 + r ----
    if (!row_major) {
      for (int j = 0; j < num_used; ++j) {
        float v = row < nrow ? ToF<T>(data[static_cast<size_t>(used[j]) * nrow + row]) : 0.f;
        if (PLAIN && isnan(v)) v = 0.f;
        rows_s[j * kTileThreads + tid] = v;
      }
    } else {
      // 32 x 32 pieces: read with the lanes along the features (coalesced), turn in a padded scratch piece that
      // borrows the still unused ring, write with the lanes along the rows (conflict-free)
      float* scratch = reinterpret_cast<float*>(ring) + warp * (32 * 33);
      const int fpieces = (num_used + 31) / 32;
      for (int piece = warp; piece < fpieces * (kTileThreads / 32); piece += kTileThreads / 32) {
        const int fp = piece % fpieces, rp = piece / fpieces;
        const int j = fp * 32 + lane;
        const int col = j < num_used ? used[j] : -1;
#pragma unroll 8
        for (int k = 0; k < 32; ++k) {
          const int r = row0 + rp * 32 + k;
          float v = (col >= 0 && r < nrow) ? ToF<T>(data[static_cast<size_t>(r) * ncol + col]) : 0.f;
          if (PLAIN && isnan(v)) v = 0.f;
          scratch[k * 33 + lane] = v;
        }
        __syncwarp();
#pragma unroll 8
        for (int k = 0; k < 32; ++k) {
          const int jj = fp * 32 + k;
          if (jj < num_used) rows_s[jj * kTileThreads + rp * 32 + lane] = scratch[lane * 33 + k];
        }
        __syncwarp();
      }
    }
    __syncthreads();
    // ---- walk the forest, chunk by chunk ----
    auto fetch = [&](int c) {
      if (c < num_chunks) {
        const ChunkDesc d = chunks[c];
        const uint4* src = reinterpret_cast<const uint4*>(blob + d.offset);
        uint4* dst = reinterpret_cast<uint4*>(ring + (c & 1) * kChunkBytes);
        for (int i = tid; i < d.bytes / 16; i += kTileThreads) __pipeline_memcpy_async(dst + i, src + i, 16);
      }
      __pipeline_commit();
    };
    fetch(0);
    double acc = 0.0;   // a forest of a thousand trees summed in float would drift from the host's double sums
    int cur_cls = num_chunks > 0 ? chunks[0].cls : 0;
    const float* my = rows_s + tid;
    for (int c = 0; c < num_chunks; ++c) {
      fetch(c + 1);
      __pipeline_wait_prior(1);
      __syncthreads();
      const ChunkDesc d = chunks[c];
      if (!LEAF && d.cls != cur_cls) {
        if (row < nrow) out[static_cast<size_t>(cur_cls) * nrow + row] = static_cast<float>(acc * inv_avg);
        acc = 0.0; cur_cls = d.cls;
      }
      const unsigned char* buf = ring + (c & 1) * kChunkBytes;
      const int* roots = reinterpret_cast<const int*>(buf);          // [ntrees] node index of every tree's root, then the nodes
      const PackedNode* nodes = reinterpret_cast<const PackedNode*>(buf + ((d.ntrees * 4 + 15) & ~15));
      for (int t = 0; t < d.ntrees; t += kWalks) {
        // kWalks walks in flight, written without branches so that their shared-memory loads overlap: a walk that has
        // reached its leaf (or has no tree) re-reads its own node and feature slot 0 until the others are done
        int at[kWalks], base[kWalks]; PackedNode nd[kWalks]; bool live[kWalks];
        bool any = false;
#pragma unroll
        for (int q = 0; q < kWalks; ++q) {
          const bool has = t + q < d.ntrees;
          base[q] = has ? roots[t + q] : 0;
          at[q] = base[q];
          nd[q] = nodes[at[q]];
          live[q] = has && (nd[q].meta & 0xFFFFu) != kLeafSlot;
          any = any || live[q];
        }
        while (any) {
          float v[kWalks];
#pragma unroll
          for (int q = 0; q < kWalks; ++q) v[q] = my[(live[q] ? (nd[q].meta & 0xFFFFu) : 0u) * kTileThreads];
#pragma unroll
          for (int q = 0; q < kWalks; ++q) {
            const int next = base[q] + static_cast<int>((nd[q].meta >> 16) & 0x1FFFu) + (GoLeft<PLAIN>(v[q], nd[q].value, nd[q].meta) ? 0 : 1);
            at[q] = live[q] ? next : at[q];
          }
          any = false;
#pragma unroll
          for (int q = 0; q < kWalks; ++q) {
            nd[q] = nodes[at[q]];
            live[q] = live[q] && (nd[q].meta & 0xFFFFu) != kLeafSlot;
            any = any || live[q];
          }
        }
#pragma unroll
        for (int q = 0; q < kWalks; ++q) {
          if (t + q < d.ntrees) {
            if (LEAF) { if (row < nrow) out_leaf[static_cast<size_t>(row) * trees_total + d.first_tree + (t + q) * num_class] = static_cast<int>((nd[q].meta >> 16) & 0x1FFFu); }
            else acc += static_cast<double>(nd[q].value);
          }
        }
      }
      __syncthreads();   // everyone is done with this buffer before the fetch after next refills it
    }
    __pipeline_wait_prior(0);
    if (!LEAF && num_chunks > 0 && row < nrow) out[static_cast<size_t>(cur_cls) * nrow + row] = static_cast<float>(acc * inv_avg);
  }
}

// Nodes of one tree in sibling-adjacent order: root first, then every split's two children next to each other.
bool PackTree(const Tree& T, const std::vector<int>& slot_of_feature, std::vector<PackedNode>* out) {
  const int L = T.num_leaves;
  if (L > 4096) return false;
  out->clear();
  if (L <= 1) { PackedNode nd; nd.value = static_cast<float>(T.leaf_value[0]); nd.meta = kLeafSlot; out->push_back(nd); return true; }
  out->resize(2 * L - 1);
  // queue of (host node id, packed position); host ids: >= 0 split, < 0 leaf ~id
  std::vector<std::pair<int, int>> queue; queue.reserve(2 * L);
  queue.emplace_back(0, 0);
  int next_free = 1;
  for (size_t qi = 0; qi < queue.size(); ++qi) {
    const int id = queue[qi].first, pos = queue[qi].second;
    PackedNode nd;
    if (id < 0) {
      const int leaf = ~id;
      nd.value = static_cast<float>(T.leaf_value[leaf]); nd.meta = kLeafSlot | (static_cast<unsigned int>(leaf) << 16);
    } else {
      if (T.decision_type[id] & kCategoricalMask) return false;
      float thr = static_cast<float>(T.threshold[id]);
      // keep "v <= threshold" exact for float inputs: round the double threshold DOWN to float
      if (static_cast<double>(thr) > T.threshold[id]) thr = std::nextafterf(thr, -std::numeric_limits<float>::infinity());
      const int slot = slot_of_feature[T.split_feature[id]];
      const int left_pos = next_free; next_free += 2;
      nd.value = thr;
      nd.meta = static_cast<unsigned int>(slot) | (static_cast<unsigned int>(left_pos) << 16) | ((T.decision_type[id] & kDefaultLeftMask) ? (1u << 29) : 0u) |
                (static_cast<unsigned int>(Tree::MissingTypeOf(T.decision_type[id])) << 30);
      queue.emplace_back(T.left_child[id], left_pos);
      queue.emplace_back(T.right_child[id], left_pos + 1);
    }
    (*out)[pos] = nd;
  }
  return true;
}

}  // namespace

// Returns false when the forest or the matrix is outside what the tiled kernel covers (the caller then takes the
// general kernel). predict_type 0/1: out[class][row] sums; 2: out_leaf[row][tree] leaf indices.
bool DevicePredictTiled(const GBDT* gbdt, const void* device_data, int dtype, int32_t nrow, int32_t ncol, bool row_major, int first_tree, int num_trees, int K,
                        bool leaf_index, float inv_avg, float* out_device, cudaStream_t s) {
  if (num_trees <= 0 || nrow <= 0) return false;
  if (dtype != kF32 && dtype != kF64 && dtype != kF16) return false;
  // features the forest reads, in ascending order
  std::vector<int> slot_of_feature(std::max(1, gbdt->max_feature_idx_ + 1), -1);
  bool plain = true;   // no node with a missing type: NaN reads as 0 everywhere, zero is an ordinary value
  for (int t = first_tree; t < first_tree + num_trees; ++t) {
    const Tree& T = *gbdt->models_[t];
    if (T.is_linear) return false;
    for (int sidx = 0; sidx < T.num_leaves - 1; ++sidx) {
      if (T.decision_type[sidx] & kCategoricalMask) return false;
      if (Tree::MissingTypeOf(T.decision_type[sidx]) != 0) plain = false;
      const int f = T.split_feature[sidx];
      if (f < 0 || f >= static_cast<int>(slot_of_feature.size())) return false;
      slot_of_feature[f] = 0;
    }
  }
  std::vector<int> used;
  for (size_t f = 0; f < slot_of_feature.size(); ++f) if (slot_of_feature[f] == 0) { slot_of_feature[f] = static_cast<int>(used.size()); used.push_back(static_cast<int>(f)); }
  if (used.size() >= kLeafSlot) return false;
  if (used.empty()) used.push_back(0);
  const size_t smem = 2 * static_cast<size_t>(kChunkBytes) + used.size() * kTileThreads * sizeof(float);
  if (smem > 220 * 1024) return false;
  // chunks: trees of one class in iteration order, as many as fit a ring buffer
  std::vector<unsigned char> blob; std::vector<ChunkDesc> chunks;
  std::vector<PackedNode> packed;
  for (int cls = 0; cls < K; ++cls) {
    std::vector<int> roots; std::vector<PackedNode> nodes; int first = -1;
    auto close = [&]() {
      if (roots.empty()) return;
      ChunkDesc d; d.offset = static_cast<long long>(blob.size()); d.ntrees = static_cast<int>(roots.size()); d.cls = cls; d.first_tree = first;
      const size_t head = (roots.size() * 4 + 15) & ~static_cast<size_t>(15);
      const size_t bytes = (head + nodes.size() * sizeof(PackedNode) + 15) & ~static_cast<size_t>(15);
      d.bytes = static_cast<int>(bytes);
      blob.resize(blob.size() + bytes, 0);
      memcpy(blob.data() + d.offset, roots.data(), roots.size() * 4);
      memcpy(blob.data() + d.offset + head, nodes.data(), nodes.size() * sizeof(PackedNode));
      chunks.push_back(d); roots.clear(); nodes.clear(); first = -1;
    };
    for (int t = cls; t < num_trees; t += K) {
      if (!PackTree(*gbdt->models_[first_tree + t], slot_of_feature, &packed)) return false;
      const size_t need = (((roots.size() + 1) * 4 + 15) & ~static_cast<size_t>(15)) + (nodes.size() + packed.size()) * sizeof(PackedNode) + 16;
      if (need > static_cast<size_t>(kChunkBytes)) {
        close();
        if (((4 + 15) & ~15) + packed.size() * sizeof(PackedNode) + 16 > static_cast<size_t>(kChunkBytes)) return false;   // a single tree larger than a buffer
      }
      if (first < 0) first = t;
      roots.push_back(static_cast<int>(nodes.size()));
      nodes.insert(nodes.end(), packed.begin(), packed.end());
    }
    close();
  }
  if (chunks.empty()) return false;
  DevBuf<unsigned char> d_blob; DevBuf<ChunkDesc> d_chunks; DevBuf<int> d_used;
  d_blob.Upload(blob, s); d_chunks.Upload(chunks, s); d_used.Upload(used, s);
  int dev = 0, sms = 0; FB_CUDA(cudaGetDevice(&dev)); FB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const int tiles = (nrow + kTileThreads - 1) / kTileThreads;
  const int grid = std::min(tiles, sms);
  const int nc = static_cast<int>(chunks.size()), nu = static_cast<int>(used.size());
#define FB_TILED_P(T, LEAF, PLAIN)                                                                                                 \
  {                                                                                                                                \
    static bool attr = false;                                                                                                      \
    if (!attr) { FB_CUDA(cudaFuncSetAttribute(PredictTiledKernel<T, LEAF, PLAIN>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024)); attr = true; } \
    PredictTiledKernel<T, LEAF, PLAIN><<<grid, kTileThreads, smem, s>>>(d_blob.get(), d_chunks.get(), nc, d_used.get(), nu, static_cast<const T*>(device_data), nrow, ncol, \
                                                                        row_major ? 1 : 0, K, num_trees, inv_avg, out_device, reinterpret_cast<int*>(out_device));          \
  }
#define FB_TILED(T, LEAF) { if (plain) FB_TILED_P(T, LEAF, true) else FB_TILED_P(T, LEAF, false) }
  if (leaf_index) {
    if (dtype == kF32) FB_TILED(float, true) else if (dtype == kF64) FB_TILED(double, true) else FB_TILED(__half, true)
  } else {
    if (dtype == kF32) FB_TILED(float, false) else if (dtype == kF64) FB_TILED(double, false) else FB_TILED(__half, false)
  }
#undef FB_TILED
#undef FB_TILED_P
  FB_LAUNCHED(); FB_KERNEL_CHECK();
  FB_CUDA(cudaStreamSynchronize(s));   // the packed forest lives in this call's buffers
  return true;
}

}  // namespace fb
