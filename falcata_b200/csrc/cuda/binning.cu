// K12: on-device binning of a dense matrix into the row-major group-bin layout, device dataset
// ownership, and upload of host-binned data.
// Parity: src/io/cuda/cuda_dense_binner.cu:L25-148 (value -> bin by binary search over per-feature
// upper bounds, NaN / zero handling, bundle encode), cuda_dense_binner.cpp:L158-581 (driver).
// Difference on purpose: the binned rows stay on the device; nothing is scattered back to the host
// unless a host copy is asked for.
#include "device_common.cuh"

#include <cuda_fp16.h>

namespace fb {

void FreeDeviceDataset(DeviceDataset* p) { delete p; }

bool CudaAvailable() {
  static int cached = -1;
  if (cached < 0) {
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) { cudaGetLastError(); n = 0; }
    cached = n > 0 ? 1 : 0;
  }
  return cached == 1;
}

namespace {

// Per used feature, what the binning kernel needs.
struct BinFeat {
  int column;          // column in the raw matrix
  int bound_begin;     // first upper bound in the concatenated array
  int num_bin;
  int missing_type;
  int bin_type;        // 0 numerical, 1 categorical
  int most_freq_bin;
  int group;           // output byte
  int bundled;
  int group_offset;
  int cat_begin, cat_count;   // categorical: sorted (value, bin) pairs
};

template <typename T> __device__ inline double LoadAsDouble(const T* p, size_t i) { return static_cast<double>(p[i]); }
template <> __device__ inline double LoadAsDouble<__half>(const __half* p, size_t i) { return static_cast<double>(__half2float(p[i])); }

__device__ inline int ValueToBinDev(double v, const BinFeat& f, const double* bounds, const int* cat_vals, const int* cat_bins) {
  if (f.bin_type == 1) {
    if (isnan(v)) return 0;
    int iv = static_cast<int>(v);
    if (iv < 0) return 0;
    int lo = 0, hi = f.cat_count - 1;
    while (lo <= hi) { int m = (lo + hi) >> 1; int c = cat_vals[f.cat_begin + m]; if (c == iv) return cat_bins[f.cat_begin + m]; if (c < iv) lo = m + 1; else hi = m - 1; }
    return 0;
  }
  if (isnan(v)) { if (f.missing_type == 2) return f.num_bin - 1; v = 0.0; }
  int l = 0, r = f.num_bin - 1;
  if (f.missing_type == 2) r -= 1;
  const double* ub = bounds + f.bound_begin;
  while (l < r) { int m = (r + l - 1) / 2; if (v <= ub[m]) r = m; else l = m + 1; }
  return l;
}

// One thread per (row, group); groups are the fast index so that the byte stores of a row coalesce.
template <typename T>
__global__ void BinRowsKernel(const T* __restrict__ data, int nrow, int ncol, bool row_major, const BinFeat* __restrict__ feats,
                              const int* __restrict__ group_feat_begin, int num_groups, const double* __restrict__ bounds,
                              const int* __restrict__ cat_vals, const int* __restrict__ cat_bins, uint8_t* __restrict__ rows, int row_stride) {
  const size_t tid = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const size_t total = static_cast<size_t>(nrow) * num_groups;
  if (tid >= total) return;
  const int g = static_cast<int>(tid % num_groups);
  const size_t i = tid / num_groups;
  int gb = 0;
  for (int k = group_feat_begin[g]; k < group_feat_begin[g + 1]; ++k) {
    const BinFeat f = feats[k];
    const size_t src = row_major ? i * ncol + f.column : static_cast<size_t>(f.column) * nrow + i;
    const int b = ValueToBinDev(LoadAsDouble<T>(data, src), f, bounds, cat_vals, cat_bins);
    if (!f.bundled) gb = b;
    else if (b != f.most_freq_bin) gb = f.group_offset + (b > f.most_freq_bin ? b - 1 : b);
  }
  rows[i * row_stride + g] = static_cast<uint8_t>(gb);
}

int RowStrideFor(int num_groups) { return ((num_groups + 4 + 15) / 16) * 16; }

// cols[g][i] = rows[i][g]; row index is the fast thread index so the stores coalesce (the strided
// loads of neighbouring groups hit the same sectors in L1/L2).
__global__ void TransposeRowsKernel(const uint8_t* __restrict__ rows, int row_stride, int n, int num_groups, uint8_t* __restrict__ cols) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const uint8_t* rp = rows + static_cast<size_t>(i) * row_stride;
  for (int g = 0; g < num_groups; ++g) cols[static_cast<size_t>(g) * n + i] = rp[g];
}

void UploadMeta(const Dataset* ds, DeviceDataset* dd, cudaStream_t s) {
  dd->feature_meta.Upload(ds->feature_meta, s);
  dd->group_bin_start.Upload(ds->group_bin_start, s);
}

}  // namespace

// Column-major copy of the bins for the partition kernels (built once, on first use).
void EnsureColumnMajor(DeviceDataset* dd, cudaStream_t s) {
  if (dd->cols.size() > 0 || dd->num_data == 0) return;
  dd->cols.Alloc(static_cast<size_t>(dd->num_groups) * dd->num_data);
  TransposeRowsKernel<<<(dd->num_data + 255) / 256, 256, 0, s>>>(dd->rows.get(), dd->row_stride, dd->num_data, dd->num_groups, dd->cols.get());
  FB_LAUNCHED(); FB_KERNEL_CHECK();
}

// Metadata that training needs on the device; called lazily by the engine (labels may be set after binning).
void SyncDeviceMetadata(const Dataset* ds, cudaStream_t s) {
  DeviceDataset* dd = ds->device;
  if (dd == nullptr) return;
  if (!ds->metadata.label.empty()) dd->label.Upload(ds->metadata.label, s);
  if (!ds->metadata.weights.empty()) dd->weight.Upload(ds->metadata.weights, s); else dd->weight.Free();
  if (!ds->metadata.query_boundaries.empty()) { dd->query_boundaries.Upload(ds->metadata.query_boundaries, s); dd->num_queries = ds->metadata.num_queries(); }
  FB_CUDA(cudaStreamSynchronize(s));
}

// Device copy of a dataset that was binned on the host.
void EnsureDeviceDataset(Dataset* ds) {
  if (ds->device != nullptr) return;
  if (!ds->has_host_bins()) Log::Fatal("Dataset has no bins to upload");
  if (ds->bin_bytes != 1) Log::Fatal("The CUDA learner stores one byte per feature group (max_bin <= 255 and bundles <= 256 bins)");
  std::unique_ptr<DeviceDataset> dd(new DeviceDataset());
  FB_CUDA(cudaGetDevice(&dd->device));
  dd->num_data = ds->num_data; dd->num_groups = ds->num_groups; dd->row_stride = RowStrideFor(ds->num_groups); dd->gh_offset = dd->row_stride - 4;
  std::vector<uint8_t> staged(static_cast<size_t>(ds->num_data) * dd->row_stride, 0);
  for (data_size_t i = 0; i < ds->num_data; ++i) memcpy(&staged[static_cast<size_t>(i) * dd->row_stride], &ds->bins8[static_cast<size_t>(i) * ds->row_stride], ds->num_groups);
  dd->rows.Upload(staged, 0);
  UploadMeta(ds, dd.get(), 0);
  FB_CUDA(cudaStreamSynchronize(0));
  ds->device = dd.release();
}

void DeviceBinDatasetChunk(Dataset* ds, const void* device_data, int dtype, int32_t nrow, int32_t ncol, bool row_major, bool keep_host_copy, int32_t start_row,
                           int32_t total_rows);

// Picks rows of a device matrix into a dense row-major block (element size `elem` bytes, any layout of the source).
__global__ void GatherRowsKernel(const unsigned char* __restrict__ src, int elem, int nrow, int ncol, int row_major, const int* __restrict__ rows, int num_rows,
                                 unsigned char* __restrict__ dst) {
  const long long total = static_cast<long long>(num_rows) * ncol;
  for (long long c = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; c < total; c += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int k = static_cast<int>(c / ncol), j = static_cast<int>(c % ncol);
    const long long r = rows[k];
    const unsigned char* s = src + (row_major ? (r * ncol + j) : (static_cast<long long>(j) * nrow + r)) * elem;
    unsigned char* d = dst + c * elem;
    for (int b = 0; b < elem; ++b) d[b] = s[b];
  }
}

// The listed rows of a device matrix, in its own element type, copied to the host (row-major).
void DeviceGatherRows(const void* device_data, int dtype, int32_t nrow, int32_t ncol, bool row_major, const int32_t* rows, int32_t num_rows, std::vector<char>* out) {
  if (!CudaAvailable()) Log::Fatal("No CUDA device is available");
  const int elem = dtype == kF64 ? 8 : (dtype == kF32 || dtype == kI32) ? 4 : (dtype == kI8 || dtype == kU8) ? 1 : 2;
  out->resize(static_cast<size_t>(num_rows) * ncol * elem);
  if (num_rows <= 0) return;
  DevBuf<int> d_rows; DevBuf<unsigned char> d_out;
  std::vector<int> h_rows(rows, rows + num_rows);
  d_rows.Upload(h_rows, 0); d_out.Alloc(out->size());
  const long long total = static_cast<long long>(num_rows) * ncol;
  const unsigned blocks = static_cast<unsigned>(std::min<long long>((total + 255) / 256, 65535));
  GatherRowsKernel<<<blocks, 256>>>(static_cast<const unsigned char*>(device_data), elem, nrow, ncol, row_major ? 1 : 0, d_rows.get(), num_rows, d_out.get());
  FB_LAUNCHED(); FB_KERNEL_CHECK();
  FB_CUDA(cudaMemcpy(out->data(), d_out.get(), out->size(), cudaMemcpyDeviceToHost));
}

void DeviceBinDataset(Dataset* ds, const void* device_data, int dtype, int32_t nrow, int32_t ncol, bool row_major, bool keep_host_copy) {
  DeviceBinDatasetChunk(ds, device_data, dtype, nrow, ncol, row_major, keep_host_copy, 0, nrow);
}

// Bins rows [start_row, start_row + nrow) of a data set of total_rows rows from a device-resident chunk of the raw
// matrix. The first chunk (start_row 0) allocates the binned rows for the whole data set; a host matrix larger than
// the device can spare is ingested as a sequence of such chunks (copy a chunk, bin it, reuse the buffer).
void DeviceBinDatasetChunk(Dataset* ds, const void* device_data, int dtype, int32_t nrow, int32_t ncol, bool row_major, bool keep_host_copy, int32_t start_row,
                           int32_t total_rows) {
  if (!CudaAvailable()) Log::Fatal("No CUDA device is available for device binning");
  if (ncol != ds->num_total_features) Log::Fatal("The number of columns (%d) differs from the dataset's (%d)", ncol, ds->num_total_features);
  if (ds->max_group_bin > 256) Log::Fatal("The CUDA learner stores one byte per feature group (max_bin <= 255)");
  if (start_row < 0 || start_row + nrow > total_rows) Log::Fatal("Chunk [%d, %d) is outside the data set of %d rows", start_row, start_row + nrow, total_rows);
  if (start_row > 0 && (ds->device == nullptr || ds->device->num_data != total_rows)) Log::Fatal("Chunks must start with the chunk at row 0");
  if (keep_host_copy && nrow != total_rows) Log::Fatal("A host copy of the bins needs the whole matrix in one chunk");
  std::unique_ptr<DeviceDataset> fresh;
  if (start_row == 0) {
    fresh.reset(new DeviceDataset());
    FB_CUDA(cudaGetDevice(&fresh->device));
    fresh->num_data = total_rows; fresh->num_groups = ds->num_groups; fresh->row_stride = RowStrideFor(ds->num_groups); fresh->gh_offset = fresh->row_stride - 4;
    ds->num_data = total_rows; ds->metadata.num_data = total_rows;
    if (ds->global_num_data == 0) ds->global_num_data = total_rows;
  }
  DeviceDataset* dd = start_row == 0 ? fresh.get() : ds->device;
  std::vector<BinFeat> feats; std::vector<int> gbegin(ds->num_groups + 1, 0); std::vector<double> bounds; std::vector<int> cat_vals, cat_bins;
  for (int g = 0; g < ds->num_groups; ++g) {
    gbegin[g] = static_cast<int>(feats.size());
    for (int f : ds->group_features[g]) {
      const BinMapper& bm = *ds->mappers[ds->real_feature_idx[f]]; const FeatureMeta& m = ds->feature_meta[f];
      BinFeat bf; bf.column = m.real_index; bf.bound_begin = static_cast<int>(bounds.size()); bf.num_bin = bm.num_bin; bf.missing_type = m.missing_type;
      bf.bin_type = m.bin_type; bf.most_freq_bin = m.most_freq_bin; bf.group = g; bf.bundled = m.bundled; bf.group_offset = m.group_offset;
      bf.cat_begin = static_cast<int>(cat_vals.size()); bf.cat_count = 0;
      if (bm.bin_type == BinType::Numerical) bounds.insert(bounds.end(), bm.bin_upper_bound.begin(), bm.bin_upper_bound.end());
      else {
        std::vector<std::pair<int, int>> pairs;
        for (int b = 1; b < bm.num_bin; ++b) pairs.emplace_back(bm.bin_2_categorical[b], b);
        std::sort(pairs.begin(), pairs.end());
        for (auto& p : pairs) { cat_vals.push_back(p.first); cat_bins.push_back(p.second); }
        bf.cat_count = static_cast<int>(pairs.size());
      }
      feats.push_back(bf);
    }
  }
  gbegin[ds->num_groups] = static_cast<int>(feats.size());
  DevBuf<BinFeat> d_feats; DevBuf<int> d_gbegin, d_cv, d_cb; DevBuf<double> d_bounds;
  d_feats.Upload(feats, 0); d_gbegin.Upload(gbegin, 0); d_bounds.Upload(bounds, 0); d_cv.Upload(cat_vals, 0); d_cb.Upload(cat_bins, 0);
  if (start_row == 0) { dd->rows.Alloc(static_cast<size_t>(total_rows) * dd->row_stride); dd->rows.Zero(0); }
  uint8_t* out_rows = dd->rows.get() + static_cast<size_t>(start_row) * dd->row_stride;
  const size_t total = static_cast<size_t>(nrow) * ds->num_groups;
  const int threads = 256; const unsigned blocks = static_cast<unsigned>((total + threads - 1) / threads);
  if (total > 0) {
#define FB_BIN_LAUNCH(T) BinRowsKernel<T><<<blocks, threads>>>(static_cast<const T*>(device_data), nrow, ncol, row_major, d_feats.get(), d_gbegin.get(), ds->num_groups, d_bounds.get(), d_cv.get(), d_cb.get(), out_rows, dd->row_stride)
    switch (dtype) {
      case kF32: FB_BIN_LAUNCH(float); break;
      case kF64: FB_BIN_LAUNCH(double); break;
      case kI8: FB_BIN_LAUNCH(int8_t); break;
      case kI16: FB_BIN_LAUNCH(int16_t); break;
      case kU8: FB_BIN_LAUNCH(uint8_t); break;
      case kU16: FB_BIN_LAUNCH(uint16_t); break;
      case kI32: FB_BIN_LAUNCH(int32_t); break;
      case kF16: FB_BIN_LAUNCH(__half); break;
      default: Log::Fatal("Unsupported dtype code %d for device binning", dtype);
    }
#undef FB_BIN_LAUNCH
    FB_LAUNCHED(); FB_KERNEL_CHECK();
  }
  if (start_row == 0) UploadMeta(ds, dd, 0);
  FB_CUDA(cudaStreamSynchronize(0));
  if (DebugFlags::Get().verify && nrow > 0) {
    // self-check: up to 1024 evenly spaced rows of the chunk are binned again by the host's bin mappers and compared
    // with the device's bytes
    const int elem = dtype == kF64 ? 8 : (dtype == kF32 || dtype == kI32) ? 4 : (dtype == kI8 || dtype == kU8) ? 1 : 2;
    const int take = std::min<int32_t>(nrow, 1024);
    std::vector<char> raw(static_cast<size_t>(take) * ncol * elem);
    std::vector<uint8_t> dev(static_cast<size_t>(take) * dd->row_stride);
    for (int k = 0; k < take; ++k) {
      const size_t r = static_cast<size_t>(static_cast<int64_t>(k) * nrow / take);
      const char* src = static_cast<const char*>(device_data);
      if (row_major) FB_CUDA(cudaMemcpy(&raw[static_cast<size_t>(k) * ncol * elem], src + r * ncol * elem, static_cast<size_t>(ncol) * elem, cudaMemcpyDeviceToHost));
      else FB_CUDA(cudaMemcpy2D(&raw[static_cast<size_t>(k) * ncol * elem], elem, src + r * elem, static_cast<size_t>(nrow) * elem, elem, ncol, cudaMemcpyDeviceToHost));
      FB_CUDA(cudaMemcpy(&dev[static_cast<size_t>(k) * dd->row_stride], out_rows + r * dd->row_stride, dd->row_stride, cudaMemcpyDeviceToHost));
    }
    Dataset host; host.CopySchemaFrom(*ds); host.keep_raw = false; host.bin_bytes = 1; host.row_stride = ds->num_groups;
    host.AllocateRows(take);
    host.PushDense(raw.data(), dtype, take, ncol, true, 0);
    for (int k = 0; k < take; ++k)
      for (int g = 0; g < ds->num_groups; ++g)
        if (host.bins8[static_cast<size_t>(k) * host.row_stride + g] != dev[static_cast<size_t>(k) * dd->row_stride + g])
          Log::Fatal("FALCATA_VERIFY: device binning differs from the host at row %lld, feature group %d: device %d, host %d",
                     static_cast<long long>(start_row + static_cast<int64_t>(k) * nrow / take), g, dev[static_cast<size_t>(k) * dd->row_stride + g],
                     host.bins8[static_cast<size_t>(k) * host.row_stride + g]);
    Log::Info("FALCATA_VERIFY: device binning equals the host's on %d sampled rows of [%d, %d)", take, start_row, start_row + nrow);
  }
  if (keep_host_copy) {
    std::vector<uint8_t> staged(static_cast<size_t>(nrow) * dd->row_stride);
    FB_CUDA(cudaMemcpy(staged.data(), dd->rows.get(), staged.size(), cudaMemcpyDeviceToHost));
    ds->bin_bytes = 1; ds->row_stride = ds->num_groups;
    ds->bins8.assign(static_cast<size_t>(nrow) * ds->num_groups, 0);
    for (int32_t i = 0; i < nrow; ++i) memcpy(&ds->bins8[static_cast<size_t>(i) * ds->num_groups], &staged[static_cast<size_t>(i) * dd->row_stride], ds->num_groups);
  }
  if (start_row == 0) {
    if (ds->device != nullptr) FreeDeviceDataset(ds->device);
    ds->device = fresh.release();
  }
}

}  // namespace fb
