// C API implementation. Parity: src/c_api.cpp (Booster wrapper L179-480, API functions L1021-3238).
#include "fb/c_api.h"

#include <omp.h>

#include <fstream>
#include <memory>
#include <map>
#include <mutex>

#include "fb/gbdt.h"

namespace fb {
// device-side entry points implemented by the CUDA module
void DeviceBinDataset(Dataset* ds, const void* device_data, int dtype, int32_t nrow, int32_t ncol, bool row_major, bool keep_host_copy);
void DeviceGatherRows(const void* device_data, int dtype, int32_t nrow, int32_t ncol, bool row_major, const int32_t* rows, int32_t num_rows, std::vector<char>* out);
void DeviceBinDatasetChunk(Dataset* ds, const void* device_data, int dtype, int32_t nrow, int32_t ncol, bool row_major, bool keep_host_copy, int32_t start_row,
                           int32_t total_rows);
void DevicePredict(const GBDT* gbdt, const void* device_data, int dtype, int32_t nrow, int32_t ncol, bool row_major, int predict_type,
                   int start_iter, int num_iter, float* out_device);
}  // namespace fb

using namespace fb;

extern "C" int FB_OpBernoulliRowsHost(int n, long long global_offset, unsigned int seed, double fraction, int* out_idx, int* out_count);

namespace {

thread_local std::string g_last_error;

struct BoosterWrap {
  Config config;
  std::unique_ptr<ObjectiveFunction> objective;
  std::unique_ptr<GBDT> gbdt;
  const Dataset* train = nullptr;
  std::mutex mu;
};

int CopyOut(const std::string& s, int64_t buffer_len, int64_t* out_len, char* out) {
  *out_len = static_cast<int64_t>(s.size()) + 1;
  if (buffer_len >= *out_len && out != nullptr) memcpy(out, s.c_str(), s.size() + 1);
  return 0;
}

std::vector<int> ParseCategorical(const Config& cfg, int ncol) {
  std::vector<int> out;
  for (auto& t : SplitAny(cfg.categorical_feature, ",")) {
    std::string s = Trim(t);
    if (s.empty() || StartsWith(s, "name:")) continue;
    int v = atoi(s.c_str()); if (v >= 0 && v < ncol) out.push_back(v);
  }
  return out;
}

}  // namespace

#define API_BEGIN() try {
#define API_END() } catch (std::exception& ex) { g_last_error = ex.what(); return -1; } catch (...) { g_last_error = "unknown exception"; return -1; } return 0;

extern "C" {

const char* FB_GetLastError() { return g_last_error.c_str(); }

int FB_RegisterLogCallback(void (*callback)(const char*)) { API_BEGIN(); Log::callback() = callback; API_END(); }
int FB_CudaAvailable(int* out) { API_BEGIN(); *out = CudaAvailable() ? 1 : 0; API_END(); }
int FB_SetLastErrorForCompat(const char* message) { g_last_error = message != nullptr ? message : "error"; return -1; }
int FB_SetNumThreads(int num_threads) { API_BEGIN(); if (num_threads > 0) omp_set_num_threads(num_threads); API_END(); }
int FB_GetNumThreads(int* out) { API_BEGIN(); *out = omp_get_max_threads(); API_END(); }
// Resolved value of an integer parameter (aliases, defaults and seed derivation applied) for the Python layer.
int FB_ResolveParamInt(const char* parameters, const char* name, int* out) {
  API_BEGIN();
  Config cfg; cfg.Set(Config::Str2Map(parameters), CudaAvailable());
  const std::string n = name;
  if (n == "data_random_seed") *out = cfg.data_random_seed;
  else if (n == "bin_construct_sample_cnt") *out = cfg.bin_construct_sample_cnt;
  else Log::Fatal("FB_ResolveParamInt does not know %s", name);
  API_END();
}
int FB_SetTimeTag(int enabled) { API_BEGIN(); StageTimer::Get().enabled = enabled != 0; if (!enabled) StageTimer::Get().Clear(); API_END(); }
int FB_GetTimeTagReport(int64_t buffer_len, int64_t* out_len, char* out_str) { API_BEGIN(); CopyOut(StageTimer::Get().Report(), buffer_len, out_len, out_str); API_END(); }

int FB_NetworkInitWithFunctions(int num_machines, int rank, void* allreduce_sum_fn, void* allgather_fn) {
  API_BEGIN();
  Network::world() = num_machines; Network::rank() = rank;
  Network::allreduce() = reinterpret_cast<Network::AllreduceSumFn>(allreduce_sum_fn);
  Network::allgather() = reinterpret_cast<Network::AllgatherFn>(allgather_fn);
  API_END();
}
int FB_NetworkInit(const char* machines, int local_listen_port, int listen_time_out, int num_machines) {
  API_BEGIN();
  if (num_machines > 1) SocketNetworkInit(machines != nullptr ? machines : "", local_listen_port, listen_time_out, num_machines);
  API_END();
}
int FB_NetworkFree() { API_BEGIN(); SocketNetworkFree(); Network::world() = 1; Network::rank() = 0; Network::allreduce() = nullptr; Network::allgather() = nullptr; API_END(); }

// ------------------------------------------------------------- Dataset ----
int FB_DatasetCreateFromMat(const void* data, int dtype, int32_t nrow, int32_t ncol, int is_row_major, const char* parameters,
                            const DatasetHandle reference, DatasetHandle* out) {
  API_BEGIN();
  Config cfg; cfg.Set(Config::Str2Map(parameters), CudaAvailable());
  std::unique_ptr<Dataset> ds(new Dataset());
  int64_t mesh_offset = 0, mesh_total = nrow;
  if (reference != nullptr) {
    ds->CopySchemaFrom(*static_cast<const Dataset*>(reference));
  } else {
    // the bin sample: a row is in iff its Philox draw (data_random_seed, row id) is below sample_cnt / nrow - the
    // draw the device ingest makes, so a matrix gets the same bin boundaries whichever way it comes in
    // Processes of the TCP mesh (FB_NetworkInit) each hold their own rows, numbered in rank order: every process draws
    // the rows of the one global sample that fall into its range and the pieces are concatenated on all of them, so the
    // bins are those of a single process holding all rows.
    // (feature-parallel training keeps all rows on every process: nothing to exchange, the same sample everywhere)
    const bool distributed = SocketNetworkActive() && Network::active() && cfg.tree_learner != "feature";
    if (distributed) GatherRowCounts(nrow, &mesh_offset, &mesh_total);
    const int64_t total_rows = distributed ? mesh_total : nrow;
    const double frac = std::min(1.0, static_cast<double>(cfg.bin_construct_sample_cnt) / static_cast<double>(std::max<int64_t>(1, total_rows)));
    std::vector<int> idx(static_cast<size_t>(std::max(1, nrow)));
    int picked = 0;
    if (FB_OpBernoulliRowsHost(nrow, distributed ? mesh_offset : 0, static_cast<unsigned int>(cfg.data_random_seed), frac, idx.data(), &picked) != 0) Log::Fatal("Row sampling failed");
    idx.resize(picked);
    if (idx.empty() && nrow > 0 && !distributed) idx.push_back(0);
    std::vector<double> sample(static_cast<size_t>(idx.size()) * ncol);
    for (size_t r = 0; r < idx.size(); ++r) for (int j = 0; j < ncol; ++j) {
      const size_t src = is_row_major ? static_cast<size_t>(idx[r]) * ncol + j : static_cast<size_t>(j) * nrow + idx[r];
      double v;
      switch (dtype) {
        case kF32: v = static_cast<const float*>(data)[src]; break;
        case kF64: v = static_cast<const double*>(data)[src]; break;
        case kI8: v = static_cast<const int8_t*>(data)[src]; break;
        case kI16: v = static_cast<const int16_t*>(data)[src]; break;
        case kU8: v = static_cast<const uint8_t*>(data)[src]; break;
        case kU16: v = static_cast<const uint16_t*>(data)[src]; break;
        case kI32: v = static_cast<const int32_t*>(data)[src]; break;
        default: Log::Fatal("Unsupported dtype code %d", dtype);
      }
      sample[r * ncol + j] = v;
    }
    if (distributed) AllGatherSampleRows(&sample, ncol);
    ds->ConstructSchema(sample.data(), static_cast<int>(sample.size() / std::max(1, ncol)), ncol, total_rows, cfg, ParseCategorical(cfg, ncol));
    if (distributed) { ds->global_row_offset = mesh_offset; ds->global_num_data = mesh_total; }
  }
  ds->AllocateRows(nrow);
  ds->PushDense(data, dtype, nrow, ncol, is_row_major != 0, 0);
  *out = ds.release();
  API_END();
}

int FB_DatasetCreateFromFile(const char* filename, const char* parameters, const DatasetHandle reference, DatasetHandle* out) {
  API_BEGIN();
  Config cfg; cfg.Set(Config::Str2Map(parameters), CudaAvailable());
  Dataset* bin = Dataset::LoadBinary(filename);
  *out = bin != nullptr ? bin : LoadDatasetFromFile(filename, cfg, static_cast<const Dataset*>(reference));
  API_END();
}

int FB_DatasetCreateFromSample(const double* sample, int32_t ns, int32_t ncol, int64_t total, const char* parameters,
                               const int32_t* categorical, int32_t num_categorical, DatasetHandle* out) {
  API_BEGIN();
  ScopedTimer api_timer("FB_DatasetCreateFromSample");
  Config cfg; cfg.Set(Config::Str2Map(parameters), CudaAvailable());
  std::unique_ptr<Dataset> ds(new Dataset());
  std::vector<int> cats = ParseCategorical(cfg, ncol);
  for (int i = 0; i < num_categorical; ++i) cats.push_back(categorical[i]);
  ds->ConstructSchema(sample, ns, ncol, total, cfg, cats);
  *out = ds.release();
  API_END();
}

int FB_DatasetCreateFromSampleTyped(const void* sample, int dtype, int32_t ns, int32_t ncol, int64_t total, const char* parameters,
                                    const int32_t* categorical, int32_t num_categorical, DatasetHandle* out) {
  API_BEGIN();
  ScopedTimer api_timer("FB_DatasetCreateFromSample");
  Config cfg; cfg.Set(Config::Str2Map(parameters), CudaAvailable());
  if (cfg.num_threads > 0) omp_set_num_threads(cfg.num_threads);
  std::unique_ptr<Dataset> ds(new Dataset());
  std::vector<int> cats = ParseCategorical(cfg, ncol);
  for (int i = 0; i < num_categorical; ++i) cats.push_back(categorical[i]);
  ds->ConstructSchemaTyped(sample, dtype, ns, ncol, total, cfg, cats);
  *out = ds.release();
  API_END();
}

int FB_DatasetCreateByReference(const DatasetHandle reference, DatasetHandle* out) {
  API_BEGIN();
  std::unique_ptr<Dataset> ds(new Dataset()); ds->CopySchemaFrom(*static_cast<const Dataset*>(reference)); *out = ds.release();
  API_END();
}

int FB_DatasetSerializeSchema(DatasetHandle handle, int64_t buffer_len, int64_t* out_len, char* out) {
  API_BEGIN();
  std::vector<char> buf; static_cast<Dataset*>(handle)->SerializeSchema(&buf);
  *out_len = static_cast<int64_t>(buf.size());
  if (buffer_len >= *out_len && out != nullptr) memcpy(out, buf.data(), buf.size());
  API_END();
}

int FB_DatasetCreateFromSchema(const char* schema, int64_t len, const char* parameters, DatasetHandle* out) {
  API_BEGIN();
  Config cfg; cfg.Set(Config::Str2Map(parameters), CudaAvailable());
  std::unique_ptr<Dataset> ds(new Dataset()); ds->DeserializeSchema(schema, static_cast<size_t>(len), cfg); *out = ds.release();
  API_END();
}

// The schema of a dataset (bin mappers, bundles, feature names) as an opaque byte buffer that another process turns
// into an empty dataset with the same bins: FB_DatasetCreateFromSerializedReference allocates num_row host rows and
// opens it for streaming pushes. Parity: FLC_DatasetSerializeReferenceToBinary / FLC_DatasetCreateFromSerializedReference
// / FLC_ByteBuffer*.
int FB_DatasetSerializeReferenceToBinary(DatasetHandle handle, void** out_buffer, int32_t* out_len) {
  API_BEGIN();
  std::unique_ptr<std::vector<char>> buf(new std::vector<char>());
  static_cast<Dataset*>(handle)->SerializeSchema(buf.get());
  if (buf->size() > static_cast<size_t>(INT32_MAX)) Log::Fatal("The serialized reference exceeds 2 GB");
  *out_len = static_cast<int32_t>(buf->size());
  *out_buffer = buf.release();
  API_END();
}
int FB_ByteBufferGetAt(void* buffer, int32_t index, uint8_t* out_val) {
  API_BEGIN();
  const std::vector<char>* b = static_cast<const std::vector<char>*>(buffer);
  if (b == nullptr || index < 0 || static_cast<size_t>(index) >= b->size()) Log::Fatal("Byte buffer index %d is out of range", index);
  *out_val = static_cast<uint8_t>((*b)[static_cast<size_t>(index)]);
  API_END();
}
int FB_ByteBufferFree(void* buffer) { API_BEGIN(); delete static_cast<std::vector<char>*>(buffer); API_END(); }
int FB_DatasetCreateFromSerializedReference(const void* ref_buffer, int32_t ref_buffer_size, int64_t num_row, int32_t num_classes, const char* parameters,
                                            DatasetHandle* out) {
  if (num_row < 0 || num_row > INT32_MAX) return FB_SetLastErrorForCompat("The row count must fit 32 bits");
  if (FB_DatasetCreateFromSchema(static_cast<const char*>(ref_buffer), ref_buffer_size, parameters, out) != 0) return -1;
  if (FB_DatasetInitRows(*out, static_cast<int32_t>(num_row), 0, num_row, 1) != 0) return -1;
  (void)num_classes;   // the init-score layout is fixed by FB_DatasetInitStreaming when the caller opens the stream
  return 0;
}

int FB_DatasetAddFeaturesFrom(DatasetHandle target, DatasetHandle source) {
  API_BEGIN();
  static_cast<Dataset*>(target)->AddFeaturesFrom(*static_cast<const Dataset*>(source));
  API_END();
}

int FB_DatasetInitRows(DatasetHandle handle, int32_t nrow, int64_t global_row_offset, int64_t global_num_row, int host_bins) {
  API_BEGIN();
  ScopedTimer api_timer("FB_DatasetInitRows");
  Dataset* ds = static_cast<Dataset*>(handle);
  ds->global_row_offset = global_row_offset; ds->global_num_data = global_num_row > 0 ? global_num_row : nrow;
  if (host_bins) ds->AllocateRows(nrow); else { ds->num_data = nrow; ds->metadata.num_data = nrow; }
  API_END();
}

int FB_DatasetPushRows(DatasetHandle handle, const void* data, int dtype, int32_t nrow, int32_t ncol, int is_row_major, int32_t start_row) {
  API_BEGIN();
  static_cast<Dataset*>(handle)->PushDense(data, dtype, nrow, ncol, is_row_major != 0, start_row);
  API_END();
}

int FB_DatasetBinDeviceMat(DatasetHandle handle, const void* device_data, int dtype, int32_t nrow, int32_t ncol, int is_row_major, int keep_host_copy) {
  API_BEGIN();
  ScopedTimer api_timer("FB_DatasetBinDeviceMat");
  DeviceBinDataset(static_cast<Dataset*>(handle), device_data, dtype, nrow, ncol, is_row_major != 0, keep_host_copy != 0);
  API_END();
}

// A Dataset from a dense matrix in device memory: the bin sample (the rows the host draw by row id picks) is gathered on
// the device and copied down, the bin boundaries are found on the host, the rows are binned on the device and stay
// there. With `reference` the schema is copied instead. Parity: include/Falcata/c_api.h FLC_DatasetCreateFromMatDevice.
int FB_DatasetCreateFromDeviceMat(const void* device_data, int dtype, int32_t nrow, int32_t ncol, int is_row_major, const char* parameters,
                                  const DatasetHandle reference, DatasetHandle* out) {
  API_BEGIN();
  if (nrow <= 0 || ncol <= 0) Log::Fatal("An empty matrix");
  Config cfg; cfg.Set(Config::Str2Map(parameters), CudaAvailable());
  std::unique_ptr<Dataset> ds(new Dataset());
  if (reference != nullptr) ds->CopySchemaFrom(*static_cast<const Dataset*>(reference));
  else {
    const double frac = std::min(1.0, static_cast<double>(cfg.bin_construct_sample_cnt) / std::max(1, nrow));
    std::vector<int32_t> idx(static_cast<size_t>(nrow));
    int picked = 0;   // the same draw by row id as for a host matrix, so a matrix gets the same bins wherever it lives
    if (FB_OpBernoulliRowsHost(nrow, 0, static_cast<unsigned int>(cfg.data_random_seed), frac, idx.data(), &picked) != 0) Log::Fatal("Row sampling failed");
    idx.resize(picked);
    if (idx.empty()) idx.push_back(0);
    std::vector<char> sample;
    DeviceGatherRows(device_data, dtype, nrow, ncol, is_row_major != 0, idx.data(), static_cast<int32_t>(idx.size()), &sample);
    ds->ConstructSchemaTyped(sample.data(), dtype, static_cast<int>(idx.size()), ncol, nrow, cfg, ParseCategorical(cfg, ncol));
  }
  DeviceBinDataset(ds.get(), device_data, dtype, nrow, ncol, is_row_major != 0, false);
  *out = ds.release();
  API_END();
}

int FB_DatasetBinDeviceChunk(DatasetHandle handle, const void* device_data, int dtype, int32_t nrow, int32_t ncol, int32_t start_row, int32_t total_rows) {
  API_BEGIN();
  DeviceBinDatasetChunk(static_cast<Dataset*>(handle), device_data, dtype, nrow, ncol, true, false, start_row, total_rows);
  API_END();
}

int FB_DatasetSetField(DatasetHandle handle, const char* field_name, const void* data, int64_t n, int dtype) {
  API_BEGIN();
  ScopedTimer api_timer("FB_DatasetSetField");
  Dataset* ds = static_cast<Dataset*>(handle); const std::string f = field_name;
  auto as_float = [&](std::vector<float>* v) {
    if (dtype == kF32) {
      // a fresh block of this size is page-faulted in on first touch, ~2 us a page on one thread: touch every page
      // of the reserved block from all threads first, then copy
      v->reserve(static_cast<size_t>(n));
      float* raw = v->data();
      if (raw != nullptr && n > (1 << 20)) {
#pragma omp parallel for schedule(static) num_threads(TeamThreads())
        for (int64_t i = 0; i < n; i += 1024) raw[i] = 0.f;
      }
      v->assign(static_cast<const float*>(data), static_cast<const float*>(data) + n);
      return;
    }
    v->resize(n);
#pragma omp parallel for schedule(static) num_threads(TeamThreads())
    for (int64_t i = 0; i < n; ++i) (*v)[i] = dtype == kF64 ? static_cast<float>(static_cast<const double*>(data)[i]) : static_cast<float>(static_cast<const int32_t*>(data)[i]);
  };
  if (f == "label" || f == "target") {
    // one value per row, or [target][row] for several regression targets (multi_regression)
    if (ds->num_data <= 0 || n < ds->num_data || n % ds->num_data != 0) Log::Fatal("Length of labels (%lld) differs from the number of rows (%d)", static_cast<long long>(n), ds->num_data);
    std::vector<float> v; as_float(&v); ds->metadata.label.swap(v);
  }
  else if (f == "weight" || f == "weights") { if (n == 0) ds->metadata.SetWeights(nullptr, 0); else { std::vector<float> v; as_float(&v); ds->metadata.SetWeights(v.data(), static_cast<data_size_t>(n)); } }
  else if (f == "group" || f == "query") { if (dtype != kI32) Log::Fatal("group must be int32"); ds->metadata.num_data = ds->num_data; ds->metadata.SetGroup(static_cast<const int32_t*>(data), static_cast<data_size_t>(n)); }
  else if (f == "init_score") {
    std::vector<double> v(n);
    for (int64_t i = 0; i < n; ++i) v[i] = dtype == kF64 ? static_cast<const double*>(data)[i] : static_cast<const float*>(data)[i];
    ds->metadata.SetInitScore(v.data(), n);
  } else Log::Fatal("Unknown field name %s", field_name);
  API_END();
}

int FB_DatasetGetField(DatasetHandle handle, const char* field_name, int64_t* out_len, const void** out_ptr, int* out_type) {
  API_BEGIN();
  Dataset* ds = static_cast<Dataset*>(handle); const std::string f = field_name;
  if (f == "label" || f == "target") { *out_len = ds->metadata.label.size(); *out_ptr = ds->metadata.label.data(); *out_type = kF32; }
  else if (f == "weight" || f == "weights") { *out_len = ds->metadata.weights.size(); *out_ptr = ds->metadata.weights.data(); *out_type = kF32; }
  else if (f == "group" || f == "query") { *out_len = ds->metadata.query_boundaries.size(); *out_ptr = ds->metadata.query_boundaries.data(); *out_type = kI32; }
  else if (f == "init_score") { *out_len = ds->metadata.init_score.size(); *out_ptr = ds->metadata.init_score.data(); *out_type = kF64; }
  else Log::Fatal("Unknown field name %s", field_name);
  API_END();
}

int FB_DatasetGetNumData(DatasetHandle handle, int32_t* out) { API_BEGIN(); *out = static_cast<Dataset*>(handle)->num_data; API_END(); }
int FB_DatasetGetNumFeature(DatasetHandle handle, int32_t* out) { API_BEGIN(); *out = static_cast<Dataset*>(handle)->num_total_features; API_END(); }
int FB_DatasetGetInfo(DatasetHandle handle, int32_t* out) {
  API_BEGIN();
  Dataset* ds = static_cast<Dataset*>(handle);
  out[0] = ds->num_features; out[1] = ds->num_groups; out[2] = ds->num_total_bin; out[3] = ds->max_group_bin; out[4] = ds->device != nullptr; out[5] = ds->has_host_bins();
  API_END();
}
int FB_DatasetSetFeatureNames(DatasetHandle handle, const char** names, int num) {
  API_BEGIN();
  Dataset* ds = static_cast<Dataset*>(handle);
  if (num != ds->num_total_features) Log::Fatal("Size of feature names (%d) differs from the number of features (%d)", num, ds->num_total_features);
  ds->feature_names.clear();
  for (int i = 0; i < num; ++i) { std::string s = names[i]; for (auto& c : s) if (c == ' ') c = '_'; ds->feature_names.push_back(s); }
  API_END();
}
int FB_DatasetGetFeatureNames(DatasetHandle handle, int64_t buffer_len, int64_t* out_len, char* out) {
  API_BEGIN();
  std::string s; for (auto& n : static_cast<Dataset*>(handle)->feature_names) { if (!s.empty()) s += "\n"; s += n; }
  CopyOut(s, buffer_len, out_len, out);
  API_END();
}
int FB_DatasetGetBinnedRow(DatasetHandle handle, int32_t row, int32_t* out_bins) {
  API_BEGIN();
  Dataset* ds = static_cast<Dataset*>(handle);
  if (!ds->has_host_bins()) Log::Fatal("Dataset has no host-resident bins");
  for (int f = 0; f < ds->num_features; ++f) out_bins[f] = ds->FeatureBin(row, f);
  API_END();
}
int FB_DatasetSaveBinary(DatasetHandle handle, const char* filename) { API_BEGIN(); static_cast<Dataset*>(handle)->SaveBinary(filename); API_END(); }
int FB_DatasetGetSubset(const DatasetHandle handle, const int32_t* idx, int32_t n, DatasetHandle* out) { API_BEGIN(); *out = static_cast<const Dataset*>(handle)->Subset(idx, n); API_END(); }
int FB_DatasetFreeDeviceData(DatasetHandle handle) { API_BEGIN(); Dataset* ds = static_cast<Dataset*>(handle); if (ds->device) { FreeDeviceDataset(ds->device); ds->device = nullptr; } API_END(); }
int FB_DatasetFeatureNumBin(DatasetHandle handle, int feature, int* out) {
  API_BEGIN();
  const Dataset* ds = static_cast<const Dataset*>(handle);
  if (feature < 0 || feature >= ds->num_total_features) Log::Fatal("Feature index %d is out of range (0..%d)", feature, ds->num_total_features - 1);
  const BinMapper* m = ds->mappers[feature].get();
  *out = (m == nullptr || m->is_trivial) ? 0 : m->num_bin;
  API_END();
}
int FB_DatasetFree(DatasetHandle handle) { API_BEGIN(); delete static_cast<Dataset*>(handle); API_END(); }

// ------------------------------------------------------------- Booster ----
int FB_BoosterCreate(const DatasetHandle train_data, const char* parameters, BoosterHandle* out) {
  API_BEGIN();
  std::unique_ptr<BoosterWrap> b(new BoosterWrap());
  const Dataset* train = static_cast<const Dataset*>(train_data);
  b->config.Set(Config::Str2Map(parameters), CudaAvailable());
  if (b->config.num_threads > 0) omp_set_num_threads(b->config.num_threads);
  if (b->config.is_cuda && !CudaAvailable()) Log::Fatal("device_type=cuda was requested but no CUDA device is available");
  if (b->config.is_cuda && train->device == nullptr) {
    // the device engine uploads host bins itself when the dataset was built on the host
    if (!train->has_host_bins()) Log::Fatal("Dataset has neither device nor host bins");
  }
  if (!b->config.is_cuda && !train->has_host_bins()) Log::Fatal("device_type=cpu needs a dataset with host-resident bins");
  b->train = train;
  b->objective.reset(CreateObjective(b->config.objective, b->config));
  if (b->objective) {
    ScopedTimer t("Booster::ObjectiveInit");
    if (b->objective->NeedQueries() && train->metadata.query_boundaries.empty()) Log::Fatal("Ranking tasks require query information");
    b->objective->Init(train->metadata, train->num_data);
  }
  b->gbdt.reset(new GBDT());
  ScopedTimer t("Booster::GBDTInit");
  b->gbdt->Init(b->config, train, b->objective.get(), b->config.metric_list);
  *out = b.release();
  API_END();
}

static int LoadBooster(const std::string& text, int* out_iters, BoosterHandle* out) {
  std::unique_ptr<BoosterWrap> b(new BoosterWrap());
  b->gbdt.reset(new GBDT());
  if (text.size() >= 4 && memcmp(text.data(), "FALB", 4) == 0) b->gbdt->LoadModelFromBinary(text.data(), text.size());
  else b->gbdt->LoadModelFromString(text.data(), text.size());
  *out_iters = b->gbdt->current_iteration();
  *out = b.release();
  return 0;
}

int FB_BoosterCreateFromModelfile(const char* filename, int* out_num_iterations, BoosterHandle* out) {
  API_BEGIN();
  std::ifstream f(filename, std::ios::binary);
  if (!f) Log::Fatal("Model file %s is not available for reads", filename);
  std::string text((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
  LoadBooster(text, out_num_iterations, out);
  API_END();
}
int FB_BoosterLoadModelFromString(const char* model_str, int64_t len, int* out_num_iterations, BoosterHandle* out) {
  API_BEGIN(); LoadBooster(std::string(model_str, len > 0 ? static_cast<size_t>(len) : strlen(model_str)), out_num_iterations, out); API_END();
}
int FB_BoosterCreateFromBinary(const char* data, int64_t len, int* out_num_iterations, BoosterHandle* out) {
  API_BEGIN(); LoadBooster(std::string(data, static_cast<size_t>(len)), out_num_iterations, out); API_END();
}
int FB_BoosterFree(BoosterHandle handle) { API_BEGIN(); delete static_cast<BoosterWrap*>(handle); API_END(); }

#define BW() BoosterWrap* b = static_cast<BoosterWrap*>(handle); std::lock_guard<std::mutex> lock(b->mu)

int FB_BoosterAddValidData(BoosterHandle handle, const DatasetHandle valid_data) { API_BEGIN(); BW(); b->gbdt->AddValidData(static_cast<const Dataset*>(valid_data)); API_END(); }
int FB_BoosterResetParameter(BoosterHandle handle, const char* parameters) {
  API_BEGIN(); BW();
  auto m = Config::Str2Map(parameters);
  for (const char* frozen : {"max_bin", "min_data_in_bin", "bin_construct_sample_cnt", "enable_bundle", "use_missing", "zero_as_missing", "categorical_feature", "num_class", "objective", "boosting", "device_type"})
    if (m.count(frozen)) Log::Fatal("Cannot change %s after the booster was constructed", frozen);
  Config merged = b->config;
  auto all = b->config.raw; for (auto& kv : m) all[kv.first] = kv.second;
  merged = Config(); merged.Set(all, CudaAvailable());
  b->config = merged; b->gbdt->ResetConfig(merged);
  API_END();
}
int FB_BoosterUpdateOneIter(BoosterHandle handle, int* is_finished) { API_BEGIN(); BW(); *is_finished = b->gbdt->TrainOneIter(nullptr, nullptr) ? 1 : 0; API_END(); }
int FB_BoosterUpdateOneIterCustom(BoosterHandle handle, const float* grad, const float* hess, int on_device, int* is_finished) {
  API_BEGIN(); BW();
  if (on_device && b->gbdt->engine() == nullptr) Log::Fatal("Device gradients need a CUDA booster");
  if (!on_device && b->gbdt->engine() != nullptr) Log::Fatal("A CUDA booster takes custom gradients as device pointers");
  *is_finished = b->gbdt->TrainOneIter(grad, hess) ? 1 : 0;
  API_END();
}
int FB_BoosterRollbackOneIter(BoosterHandle handle) { API_BEGIN(); BW(); b->gbdt->RollbackOneIter(); API_END(); }
int FB_BoosterGetCurrentIteration(BoosterHandle handle, int* out) { API_BEGIN(); BW(); *out = b->gbdt->current_iteration(); API_END(); }
int FB_BoosterNumModelPerIteration(BoosterHandle handle, int* out) { API_BEGIN(); BW(); *out = b->gbdt->num_tree_per_iteration_; API_END(); }
int FB_BoosterNumberOfTotalModel(BoosterHandle handle, int* out) { API_BEGIN(); BW(); *out = b->gbdt->NumModels(); API_END(); }
int FB_BoosterGetNumClasses(BoosterHandle handle, int* out) { API_BEGIN(); BW(); *out = b->gbdt->num_class_; API_END(); }
int FB_BoosterGetNumFeature(BoosterHandle handle, int* out) { API_BEGIN(); BW(); *out = b->gbdt->max_feature_idx_ + 1; API_END(); }
int FB_BoosterGetEvalCounts(BoosterHandle handle, int* out) { API_BEGIN(); BW(); *out = static_cast<int>(b->gbdt->EvalNames().size()); API_END(); }
int FB_BoosterGetEvalNames(BoosterHandle handle, int64_t buffer_len, int64_t* out_len, char* out) {
  API_BEGIN(); BW();
  auto names = b->gbdt->EvalNames(); auto hb = b->gbdt->EvalHigherBetter();
  std::string s; for (size_t i = 0; i < names.size(); ++i) { if (i) s += "\n"; s += (hb[i] ? "+" : "-") + names[i]; }
  CopyOut(s, buffer_len, out_len, out);
  API_END();
}
int FB_BoosterGetEval(BoosterHandle handle, int data_idx, int* out_len, double* out_results) {
  API_BEGIN(); BW();
  auto v = b->gbdt->GetEval(data_idx); *out_len = static_cast<int>(v.size());
  for (size_t i = 0; i < v.size(); ++i) out_results[i] = v[i];
  API_END();
}
int FB_BoosterGetNumPredict(BoosterHandle handle, int data_idx, int64_t* out_len) { API_BEGIN(); BW(); *out_len = b->gbdt->GetNumPredict(data_idx); API_END(); }
int FB_BoosterGetPredict(BoosterHandle handle, int data_idx, int64_t* out_len, double* out_result) { API_BEGIN(); BW(); *out_len = b->gbdt->GetNumPredict(data_idx); b->gbdt->GetPredictAt(data_idx, out_result); API_END(); }
int FB_BoosterGetTrainScoreDevicePtr(BoosterHandle handle, void** out_ptr) { API_BEGIN(); BW(); *out_ptr = b->gbdt->TrainScoreDevicePtr(); API_END(); }
int FB_BoosterCalcNumPredict(BoosterHandle handle, int num_row, int predict_type, int start_iteration, int num_iteration, int64_t* out_len) {
  API_BEGIN(); BW(); *out_len = static_cast<int64_t>(num_row) * b->gbdt->NumPredictOneRow(predict_type, start_iteration, num_iteration); API_END();
}
int FB_BoosterPredictForMat(BoosterHandle handle, const void* data, int dtype, int32_t nrow, int32_t ncol, int is_row_major, int predict_type,
                            int start_iteration, int num_iteration, const char* parameter, int64_t* out_len, double* out_result) {
  API_BEGIN(); BW();
  // the options of this call only: nothing is written into the booster, so a later call that omits them gets the defaults
  const PredictParams pp = PredictParams::FromString(parameter);
  *out_len = static_cast<int64_t>(nrow) * b->gbdt->NumPredictOneRow(predict_type, start_iteration, num_iteration);
  b->gbdt->PredictMat(data, dtype, nrow, ncol, is_row_major != 0, predict_type, start_iteration, num_iteration, out_result, pp);
  API_END();
}
// ---- single-row and sparse entry points --------------------------------------------------------------------
// Parity: src/c_api.cpp (LGBM_BoosterPredictForMatSingleRow[Fast[Init]], LGBM_BoosterPredictForCSR, LGBM_DatasetCreateFromCSR,
// LGBM_GetSampleCount, LGBM_SampleIndices, LGBM_DumpParamAliases, LGBM_BoosterValidateFeatureNames, LGBM_DatasetDumpText).
int FB_BoosterPredictForMatSingleRow(BoosterHandle handle, const void* data, int dtype, int32_t ncol, int is_row_major, int predict_type, int start_iteration,
                                     int num_iteration, const char* parameter, int64_t* out_len, double* out_result) {
  return FB_BoosterPredictForMat(handle, data, dtype, 1, ncol, is_row_major, predict_type, start_iteration, num_iteration, parameter, out_len, out_result);
}

namespace {
// Everything a single-row prediction needs, resolved once: the parameter string is parsed at FastInit, not per row.
struct FastConfig { BoosterHandle booster; int predict_type, start_iteration, num_iteration, dtype; int32_t ncol; PredictParams pp; int per_row; };
// rows [r0, r1) of a CSR matrix as a dense row-major double block
void DensifyCSR(const void* indptr, int indptr_type, const int32_t* indices, const void* data, int data_type, int64_t r0, int64_t r1, int64_t num_col, std::vector<double>* out) {
  out->assign(static_cast<size_t>(r1 - r0) * num_col, 0.0);
  auto ptr = [&](int64_t i) -> int64_t { return indptr_type == kI32 ? static_cast<const int32_t*>(indptr)[i] : static_cast<const int64_t*>(indptr)[i]; };
  for (int64_t r = r0; r < r1; ++r)
    for (int64_t k = ptr(r); k < ptr(r + 1); ++k) {
      const int32_t c = indices[k];
      if (c < 0 || c >= num_col) continue;
      (*out)[static_cast<size_t>(r - r0) * num_col + c] = data_type == kF32 ? static_cast<double>(static_cast<const float*>(data)[k]) : static_cast<const double*>(data)[k];
    }
}
}  // namespace

int FB_BoosterPredictForMatSingleRowFastInit(BoosterHandle handle, int predict_type, int start_iteration, int num_iteration, int dtype, int32_t ncol,
                                             const char* parameter, void** out_fast_config) {
  API_BEGIN();
  BW();
  FastConfig* fc = new FastConfig{handle, predict_type, start_iteration, num_iteration, dtype, ncol, PredictParams::FromString(parameter),
                                  b->gbdt->NumPredictOneRow(predict_type, start_iteration, num_iteration)};
  *out_fast_config = fc;
  API_END();
}
int FB_BoosterPredictForMatSingleRowFast(void* fast_config, const void* data, int64_t* out_len, double* out_result) {
  API_BEGIN();
  const FastConfig* fc = static_cast<const FastConfig*>(fast_config);
  BoosterHandle handle = fc->booster; BW();
  *out_len = fc->per_row;
  b->gbdt->PredictMat(data, fc->dtype, 1, fc->ncol, true, fc->predict_type, fc->start_iteration, fc->num_iteration, out_result, fc->pp);
  API_END();
}
// Prepared single-row prediction from one CSR row: the row is scattered into a dense buffer of the prepared width.
int FB_BoosterPredictForCSRSingleRowFastInit(BoosterHandle handle, int predict_type, int start_iteration, int num_iteration, int data_type, int64_t num_col,
                                             const char* parameter, void** out_fast_config) {
  if (num_col <= 0 || num_col > INT32_MAX) return FB_SetLastErrorForCompat("The number of columns must be a positive 32-bit value");
  (void)data_type;   // the row is densified to f64
  return FB_BoosterPredictForMatSingleRowFastInit(handle, predict_type, start_iteration, num_iteration, kF64, static_cast<int32_t>(num_col), parameter, out_fast_config);
}
int FB_BoosterPredictForCSRSingleRowFast(void* fast_config, const void* indptr, int indptr_type, const int32_t* indices, const void* data, int data_type, int64_t nindptr,
                                         int64_t nelem, int64_t* out_len, double* out_result) {
  API_BEGIN();
  (void)nelem;
  if (nindptr != 2) Log::Fatal("A single row has two row pointers (got %lld)", static_cast<long long>(nindptr));
  const FastConfig* fc = static_cast<const FastConfig*>(fast_config);
  static thread_local std::vector<double> dense;
  DensifyCSR(indptr, indptr_type, indices, data, data_type, 0, 1, fc->ncol, &dense);
  if (FB_BoosterPredictForMatSingleRowFast(fast_config, dense.data(), out_len, out_result) != 0) return -1;
  API_END();
}
int FB_FastConfigFree(void* fast_config) { API_BEGIN(); delete static_cast<FastConfig*>(fast_config); API_END(); }

int FB_BoosterPredictForCSR(BoosterHandle handle, const void* indptr, int indptr_type, const int32_t* indices, const void* data, int data_type, int64_t nindptr,
                            int64_t nelem, int64_t num_col, int predict_type, int start_iteration, int num_iteration, const char* parameter, int64_t* out_len,
                            double* out_result) {
  (void)nelem;
  const int64_t nrow = nindptr - 1;
  int64_t total = 0;
  std::vector<double> block;
  const int64_t step = std::max<int64_t>(1, (8 << 20) / std::max<int64_t>(1, num_col));
  for (int64_t r0 = 0; r0 < nrow; r0 += step) {
    const int64_t r1 = std::min(nrow, r0 + step);
    try { DensifyCSR(indptr, indptr_type, indices, data, data_type, r0, r1, num_col, &block); } catch (std::exception& ex) { g_last_error = ex.what(); return -1; }
    int64_t len = 0;
    if (FB_BoosterPredictForMat(handle, block.data(), kF64, static_cast<int32_t>(r1 - r0), static_cast<int32_t>(num_col), 1, predict_type, start_iteration, num_iteration,
                                parameter, &len, out_result + total) != 0) return -1;
    total += len;
  }
  *out_len = total;
  return 0;
}

// Feature contributions of CSR rows as a CSR matrix (zeros dropped): [rows x (features + 1) * trees-per-round]. The three
// output arrays are allocated here and released by FB_BoosterFreePredictSparse. out_len[0] = stored values, out_len[1] =
// entries of the row pointer. matrix_type 1: CSC in and out (num_col is then the number of rows, the pointer array runs
// over the output's columns). Parity: FLC_BoosterPredictSparseOutput.
int FB_BoosterPredictSparseOutput(BoosterHandle handle, const void* indptr, int indptr_type, const int32_t* indices, const void* data, int data_type, int64_t nindptr,
                                  int64_t nelem, int64_t num_col, int predict_type, int start_iteration, int num_iteration, const char* parameter, int matrix_type,
                                  int64_t* out_len, void** out_indptr, int32_t** out_indices, void** out_data) {
  if (predict_type != 3) return FB_SetLastErrorForCompat("Sparse output is for feature contributions (predict_type = contrib)");
  if (matrix_type != 0 && matrix_type != 1) return FB_SetLastErrorForCompat("matrix_type is 0 (CSR) or 1 (CSC)");
  int64_t per_row = 0;
  if (FB_BoosterCalcNumPredict(handle, 1, predict_type, start_iteration, num_iteration, &per_row) != 0) return -1;
  if (matrix_type == 1) {
    // CSC in (num_col here = the number of rows), CSC out: column c of the output lists the rows with a non-zero contribution
    const int64_t rows = num_col;
    std::vector<double> dense_c(static_cast<size_t>(std::max<int64_t>(1, rows * per_row)));
    int64_t len_c = 0;
    if (FB_BoosterPredictForCSC(handle, indptr, indptr_type, indices, data, data_type, nindptr, nelem, rows, predict_type, start_iteration, num_iteration, parameter, &len_c,
                                dense_c.data()) != 0) return -1;
    int64_t nnz_c = 0; for (int64_t i = 0; i < rows * per_row; ++i) if (dense_c[static_cast<size_t>(i)] != 0.0) ++nnz_c;
    const bool p64 = indptr_type != kI32, v32 = data_type == kF32;
    void* cp = malloc(static_cast<size_t>(per_row + 1) * (p64 ? 8 : 4));
    int32_t* ci = static_cast<int32_t*>(malloc(static_cast<size_t>(std::max<int64_t>(1, nnz_c)) * 4));
    void* cd = malloc(static_cast<size_t>(std::max<int64_t>(1, nnz_c)) * (v32 ? 4 : 8));
    if (cp == nullptr || ci == nullptr || cd == nullptr) { free(cp); free(ci); free(cd); return FB_SetLastErrorForCompat("Out of memory for the sparse output"); }
    int64_t w = 0;
    for (int64_t c = 0; c <= per_row; ++c) {
      if (p64) static_cast<int64_t*>(cp)[c] = w; else static_cast<int32_t*>(cp)[c] = static_cast<int32_t>(w);
      if (c == per_row) break;
      for (int64_t r = 0; r < rows; ++r) {
        const double v = dense_c[static_cast<size_t>(r * per_row + c)];
        if (v == 0.0) continue;
        ci[w] = static_cast<int32_t>(r);
        if (v32) static_cast<float*>(cd)[w] = static_cast<float>(v); else static_cast<double*>(cd)[w] = v;
        ++w;
      }
    }
    out_len[0] = nnz_c; out_len[1] = per_row + 1;
    *out_indptr = cp; *out_indices = ci; *out_data = cd;
    return 0;
  }
  const int64_t nrow = nindptr - 1;
  std::vector<double> dense(static_cast<size_t>(std::max<int64_t>(1, nrow * per_row)));
  int64_t len = 0;
  if (FB_BoosterPredictForCSR(handle, indptr, indptr_type, indices, data, data_type, nindptr, nelem, num_col, predict_type, start_iteration, num_iteration, parameter, &len,
                              dense.data()) != 0) return -1;
  int64_t nnz = 0; for (int64_t i = 0; i < nrow * per_row; ++i) if (dense[static_cast<size_t>(i)] != 0.0) ++nnz;
  const bool ptr64 = indptr_type != kI32, val32 = data_type == kF32;
  void* op = malloc(static_cast<size_t>(nrow + 1) * (ptr64 ? 8 : 4));
  int32_t* oi = static_cast<int32_t*>(malloc(static_cast<size_t>(std::max<int64_t>(1, nnz)) * 4));
  void* od = malloc(static_cast<size_t>(std::max<int64_t>(1, nnz)) * (val32 ? 4 : 8));
  if (op == nullptr || oi == nullptr || od == nullptr) { free(op); free(oi); free(od); return FB_SetLastErrorForCompat("Out of memory for the sparse output"); }
  int64_t k = 0;
  for (int64_t r = 0; r <= nrow; ++r) {
    if (ptr64) static_cast<int64_t*>(op)[r] = k; else static_cast<int32_t*>(op)[r] = static_cast<int32_t>(k);
    if (r == nrow) break;
    for (int64_t c = 0; c < per_row; ++c) {
      const double v = dense[static_cast<size_t>(r * per_row + c)];
      if (v == 0.0) continue;
      oi[k] = static_cast<int32_t>(c);
      if (val32) static_cast<float*>(od)[k] = static_cast<float>(v); else static_cast<double*>(od)[k] = v;
      ++k;
    }
  }
  out_len[0] = nnz; out_len[1] = nrow + 1;
  *out_indptr = op; *out_indices = oi; *out_data = od;
  return 0;
}
int FB_BoosterFreePredictSparse(void* indptr, int32_t* indices, void* data) { free(indptr); free(indices); free(data); return 0; }

int FB_DatasetCreateFromCSR(const void* indptr, int indptr_type, const int32_t* indices, const void* data, int data_type, int64_t nindptr, int64_t nelem,
                            int64_t num_col, const char* parameters, const DatasetHandle reference, DatasetHandle* out) {
  API_BEGIN();
  (void)nelem;
  const int32_t nrow = static_cast<int32_t>(nindptr - 1), ncol = static_cast<int32_t>(num_col);
  Config cfg; cfg.Set(Config::Str2Map(parameters), CudaAvailable());
  std::unique_ptr<Dataset> ds(new Dataset());
  std::vector<double> block;
  if (reference != nullptr) ds->CopySchemaFrom(*static_cast<const Dataset*>(reference));
  else {
    // the same draw by row id as for a dense matrix, so a matrix gets the same bins in either form
    const double frac = std::min(1.0, static_cast<double>(cfg.bin_construct_sample_cnt) / std::max(1, nrow));
    std::vector<int> idx(static_cast<size_t>(std::max(1, nrow)));
    int picked = 0;
    if (FB_OpBernoulliRowsHost(nrow, 0, static_cast<unsigned int>(cfg.data_random_seed), frac, idx.data(), &picked) != 0) Log::Fatal("Row sampling failed");
    idx.resize(picked);
    if (idx.empty() && nrow > 0) idx.push_back(0);
    std::vector<double> sample(static_cast<size_t>(idx.size()) * ncol), one;
    for (size_t r = 0; r < idx.size(); ++r) { DensifyCSR(indptr, indptr_type, indices, data, data_type, idx[r], idx[r] + 1, ncol, &one); std::copy(one.begin(), one.end(), sample.begin() + r * ncol); }
    ds->ConstructSchema(sample.data(), static_cast<int>(idx.size()), ncol, nrow, cfg, ParseCategorical(cfg, ncol));
  }
  ds->AllocateRows(nrow);
  const int64_t step = std::max<int64_t>(1, (8 << 20) / std::max<int64_t>(1, num_col));
  for (int64_t r0 = 0; r0 < nrow; r0 += step) {
    const int64_t r1 = std::min<int64_t>(nrow, r0 + step);
    DensifyCSR(indptr, indptr_type, indices, data, data_type, r0, r1, ncol, &block);
    ds->PushDense(block.data(), kF64, static_cast<data_size_t>(r1 - r0), ncol, true, static_cast<data_size_t>(r0));
  }
  *out = ds.release();
  API_END();
}

namespace {
// column-compressed -> row-compressed (32-bit row pointers are enough below 2^31 elements; 64-bit ones are kept otherwise)
void CscToCsr(const void* col_ptr, int col_ptr_type, const int32_t* indices, const void* data, int data_type, int64_t ncol_ptr, int64_t nelem, int64_t num_row,
              std::vector<int64_t>* indptr, std::vector<int32_t>* out_idx, std::vector<double>* out_val) {
  auto ptr = [&](int64_t i) -> int64_t { return col_ptr_type == kI32 ? static_cast<const int32_t*>(col_ptr)[i] : static_cast<const int64_t*>(col_ptr)[i]; };
  indptr->assign(static_cast<size_t>(num_row) + 1, 0);
  for (int64_t k = 0; k < nelem; ++k) { const int32_t r = indices[k]; if (r >= 0 && r < num_row) ++(*indptr)[r + 1]; }
  for (int64_t r = 0; r < num_row; ++r) (*indptr)[r + 1] += (*indptr)[r];
  out_idx->resize(static_cast<size_t>(nelem)); out_val->resize(static_cast<size_t>(nelem));
  std::vector<int64_t> cursor(indptr->begin(), indptr->end() - 1);
  for (int64_t c = 0; c + 1 < ncol_ptr; ++c)
    for (int64_t k = ptr(c); k < ptr(c + 1); ++k) {
      const int32_t r = indices[k];
      if (r < 0 || r >= num_row) continue;
      const int64_t at = cursor[r]++;
      (*out_idx)[at] = static_cast<int32_t>(c);
      (*out_val)[at] = data_type == kF32 ? static_cast<double>(static_cast<const float*>(data)[k]) : static_cast<const double*>(data)[k];
    }
}
constexpr int kI64 = 8;   // row-pointer type code of the CSR entry points for 64-bit pointers (anything but kI32)
}  // namespace

int FB_DatasetCreateFromCSC(const void* col_ptr, int col_ptr_type, const int32_t* indices, const void* data, int data_type, int64_t ncol_ptr, int64_t nelem,
                            int64_t num_row, const char* parameters, const DatasetHandle reference, DatasetHandle* out) {
  std::vector<int64_t> indptr; std::vector<int32_t> idx; std::vector<double> val;
  try { CscToCsr(col_ptr, col_ptr_type, indices, data, data_type, ncol_ptr, nelem, num_row, &indptr, &idx, &val); } catch (std::exception& ex) { g_last_error = ex.what(); return -1; }
  return FB_DatasetCreateFromCSR(indptr.data(), kI64, idx.data(), val.data(), kF64, num_row + 1, nelem, ncol_ptr - 1, parameters, reference, out);
}
int FB_BoosterPredictForCSC(BoosterHandle handle, const void* col_ptr, int col_ptr_type, const int32_t* indices, const void* data, int data_type, int64_t ncol_ptr,
                            int64_t nelem, int64_t num_row, int predict_type, int start_iteration, int num_iteration, const char* parameter, int64_t* out_len,
                            double* out_result) {
  std::vector<int64_t> indptr; std::vector<int32_t> idx; std::vector<double> val;
  try { CscToCsr(col_ptr, col_ptr_type, indices, data, data_type, ncol_ptr, nelem, num_row, &indptr, &idx, &val); } catch (std::exception& ex) { g_last_error = ex.what(); return -1; }
  return FB_BoosterPredictForCSR(handle, indptr.data(), kI64, idx.data(), val.data(), kF64, num_row + 1, nelem, ncol_ptr - 1, predict_type, start_iteration, num_iteration,
                                 parameter, out_len, out_result);
}
// Several row blocks that together form one matrix (all row-major or all column-major, same element type).
int FB_BoosterPredictForMats(BoosterHandle handle, const void** data, int dtype, int32_t nmat, const int32_t* nrow, int32_t ncol, int is_row_major, int predict_type,
                             int start_iteration, int num_iteration, const char* parameter, int64_t* out_len, double* out_result) {
  int64_t total = 0;
  for (int32_t m = 0; m < nmat; ++m) {
    int64_t len = 0;
    if (FB_BoosterPredictForMat(handle, data[m], dtype, nrow[m], ncol, is_row_major, predict_type, start_iteration, num_iteration, parameter, &len, out_result + total) != 0) return -1;
    total += len;
  }
  *out_len = total;
  return 0;
}
int FB_DatasetCreateFromMats(int32_t nmat, const void** data, int dtype, const int32_t* nrow, int32_t ncol, int is_row_major, const char* parameters,
                             const DatasetHandle reference, DatasetHandle* out) {
  API_BEGIN();
  // the blocks are read as one row-major double matrix (a copy; the single-matrix entry point then does the rest)
  int64_t total = 0; for (int32_t m = 0; m < nmat; ++m) total += nrow[m];
  std::vector<double> all(static_cast<size_t>(total) * ncol);
  int64_t at = 0;
  for (int32_t m = 0; m < nmat; ++m) {
    for (int32_t i = 0; i < nrow[m]; ++i) for (int32_t j = 0; j < ncol; ++j) {
      const size_t src = is_row_major ? static_cast<size_t>(i) * ncol + j : static_cast<size_t>(j) * nrow[m] + i;
      double v;
      switch (dtype) {
        case kF32: v = static_cast<const float*>(data[m])[src]; break;
        case kF64: v = static_cast<const double*>(data[m])[src]; break;
        case kI32: v = static_cast<const int32_t*>(data[m])[src]; break;
        default: Log::Fatal("FB_DatasetCreateFromMats takes float32, float64 or int32 blocks"); v = 0;
      }
      all[static_cast<size_t>(at + i) * ncol + j] = v;
    }
    at += nrow[m];
  }
  if (FB_DatasetCreateFromMat(all.data(), kF64, static_cast<int32_t>(total), ncol, 1, parameters, reference, out) != 0) throw std::runtime_error(g_last_error);
  API_END();
}

// ---- streaming: rows and their metadata arrive in blocks, in any order of blocks --------------------------------
// Parity: src/c_api.cpp (LGBM_DatasetInitStreaming, LGBM_DatasetPushRowsWithMetadata, LGBM_DatasetMarkFinished). The
// dataset comes from FB_DatasetCreateByReference / FB_DatasetCreateFromSampleTyped and FB_DatasetInitRows(host_bins=1).
namespace {
struct StreamState { std::vector<int32_t> query_of_row; int nclasses = 1; };
std::mutex g_stream_mu;
std::map<const Dataset*, StreamState> g_stream;
}  // namespace

int FB_DatasetInitStreaming(DatasetHandle handle, int32_t has_weights, int32_t has_init_scores, int32_t has_queries, int32_t nclasses) {
  API_BEGIN();
  Dataset* ds = static_cast<Dataset*>(handle);
  if (!ds->has_host_bins()) Log::Fatal("Streaming needs host bins: call FB_DatasetInitRows(handle, nrow, 0, 0, 1) first");
  const size_t n = static_cast<size_t>(ds->num_data);
  ds->metadata.label.assign(n, 0.f);
  if (has_weights) ds->metadata.weights.assign(n, 1.f);
  if (has_init_scores) ds->metadata.init_score.assign(n * std::max(1, nclasses), 0.0);
  std::lock_guard<std::mutex> g(g_stream_mu);
  StreamState& st = g_stream[ds];
  st.nclasses = std::max(1, nclasses);
  if (has_queries) st.query_of_row.assign(n, 0); else st.query_of_row.clear();
  API_END();
}
int FB_DatasetPushRowsWithMetadata(DatasetHandle handle, const void* data, int dtype, int32_t nrow, int32_t ncol, int32_t start_row, const float* label,
                                   const float* weight, const double* init_score, const int32_t* query) {
  API_BEGIN();
  Dataset* ds = static_cast<Dataset*>(handle);
  if (start_row < 0 || static_cast<int64_t>(start_row) + nrow > ds->num_data) Log::Fatal("Pushed rows [%d, %d) are outside the dataset (%d rows)", start_row, start_row + nrow, ds->num_data);
  ds->PushDense(data, dtype, nrow, ncol, true, start_row);
  if (label != nullptr) std::copy(label, label + nrow, ds->metadata.label.begin() + start_row);
  if (weight != nullptr && !ds->metadata.weights.empty()) std::copy(weight, weight + nrow, ds->metadata.weights.begin() + start_row);
  std::lock_guard<std::mutex> g(g_stream_mu);
  StreamState& st = g_stream[ds];
  if (init_score != nullptr && !ds->metadata.init_score.empty())   // block layout: class-major within the pushed block
    for (int k = 0; k < st.nclasses; ++k) std::copy(init_score + static_cast<size_t>(k) * nrow, init_score + static_cast<size_t>(k + 1) * nrow,
                                                     ds->metadata.init_score.begin() + static_cast<size_t>(k) * ds->num_data + start_row);
  if (query != nullptr && !st.query_of_row.empty()) std::copy(query, query + nrow, st.query_of_row.begin() + start_row);
  API_END();
}
// CSR rows with their metadata: the rows go through the CSR push, the metadata through the dense one's bookkeeping
int FB_DatasetPushRowsByCSRWithMetadata(DatasetHandle handle, const void* indptr, int indptr_type, const int32_t* indices, const void* data, int data_type,
                                        int64_t nindptr, int64_t nelem, int64_t start_row, const float* label, const float* weight, const double* init_score,
                                        const int32_t* query) {
  API_BEGIN();
  Dataset* ds = static_cast<Dataset*>(handle);
  const int64_t nrow = nindptr - 1;
  if (start_row < 0 || start_row + nrow > ds->num_data) Log::Fatal("Pushed rows [%lld, %lld) are outside the dataset (%d rows)", static_cast<long long>(start_row), static_cast<long long>(start_row + nrow), ds->num_data);
  if (FB_DatasetPushRowsByCSR(handle, indptr, indptr_type, indices, data, data_type, nindptr, nelem, ds->num_total_features, start_row) != 0) return -1;
  if (label != nullptr) std::copy(label, label + nrow, ds->metadata.label.begin() + start_row);
  if (weight != nullptr && !ds->metadata.weights.empty()) std::copy(weight, weight + nrow, ds->metadata.weights.begin() + start_row);
  std::lock_guard<std::mutex> g(g_stream_mu);
  StreamState& st = g_stream[ds];
  if (init_score != nullptr && !ds->metadata.init_score.empty())
    for (int k = 0; k < st.nclasses; ++k) std::copy(init_score + static_cast<size_t>(k) * nrow, init_score + static_cast<size_t>(k + 1) * nrow,
                                                     ds->metadata.init_score.begin() + static_cast<size_t>(k) * ds->num_data + start_row);
  if (query != nullptr && !st.query_of_row.empty()) std::copy(query, query + nrow, st.query_of_row.begin() + start_row);
  API_END();
}

// Schema from per-column samples: column j holds num_per_col[j] sampled non-zero values with the sample rows they came
// from; everything else in the num_sample_row sampled rows is zero. The rows (num_local_row of num_dist_row over all
// machines) are pushed afterwards. Parity: include/Falcata/c_api.h FLC_DatasetCreateFromSampledColumn.
int FB_DatasetCreateFromSampledColumn(double** sample_data, int** sample_indices, int32_t ncol, const int* num_per_col, int32_t num_sample_row,
                                      int32_t num_local_row, int64_t num_dist_row, const char* parameters, DatasetHandle* out) {
  API_BEGIN();
  if (ncol <= 0 || num_sample_row <= 0) Log::Fatal("An empty sample");
  std::vector<double> dense(static_cast<size_t>(num_sample_row) * ncol, 0.0);
  for (int j = 0; j < ncol; ++j)
    for (int k = 0; k < num_per_col[j]; ++k) {
      const int r = sample_indices[j][k];
      if (r < 0 || r >= num_sample_row) Log::Fatal("Sample row %d of column %d is outside the %d sampled rows", r, j, num_sample_row);
      dense[static_cast<size_t>(r) * ncol + j] = sample_data[j][k];
    }
  if (FB_DatasetCreateFromSample(dense.data(), num_sample_row, ncol, num_dist_row > 0 ? num_dist_row : num_local_row, parameters, nullptr, 0, out) != 0) return -1;
  if (FB_DatasetInitRows(*out, num_local_row, 0, num_dist_row > 0 ? num_dist_row : num_local_row, 1) != 0) return -1;
  API_END();
}

// Rows from a callback: get_row_funptr points to a std::function<void(int row, std::vector<std::pair<int, double>>& out)>
// that clears and fills `out` with the row's (column, value) pairs. Parity: FLC_DatasetCreateFromCSRFunc.
int FB_DatasetCreateFromCSRFunc(void* get_row_funptr, int num_rows, int64_t num_col, const char* parameters, const DatasetHandle reference, DatasetHandle* out) {
  API_BEGIN();
  if (get_row_funptr == nullptr) Log::Fatal("The row callback is null");
  auto& get_row = *static_cast<std::function<void(int, std::vector<std::pair<int, double>>&)>*>(get_row_funptr);
  std::vector<int64_t> indptr(1, 0); std::vector<int32_t> indices; std::vector<double> values; std::vector<std::pair<int, double>> row;
  for (int i = 0; i < num_rows; ++i) {
    get_row(i, row);
    for (const auto& kv : row) { indices.push_back(kv.first); values.push_back(kv.second); }
    indptr.push_back(static_cast<int64_t>(indices.size()));
  }
  if (FB_DatasetCreateFromCSR(indptr.data(), 8 /* int64 row pointers */, indices.data(), values.data(), kF64, static_cast<int64_t>(indptr.size()), static_cast<int64_t>(values.size()), num_col, parameters,
                              reference, out) != 0) return -1;
  API_END();
}

int FB_DatasetMarkFinished(DatasetHandle handle) {
  API_BEGIN();
  Dataset* ds = static_cast<Dataset*>(handle);
  std::lock_guard<std::mutex> g(g_stream_mu);
  auto it = g_stream.find(ds);
  if (it != g_stream.end()) {
    const auto& q = it->second.query_of_row;
    if (!q.empty()) {   // consecutive rows with the same query id form one query
      std::vector<int32_t> sizes;
      for (size_t i = 0; i < q.size(); ++i) { if (i == 0 || q[i] != q[i - 1]) sizes.push_back(0); ++sizes.back(); }
      ds->metadata.num_data = ds->num_data;
      ds->metadata.SetGroup(sizes.data(), static_cast<data_size_t>(sizes.size()));
    }
    g_stream.erase(it);
  }
  ds->metadata.UpdateQueryWeights();
  API_END();
}

// ---- Arrow C data interface ---------------------------------------------------------------------------------
// Record batches (struct arrays) whose columns are primitive numbers or booleans; nulls read as NaN. The batches are
// copied into one dense matrix and released, as the producer expects of a consumer.
// Parity: src/c_api.cpp (LGBM_DatasetCreateFromArrow, LGBM_BoosterPredictForArrow), include/Falcata/arrow.h.
namespace {
struct FBArrowSchema { const char* format; const char* name; const char* metadata; int64_t flags; int64_t n_children; FBArrowSchema** children; FBArrowSchema* dictionary;
                       void (*release)(FBArrowSchema*); void* private_data; };
struct FBArrowArray { int64_t length; int64_t null_count; int64_t offset; int64_t n_buffers; int64_t n_children; const void** buffers; FBArrowArray** children;
                      FBArrowArray* dictionary; void (*release)(FBArrowArray*); void* private_data; };

double ArrowValue(const FBArrowArray* col, const char* fmt, int64_t i) {
  const int64_t k = col->offset + i;
  const uint8_t* valid = col->n_buffers > 0 ? static_cast<const uint8_t*>(col->buffers[0]) : nullptr;
  if (valid != nullptr && col->null_count != 0 && !((valid[k >> 3] >> (k & 7)) & 1)) return std::numeric_limits<double>::quiet_NaN();
  const void* d = col->buffers[1];
  switch (fmt[0]) {
    case 'g': return static_cast<const double*>(d)[k];
    case 'f': return static_cast<const float*>(d)[k];
    case 'l': return static_cast<double>(static_cast<const int64_t*>(d)[k]);
    case 'L': return static_cast<double>(static_cast<const uint64_t*>(d)[k]);
    case 'i': return static_cast<const int32_t*>(d)[k];
    case 'I': return static_cast<const uint32_t*>(d)[k];
    case 's': return static_cast<const int16_t*>(d)[k];
    case 'S': return static_cast<const uint16_t*>(d)[k];
    case 'c': return static_cast<const int8_t*>(d)[k];
    case 'C': return static_cast<const uint8_t*>(d)[k];
    case 'b': return (static_cast<const uint8_t*>(d)[k >> 3] >> (k & 7)) & 1;
    default: Log::Fatal("Arrow column type '%s' is not a primitive number", fmt); return 0.0;
  }
}

// Releases the batches and the schema when it goes out of scope, whichever way the call ends: the consumer of an Arrow C
// data structure owns it from the moment it is handed over.
struct ArrowOwner {
  int64_t n; FBArrowArray* chunks; FBArrowSchema* schema;
  ~ArrowOwner() {
    for (int64_t c = 0; c < n; ++c) if (chunks != nullptr && chunks[c].release != nullptr) chunks[c].release(&chunks[c]);
    if (schema != nullptr && schema->release != nullptr) schema->release(schema);
  }
};

// all batches as one row-major double matrix
void ArrowToDense(int64_t n_chunks, FBArrowArray* chunks, FBArrowSchema* schema, std::vector<double>* out, int64_t* nrow, int32_t* ncol) {
  ArrowOwner owner{n_chunks, chunks, schema};
  if (schema == nullptr || schema->format == nullptr || schema->format[0] != '+' || schema->format[1] != 's') Log::Fatal("The Arrow data must be record batches (struct arrays)");
  *ncol = static_cast<int32_t>(schema->n_children);
  *nrow = 0;
  for (int64_t c = 0; c < n_chunks; ++c) *nrow += chunks[c].length;
  if (*nrow > 2147483647LL) Log::Fatal("Arrow input has %lld rows; at most 2^31 - 1 are supported", static_cast<long long>(*nrow));
  out->assign(static_cast<size_t>(*nrow) * (*ncol), 0.0);
  int64_t at = 0;
  for (int64_t c = 0; c < n_chunks; ++c) {
    const FBArrowArray& batch = chunks[c];
    if (batch.n_children != schema->n_children) Log::Fatal("An Arrow batch has %lld columns, the schema %lld", static_cast<long long>(batch.n_children), static_cast<long long>(schema->n_children));
    // validity bitmap of the record batch itself: a null struct row reads as missing in every column
    const uint8_t* row_valid = (batch.n_buffers > 0 && batch.buffers != nullptr) ? static_cast<const uint8_t*>(batch.buffers[0]) : nullptr;
    for (int32_t j = 0; j < *ncol; ++j) {
      const FBArrowArray* col = batch.children[j];
      const char* fmt = schema->children[j]->format;
      for (int64_t i = 0; i < batch.length; ++i) {
        const int64_t r = batch.offset + i;
        const bool row_null = row_valid != nullptr && !((row_valid[r >> 3] >> (r & 7)) & 1);
        (*out)[static_cast<size_t>(at + i) * (*ncol) + j] = row_null ? std::numeric_limits<double>::quiet_NaN() : ArrowValue(col, fmt, r);
      }
    }
    at += batch.length;
  }
}
}  // namespace

int FB_DatasetCreateFromArrow(int64_t n_chunks, void* chunks, void* schema, const char* parameters, const DatasetHandle reference, DatasetHandle* out) {
  std::vector<double> dense; int64_t nrow = 0; int32_t ncol = 0;
  try { ArrowToDense(n_chunks, static_cast<FBArrowArray*>(chunks), static_cast<FBArrowSchema*>(schema), &dense, &nrow, &ncol); }
  catch (std::exception& ex) { g_last_error = ex.what(); return -1; }
  return FB_DatasetCreateFromMat(dense.data(), kF64, static_cast<int32_t>(nrow), ncol, 1, parameters, reference, out);
}
int FB_BoosterPredictForArrow(BoosterHandle handle, int64_t n_chunks, void* chunks, void* schema, int predict_type, int start_iteration, int num_iteration,
                              const char* parameter, int64_t* out_len, double* out_result) {
  std::vector<double> dense; int64_t nrow = 0; int32_t ncol = 0;
  try { ArrowToDense(n_chunks, static_cast<FBArrowArray*>(chunks), static_cast<FBArrowSchema*>(schema), &dense, &nrow, &ncol); }
  catch (std::exception& ex) { g_last_error = ex.what(); return -1; }
  return FB_BoosterPredictForMat(handle, dense.data(), kF64, static_cast<int32_t>(nrow), ncol, 1, predict_type, start_iteration, num_iteration, parameter, out_len, out_result);
}

// ---- Arrow C stream interface: the stream is drained into a list of batches, then handled like an array of chunks ----
namespace {
struct FBArrowArrayStream {
  int (*get_schema)(FBArrowArrayStream*, FBArrowSchema* out);
  int (*get_next)(FBArrowArrayStream*, FBArrowArray* out);
  const char* (*get_last_error)(FBArrowArrayStream*);
  void (*release)(FBArrowArrayStream*);
  void* private_data;
};
// Pulls every batch out of the stream and releases the stream. On an error of the producer the batches already pulled are
// released and the call fails with the producer's message.
bool DrainArrowStream(void* stream_ptr, std::vector<FBArrowArray>* batches, FBArrowSchema* schema) {
  FBArrowArrayStream* st = static_cast<FBArrowArrayStream*>(stream_ptr);
  if (st == nullptr || st->get_schema == nullptr || st->get_next == nullptr) { g_last_error = "The Arrow stream is empty or already released"; return false; }
  auto fail = [&](const char* what) {
    const char* why = st->get_last_error != nullptr ? st->get_last_error(st) : nullptr;
    g_last_error = std::string(what) + (why != nullptr ? std::string(": ") + why : std::string());
    for (auto& b : *batches) if (b.release != nullptr) b.release(&b);
    batches->clear();
    if (st->release != nullptr) st->release(st);
    return false;
  };
  memset(schema, 0, sizeof(*schema));
  if (st->get_schema(st, schema) != 0) return fail("The Arrow stream gave no schema");
  for (;;) {
    FBArrowArray next; memset(&next, 0, sizeof(next));
    if (st->get_next(st, &next) != 0) { if (schema->release != nullptr) schema->release(schema); return fail("The Arrow stream failed while reading a batch"); }
    if (next.release == nullptr) break;   // end of the stream
    batches->push_back(next);
  }
  if (st->release != nullptr) st->release(st);
  return true;
}
// One numeric column (a plain array or the single child of a struct), all chunks in order, as doubles.
void ArrowColumnToDoubles(int64_t n_chunks, FBArrowArray* chunks, FBArrowSchema* schema, std::vector<double>* out) {
  ArrowOwner owner{n_chunks, chunks, schema};
  if (schema == nullptr || schema->format == nullptr) Log::Fatal("The Arrow field has no schema");
  const bool is_struct = schema->format[0] == '+' && schema->format[1] == 's';
  if (is_struct && schema->n_children != 1) Log::Fatal("A field takes one Arrow column, not %lld", static_cast<long long>(schema->n_children));
  const char* fmt = is_struct ? schema->children[0]->format : schema->format;
  out->clear();
  for (int64_t c = 0; c < n_chunks; ++c) {
    const FBArrowArray* col = is_struct ? chunks[c].children[0] : &chunks[c];
    const int64_t len = is_struct ? chunks[c].length : col->length;
    for (int64_t i = 0; i < len; ++i) out->push_back(ArrowValue(col, fmt, is_struct ? chunks[c].offset + i : i));
  }
}
int SetFieldFromDoubles(DatasetHandle handle, const char* field_name, const std::vector<double>& v) {
  const std::string f = field_name;
  if (f == "group" || f == "query") {
    std::vector<int32_t> g(v.size()); for (size_t i = 0; i < v.size(); ++i) g[i] = static_cast<int32_t>(v[i]);
    return FB_DatasetSetField(handle, field_name, g.data(), static_cast<int64_t>(g.size()), kI32);
  }
  if (f == "init_score") return FB_DatasetSetField(handle, field_name, v.data(), static_cast<int64_t>(v.size()), kF64);
  std::vector<float> x(v.begin(), v.end());
  return FB_DatasetSetField(handle, field_name, x.data(), static_cast<int64_t>(x.size()), kF32);
}
}  // namespace

// Parity: src/c_api.cpp (dataset creation, field setting and prediction from an ArrowArrayStream).
int FB_DatasetCreateFromArrowStream(void* stream, const char* parameters, const DatasetHandle reference, DatasetHandle* out) {
  std::vector<FBArrowArray> batches; FBArrowSchema schema;
  if (!DrainArrowStream(stream, &batches, &schema)) return -1;
  return FB_DatasetCreateFromArrow(static_cast<int64_t>(batches.size()), batches.data(), &schema, parameters, reference, out);
}
int FB_BoosterPredictForArrowStream(BoosterHandle handle, void* stream, int predict_type, int start_iteration, int num_iteration, const char* parameter,
                                    int64_t* out_len, double* out_result) {
  std::vector<FBArrowArray> batches; FBArrowSchema schema;
  if (!DrainArrowStream(stream, &batches, &schema)) return -1;
  return FB_BoosterPredictForArrow(handle, static_cast<int64_t>(batches.size()), batches.data(), &schema, predict_type, start_iteration, num_iteration, parameter, out_len, out_result);
}
int FB_DatasetSetFieldFromArrow(DatasetHandle handle, const char* field_name, int64_t n_chunks, void* chunks, void* schema) {
  std::vector<double> v;
  try { ArrowColumnToDoubles(n_chunks, static_cast<FBArrowArray*>(chunks), static_cast<FBArrowSchema*>(schema), &v); }
  catch (std::exception& ex) { g_last_error = ex.what(); return -1; }
  return SetFieldFromDoubles(handle, field_name, v);
}
int FB_DatasetSetFieldFromArrowStream(DatasetHandle handle, const char* field_name, void* stream) {
  std::vector<FBArrowArray> batches; FBArrowSchema schema;
  if (!DrainArrowStream(stream, &batches, &schema)) return -1;
  return FB_DatasetSetFieldFromArrow(handle, field_name, static_cast<int64_t>(batches.size()), batches.data(), &schema);
}

// Rows [start_row, start_row + nindptr - 1) of a streamed data set, given as CSR: densified block by block and pushed.
// Parity: src/c_api.cpp (LGBM_DatasetPushRowsByCSR).
int FB_DatasetPushRowsByCSR(DatasetHandle handle, const void* indptr, int indptr_type, const int32_t* indices, const void* data, int data_type, int64_t nindptr,
                            int64_t nelem, int64_t num_col, int64_t start_row) {
  API_BEGIN();
  (void)nelem;
  const int64_t nrow = nindptr - 1;
  const int64_t block = std::max<int64_t>(1, (int64_t{32} << 20) / std::max<int64_t>(1, num_col * 8));
  std::vector<double> dense;
  for (int64_t a = 0; a < nrow; a += block) {
    const int64_t b = std::min(nrow, a + block);
    DensifyCSR(indptr, indptr_type, indices, data, data_type, a, b, num_col, &dense);
    if (FB_DatasetPushRows(handle, dense.data(), kF64, static_cast<int32_t>(b - a), static_cast<int32_t>(num_col), 1, static_cast<int32_t>(start_row + a)) != 0) return -1;
  }
  API_END();
}

// Fails when `new_parameters` changes a parameter that the binned data depends on.
// Parity: src/c_api.cpp (LGBM_DatasetUpdateParamChecking).
int FB_DatasetUpdateParamChecking(const char* old_parameters, const char* new_parameters) {
  API_BEGIN();
  static const char* const kBinned[] = {"max_bin", "max_bin_by_feature", "min_data_in_bin", "bin_construct_sample_cnt", "use_missing", "zero_as_missing",
                                        "categorical_feature", "feature_pre_filter", "enable_bundle", "data_random_seed", "is_enable_sparse", "two_round",
                                        "header", "label_column", "weight_column", "group_column", "ignore_column", "forcedbins_filename", "linear_tree",
                                        "min_data_in_leaf", "max_cat_to_onehot", "precise_float_parser"};
  auto old_map = Config::Str2Map(old_parameters), new_map = Config::Str2Map(new_parameters);
  Config old_cfg; old_cfg.Set(old_map, CudaAvailable());
  for (const char* key : kBinned) {
    auto it = new_map.find(key);
    if (it == new_map.end()) continue;
    auto was = old_map.find(key);
    const std::string before = was != old_map.end() ? was->second : std::string();
    if (was == old_map.end()) {
      // the parameter was at its default when the data was binned: only min_data_in_leaf may then be raised freely
      if (std::string(key) == "min_data_in_leaf" && atoi(it->second.c_str()) >= old_cfg.min_data_in_leaf) continue;
      Config probe; std::unordered_map<std::string, std::string> one{{key, it->second}}; probe.Set(one, CudaAvailable());
      if (probe.ToString() == Config().ToString()) continue;   // set to its default value: no change
      Log::Fatal("Cannot change %s after constructed Dataset handle.", key);
    }
    if (before != it->second) {
      if (std::string(key) == "min_data_in_leaf" && atoi(it->second.c_str()) >= atoi(before.c_str()) && !old_cfg.feature_pre_filter) continue;
      Log::Fatal("Cannot change %s after constructed Dataset handle.", key);
    }
  }
  API_END();
}

int FB_GetSampleCount(int32_t num_total_row, const char* parameters, int* out) {
  API_BEGIN();
  Config cfg; cfg.Set(Config::Str2Map(parameters), CudaAvailable());
  *out = std::min<int>(num_total_row, cfg.bin_construct_sample_cnt);
  API_END();
}
// The rows of the bin sample (ascending): the counter-based draw by row id that every ingest path makes.
int FB_SampleIndices(int32_t num_total_row, const char* parameters, void* out, int32_t* out_len) {
  API_BEGIN();
  Config cfg; cfg.Set(Config::Str2Map(parameters), CudaAvailable());
  const double frac = std::min(1.0, static_cast<double>(cfg.bin_construct_sample_cnt) / std::max(1, num_total_row));
  int picked = 0;
  if (FB_OpBernoulliRowsHost(num_total_row, 0, static_cast<unsigned int>(cfg.data_random_seed), frac, static_cast<int*>(out), &picked) != 0) Log::Fatal("Row sampling failed");
  *out_len = picked;
  API_END();
}
int FB_DumpParamAliases(int64_t buffer_len, int64_t* out_len, char* out_str) {
  API_BEGIN();
  std::map<std::string, std::vector<std::string>> by_name;
  for (const auto& kv : Config::AliasTable()) by_name[kv.second].push_back(kv.first);
  std::string s = "{";
  bool first = true;
  for (auto& kv : by_name) {
    std::sort(kv.second.begin(), kv.second.end());
    if (!first) s += ", ";
    first = false;
    s += "\"" + kv.first + "\": [";
    for (size_t i = 0; i < kv.second.size(); ++i) { if (i) s += ", "; s += "\"" + kv.second[i] + "\""; }
    s += "]";
  }
  s += "}";
  *out_len = static_cast<int64_t>(s.size()) + 1;
  if (buffer_len >= *out_len && out_str != nullptr) memcpy(out_str, s.c_str(), s.size() + 1);
  API_END();
}
int FB_BoosterValidateFeatureNames(BoosterHandle handle, const char** data_names, int data_num_features) {
  API_BEGIN(); BW();
  const auto& names = b->gbdt->feature_names_;
  if (static_cast<int>(names.size()) != data_num_features) Log::Fatal("Model was trained on %d features, but got %d input features to predict", static_cast<int>(names.size()), data_num_features);
  for (int i = 0; i < data_num_features; ++i)
    if (names[i] != data_names[i]) Log::Fatal("Expected '%s' at position %d but found '%s'", names[i].c_str(), i, data_names[i]);
  API_END();
}
int FB_BoosterResetTrainingData(BoosterHandle handle, const DatasetHandle train_data) {
  API_BEGIN(); BW();
  const Dataset* train = static_cast<const Dataset*>(train_data);
  if (b->train != nullptr && train->num_total_features != b->train->num_total_features) Log::Fatal("Cannot reset training data: the new dataset has %d features, the model %d", train->num_total_features, b->train->num_total_features);
  b->objective.reset(CreateObjective(b->config.objective, b->config));
  if (b->objective) {
    if (b->objective->NeedQueries() && train->metadata.query_boundaries.empty()) Log::Fatal("Ranking tasks require query information");
    b->objective->Init(train->metadata, train->num_data);
  }
  b->train = train;
  b->gbdt->ResetTrainingData(b->config, train, b->objective.get(), b->config.metric_list);
  API_END();
}
int FB_BoosterGetLinear(BoosterHandle handle, int* out) { API_BEGIN(); BW(); *out = b->config.linear_tree ? 1 : 0; API_END(); }
int FB_DatasetGetFeatureNumBin(DatasetHandle handle, int feature, int* out) { return FB_DatasetFeatureNumBin(handle, feature, out); }
int FB_DatasetDumpText(DatasetHandle handle, const char* filename) {
  API_BEGIN();
  const Dataset* ds = static_cast<const Dataset*>(handle);
  if (!ds->has_host_bins()) Log::Fatal("Dataset has no host-resident bins to dump");
  std::ofstream f(filename);
  if (!f) Log::Fatal("Cannot write %s", filename);
  f << "num_features: " << ds->num_features << "\nnum_total_features: " << ds->num_total_features << "\nnum_groups: " << ds->num_groups << "\nnum_data: " << ds->num_data << "\n";
  f << "feature_names: "; for (auto& n : ds->feature_names) f << n << ", "; f << "\n";
  for (data_size_t i = 0; i < ds->num_data; ++i) { for (int fi = 0; fi < ds->num_features; ++fi) f << ds->FeatureBin(i, fi) << ", "; f << "\n"; }
  API_END();
}
int FB_SetLastError(const char* msg) { g_last_error = msg ? msg : ""; return 0; }
int FB_GetMaxThreads(int* out) { return FB_GetNumThreads(out); }
int FB_SetMaxThreads(int num_threads) { return FB_SetNumThreads(num_threads); }

// Predict every row of a text data file (CSV / TSV / LibSVM) and write one line per row (tab-separated
// values for multi-output predictions). Parity: src/c_api.cpp LGBM_BoosterPredictForFile, src/application/predictor.hpp.
int FB_BoosterPredictForFile(BoosterHandle handle, const char* data_filename, int data_has_header, int predict_type, int start_iteration, int num_iteration,
                             const char* parameter, const char* result_filename) {
  API_BEGIN(); BW();
  Config cfg; auto m = Config::Str2Map(parameter); m["header"] = data_has_header ? "true" : "false";
  cfg.Set(m, CudaAvailable());
  ParsedFile pf;
  ParseDataFile(data_filename, cfg, b->gbdt->max_feature_idx_ + 1, &pf);
  const int per_row = b->gbdt->NumPredictOneRow(predict_type, start_iteration, num_iteration);
  std::vector<double> out(static_cast<size_t>(pf.num_rows) * per_row);
  b->gbdt->PredictMat(pf.dense.data(), kF64, pf.num_rows, pf.num_features, true, predict_type, start_iteration, num_iteration, out.data());
  std::ofstream f(result_filename);
  if (!f) Log::Fatal("Prediction results file %s cannot be written", result_filename);
  for (data_size_t i = 0; i < pf.num_rows; ++i) {
    for (int k = 0; k < per_row; ++k) { if (k) f << '\t'; f << DoubleToStr17(out[static_cast<size_t>(i) * per_row + k]); }
    f << '\n';
  }
  API_END();
}
int FB_BoosterPredictForDeviceMat(BoosterHandle handle, const void* device_data, int dtype, int32_t nrow, int32_t ncol, int is_row_major,
                                  int predict_type, int start_iteration, int num_iteration, float* out_device) {
  API_BEGIN(); BW();
  DevicePredict(b->gbdt.get(), device_data, dtype, nrow, ncol, is_row_major != 0, predict_type, start_iteration, num_iteration, out_device);
  API_END();
}
int FB_BoosterSaveModel(BoosterHandle handle, int start_iteration, int num_iteration, int feature_importance_type, const char* filename) {
  API_BEGIN(); BW();
  std::ofstream f(filename, std::ios::binary);
  if (!f) Log::Fatal("Model file %s is not available for writes", filename);
  f << b->gbdt->SaveModelToString(start_iteration, num_iteration, feature_importance_type);
  API_END();
}
int FB_BoosterSaveModelToString(BoosterHandle handle, int start_iteration, int num_iteration, int feature_importance_type, int64_t buffer_len,
                                int64_t* out_len, char* out_str) {
  API_BEGIN(); BW(); CopyOut(b->gbdt->SaveModelToString(start_iteration, num_iteration, feature_importance_type), buffer_len, out_len, out_str); API_END();
}
int FB_BoosterDumpModel(BoosterHandle handle, int start_iteration, int num_iteration, int feature_importance_type, int64_t buffer_len,
                        int64_t* out_len, char* out_str) {
  API_BEGIN(); BW(); CopyOut(b->gbdt->DumpModel(start_iteration, num_iteration, feature_importance_type), buffer_len, out_len, out_str); API_END();
}
int FB_BoosterModelToIfElse(BoosterHandle handle, int num_iteration, int64_t buffer_len, int64_t* out_len, char* out_str) {
  API_BEGIN(); BW(); CopyOut(b->gbdt->ModelToIfElse(num_iteration), buffer_len, out_len, out_str); API_END();
}
int FB_BoosterSaveModelToBinary(BoosterHandle handle, int start_iteration, int num_iteration, int feature_importance_type, int with_stats,
                                int with_diagnostics, int f32_leaves, int compress_level, int64_t buffer_len, int64_t* out_len, char* out) {
  API_BEGIN(); BW();
  auto buf = b->gbdt->SaveModelToBinary(start_iteration, num_iteration, feature_importance_type, with_stats != 0, with_diagnostics != 0, f32_leaves != 0, compress_level);
  *out_len = static_cast<int64_t>(buf.size());
  if (buffer_len >= *out_len && out != nullptr) memcpy(out, buf.data(), buf.size());
  API_END();
}
int FB_BoosterGetLeafValue(BoosterHandle handle, int tree_idx, int leaf_idx, double* out_val) { API_BEGIN(); BW(); *out_val = b->gbdt->GetLeafValue(tree_idx, leaf_idx); API_END(); }
int FB_BoosterSetLeafValue(BoosterHandle handle, int tree_idx, int leaf_idx, double val) { API_BEGIN(); BW(); b->gbdt->SetLeafValue(tree_idx, leaf_idx, val); API_END(); }
int FB_BoosterFeatureImportance(BoosterHandle handle, int num_iteration, int importance_type, double* out_results) {
  API_BEGIN(); BW(); auto v = b->gbdt->FeatureImportance(num_iteration, importance_type); for (size_t i = 0; i < v.size(); ++i) out_results[i] = v[i]; API_END();
}
int FB_BoosterGetFeatureNames(BoosterHandle handle, int64_t buffer_len, int64_t* out_len, char* out) {
  API_BEGIN(); BW(); std::string s; for (auto& n : b->gbdt->feature_names_) { if (!s.empty()) s += "\n"; s += n; } CopyOut(s, buffer_len, out_len, out); API_END();
}
int FB_BoosterRefit(BoosterHandle handle, const int32_t* leaf_preds, int32_t nrow, int32_t ncol) { API_BEGIN(); BW(); b->gbdt->RefitTree(leaf_preds, nrow, ncol); API_END(); }
int FB_BoosterMerge(BoosterHandle handle, BoosterHandle other_handle) { API_BEGIN(); BW(); b->gbdt->MergeFrom(static_cast<BoosterWrap*>(other_handle)->gbdt.get()); API_END(); }
int FB_BoosterShuffleModels(BoosterHandle handle, int start_iter, int end_iter) { API_BEGIN(); BW(); b->gbdt->ShuffleModels(start_iter, end_iter); API_END(); }
int FB_BoosterGetUpperBoundValue(BoosterHandle handle, double* out) { API_BEGIN(); BW(); *out = b->gbdt->UpperBound(); API_END(); }
int FB_BoosterGetLowerBoundValue(BoosterHandle handle, double* out) { API_BEGIN(); BW(); *out = b->gbdt->LowerBound(); API_END(); }
int FB_BoosterGetLoadedParam(BoosterHandle handle, int64_t buffer_len, int64_t* out_len, char* out_str) {
  API_BEGIN(); BW(); CopyOut(b->gbdt->loaded_parameter_.empty() ? b->gbdt->config_.ToString() : b->gbdt->loaded_parameter_, buffer_len, out_len, out_str); API_END();
}
int FB_BoosterGpuLaunches(BoosterHandle handle, int64_t* out) { API_BEGIN(); BW(); *out = b->gbdt->engine() ? b->gbdt->engine()->GpuLaunches() : 0; API_END(); }
int FB_BoosterStageReport(BoosterHandle handle, int64_t buffer_len, int64_t* out_len, char* out_str) {
  API_BEGIN(); BW(); CopyOut(b->gbdt->engine() ? b->gbdt->engine()->StageReport() : std::string(), buffer_len, out_len, out_str); API_END();
}

}  // extern "C"
