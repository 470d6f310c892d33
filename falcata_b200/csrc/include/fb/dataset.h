// Binned training data: bin mappers, feature groups (EFB bundles), row-major bin storage,
// and metadata (label / weight / query boundaries / init score).
//
// Parity: src/io/dataset.cpp (Construct L533-676, EFB L125-262 + L414-531, FixHistogram
// L1965-2061), src/io/dataset_loader.cpp:L607-768 (ConstructFromSampleData),
// src/io/metadata.cpp, include/Falcata/feature_group.h.
//
// Layout decisions that differ from the reference on purpose:
//  * one dense row-major matrix [num_data x num_groups] of group bins (uint8, or uint16 when a
//    group has more than 256 bins) serves histogram construction, row partition and binned
//    prediction alike: with a 32-byte row the gather of one row is exactly one DRAM sector;
//  * every bin of a single-feature group is stored in the histogram (no most-frequent-bin
//    elision), so only bundled features need the "total minus the rest" reconstruction.
#pragma once
#include <memory>
#include <string>
#include <vector>
#include "fb/bin.h"
#include "fb/config.h"

namespace fb {

struct Metadata {
  data_size_t num_data = 0;
  std::vector<label_t> label;
  std::vector<label_t> weights;
  std::vector<data_size_t> query_boundaries;   // size num_queries + 1
  std::vector<double> init_score;              // class-major, size k * num_data
  std::vector<label_t> query_weights;
  data_size_t num_queries() const { return query_boundaries.empty() ? 0 : static_cast<data_size_t>(query_boundaries.size()) - 1; }
  void SetLabel(const float* p, data_size_t n) { label.assign(p, p + n); }
  void SetWeights(const float* p, data_size_t n) { if (p == nullptr || n == 0) weights.clear(); else weights.assign(p, p + n); UpdateQueryWeights(); }
  void SetGroup(const int32_t* sizes, data_size_t n);
  void SetInitScore(const double* p, int64_t n) { if (p == nullptr || n == 0) init_score.clear(); else init_score.assign(p, p + n); }
  void UpdateQueryWeights();
};

// What split finding needs to know about one inner feature.
struct FeatureMeta {
  int hist_offset;     // first histogram slot of this feature's bins (group start + offset in group)
  int num_bin;         // bins of the feature itself
  int missing_type;    // MissingType
  int default_bin;
  int most_freq_bin;
  int bundled;         // 1: the most_freq_bin slot is not stored, remaining bins are contiguous
  int bin_type;        // BinType
  int group;           // column of the row-major bin matrix
  int group_offset;    // bundled: group bin of the feature's first stored bin
  int monotone;        // -1, 0, +1
  float penalty;       // feature_contri multiplier
  int real_index;      // column in the user's matrix
};

struct DeviceDataset;   // defined by the CUDA module
void FreeDeviceDataset(DeviceDataset* p);

class Dataset {
 public:
  Dataset() = default;
  ~Dataset();
  data_size_t num_data = 0;
  int num_total_features = 0;
  int num_features = 0;                 // inner (non-trivial) features
  int num_groups = 0;
  int num_total_bin = 0;                // histogram slots over all groups
  int max_group_bin = 0;
  std::vector<std::unique_ptr<BinMapper>> mappers;   // per total feature
  std::vector<int> used_feature_map;                 // total -> inner or -1
  std::vector<int> real_feature_idx;                 // inner -> total
  std::vector<std::vector<int>> group_features;      // group -> inner features
  std::vector<int> group_bin_start;                  // group -> first histogram slot
  std::vector<int> group_num_bin;
  std::vector<FeatureMeta> feature_meta;             // per inner feature
  std::vector<std::string> feature_names;
  std::vector<int> categorical_features;             // total-feature indices
  Metadata metadata;
  // storage (host). Exactly one of bins8 / bins16 is used; empty when data lives on the device only.
  int bin_bytes = 1;
  int row_stride = 0;                                // elements per row (>= num_groups, padded)
  std::vector<uint8_t> bins8;
  std::vector<uint16_t> bins16;
  DeviceDataset* device = nullptr;                   // device copy / device-only storage
  // global row id of local row 0 and global row count (rows are sharded over ranks)
  int64_t global_row_offset = 0;
  int64_t global_num_data = 0;
  int max_bin_param = 255;
  // raw feature values [num_data x num_total_features], kept only for linear_tree (the leaf regressions need them)
  bool keep_raw = false;
  std::vector<float> raw;
  bool has_raw() const { return !raw.empty(); }

  // Build mappers + groups from a dense sample [ns x ncol] (row-major doubles).
  void ConstructSchema(const double* sample, int ns, int ncol, int64_t total_rows, const Config& cfg,
                       const std::vector<int>& categorical);
  // same, with the sample in any supported element type (DType code)
  void ConstructSchemaTyped(const void* sample, int dtype, int ns, int ncol, int64_t total_rows, const Config& cfg,
                       const std::vector<int>& categorical);
  // Copy mappers/groups from another dataset (validation data aligned with training data).
  void CopySchemaFrom(const Dataset& ref);
  // Appends the features of `other` (the same rows, binned on the host) behind this dataset's: mappers, feature groups
  // and bin columns are concatenated, nothing is binned again. Parity: Dataset::AddFeaturesFrom (src/io/dataset.cpp).
  void AddFeaturesFrom(const Dataset& other);
  void AllocateRows(data_size_t n);
  // Bin rows [row_begin, row_begin+n) from a dense host matrix.
  void PushDense(const void* data, int dtype, data_size_t n, int ncol, bool row_major, data_size_t row_begin);
  inline int GroupBin(data_size_t row, int group) const {
    return bin_bytes == 1 ? bins8[static_cast<size_t>(row) * row_stride + group] : bins16[static_cast<size_t>(row) * row_stride + group];
  }
  // feature bin of a row (undoing the bundle encoding).
  inline int FeatureBin(data_size_t row, int inner) const {
    const FeatureMeta& m = feature_meta[inner];
    int gb = GroupBin(row, m.group);
    return DecodeFeatureBin(m, gb);
  }
  static inline int DecodeFeatureBin(const FeatureMeta& m, int gb) {
    if (!m.bundled) return gb;
    int rel = gb - m.group_offset;
    if (rel < 0 || rel >= m.num_bin - 1) return m.most_freq_bin;
    return rel >= m.most_freq_bin ? rel + 1 : rel;
  }
  std::string FeatureInfos() const;
  // True when `other` bins values exactly like this dataset: same features in use, same groups and, per feature, the same
  // bin boundaries / categories, missing handling and default / most frequent bins. Trees refer to data by bin index, so
  // only aligned datasets can replay a model's trees. Parity: Dataset::CheckAlign (include/Falcata/dataset.h).
  bool CheckAlign(const Dataset& other) const;
  bool has_host_bins() const { return !bins8.empty() || !bins16.empty(); }
  void SerializeSchema(std::vector<char>* out) const;
  void DeserializeSchema(const char* p, size_t n, const Config& cfg);
  void SaveBinary(const std::string& path) const;
  static Dataset* LoadBinary(const std::string& path);
  Dataset* Subset(const data_size_t* idx, data_size_t n) const;
 private:
  void BuildGroups(const std::vector<std::vector<int>>& groups, const Config& cfg);
};

// dtype codes shared with the Python layer
enum DType : int { kF32 = 0, kF64 = 1, kI8 = 2, kI16 = 3, kU8 = 4, kU16 = 5, kF16 = 6, kI32 = 7 };

// Text file loader (CSV / TSV / LibSVM with optional header, label/weight/group columns).
Dataset* LoadDatasetFromFile(const std::string& path, const Config& cfg, const Dataset* reference);
// A text data file (CSV / TSV / LibSVM) as a dense row-major matrix plus its label / weight / group columns.
struct ParsedFile {
  data_size_t num_rows = 0; int num_features = 0; bool has_header = false;
  std::vector<double> dense; std::vector<float> label, weight; std::vector<double> group_ids; std::vector<std::string> names;
};
void ParseDataFile(const std::string& path, const Config& cfg, int force_num_features, ParsedFile* out);

}  // namespace fb
