// Value -> bin mapping for one feature.
// Parity: src/io/bin.cpp:L81-511 (FindBin and helpers), include/Falcata/bin.h:L644-682
// (ValueToBin), L230-239 (feature_infos string).
#pragma once
#include <string>
#include <unordered_map>
#include <vector>
#include "fb/common.h"

namespace fb {

enum class BinType : int { Numerical = 0, Categorical = 1 };
enum class MissingType : int { None = 0, Zero = 1, NaN = 2 };

class BinMapper {
 public:
  int num_bin = 1;
  MissingType missing_type = MissingType::None;
  BinType bin_type = BinType::Numerical;
  bool is_trivial = true;
  double sparse_rate = 0.0;
  double min_val = 0.0, max_val = 0.0;
  int default_bin = 0;     // bin of value 0
  int most_freq_bin = 0;
  std::vector<double> bin_upper_bound;        // numerical: size num_bin (last = +inf or NaN)
  std::vector<int> bin_2_categorical;         // categorical: bin -> category value
  std::unordered_map<int, int> categorical_2_bin;

  // `values` are the sampled non-zero (and NaN) values of the feature; zeros are
  // implied: total_sample_cnt - num_values.
  void FindBin(double* values, int num_values, size_t total_sample_cnt, int max_bin, int min_data_in_bin,
               int min_split_data, bool pre_filter, BinType type, bool use_missing, bool zero_as_missing,
               const std::vector<double>& forced_upper_bounds);

  inline int ValueToBin(double value) const {
    if (std::isnan(value)) {
      if (bin_type == BinType::Categorical) return 0;
      if (missing_type == MissingType::NaN) return num_bin - 1;
      value = 0.0;
    }
    if (bin_type == BinType::Numerical) {
      int l = 0, r = num_bin - 1;
      if (missing_type == MissingType::NaN) r -= 1;
      while (l < r) {
        int m = (r + l - 1) / 2;
        if (value <= bin_upper_bound[m]) r = m; else l = m + 1;
      }
      return l;
    } else {
      int iv = static_cast<int>(value);
      if (iv < 0) return 0;
      auto it = categorical_2_bin.find(iv);
      return it == categorical_2_bin.end() ? 0 : it->second;
    }
  }
  // Real-valued threshold written into the model for "bin <= t goes left".
  inline double BinToValue(int bin) const {
    return bin_type == BinType::Numerical ? bin_upper_bound[bin] : static_cast<double>(bin_2_categorical[bin]);
  }
  std::string InfoString() const;
  // Compact serialisation used to move mappers between ranks and into dataset files.
  void Serialize(std::vector<char>* out) const;
  const char* Deserialize(const char* p);
};

}  // namespace fb
