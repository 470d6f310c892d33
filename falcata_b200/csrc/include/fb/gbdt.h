// Boosting driver: gbdt / dart / rf, bagging and GOSS row sampling, evaluation, prediction,
// text / JSON / binary model IO, refit, rollback, snapshots.
// Parity: src/boosting/gbdt.cpp (Init L159-271, TrainOneIter L455-565, RollbackOneIter L567-585,
// UpdateScore L606-638, RefitTree L369-407, divergence monitor L38-128), dart.hpp, rf.hpp, goss.hpp,
// bagging.hpp, gbdt_model_text.cpp:L315-675, gbdt_prediction.cpp, gbdt_model_binary.cpp + falb.h.
#pragma once
#include <memory>
#include <string>
#include <vector>
#include "fb/config.h"
#include "fb/dataset.h"
#include "fb/learner.h"
#include "fb/objective.h"
#include "fb/tree.h"

namespace fb {

// The device-resident half of training (scores, gradients, learner, validation scores, metrics).
// Implemented by the CUDA module; GBDT drives it when device_type=cuda.
class DeviceEngine {
 public:
  virtual ~DeviceEngine() {}
  virtual void AddValid(const Dataset* valid) = 0;
  virtual void AddConstantToScores(double v, int class_id) = 0;
  // Copies host gradients (n * trees-per-round values each) into device buffers owned by the engine and returns the device
  // pointers, which TrainOneIter takes as its custom gradients (it reads device memory only).
  virtual void UploadGradients(const float* host_grad, const float* host_hess, const float** dev_grad, const float** dev_hess) = 0;
  // This round's gradients of one class tree (as the trees were trained on them), copied to the host.
  virtual void DownloadGradients(int class_id, float* host_grad, float* host_hess) = 0;
  // score[class][row] += host_values[row] on data set data_idx (0 = training, v + 1 = validation set v)
  virtual void AddRowValuesToScores(int data_idx, int class_id, const float* host_values) = 0;
  // score = a * score + b[class] on the training and every validation set (random forests keep running means)
  virtual void ScaleScores(double a, const std::vector<double>& b) = 0;
  // Computes gradients on the device (or takes custom device gradients), grows one tree per
  // class, shrinks them, adds them to the train and validation scores. Returns host trees.
  virtual void TrainOneIter(const float* custom_grad, const float* custom_hess, int iter, double shrinkage,
                            const std::vector<double>& init_scores, std::vector<std::unique_ptr<Tree>>* out, bool* all_constant) = 0;
  virtual std::vector<double> EvalMetric(int data_idx, const std::string& metric_name, bool* supported) = 0;
  virtual void CopyScoresToHost(int data_idx, double* out) = 0;
  // by traversal of the binned rows; which: 0 = training and validation scores, 1 = training only, 2 = validation only
  virtual void AddTreeToScores(const Tree& tree, int class_id, double scale, int which = 0) = 0;
  virtual void* TrainScorePtr() = 0;       // float* on the device, class-major
  virtual int64_t GpuLaunches() const = 0;
  virtual std::string StageReport() const = 0;
  virtual void SetBagging(double fraction, int freq, int seed) = 0;
};
DeviceEngine* CreateDeviceEngine(const Config& cfg, const Dataset* train, const ObjectiveFunction* obj, int num_tree_per_iter);
bool CudaAvailable();

// Options of ONE predict call (parsed from its parameter string; nothing of them outlives the call).
struct PredictParams {
  bool early_stop = false; int early_stop_freq = 10; double early_stop_margin = 10.0; bool disable_shape_check = false;
  static PredictParams FromString(const char* parameter);
};

class GBDT {
 public:
  GBDT() {}
  ~GBDT();
  void Init(const Config& cfg, const Dataset* train, ObjectiveFunction* obj, const std::vector<std::string>& metric_names);
  // Continue boosting the trees trained so far on another dataset with the same bin mappers: scores are rebuilt by
  // replaying the model on the new rows; validation sets have to be added again.
  void ResetTrainingData(const Config& cfg, const Dataset* train, ObjectiveFunction* obj, const std::vector<std::string>& metric_names);
  void AddValidData(const Dataset* valid);
  // Returns true when training cannot continue (no splittable leaf).
  bool TrainOneIter(const float* grad, const float* hess);
  void RollbackOneIter();
  int current_iteration() const { return static_cast<int>(models_.size()) / std::max(1, num_tree_per_iteration_); }
  int NumModels() const { return static_cast<int>(models_.size()); }
  std::vector<double> GetEval(int data_idx) const;
  std::vector<std::string> EvalNames() const;
  std::vector<bool> EvalHigherBetter() const;
  int64_t GetNumPredict(int data_idx) const;
  void GetPredictAt(int data_idx, double* out) const;       // converted outputs of the training / validation scores
  void RefitTree(const int* leaf_preds, int nrow, int ncol);
  void ResetConfig(const Config& cfg);
  void ShuffleModels(int start, int end);
  void MergeFrom(const GBDT* other);

  // ---- prediction on raw feature rows ----
  // predict_type: 0 normal, 1 raw, 2 leaf index, 3 contrib
  int NumPredictOneRow(int predict_type, int start_iter, int num_iter) const;
  void PredictRow(const double* row, int predict_type, int start_iter, int num_iter, double* out, const PredictParams& pp = PredictParams()) const;
  void PredictMat(const void* data, int dtype, int nrow, int ncol, bool row_major, int predict_type, int start_iter, int num_iter, double* out,
                  const PredictParams& pp = PredictParams()) const;

  // ---- model IO ----
  std::string SaveModelToString(int start_iter, int num_iter, int importance_type) const;
  bool LoadModelFromString(const char* str, size_t len);
  std::string DumpModel(int start_iter, int num_iter, int importance_type) const;
  std::string ModelToIfElse(int num_iter) const;
  std::vector<double> FeatureImportance(int num_iter, int importance_type) const;
  // FALB container (the reference's layout). Node statistics (counts / weights: needed by TreeSHAP, JSON dumps, refit) and
  // diagnostics (split gains, internal values: needed by gain importance) are optional sections; compress_level 0 leaves every
  // section raw.
  std::vector<char> SaveModelToBinary(int start_iter, int num_iter, int importance_type, bool with_stats, bool with_diagnostics, bool f32_leaves,
                                      int compress_level) const;
  bool falb_without_stats_ = false;   // loaded from a FALB file that carries no node statistics: contributions cannot be computed
  bool LoadModelFromBinary(const char* data, size_t len);

  double GetLeafValue(int tree, int leaf) const { return models_[tree]->leaf_value[leaf]; }
  void SetLeafValue(int tree, int leaf, double v) { models_[tree]->SetLeafOutput(leaf, v); }
  double UpperBound() const; double LowerBound() const;

  int num_class_ = 1;
  int num_tree_per_iteration_ = 1;
  int max_feature_idx_ = 0;
  int label_idx_ = 0;
  bool average_output_ = false;
  std::vector<std::string> feature_names_;
  std::vector<std::string> feature_infos_;
  std::vector<std::unique_ptr<Tree>> models_;
  std::unique_ptr<ObjectiveFunction> loaded_objective_;
  const ObjectiveFunction* objective_ = nullptr;
  std::string loaded_parameter_;
  Config config_;
  DeviceEngine* engine() const { return engine_.get(); }
  void* TrainScoreDevicePtr() const { return engine_ ? engine_->TrainScorePtr() : nullptr; }
  const double* TrainScoreHost() const { return train_score_.data(); }
  int iter_ = 0;

 private:
  void Bagging(int iter, const float* grad, const float* hess);
  void BoostFromAverage(int class_id, double* out_init);
  void UpdateScore(const Tree* tree, int class_id);
  void DartDropTrees();
  void DartNormalize();
  bool CheckDivergence(const float* grad, int64_t n);
  void AddTreeScore(const Tree* tree, const Dataset* ds, double* score, double scale) const;
  // linear_tree: replace the constant leaf outputs by a ridge regression on the leaf's path features
  void FitLinearLeaves(Tree* tree, const float* grad, const float* hess, bool constant_only) const;

  const Dataset* train_ = nullptr;
  std::vector<const Dataset*> valid_;
  std::unique_ptr<TreeLearner> learner_;
  std::unique_ptr<DeviceEngine> engine_;
  std::vector<std::vector<std::unique_ptr<Metric>>> metrics_;   // [0] train, [1+] valid
  std::vector<std::string> metric_names_;
  std::vector<double> train_score_;                    // class-major
  std::vector<std::vector<double>> valid_score_;
  std::vector<float> grad_, hess_;
  std::vector<data_size_t> bag_indices_;
  data_size_t bag_cnt_ = 0;
  bool is_bagging_ = false, is_goss_ = false;
  bool is_dart_ = false, is_rf_ = false, is_cuda_ = false;
  double shrinkage_rate_ = 0.1;
  std::vector<int> drop_index_;
  std::vector<double> tree_weight_;
  double sum_weight_ = 0;
  Random drop_rand_{4};
  std::vector<double> init_scores_;
  std::vector<bool> class_need_train_;
  bool boosted_from_average_ = false;
  double first_grad_norm_ = -1;
  void FitLinearLeavesOnDeviceTrees(std::vector<std::unique_ptr<Tree>>* trees);
  std::vector<double> rf_init_scores_;
  const float* rf_dev_grad_ = nullptr; const float* rf_dev_hess_ = nullptr;   // device copies of the forest's fixed gradients (owned by the engine)
};

}  // namespace fb
