// Objective functions (host) and metrics.
// Parity: src/objective/{regression,binary,multiclass,xentropy,rank}_objective.hpp,
// src/objective/objective_function.cpp:L28-82 (factory), include/Falcata/objective_function.h;
// metrics: src/metric/*.hpp, src/metric/metric.cpp:L23-89, src/metric/dcg_calculator.cpp.
#pragma once
#include <memory>
#include <string>
#include <vector>
#include "fb/config.h"
#include "fb/dataset.h"

namespace fb {

class ObjectiveFunction {
 public:
  virtual ~ObjectiveFunction() {}
  virtual void Init(const Metadata& md, data_size_t num_data) = 0;
  // score is class-major: score[k * num_data + i]
  virtual void GetGradients(const double* score, score_t* grad, score_t* hess) const = 0;
  virtual const char* GetName() const = 0;
  virtual bool IsConstantHessian() const { return false; }
  virtual bool IsRenewTreeOutput() const { return false; }
  virtual double RenewTreeOutput(double ori, const double* /*score*/, const data_size_t* /*idx*/, int /*cnt*/) const { return ori; }
  virtual double BoostFromScore(int /*class_id*/) const { return 0.0; }
  virtual bool ClassNeedTrain(int /*class_id*/) const { return true; }
  virtual int NumModelPerIteration() const { return 1; }
  virtual int NumPredictOneRow() const { return 1; }
  virtual void ConvertOutput(const double* in, double* out) const { out[0] = in[0]; }
  virtual std::string ToString() const = 0;
  // Code the device kernels switch on (see cuda/objective_kernels.cu); -1: host only.
  virtual int DeviceKind() const { return -1; }
  virtual double DeviceParam(int) const { return 0.0; }
  virtual bool NeedQueries() const { return false; }
};

ObjectiveFunction* CreateObjective(const std::string& name, const Config& cfg);
// Re-create from the "objective=" line of a model file (e.g. "binary sigmoid:1").
ObjectiveFunction* CreateObjectiveFromModelString(const std::string& str, Config* cfg);

class Metric {
 public:
  virtual ~Metric() {}
  virtual void Init(const Metadata& md, data_size_t num_data) = 0;
  virtual std::vector<std::string> Names() const = 0;
  virtual bool HigherBetter() const = 0;
  // score: raw class-major scores; objective used to convert outputs where needed
  virtual std::vector<double> Eval(const double* score, const ObjectiveFunction* obj) const = 0;
};

Metric* CreateMetric(const std::string& name, const Config& cfg);

// DCG helpers shared by lambdarank and the ndcg metric.
struct DCG {
  static std::vector<double> Discounts(int n);
  static double MaxDCGAtK(int k, const label_t* label, int n, const std::vector<double>& gains);
  static void CalDCG(const std::vector<int>& ks, const label_t* label, const double* score, int n, const std::vector<double>& gains, std::vector<double>* out);
  static void CalMaxDCG(const std::vector<int>& ks, const label_t* label, int n, const std::vector<double>& gains, std::vector<double>* out);
};

}  // namespace fb
