// Command-line application: `falcata config=train.conf [key=value ...]`.
// Tasks: train (optionally continued from input_model, with validation files, metric output every
// metric_freq rounds, early stopping and snapshots), predict (file in, one line per row out), convert_model
// (if-else C++ source), refit (leaf values re-estimated on new data), save_binary (binned data set file).
// Parameters come from the config file (key = value lines, '#' comments) and are overridden by key=value
// arguments. Parity: src/main.cpp, src/application/application.cpp (LoadParameters L48-104, InitTrain L165-212,
// Train L214-244, Predict L246-281, ConvertModel L283-290).
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <iostream>
#include <sstream>
#include <string>
#include <unordered_map>
#include <vector>

#include "fb/c_api.h"
#include "fb/common.h"
#include "fb/config.h"

using namespace fb;

namespace {

void Check(int rc) { if (rc != 0) { std::fprintf(stderr, "[Fatal] %s\n", FB_GetLastError()); std::exit(1); } }

std::string GetString(int (*fn)(BoosterHandle, int64_t, int64_t*, char*), BoosterHandle h) {
  int64_t len = 0; Check(fn(h, 0, &len, nullptr));
  std::string s(static_cast<size_t>(len), '\0'); Check(fn(h, len, &len, &s[0]));
  if (!s.empty() && s.back() == '\0') s.pop_back();
  return s;
}

std::unordered_map<std::string, std::string> LoadParameters(int argc, char** argv) {
  std::unordered_map<std::string, std::string> cmd, file;
  auto put = [](std::unordered_map<std::string, std::string>* m, const std::string& kv) {
    const size_t eq = kv.find('=');
    if (eq == std::string::npos) { if (!Trim(kv).empty()) Log::Warning("Unknown parameter %s (expected key=value)", kv.c_str()); return; }
    const std::string k = Trim(kv.substr(0, eq)), v = Trim(kv.substr(eq + 1));
    if (!k.empty() && !m->count(k)) (*m)[k] = v;   // first occurrence wins
  };
  for (int i = 1; i < argc; ++i) put(&cmd, argv[i]);
  std::string conf;
  for (const char* k : {"config", "config_file"}) if (cmd.count(k)) conf = cmd[k];
  if (!conf.empty()) {
    std::ifstream f(conf);
    if (!f) Log::Fatal("Config file %s doesn't exist", conf.c_str());
    std::string line;
    while (std::getline(f, line)) { const size_t hash = line.find('#'); if (hash != std::string::npos) line = line.substr(0, hash); put(&file, line); }
  }
  for (auto& kv : file) if (!cmd.count(kv.first)) cmd[kv.first] = kv.second;   // the command line overrides the file
  cmd.erase("config"); cmd.erase("config_file");
  return cmd;
}

std::string ToParamString(const std::unordered_map<std::string, std::string>& m) {
  std::string s; for (auto& kv : m) { if (!s.empty()) s += ' '; s += kv.first + "=" + kv.second; } return s;
}

struct EvalNames { std::vector<std::string> names; std::vector<bool> higher; };
EvalNames GetEvalNames(BoosterHandle h) {
  EvalNames e; const std::string s = GetString(FB_BoosterGetEvalNames, h);
  for (auto& n : Split(s, '\n')) { if (n.empty()) continue; e.higher.push_back(n[0] == '+'); e.names.push_back(n.substr(1)); }
  return e;
}

int TaskTrain(const Config& cfg, const std::string& params_in) {
  if (cfg.data.empty()) Log::Fatal("No training data: set data=<file>");
  std::string params = params_in;
  if (cfg.num_machines > 1) {
    // distributed training on CPUs: one process per machine list entry, collectives over TCP; every process loads its own
    // rows (pre_partition=true: its own file; else its block of the shared file) and writes its own copy of the model
    std::string machines = cfg.machines;
    if (machines.empty() && !cfg.machine_list_filename.empty()) {
      std::ifstream f(cfg.machine_list_filename);
      if (!f) Log::Fatal("Cannot open machine list file %s", cfg.machine_list_filename.c_str());
      std::stringstream ss; ss << f.rdbuf(); machines = ss.str();
    }
    if (machines.empty()) Log::Fatal("num_machines=%d needs machines=host:port,... or machine_list_filename", cfg.num_machines);
    Check(FB_NetworkInit(machines.c_str(), cfg.local_listen_port, cfg.time_out, cfg.num_machines));
    params += " device_type=cpu";
    if (cfg.tree_learner == "serial") { Log::Warning("num_machines > 1 with tree_learner=serial: using tree_learner=data"); params += " tree_learner=data"; }
  }
  DatasetHandle train = nullptr; Check(FB_DatasetCreateFromFile(cfg.data.c_str(), params.c_str(), nullptr, &train));
  std::vector<DatasetHandle> valids; std::vector<std::string> valid_names;
  for (auto& v : SplitAny(cfg.valid, ",")) { const std::string p = Trim(v); if (p.empty()) continue; DatasetHandle d = nullptr; Check(FB_DatasetCreateFromFile(p.c_str(), params.c_str(), train, &d)); valids.push_back(d); valid_names.push_back(p); }
  BoosterHandle bst = nullptr; Check(FB_BoosterCreate(train, params.c_str(), &bst));
  if (!cfg.input_model.empty()) {
    // continued training: the loaded model's trees come first
    int it = 0; BoosterHandle init = nullptr; Check(FB_BoosterCreateFromModelfile(cfg.input_model.c_str(), &it, &init));
    Check(FB_BoosterMerge(bst, init)); Check(FB_BoosterFree(init));
    Log::Info("Continued training from %s (%d iterations)", cfg.input_model.c_str(), it);
  }
  for (DatasetHandle d : valids) Check(FB_BoosterAddValidData(bst, d));
  const EvalNames en = GetEvalNames(bst);
  int neval = 0; Check(FB_BoosterGetEvalCounts(bst, &neval));
  std::vector<double> vals(std::max(1, neval));
  double best = 0; int best_iter = 0; bool have_best = false;
  for (int it = 0; it < cfg.num_iterations; ++it) {
    int finished = 0; Check(FB_BoosterUpdateOneIter(bst, &finished));
    const bool report = cfg.metric_freq > 0 && (it + 1) % cfg.metric_freq == 0;
    if (report && cfg.is_provide_training_metric && neval > 0) {
      int n = 0; Check(FB_BoosterGetEval(bst, 0, &n, vals.data()));
      for (int k = 0; k < n; ++k) Log::Info("Iteration:%d, training %s : %g", it + 1, en.names[k].c_str(), vals[k]);
    }
    bool stop = false;
    for (size_t v = 0; v < valids.size() && neval > 0; ++v) {
      int n = 0; Check(FB_BoosterGetEval(bst, static_cast<int>(v) + 1, &n, vals.data()));
      if (report) for (int k = 0; k < n; ++k) Log::Info("Iteration:%d, valid_%d %s : %g", it + 1, static_cast<int>(v) + 1, en.names[k].c_str(), vals[k]);
      if (v == 0 && cfg.early_stopping_round > 0 && n > 0) {
        const double cur = vals[0]; const bool better = !have_best || (en.higher[0] ? cur > best + cfg.early_stopping_min_delta : cur < best - cfg.early_stopping_min_delta);
        if (better) { best = cur; best_iter = it + 1; have_best = true; }
        else if (it + 1 - best_iter >= cfg.early_stopping_round) { Log::Info("Early stopping at iteration %d, the best iteration round is %d", it + 1, best_iter); stop = true; }
      }
    }
    if (cfg.snapshot_freq > 0 && (it + 1) % cfg.snapshot_freq == 0) {
      const std::string snap = cfg.output_model + ".snapshot_iter_" + std::to_string(it + 1);
      Check(FB_BoosterSaveModel(bst, 0, -1, 0, snap.c_str()));
    }
    if (finished || stop) break;
  }
  Check(FB_BoosterSaveModel(bst, 0, (cfg.early_stopping_round > 0 && have_best) ? best_iter : -1, 0, cfg.output_model.c_str()));
  Log::Info("Finished training, model saved to %s", cfg.output_model.c_str());
  Check(FB_BoosterFree(bst)); for (DatasetHandle d : valids) Check(FB_DatasetFree(d)); Check(FB_DatasetFree(train));
  return 0;
}

int PredictType(const Config& cfg) { return cfg.predict_contrib ? 3 : (cfg.predict_leaf_index ? 2 : (cfg.predict_raw_score ? 1 : 0)); }

int TaskPredict(const Config& cfg, const std::string& params) {
  if (cfg.input_model.empty()) Log::Fatal("task=predict needs input_model");
  if (cfg.data.empty()) Log::Fatal("task=predict needs data=<file>");
  int it = 0; BoosterHandle bst = nullptr; Check(FB_BoosterCreateFromModelfile(cfg.input_model.c_str(), &it, &bst));
  Check(FB_BoosterPredictForFile(bst, cfg.data.c_str(), cfg.header ? 1 : 0, PredictType(cfg), cfg.start_iteration_predict, cfg.num_iteration_predict, params.c_str(),
                                 cfg.output_result.c_str()));
  Log::Info("Finished prediction, results saved to %s", cfg.output_result.c_str());
  return FB_BoosterFree(bst);
}

int TaskConvertModel(const Config& cfg) {
  if (cfg.input_model.empty()) Log::Fatal("task=convert_model needs input_model");
  if (cfg.convert_model_language != "cpp") Log::Fatal("convert_model_language must be cpp");
  int it = 0; BoosterHandle bst = nullptr; Check(FB_BoosterCreateFromModelfile(cfg.input_model.c_str(), &it, &bst));
  int64_t len = 0; Check(FB_BoosterModelToIfElse(bst, -1, 0, &len, nullptr));
  std::string code(static_cast<size_t>(len), '\0'); Check(FB_BoosterModelToIfElse(bst, -1, len, &len, &code[0]));
  if (!code.empty() && code.back() == '\0') code.pop_back();
  std::ofstream f(cfg.convert_model); if (!f) Log::Fatal("Cannot write %s", cfg.convert_model.c_str());
  f << code;
  Log::Info("Finished converting the model to %s", cfg.convert_model.c_str());
  return FB_BoosterFree(bst);
}

int TaskRefit(const Config& cfg, const std::string& params) {
  if (cfg.input_model.empty() || cfg.data.empty()) Log::Fatal("task=refit needs input_model and data");
  int it = 0; BoosterHandle old = nullptr; Check(FB_BoosterCreateFromModelfile(cfg.input_model.c_str(), &it, &old));
  // leaf index of every row under the existing model
  const std::string leaf_file = cfg.output_model + ".leaf_idx.tmp";
  Check(FB_BoosterPredictForFile(old, cfg.data.c_str(), cfg.header ? 1 : 0, 2, 0, -1, params.c_str(), leaf_file.c_str()));
  std::vector<int32_t> leaves; int32_t nrow = 0, ncol = 0;
  { std::ifstream f(leaf_file); std::string line; while (std::getline(f, line)) { if (line.empty()) continue; auto toks = Split(line, '\t'); ncol = static_cast<int32_t>(toks.size()); for (auto& t : toks) leaves.push_back(static_cast<int32_t>(ParseDouble(t))); ++nrow; } }
  std::remove(leaf_file.c_str());
  DatasetHandle train = nullptr; Check(FB_DatasetCreateFromFile(cfg.data.c_str(), params.c_str(), nullptr, &train));
  std::string p2 = params + " device_type=cpu";
  BoosterHandle bst = nullptr; Check(FB_BoosterCreate(train, p2.c_str(), &bst));
  Check(FB_BoosterMerge(bst, old));
  Check(FB_BoosterRefit(bst, leaves.data(), nrow, ncol));
  Check(FB_BoosterSaveModel(bst, 0, -1, 0, cfg.output_model.c_str()));
  Log::Info("Finished refitting, model saved to %s", cfg.output_model.c_str());
  Check(FB_BoosterFree(bst)); Check(FB_BoosterFree(old)); return FB_DatasetFree(train);
}

int TaskSaveBinary(const Config& cfg, const std::string& params) {
  if (cfg.data.empty()) Log::Fatal("task=save_binary needs data=<file>");
  DatasetHandle d = nullptr; Check(FB_DatasetCreateFromFile(cfg.data.c_str(), params.c_str(), nullptr, &d));
  const std::string out = cfg.data + ".bin";
  Check(FB_DatasetSaveBinary(d, out.c_str()));
  Log::Info("Saved the binned data set to %s", out.c_str());
  return FB_DatasetFree(d);
}

}  // namespace

int main(int argc, char** argv) {
  try {
    if (argc < 2) {
      std::printf("usage: %s config=<file> [key=value ...]\n  tasks: train | predict | convert_model | refit | save_binary\n", argv[0]);
      return 1;
    }
    auto m = LoadParameters(argc, argv);
    int has_cuda = 0; FB_CudaAvailable(&has_cuda);
    Config cfg; cfg.Set(m, has_cuda != 0);
    const std::string params = ToParamString(m);
    const std::string task = ToLower(cfg.task);
    if (task == "train" || task == "training") return TaskTrain(cfg, params);
    if (task == "predict" || task == "prediction" || task == "test") return TaskPredict(cfg, params);
    if (task == "convert_model") return TaskConvertModel(cfg);
    if (task == "refit" || task == "refit_tree") return TaskRefit(cfg, params);
    if (task == "save_binary") return TaskSaveBinary(cfg, params);
    Log::Fatal("Unknown task %s", cfg.task.c_str());
  } catch (const std::exception& e) {
    std::fprintf(stderr, "[Fatal] %s\n", e.what());
    return 1;
  }
  return 0;
}
