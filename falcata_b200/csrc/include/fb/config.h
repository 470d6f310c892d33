// Flat parameter struct with alias normalisation, typed parsing, cross-checks and
// a ToString() dump for the model file.
//
// Parity: include/Falcata/config.h (parameter names, defaults, aliases),
// src/io/config.cpp:L273-649 (Set, ResolveFalcataParams, CheckParamConflict).
// The table below is the single source of truth: one line per parameter.
#pragma once
#include <string>
#include <unordered_map>
#include <vector>
#include "fb/common.h"

namespace fb {

// X(type, name, default, "alias1,alias2")
#define FB_CONFIG_PARAMS(X) \
  X(std::string, task, "train", "task_type") \
  X(std::string, objective, "regression", "objective_type,app,application,loss") \
  X(std::string, boosting, "gbdt", "boosting_type,boost") \
  X(std::string, data_sample_strategy, "bagging", "") \
  X(std::string, data, "", "train,train_data,train_data_file,data_filename") \
  X(std::string, valid, "", "test,valid_data,valid_data_file,test_data,test_data_file,valid_filenames") \
  X(int, num_iterations, 100, "num_iteration,n_iter,num_tree,num_trees,num_round,num_rounds,nrounds,num_boost_round,n_estimators,max_iter") \
  X(double, learning_rate, 0.1, "shrinkage_rate,eta") \
  X(int, num_leaves, 31, "num_leaf,max_leaves,max_leaf,max_leaf_nodes") \
  X(std::string, tree_learner, "serial", "tree,tree_type,tree_learner_type") \
  X(int, num_threads, 0, "num_thread,nthread,nthreads,n_jobs") \
  X(std::string, device_type, "", "device") \
  X(int, seed, 0, "random_seed,random_state") \
  X(bool, deterministic, false, "") \
  X(int, max_depth, -1, "") \
  X(int, min_data_in_leaf, 20, "min_data_per_leaf,min_data,min_child_samples,min_samples_leaf") \
  X(double, min_sum_hessian_in_leaf, 1e-3, "min_sum_hessian_per_leaf,min_sum_hessian,min_hessian,min_child_weight") \
  X(double, bagging_fraction, 1.0, "sub_row,subsample,bagging") \
  X(double, pos_bagging_fraction, 1.0, "pos_sub_row,pos_subsample,pos_bagging") \
  X(double, neg_bagging_fraction, 1.0, "neg_sub_row,neg_subsample,neg_bagging") \
  X(int, bagging_freq, 0, "subsample_freq") \
  X(int, bagging_seed, 3, "bagging_fraction_seed") \
  X(bool, bagging_by_query, false, "") \
  X(double, feature_fraction, 1.0, "sub_feature,colsample_bytree") \
  X(double, feature_fraction_bynode, 1.0, "sub_feature_bynode,colsample_bynode") \
  X(int, feature_fraction_seed, 2, "") \
  X(bool, extra_trees, false, "extra_tree") \
  X(int, extra_seed, 6, "") \
  X(int, early_stopping_round, 0, "early_stopping_rounds,early_stopping,n_iter_no_change") \
  X(double, early_stopping_min_delta, 0.0, "") \
  X(bool, first_metric_only, false, "") \
  X(double, max_delta_step, 0.0, "max_tree_output,max_leaf_output") \
  X(double, lambda_l1, 0.0, "reg_alpha,l1_regularization") \
  X(double, lambda_l2, 0.0, "reg_lambda,lambda,l2_regularization") \
  X(double, linear_lambda, 0.0, "") \
  X(double, min_gain_to_split, 0.0, "min_split_gain") \
  X(double, drop_rate, 0.1, "rate_drop") \
  X(int, max_drop, 50, "") \
  X(double, skip_drop, 0.5, "") \
  X(bool, xgboost_dart_mode, false, "") \
  X(bool, uniform_drop, false, "") \
  X(int, drop_seed, 4, "") \
  X(double, top_rate, 0.2, "") \
  X(double, other_rate, 0.1, "") \
  X(int, min_data_per_group, 100, "") \
  X(int, max_cat_threshold, 32, "") \
  X(double, cat_l2, 10.0, "") \
  X(double, cat_smooth, 10.0, "") \
  X(int, max_cat_to_onehot, 4, "") \
  X(int, top_k, 20, "topk") \
  X(std::string, monotone_constraints, "", "mc,monotone_constraint,monotonic_cst") \
  X(std::string, monotone_constraints_method, "basic", "monotone_constraining_method,mc_method") \
  X(double, monotone_penalty, 0.0, "monotone_splits_penalty,ms_penalty,mc_penalty") \
  X(std::string, feature_contri, "", "feature_contrib,fc,fp,feature_penalty") \
  X(std::string, forcedsplits_filename, "", "fs,forced_splits_filename,forced_splits_file,forced_splits") \
  X(double, refit_decay_rate, 0.9, "") \
  X(double, cegb_tradeoff, 1.0, "") \
  X(double, cegb_penalty_split, 0.0, "") \
  X(std::string, cegb_penalty_feature_lazy, "", "") \
  X(std::string, cegb_penalty_feature_coupled, "", "") \
  X(bool, force_col_wise, false, "") \
  X(bool, force_row_wise, false, "") \
  X(double, histogram_pool_size, -1.0, "hist_pool_size") \
  X(std::string, parser_config_file, "", "") \
  X(bool, precise_float_parser, false, "") \
  X(int, file_load_progress_interval_bytes, 0, "") \
  X(double, path_smooth, 0.0, "") \
  X(std::string, interaction_constraints, "", "") \
  X(int, verbosity, 1, "verbose") \
  X(std::string, input_model, "", "model_input,model_in") \
  X(std::string, output_model, "Falcata_model.txt", "model_output,model_out") \
  X(int, saved_feature_importance_type, 0, "") \
  X(int, snapshot_freq, -1, "save_period") \
  X(bool, use_quantized_grad, false, "") \
  X(std::string, quant_mode, "auto", "") \
  X(int, quant_bins, 0, "num_grad_quant_bins") \
  X(bool, quant_train_renew_leaf, false, "") \
  X(bool, stochastic_rounding, true, "") \
  X(bool, linear_tree, false, "linear_trees") \
  X(int, max_bin, 255, "max_bins") \
  X(std::string, max_bin_by_feature, "", "") \
  X(int, min_data_in_bin, 3, "") \
  X(int, bin_construct_sample_cnt, 200000, "subsample_for_bin") \
  X(int, data_random_seed, 1, "data_seed") \
  X(bool, is_enable_sparse, true, "is_sparse,enable_sparse,sparse") \
  X(bool, enable_bundle, true, "is_enable_bundle,bundle") \
  X(bool, use_missing, true, "") \
  X(bool, zero_as_missing, false, "") \
  X(bool, feature_pre_filter, true, "") \
  X(bool, pre_partition, false, "is_pre_partition") \
  X(bool, distributed_bin_finding, false, "") \
  X(bool, two_round, false, "two_round_loading,use_two_round_loading") \
  X(bool, header, false, "has_header") \
  X(std::string, label_column, "", "label") \
  X(std::string, weight_column, "", "weight") \
  X(std::string, group_column, "", "group,group_id,query_column,query,query_id") \
  X(std::string, ignore_column, "", "ignore_feature,blacklist") \
  X(std::string, categorical_feature, "", "cat_feature,categorical_column,cat_column,categorical_features") \
  X(std::string, forcedbins_filename, "", "") \
  X(bool, save_binary, false, "is_save_binary,is_save_binary_file") \
  X(int, start_iteration_predict, 0, "") \
  X(int, num_iteration_predict, -1, "") \
  X(bool, predict_raw_score, false, "is_predict_raw_score,predict_rawscore,raw_score") \
  X(bool, predict_leaf_index, false, "is_predict_leaf_index,leaf_index") \
  X(bool, predict_contrib, false, "is_predict_contrib,contrib") \
  X(bool, predict_disable_shape_check, false, "") \
  X(bool, pred_early_stop, false, "") \
  X(int, pred_early_stop_freq, 10, "") \
  X(double, pred_early_stop_margin, 10.0, "") \
  X(std::string, output_result, "Falcata_predict_result.txt", "predict_result,prediction_result,predict_name,prediction_name,pred_name,name_pred") \
  X(std::string, convert_model_language, "", "") \
  X(std::string, convert_model, "gbdt_prediction.cpp", "convert_model_file") \
  X(int, objective_seed, 5, "") \
  X(int, num_class, 1, "num_classes") \
  X(bool, is_unbalance, false, "unbalance,unbalanced_sets") \
  X(double, scale_pos_weight, 1.0, "") \
  X(double, sigmoid, 1.0, "") \
  X(bool, boost_from_average, true, "") \
  X(bool, reg_sqrt, false, "") \
  X(double, alpha, 0.9, "") \
  X(double, fair_c, 1.0, "") \
  X(double, poisson_max_delta_step, 0.7, "") \
  X(double, tweedie_variance_power, 1.5, "") \
  X(int, lambdarank_truncation_level, 30, "") \
  X(bool, lambdarank_norm, true, "") \
  X(std::string, label_gain, "", "") \
  X(bool, lambdarank_position_bias_regularization, false, "") \
  X(std::string, metric, "", "metrics,metric_types") \
  X(int, metric_freq, 1, "output_freq") \
  X(bool, is_provide_training_metric, false, "training_metric,is_training_metric,train_metric") \
  X(std::string, eval_at, "1,2,3,4,5", "ndcg_eval_at,ndcg_at,map_eval_at,map_at") \
  X(int, multi_error_top_k, 1, "") \
  X(std::string, auc_mu_weights, "", "") \
  X(int, num_machines, 1, "num_machine") \
  X(int, local_listen_port, 12400, "local_port,port") \
  X(int, time_out, 120, "") \
  X(std::string, machine_list_filename, "", "machine_list_file,machine_list,mlist") \
  X(std::string, machines, "", "workers,nodes") \
  X(int, gpu_platform_id, -1, "") \
  X(int, gpu_device_id, -1, "") \
  X(bool, gpu_use_dp, false, "") \
  X(int, num_gpu, 1, "") \
  X(std::string, gpu_device_id_list, "", "") \
  X(std::string, cuda_precision, "fp64", "") \
  X(std::string, cuda_plan, "auto", "") \
  X(std::string, grow_policy, "level", "") \

enum class QuantMode : int { None = 0, Stochastic = 1, FixedPoint = 2 };

struct Config {
#define FB_DECL(type, name, def, aliases) type name = def;
  FB_CONFIG_PARAMS(FB_DECL)
#undef FB_DECL

  // ---- derived (filled by Resolve) ----
  QuantMode quant = QuantMode::None;
  int quant_bins_resolved = 0;
  bool quant_bins_from_auto = false;   // quant_bins was left at its default: the learner may pick a safer or finer count
  bool is_cuda = false;
  std::vector<double> label_gain_vec;
  std::vector<int> eval_at_vec;
  std::vector<std::string> metric_list;
  std::vector<int8_t> monotone_vec;
  std::vector<double> feature_contri_vec;
  std::vector<int> max_bin_by_feature_vec;
  int num_tree_per_iteration = 1;
  // keys the user set explicitly (post alias normalisation)
  std::unordered_map<std::string, std::string> raw;

  static const std::unordered_map<std::string, std::string>& AliasTable();
  static std::unordered_map<std::string, std::string> Str2Map(const char* parameters);
  static void NormalizeAliases(std::unordered_map<std::string, std::string>* params);
  void Set(const std::unordered_map<std::string, std::string>& params, bool cuda_available);
  void Resolve(bool cuda_available);
  void CheckParamConflict();
  // "[name: value]" lines of the model file's parameters section.
  std::string ToString() const;
  static std::string ParseObjectiveAlias(const std::string& name);
  static std::string ParseMetricAlias(const std::string& name);
};

// ---------------------------------------------------------------- planner ----
// Process-independent set of on/off decisions for performance-only choices,
// grammar "auto[,key:on|off]*" (parity: include/Falcata/falcata_plan.h:L44-258).
// Every key must leave quantized models bit-identical; tests flip each key.
struct Plan {
  bool hist_tc = false;          // root level of the quantized construct on the tensor cores (one-hot tcgen05 instance, 1 GPU)
  bool device_controller = true; // split arbitration on the device (no per-level host decision)
  bool fused_tail = true;        // split search, per-leaf argmax, cross-rank argmax and the level controller in ONE launch
  bool fused_scan = true;        // the partition's scan + child set-up step inside the flags launch (last chunk block of each split)
  bool pack4 = true;             // 4-bit row storage when every group has <= 16 bins
  bool compact_view = true;      // per-tree gather of feature_fraction-sampled columns
  bool gh_in_row = false;        // packed gradient word stored next to the row's bins (measured slower on B200: the separate 4 B/row array stays L2-resident)
  bool hist_lane = true;         // lane-per-group construct with bank-interleaved warp-private tiles (groups with <= 64 bins)
  bool hist_lane_atomic = false; // lane-per-group construct with one shared tile per block and shared atomics
  bool hist_lane_red = true;     // lane construct adds with shared-memory reduction instructions into tiles shared by 8 warps (off: load-add-store with forwarding, a tile per warp)
  bool robust_scale = true;      // fixed-point quantization: outlier-robust gradient scale (changes the model only where it fires: a small outlier cluster above an empty octave)
  bool quant_ef = true;          // fixed-point quantization: int8 error feedback of the rounding residuals from round to round
  bool hist_float_red = false;   // fp32 lane construct with shared-memory reduction adds into shared tiles (off: a tile per warp, load-add-store, sums in row order)
  bool col_major_part = true;    // partition reads the split column from a column-major copy of the bins
  bool bulk_root = true;         // root level of the lane construct staged by bulk asynchronous copies (TMA engine, mbarrier completion)
  static Plan FromString(const std::string& s);
  std::string ToString() const;
};

}  // namespace fb
