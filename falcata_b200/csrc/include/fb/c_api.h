/* C API of the falcata_b200 core, consumed by the Python layer through ctypes.
 * Every function returns 0 on success and -1 on error; FB_GetLastError() gives the message.
 * Parity: include/Falcata/c_api.h (FLC_Dataset*, FLC_Booster*, FLC_Network* families), src/c_api.cpp.
 * dtype codes: 0 f32, 1 f64, 2 i8, 3 i16, 4 u8, 5 u16, 6 f16, 7 i32.
 * predict_type: 0 normal, 1 raw score, 2 leaf index, 3 feature contributions. */
#ifndef FB_C_API_H_
#define FB_C_API_H_
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* DatasetHandle;
typedef void* BoosterHandle;

const char* FB_GetLastError();
int FB_RegisterLogCallback(void (*callback)(const char*));
int FB_CudaAvailable(int* out);
int FB_ResolveParamInt(const char* parameters, const char* name, int* out);
int FB_SetTimeTag(int enabled);
// Host worker threads of the OpenMP loops (bin finding, label scans, host learners). <= 0: leave as is.
int FB_SetLastErrorForCompat(const char* message);   /* records `message` as the last error and returns -1 (used by fb/c_api_compat.h) */
int FB_SetNumThreads(int num_threads);
int FB_GetNumThreads(int* out);
int FB_GetTimeTagReport(int64_t buffer_len, int64_t* out_len, char* out_str);

/* Host collectives supplied by the embedding process (torch.distributed in the Python layer). */
/* Host collectives over TCP: `machines` = "host:port,host:port,..." (or "host port" lines), this process is the entry that is
   local and listens on local_listen_port; listen_time_out in minutes. */
int FB_NetworkInit(const char* machines, int local_listen_port, int listen_time_out, int num_machines);
int FB_NetworkInitWithFunctions(int num_machines, int rank, void* allreduce_sum_fn, void* allgather_fn);
int FB_NetworkFree();

/* ---- Dataset ---- */
int FB_DatasetCreateFromMat(const void* data, int dtype, int32_t nrow, int32_t ncol, int is_row_major, const char* parameters,
                            const DatasetHandle reference, DatasetHandle* out);
int FB_DatasetCreateFromFile(const char* filename, const char* parameters, const DatasetHandle reference, DatasetHandle* out);
/* Schema only (bin mappers + bundles) from a dense f64 sample; rows are attached afterwards. */
int FB_DatasetCreateFromSample(const double* sample, int32_t num_sample_row, int32_t ncol, int64_t num_total_row, const char* parameters,
                               const int32_t* categorical, int32_t num_categorical, DatasetHandle* out);
// The sample in its own element type (DType code): no widening to double on the way in.
int FB_DatasetCreateFromSampleTyped(const void* sample, int dtype, int32_t num_sample_row, int32_t ncol, int64_t num_total_row, const char* parameters,
                                    const int32_t* categorical, int32_t num_categorical, DatasetHandle* out);
int FB_DatasetCreateByReference(const DatasetHandle reference, DatasetHandle* out);
int FB_DatasetSerializeSchema(DatasetHandle handle, int64_t buffer_len, int64_t* out_len, char* out);
int FB_DatasetCreateFromSchema(const char* schema, int64_t len, const char* parameters, DatasetHandle* out);
int FB_DatasetInitRows(DatasetHandle handle, int32_t nrow, int64_t global_row_offset, int64_t global_num_row, int host_bins);
int FB_DatasetPushRows(DatasetHandle handle, const void* data, int dtype, int32_t nrow, int32_t ncol, int is_row_major, int32_t start_row);
/* Bin a dense device matrix on the GPU; the binned rows stay on the device. */
int FB_DatasetBinDeviceMat(DatasetHandle handle, const void* device_data, int dtype, int32_t nrow, int32_t ncol, int is_row_major, int keep_host_copy);
// Rows [start_row, start_row + nrow) of a total_rows data set from a device-resident row-major chunk (first chunk: start_row 0).
/* A whole Dataset from a dense device matrix: sample gathered on the device, bin boundaries on the host, rows binned on the device. */
int FB_DatasetCreateFromDeviceMat(const void* device_data, int dtype, int32_t nrow, int32_t ncol, int is_row_major, const char* parameters,
                                  const DatasetHandle reference, DatasetHandle* out);
int FB_DatasetBinDeviceChunk(DatasetHandle handle, const void* device_data, int dtype, int32_t nrow, int32_t ncol, int32_t start_row, int32_t total_rows);
int FB_DatasetSetField(DatasetHandle handle, const char* field_name, const void* data, int64_t num_element, int dtype);
int FB_DatasetGetField(DatasetHandle handle, const char* field_name, int64_t* out_len, const void** out_ptr, int* out_type);
int FB_DatasetGetNumData(DatasetHandle handle, int32_t* out);
int FB_DatasetGetNumFeature(DatasetHandle handle, int32_t* out);
int FB_DatasetGetInfo(DatasetHandle handle, int32_t* out /* [num_used_features, num_groups, num_total_bin, max_group_bin, has_device, has_host] */);
int FB_DatasetSetFeatureNames(DatasetHandle handle, const char** names, int num);
int FB_DatasetGetFeatureNames(DatasetHandle handle, int64_t buffer_len, int64_t* out_len, char* out /* '\n' joined */);
int FB_DatasetGetBinnedRow(DatasetHandle handle, int32_t row, int32_t* out_feature_bins /* num_used_features */);
int FB_DatasetSaveBinary(DatasetHandle handle, const char* filename);
int FB_DatasetGetSubset(const DatasetHandle handle, const int32_t* used_row_indices, int32_t num_used_row_indices, DatasetHandle* out);
int FB_DatasetFreeDeviceData(DatasetHandle handle);
int FB_DatasetFeatureNumBin(DatasetHandle handle, int feature, int* out);
int FB_DatasetFree(DatasetHandle handle);

/* ---- Booster ---- */
int FB_BoosterCreate(const DatasetHandle train_data, const char* parameters, BoosterHandle* out);
int FB_BoosterCreateFromModelfile(const char* filename, int* out_num_iterations, BoosterHandle* out);
int FB_BoosterLoadModelFromString(const char* model_str, int64_t len, int* out_num_iterations, BoosterHandle* out);
int FB_BoosterCreateFromBinary(const char* data, int64_t len, int* out_num_iterations, BoosterHandle* out);
int FB_BoosterFree(BoosterHandle handle);
int FB_BoosterAddValidData(BoosterHandle handle, const DatasetHandle valid_data);
int FB_BoosterResetParameter(BoosterHandle handle, const char* parameters);
int FB_BoosterUpdateOneIter(BoosterHandle handle, int* is_finished);
/* grad/hess: host pointers, or device pointers when on_device != 0 (CUDA boosters). */
int FB_BoosterUpdateOneIterCustom(BoosterHandle handle, const float* grad, const float* hess, int on_device, int* is_finished);
int FB_BoosterRollbackOneIter(BoosterHandle handle);
int FB_BoosterGetCurrentIteration(BoosterHandle handle, int* out);
int FB_BoosterNumModelPerIteration(BoosterHandle handle, int* out);
int FB_BoosterNumberOfTotalModel(BoosterHandle handle, int* out);
int FB_BoosterGetNumClasses(BoosterHandle handle, int* out);
int FB_BoosterGetNumFeature(BoosterHandle handle, int* out);
int FB_BoosterGetEvalCounts(BoosterHandle handle, int* out);
int FB_BoosterGetEvalNames(BoosterHandle handle, int64_t buffer_len, int64_t* out_len, char* out /* '\n' joined, with a leading +/- for higher/lower better */);
int FB_BoosterGetEval(BoosterHandle handle, int data_idx, int* out_len, double* out_results);
int FB_BoosterGetNumPredict(BoosterHandle handle, int data_idx, int64_t* out_len);
int FB_BoosterGetPredict(BoosterHandle handle, int data_idx, int64_t* out_len, double* out_result);
int FB_BoosterGetTrainScoreDevicePtr(BoosterHandle handle, void** out_ptr);
int FB_BoosterCalcNumPredict(BoosterHandle handle, int num_row, int predict_type, int start_iteration, int num_iteration, int64_t* out_len);
int FB_BoosterPredictForMat(BoosterHandle handle, const void* data, int dtype, int32_t nrow, int32_t ncol, int is_row_major, int predict_type,
                            int start_iteration, int num_iteration, const char* parameter, int64_t* out_len, double* out_result);
/* Device traversal predict: data and out_result are device pointers (out: f32, class-major when raw/normal). */
int FB_BoosterPredictForFile(BoosterHandle handle, const char* data_filename, int data_has_header, int predict_type, int start_iteration,
                             int num_iteration, const char* parameter, const char* result_filename);
int FB_BoosterPredictForDeviceMat(BoosterHandle handle, const void* device_data, int dtype, int32_t nrow, int32_t ncol, int is_row_major,
                                  int predict_type, int start_iteration, int num_iteration, float* out_device);
int FB_BoosterSaveModel(BoosterHandle handle, int start_iteration, int num_iteration, int feature_importance_type, const char* filename);
int FB_BoosterSaveModelToString(BoosterHandle handle, int start_iteration, int num_iteration, int feature_importance_type, int64_t buffer_len,
                                int64_t* out_len, char* out_str);
int FB_BoosterDumpModel(BoosterHandle handle, int start_iteration, int num_iteration, int feature_importance_type, int64_t buffer_len,
                        int64_t* out_len, char* out_str);
int FB_BoosterModelToIfElse(BoosterHandle handle, int num_iteration, int64_t buffer_len, int64_t* out_len, char* out_str);
int FB_BoosterSaveModelToBinary(BoosterHandle handle, int start_iteration, int num_iteration, int feature_importance_type, int with_stats,
                                int with_diagnostics, int f32_leaves, int compress_level, int64_t buffer_len, int64_t* out_len, char* out);
int FB_BoosterGetLeafValue(BoosterHandle handle, int tree_idx, int leaf_idx, double* out_val);
int FB_BoosterSetLeafValue(BoosterHandle handle, int tree_idx, int leaf_idx, double val);
int FB_BoosterFeatureImportance(BoosterHandle handle, int num_iteration, int importance_type, double* out_results);
int FB_BoosterGetFeatureNames(BoosterHandle handle, int64_t buffer_len, int64_t* out_len, char* out);
int FB_BoosterRefit(BoosterHandle handle, const int32_t* leaf_preds, int32_t nrow, int32_t ncol);
int FB_BoosterMerge(BoosterHandle handle, BoosterHandle other_handle);
int FB_BoosterShuffleModels(BoosterHandle handle, int start_iter, int end_iter);
int FB_BoosterGetUpperBoundValue(BoosterHandle handle, double* out);
int FB_BoosterGetLowerBoundValue(BoosterHandle handle, double* out);
int FB_BoosterGetLoadedParam(BoosterHandle handle, int64_t buffer_len, int64_t* out_len, char* out_str);
int FB_BoosterGpuLaunches(BoosterHandle handle, int64_t* out);
int FB_BoosterStageReport(BoosterHandle handle, int64_t buffer_len, int64_t* out_len, char* out_str);

/* single-row, sparse and introspection entry points */
int FB_BoosterPredictForMatSingleRow(BoosterHandle handle, const void* data, int dtype, int32_t ncol, int is_row_major, int predict_type, int start_iteration,
                                     int num_iteration, const char* parameter, int64_t* out_len, double* out_result);
int FB_BoosterPredictForMatSingleRowFastInit(BoosterHandle handle, int predict_type, int start_iteration, int num_iteration, int dtype, int32_t ncol,
                                             const char* parameter, void** out_fast_config);
int FB_BoosterPredictForMatSingleRowFast(void* fast_config, const void* data, int64_t* out_len, double* out_result);
int FB_FastConfigFree(void* fast_config);
int FB_BoosterPredictForCSR(BoosterHandle handle, const void* indptr, int indptr_type, const int32_t* indices, const void* data, int data_type, int64_t nindptr,
                            int64_t nelem, int64_t num_col, int predict_type, int start_iteration, int num_iteration, const char* parameter, int64_t* out_len,
                            double* out_result);
int FB_DatasetCreateFromCSR(const void* indptr, int indptr_type, const int32_t* indices, const void* data, int data_type, int64_t nindptr, int64_t nelem,
                            int64_t num_col, const char* parameters, const DatasetHandle reference, DatasetHandle* out);
int FB_DatasetCreateFromCSC(const void* col_ptr, int col_ptr_type, const int32_t* indices, const void* data, int data_type, int64_t ncol_ptr, int64_t nelem,
                            int64_t num_row, const char* parameters, const DatasetHandle reference, DatasetHandle* out);
int FB_BoosterPredictForCSC(BoosterHandle handle, const void* col_ptr, int col_ptr_type, const int32_t* indices, const void* data, int data_type, int64_t ncol_ptr,
                            int64_t nelem, int64_t num_row, int predict_type, int start_iteration, int num_iteration, const char* parameter, int64_t* out_len,
                            double* out_result);
int FB_BoosterPredictForMats(BoosterHandle handle, const void** data, int dtype, int32_t nmat, const int32_t* nrow, int32_t ncol, int is_row_major, int predict_type,
                             int start_iteration, int num_iteration, const char* parameter, int64_t* out_len, double* out_result);
int FB_DatasetCreateFromMats(int32_t nmat, const void** data, int dtype, const int32_t* nrow, int32_t ncol, int is_row_major, const char* parameters,
                             const DatasetHandle reference, DatasetHandle* out);
/* streaming ingest: FB_DatasetCreateByReference / ...FromSampleTyped, FB_DatasetInitRows(host_bins=1), then these */
int FB_DatasetInitStreaming(DatasetHandle handle, int32_t has_weights, int32_t has_init_scores, int32_t has_queries, int32_t nclasses);
int FB_DatasetPushRowsWithMetadata(DatasetHandle handle, const void* data, int dtype, int32_t nrow, int32_t ncol, int32_t start_row, const float* label,
                                   const float* weight, const double* init_score, const int32_t* query);
int FB_DatasetMarkFinished(DatasetHandle handle);
/* Arrow C data interface: `chunks` is an array of n_chunks ArrowArray structs (record batches), `schema` one ArrowSchema; both are released */
int FB_DatasetCreateFromArrow(int64_t n_chunks, void* chunks, void* schema, const char* parameters, const DatasetHandle reference, DatasetHandle* out);
/* Arrow C stream interface (`stream`: an ArrowArrayStream*; it is drained and released) and single fields from Arrow */
int FB_DatasetCreateFromArrowStream(void* stream, const char* parameters, const DatasetHandle reference, DatasetHandle* out);
int FB_BoosterPredictForArrowStream(BoosterHandle handle, void* stream, int predict_type, int start_iteration, int num_iteration, const char* parameter,
                                    int64_t* out_len, double* out_result);
int FB_DatasetSetFieldFromArrow(DatasetHandle handle, const char* field_name, int64_t n_chunks, void* chunks, void* schema);
int FB_DatasetSetFieldFromArrowStream(DatasetHandle handle, const char* field_name, void* stream);
int FB_DatasetPushRowsByCSR(DatasetHandle handle, const void* indptr, int indptr_type, const int32_t* indices, const void* data, int data_type, int64_t nindptr,
                            int64_t nelem, int64_t num_col, int64_t start_row);
int FB_DatasetPushRowsByCSRWithMetadata(DatasetHandle handle, const void* indptr, int indptr_type, const int32_t* indices, const void* data, int data_type,
                                        int64_t nindptr, int64_t nelem, int64_t start_row, const float* label, const float* weight, const double* init_score,
                                        const int32_t* query);
int FB_DatasetCreateFromSampledColumn(double** sample_data, int** sample_indices, int32_t ncol, const int* num_per_col, int32_t num_sample_row,
                                      int32_t num_local_row, int64_t num_dist_row, const char* parameters, DatasetHandle* out);
/* get_row_funptr: std::function<void(int row, std::vector<std::pair<int, double>>& out)>* (C++ callers only) */
int FB_DatasetCreateFromCSRFunc(void* get_row_funptr, int num_rows, int64_t num_col, const char* parameters, const DatasetHandle reference, DatasetHandle* out);
int FB_BoosterPredictForCSRSingleRowFastInit(BoosterHandle handle, int predict_type, int start_iteration, int num_iteration, int data_type, int64_t num_col,
                                             const char* parameter, void** out_fast_config);
int FB_BoosterPredictForCSRSingleRowFast(void* fast_config, const void* indptr, int indptr_type, const int32_t* indices, const void* data, int data_type, int64_t nindptr,
                                         int64_t nelem, int64_t* out_len, double* out_result);
int FB_DatasetSerializeReferenceToBinary(DatasetHandle handle, void** out_buffer, int32_t* out_len);
int FB_ByteBufferGetAt(void* buffer, int32_t index, uint8_t* out_val);
int FB_ByteBufferFree(void* buffer);
int FB_DatasetCreateFromSerializedReference(const void* ref_buffer, int32_t ref_buffer_size, int64_t num_row, int32_t num_classes, const char* parameters,
                                            DatasetHandle* out);
/* contributions of CSR rows as CSR (matrix_type 0); the outputs are allocated here, free them with FB_BoosterFreePredictSparse */
int FB_BoosterPredictSparseOutput(BoosterHandle handle, const void* indptr, int indptr_type, const int32_t* indices, const void* data, int data_type, int64_t nindptr,
                                  int64_t nelem, int64_t num_col, int predict_type, int start_iteration, int num_iteration, const char* parameter, int matrix_type,
                                  int64_t* out_len, void** out_indptr, int32_t** out_indices, void** out_data);
int FB_BoosterFreePredictSparse(void* indptr, int32_t* indices, void* data);
/* appends the (host-binned) features of `source` behind those of `target`; both hold the same rows */
int FB_DatasetAddFeaturesFrom(DatasetHandle target, DatasetHandle source);
int FB_DatasetUpdateParamChecking(const char* old_parameters, const char* new_parameters);
int FB_BoosterPredictForArrow(BoosterHandle handle, int64_t n_chunks, void* chunks, void* schema, int predict_type, int start_iteration, int num_iteration,
                              const char* parameter, int64_t* out_len, double* out_result);
int FB_GetSampleCount(int32_t num_total_row, const char* parameters, int* out);
int FB_SampleIndices(int32_t num_total_row, const char* parameters, void* out, int32_t* out_len);
int FB_DumpParamAliases(int64_t buffer_len, int64_t* out_len, char* out_str);
int FB_BoosterValidateFeatureNames(BoosterHandle handle, const char** data_names, int data_num_features);
int FB_BoosterResetTrainingData(BoosterHandle handle, const DatasetHandle train_data);
int FB_BoosterGetLinear(BoosterHandle handle, int* out);
int FB_DatasetGetFeatureNumBin(DatasetHandle handle, int feature, int* out);
int FB_DatasetDumpText(DatasetHandle handle, const char* filename);
int FB_SetLastError(const char* msg);
int FB_GetMaxThreads(int* out);
int FB_SetMaxThreads(int num_threads);

#ifdef __cplusplus
}
#endif
#endif  /* FB_C_API_H_ */
