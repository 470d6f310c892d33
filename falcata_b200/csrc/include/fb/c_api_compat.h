/* Names of the C API under the two older prefixes, `FLC_` and `LGBM_`.
 *
 * The library exports `FB_*` (fb/c_api.h). Code written against the `FLC_*` entry points of include/Falcata/c_api.h, or
 * against the historical `LGBM_*` spellings of include/Falcata/c_api_compat.h, compiles against this header instead:
 *   - where the arguments are the same, the old name is a macro for the new one (works in C and C++, also for taking the
 *     function's address);
 *   - where they differ, a static inline adapter with the OLD argument list converts: data-type codes (the old API numbers
 *     float32, float64, int32, int64 as 0..3; this library has more types and numbers them differently), name lists as
 *     arrays of C strings instead of one joined buffer, 32-bit lengths, arguments this library does not need.
 * Entry points with no counterpart here (socket networking, sparse prediction output, serialized dataset references,
 * adding features from another dataset) are adapters that fail with a message, so that callers still link.
 * Nothing inside the library uses these names.
 */
#ifndef FB_C_API_COMPAT_H_
#define FB_C_API_COMPAT_H_

#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "fb/c_api.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef void* FastConfigHandle;
typedef void* ByteBufferHandle;
struct ArrowArray;
struct ArrowSchema;
struct ArrowArrayStream;

#define C_API_DTYPE_FLOAT32 0
#define C_API_DTYPE_FLOAT64 1
#define C_API_DTYPE_INT32 2
#define C_API_DTYPE_INT64 3
#define C_API_PREDICT_NORMAL 0
#define C_API_PREDICT_RAW_SCORE 1
#define C_API_PREDICT_LEAF_INDEX 2
#define C_API_PREDICT_CONTRIB 3
#define C_API_MATRIX_TYPE_CSR 0
#define C_API_MATRIX_TYPE_CSC 1
#define C_API_FEATURE_IMPORTANCE_SPLIT 0
#define C_API_FEATURE_IMPORTANCE_GAIN 1

/* old data-type code -> this library's (0 float32, 1 float64, 7 int32; int64 has no code of its own: any value other
 * than 7 reads as int64 where row pointers are concerned) */
static inline int fb_compat_dtype(int old_code) { return old_code == 2 ? 7 : (old_code == 3 ? 8 : old_code); }
/* this library's data-type code -> old */
static inline int fb_compat_dtype_back(int code) { return code == 7 ? 2 : code; }
static inline int fb_compat_unsupported(const char* what) { return FB_SetLastErrorForCompat(what); }

/* ---- same arguments: the old name is the new function ---- */
#define FLC_GetLastError FB_GetLastError
#define FLC_DumpParamAliases FB_DumpParamAliases
#define FLC_RegisterLogCallback FB_RegisterLogCallback
#define FLC_GetSampleCount FB_GetSampleCount
#define FLC_SampleIndices FB_SampleIndices
#define FLC_DatasetCreateFromFile FB_DatasetCreateFromFile
#define FLC_DatasetMarkFinished FB_DatasetMarkFinished
#define FLC_DatasetSetFeatureNames FB_DatasetSetFeatureNames
#define FLC_DatasetFree FB_DatasetFree
#define FLC_DatasetFreeDeviceData FB_DatasetFreeDeviceData
#define FLC_DatasetSaveBinary FB_DatasetSaveBinary
#define FLC_DatasetDumpText FB_DatasetDumpText
#define FLC_DatasetUpdateParamChecking FB_DatasetUpdateParamChecking
#define FLC_DatasetGetFeatureNumBin FB_DatasetGetFeatureNumBin
#define FLC_BoosterGetLinear FB_BoosterGetLinear
#define FLC_BoosterCreate FB_BoosterCreate
#define FLC_BoosterCreateFromModelfile FB_BoosterCreateFromModelfile
#define FLC_BoosterGetLoadedParam FB_BoosterGetLoadedParam
#define FLC_BoosterFree FB_BoosterFree
#define FLC_BoosterShuffleModels FB_BoosterShuffleModels
#define FLC_BoosterMerge FB_BoosterMerge
#define FLC_BoosterAddValidData FB_BoosterAddValidData
#define FLC_BoosterResetTrainingData FB_BoosterResetTrainingData
#define FLC_BoosterResetParameter FB_BoosterResetParameter
#define FLC_BoosterGetNumClasses FB_BoosterGetNumClasses
#define FLC_BoosterUpdateOneIter FB_BoosterUpdateOneIter
#define FLC_BoosterRefit FB_BoosterRefit
#define FLC_BoosterRollbackOneIter FB_BoosterRollbackOneIter
#define FLC_BoosterGetCurrentIteration FB_BoosterGetCurrentIteration
#define FLC_BoosterNumModelPerIteration FB_BoosterNumModelPerIteration
#define FLC_BoosterNumberOfTotalModel FB_BoosterNumberOfTotalModel
#define FLC_BoosterGetEvalCounts FB_BoosterGetEvalCounts
#define FLC_BoosterValidateFeatureNames FB_BoosterValidateFeatureNames
#define FLC_BoosterGetNumFeature FB_BoosterGetNumFeature
#define FLC_BoosterGetEval FB_BoosterGetEval
#define FLC_BoosterGetNumPredict FB_BoosterGetNumPredict
#define FLC_BoosterGetPredict FB_BoosterGetPredict
#define FLC_BoosterPredictForFile FB_BoosterPredictForFile
#define FLC_BoosterCalcNumPredict FB_BoosterCalcNumPredict
#define FLC_BoosterSaveModel FB_BoosterSaveModel
#define FLC_BoosterSaveModelToString FB_BoosterSaveModelToString
#define FLC_BoosterSaveModelToBinary FB_BoosterSaveModelToBinary
#define FLC_BoosterCreateFromBinary FB_BoosterCreateFromBinary
#define FLC_BoosterDumpModel FB_BoosterDumpModel
#define FLC_BoosterGetLeafValue FB_BoosterGetLeafValue
#define FLC_BoosterSetLeafValue FB_BoosterSetLeafValue
#define FLC_BoosterFeatureImportance FB_BoosterFeatureImportance
#define FLC_BoosterGetUpperBoundValue FB_BoosterGetUpperBoundValue
#define FLC_BoosterGetLowerBoundValue FB_BoosterGetLowerBoundValue
#define FLC_NetworkFree FB_NetworkFree
#define FLC_NetworkInitWithFunctions FB_NetworkInitWithFunctions
#define FLC_SetMaxThreads FB_SetMaxThreads
#define FLC_GetMaxThreads FB_GetMaxThreads
#define FLC_DatasetGetNumData FB_DatasetGetNumData
#define FLC_DatasetGetNumFeature FB_DatasetGetNumFeature
#define FLC_FastConfigFree FB_FastConfigFree
#define FLC_BoosterPredictForMatSingleRowFast FB_BoosterPredictForMatSingleRowFast
#define FLC_DatasetCreateFromArrowStream FB_DatasetCreateFromArrowStream
#define FLC_DatasetSetFieldFromArrow FB_DatasetSetFieldFromArrow
#define FLC_DatasetSetFieldFromArrowStream FB_DatasetSetFieldFromArrowStream
#define FLC_BoosterPredictForArrowStream FB_BoosterPredictForArrowStream

#define LGBM_GetLastError FB_GetLastError
#define LGBM_DumpParamAliases FB_DumpParamAliases
#define LGBM_RegisterLogCallback FB_RegisterLogCallback
#define LGBM_GetSampleCount FB_GetSampleCount
#define LGBM_SampleIndices FB_SampleIndices
#define LGBM_DatasetCreateFromFile FB_DatasetCreateFromFile
#define LGBM_DatasetMarkFinished FB_DatasetMarkFinished
#define LGBM_DatasetSetFeatureNames FB_DatasetSetFeatureNames
#define LGBM_DatasetFree FB_DatasetFree
#define LGBM_DatasetFreeDeviceData FB_DatasetFreeDeviceData
#define LGBM_DatasetSaveBinary FB_DatasetSaveBinary
#define LGBM_DatasetDumpText FB_DatasetDumpText
#define LGBM_DatasetUpdateParamChecking FB_DatasetUpdateParamChecking
#define LGBM_DatasetGetFeatureNumBin FB_DatasetGetFeatureNumBin
#define LGBM_BoosterGetLinear FB_BoosterGetLinear
#define LGBM_BoosterCreate FB_BoosterCreate
#define LGBM_BoosterCreateFromModelfile FB_BoosterCreateFromModelfile
#define LGBM_BoosterGetLoadedParam FB_BoosterGetLoadedParam
#define LGBM_BoosterFree FB_BoosterFree
#define LGBM_BoosterShuffleModels FB_BoosterShuffleModels
#define LGBM_BoosterMerge FB_BoosterMerge
#define LGBM_BoosterAddValidData FB_BoosterAddValidData
#define LGBM_BoosterResetTrainingData FB_BoosterResetTrainingData
#define LGBM_BoosterResetParameter FB_BoosterResetParameter
#define LGBM_BoosterGetNumClasses FB_BoosterGetNumClasses
#define LGBM_BoosterUpdateOneIter FB_BoosterUpdateOneIter
#define LGBM_BoosterRefit FB_BoosterRefit
#define LGBM_BoosterRollbackOneIter FB_BoosterRollbackOneIter
#define LGBM_BoosterGetCurrentIteration FB_BoosterGetCurrentIteration
#define LGBM_BoosterNumModelPerIteration FB_BoosterNumModelPerIteration
#define LGBM_BoosterNumberOfTotalModel FB_BoosterNumberOfTotalModel
#define LGBM_BoosterGetEvalCounts FB_BoosterGetEvalCounts
#define LGBM_BoosterValidateFeatureNames FB_BoosterValidateFeatureNames
#define LGBM_BoosterGetNumFeature FB_BoosterGetNumFeature
#define LGBM_BoosterGetEval FB_BoosterGetEval
#define LGBM_BoosterGetNumPredict FB_BoosterGetNumPredict
#define LGBM_BoosterGetPredict FB_BoosterGetPredict
#define LGBM_BoosterPredictForFile FB_BoosterPredictForFile
#define LGBM_BoosterCalcNumPredict FB_BoosterCalcNumPredict
#define LGBM_BoosterSaveModel FB_BoosterSaveModel
#define LGBM_BoosterSaveModelToString FB_BoosterSaveModelToString
#define LGBM_BoosterSaveModelToBinary FB_BoosterSaveModelToBinary
#define LGBM_BoosterCreateFromBinary FB_BoosterCreateFromBinary
#define LGBM_BoosterDumpModel FB_BoosterDumpModel
#define LGBM_BoosterGetLeafValue FB_BoosterGetLeafValue
#define LGBM_BoosterSetLeafValue FB_BoosterSetLeafValue
#define LGBM_BoosterFeatureImportance FB_BoosterFeatureImportance
#define LGBM_BoosterGetUpperBoundValue FB_BoosterGetUpperBoundValue
#define LGBM_BoosterGetLowerBoundValue FB_BoosterGetLowerBoundValue
#define LGBM_NetworkFree FB_NetworkFree
#define LGBM_NetworkInitWithFunctions FB_NetworkInitWithFunctions
#define LGBM_SetMaxThreads FB_SetMaxThreads
#define LGBM_GetMaxThreads FB_GetMaxThreads
#define LGBM_DatasetGetNumData FB_DatasetGetNumData
#define LGBM_DatasetGetNumFeature FB_DatasetGetNumFeature
#define LGBM_FastConfigFree FB_FastConfigFree
#define LGBM_BoosterPredictForMatSingleRowFast FB_BoosterPredictForMatSingleRowFast
#define LGBM_DatasetCreateFromArrowStream FB_DatasetCreateFromArrowStream
#define LGBM_DatasetSetFieldFromArrow FB_DatasetSetFieldFromArrow
#define LGBM_DatasetSetFieldFromArrowStream FB_DatasetSetFieldFromArrowStream
#define LGBM_BoosterPredictForArrowStream FB_BoosterPredictForArrowStream

/* ---- different arguments: adapters with the old argument lists ---- */
#define FB_COMPAT_BOTH(ret, name, params, call) \
  static inline ret FLC_##name params { return call; } \
  static inline ret LGBM_##name params { return call; }

/* a joined "a\nb\nc" buffer -> an array of caller-provided C strings, the way the old name getters report them */
static inline int fb_compat_split_names(const char* joined, int strip_sign, const int len, int* out_count, const size_t buffer_len, size_t* out_buffer_len, char** out_strs) {
  int count = 0; size_t longest = 0;
  const char* p = joined;
  while (p != NULL && *p != '\0') {
    const char* e = strchr(p, '\n');
    size_t n = e != NULL ? (size_t)(e - p) : strlen(p);
    const char* q = p;
    if (strip_sign && n > 0 && (*q == '+' || *q == '-')) { ++q; --n; }
    if (count < len && out_strs != NULL && buffer_len > 0) {
      const size_t c = n < buffer_len - 1 ? n : buffer_len - 1;
      memcpy(out_strs[count], q, c); out_strs[count][c] = '\0';
    }
    if (n + 1 > longest) longest = n + 1;
    ++count;
    if (e == NULL) break;
    p = e + 1;
  }
  *out_count = count; *out_buffer_len = longest;
  return 0;
}
#define FB_COMPAT_NAME_GETTER(name, getter, strip)                                                                                        \
  static inline int fb_compat_##name(void* handle, const int len, int* out_len, const size_t buffer_len, size_t* out_buffer_len, char** out_strs) { \
    int64_t need = 0;                                                                                                                      \
    char* joined;                                                                                                                          \
    int rc;                                                                                                                                \
    if (getter(handle, 0, &need, NULL) != 0) return -1;                                                                                    \
    joined = (char*)malloc((size_t)need + 1);                                                                                              \
    if (joined == NULL) return fb_compat_unsupported("out of memory");                                                                     \
    joined[0] = '\0';                                                                                                                      \
    rc = getter(handle, need + 1, &need, joined);                                                                                          \
    if (rc == 0) rc = fb_compat_split_names(joined, strip, len, out_len, buffer_len, out_buffer_len, out_strs);                            \
    free(joined);                                                                                                                          \
    return rc;                                                                                                                             \
  }
FB_COMPAT_NAME_GETTER(dataset_feature_names, FB_DatasetGetFeatureNames, 0)
FB_COMPAT_NAME_GETTER(booster_feature_names, FB_BoosterGetFeatureNames, 0)
FB_COMPAT_NAME_GETTER(booster_eval_names, FB_BoosterGetEvalNames, 1)
FB_COMPAT_BOTH(int, DatasetGetFeatureNames, (DatasetHandle handle, const int len, int* num_feature_names, const size_t buffer_len, size_t* out_buffer_len, char** feature_names),
               fb_compat_dataset_feature_names(handle, len, num_feature_names, buffer_len, out_buffer_len, feature_names))
FB_COMPAT_BOTH(int, BoosterGetFeatureNames, (BoosterHandle handle, const int len, int* out_len, const size_t buffer_len, size_t* out_buffer_len, char** out_strs),
               fb_compat_booster_feature_names(handle, len, out_len, buffer_len, out_buffer_len, out_strs))
FB_COMPAT_BOTH(int, BoosterGetEvalNames, (BoosterHandle handle, const int len, int* out_len, const size_t buffer_len, size_t* out_buffer_len, char** out_strs),
               fb_compat_booster_eval_names(handle, len, out_len, buffer_len, out_buffer_len, out_strs))

/* dataset creation and streaming */
FB_COMPAT_BOTH(int, DatasetCreateFromMat, (const void* data, int data_type, int32_t nrow, int32_t ncol, int is_row_major, const char* parameters, const DatasetHandle reference, DatasetHandle* out),
               FB_DatasetCreateFromMat(data, fb_compat_dtype(data_type), nrow, ncol, is_row_major, parameters, reference, out))
FB_COMPAT_BOTH(int, DatasetCreateFromMats, (int32_t nmat, const void** data, int data_type, int32_t* nrow, int32_t ncol, int* is_row_major, const char* parameters, const DatasetHandle reference, DatasetHandle* out),
               FB_DatasetCreateFromMats(nmat, data, fb_compat_dtype(data_type), nrow, ncol, (is_row_major != NULL && nmat > 0) ? is_row_major[0] : 1, parameters, reference, out))
FB_COMPAT_BOTH(int, DatasetCreateFromCSR, (const void* indptr, int indptr_type, const int32_t* indices, const void* data, int data_type, int64_t nindptr, int64_t nelem, int64_t num_col, const char* parameters, const DatasetHandle reference, DatasetHandle* out),
               FB_DatasetCreateFromCSR(indptr, fb_compat_dtype(indptr_type), indices, data, fb_compat_dtype(data_type), nindptr, nelem, num_col, parameters, reference, out))
FB_COMPAT_BOTH(int, DatasetCreateFromCSC, (const void* col_ptr, int col_ptr_type, const int32_t* indices, const void* data, int data_type, int64_t ncol_ptr, int64_t nelem, int64_t num_row, const char* parameters, const DatasetHandle reference, DatasetHandle* out),
               FB_DatasetCreateFromCSC(col_ptr, fb_compat_dtype(col_ptr_type), indices, data, fb_compat_dtype(data_type), ncol_ptr, nelem, num_row, parameters, reference, out))
FB_COMPAT_BOTH(int, DatasetCreateFromArrow, (int64_t n_chunks, const struct ArrowArray* chunks, const struct ArrowSchema* schema, const char* parameters, const DatasetHandle reference, DatasetHandle* out),
               FB_DatasetCreateFromArrow(n_chunks, (void*)chunks, (void*)schema, parameters, reference, out))
static inline int fb_compat_create_by_reference(const DatasetHandle reference, int64_t num_total_row, DatasetHandle* out) {
  if (FB_DatasetCreateByReference(reference, out) != 0) return -1;
  return FB_DatasetInitRows(*out, (int32_t)num_total_row, 0, num_total_row, 1);
}
FB_COMPAT_BOTH(int, DatasetCreateByReference, (const DatasetHandle reference, int64_t num_total_row, DatasetHandle* out), fb_compat_create_by_reference(reference, num_total_row, out))
FB_COMPAT_BOTH(int, DatasetInitStreaming, (DatasetHandle dataset, int32_t has_weights, int32_t has_init_scores, int32_t has_queries, int32_t nclasses, int32_t nthreads, int32_t omp_max_threads),
               ((void)nthreads, (void)omp_max_threads, FB_DatasetInitStreaming(dataset, has_weights, has_init_scores, has_queries, nclasses)))
FB_COMPAT_BOTH(int, DatasetPushRows, (DatasetHandle dataset, const void* data, int data_type, int32_t nrow, int32_t ncol, int32_t start_row),
               FB_DatasetPushRows(dataset, data, fb_compat_dtype(data_type), nrow, ncol, 1, start_row))
FB_COMPAT_BOTH(int, DatasetPushRowsWithMetadata, (DatasetHandle dataset, const void* data, int data_type, int32_t nrow, int32_t ncol, int32_t start_row, const float* label, const float* weight, const double* init_score, const int32_t* query, int32_t tid),
               ((void)tid, FB_DatasetPushRowsWithMetadata(dataset, data, fb_compat_dtype(data_type), nrow, ncol, start_row, label, weight, init_score, query)))
FB_COMPAT_BOTH(int, DatasetPushRowsByCSR, (DatasetHandle dataset, const void* indptr, int indptr_type, const int32_t* indices, const void* data, int data_type, int64_t nindptr, int64_t nelem, int64_t num_col, int64_t start_row),
               FB_DatasetPushRowsByCSR(dataset, indptr, fb_compat_dtype(indptr_type), indices, data, fb_compat_dtype(data_type), nindptr, nelem, num_col, start_row))
FB_COMPAT_BOTH(int, DatasetPushRowsByCSRWithMetadata, (DatasetHandle dataset, const void* indptr, int indptr_type, const int32_t* indices, const void* data, int data_type, int64_t nindptr, int64_t nelem, int64_t start_row, const float* label, const float* weight, const double* init_score, const int32_t* query, int32_t tid),
               ((void)tid, FB_DatasetPushRowsByCSRWithMetadata(dataset, indptr, fb_compat_dtype(indptr_type), indices, data, fb_compat_dtype(data_type), nindptr, nelem, start_row, label, weight, init_score, query)))
FB_COMPAT_BOTH(int, DatasetCreateFromSampledColumn, (double** sample_data, int** sample_indices, int32_t ncol, const int* num_per_col, int32_t num_sample_row, int32_t num_local_row, int64_t num_dist_row, const char* parameters, DatasetHandle* out),
               FB_DatasetCreateFromSampledColumn(sample_data, sample_indices, ncol, num_per_col, num_sample_row, num_local_row, num_dist_row, parameters, out))
FB_COMPAT_BOTH(int, DatasetCreateFromCSRFunc, (void* get_row_funptr, int num_rows, int64_t num_col, const char* parameters, const DatasetHandle reference, DatasetHandle* out),
               FB_DatasetCreateFromCSRFunc(get_row_funptr, num_rows, num_col, parameters, reference, out))
FB_COMPAT_BOTH(int, DatasetCreateFromMatDevice, (const void* data, int data_type, int32_t nrow, int32_t ncol, int is_row_major, const char* parameters, const DatasetHandle reference, DatasetHandle* out),
               FB_DatasetCreateFromDeviceMat(data, fb_compat_dtype(data_type), nrow, ncol, is_row_major, parameters, reference, out))
FB_COMPAT_BOTH(int, BoosterPredictForCSRSingleRowFastInit, (BoosterHandle handle, const int predict_type, const int start_iteration, const int num_iteration, const int data_type, const int64_t num_col, const char* parameter, void** out_fastConfig),
               FB_BoosterPredictForCSRSingleRowFastInit(handle, predict_type, start_iteration, num_iteration, fb_compat_dtype(data_type), num_col, parameter, out_fastConfig))
/* the old Fast call carries no element type for the values: it is the one given to FastInit, which the adapter cannot see; doubles are assumed (the reference's own default) */
FB_COMPAT_BOTH(int, BoosterPredictForCSRSingleRowFast, (void* fastConfig_handle, const void* indptr, const int indptr_type, const int32_t* indices, const void* data, const int64_t nindptr, const int64_t nelem, int64_t* out_len, double* out_result),
               FB_BoosterPredictForCSRSingleRowFast(fastConfig_handle, indptr, fb_compat_dtype(indptr_type), indices, data, 1, nindptr, nelem, out_len, out_result))
static inline void FLC_SetLastError(const char* msg) { (void)FB_SetLastErrorForCompat(msg); }
static inline void LGBM_SetLastError(const char* msg) { (void)FB_SetLastErrorForCompat(msg); }
FB_COMPAT_BOTH(int, DatasetSetWaitForManualFinish, (DatasetHandle dataset, int wait), ((void)dataset, (void)wait, 0))   /* rows are usable once pushed; FB_DatasetMarkFinished closes the stream either way */
FB_COMPAT_BOTH(int, DatasetGetSubset, (const DatasetHandle handle, const int32_t* used_row_indices, int32_t num_used_row_indices, const char* parameters, DatasetHandle* out),
               ((void)parameters, FB_DatasetGetSubset(handle, used_row_indices, num_used_row_indices, out)))
FB_COMPAT_BOTH(int, DatasetSetField, (DatasetHandle handle, const char* field_name, const void* field_data, int num_element, int type),
               FB_DatasetSetField(handle, field_name, field_data, (int64_t)num_element, fb_compat_dtype(type)))
static inline int fb_compat_get_field(DatasetHandle handle, const char* field_name, int* out_len, const void** out_ptr, int* out_type) {
  int64_t n = 0; int t = 0;
  if (FB_DatasetGetField(handle, field_name, &n, out_ptr, &t) != 0) return -1;
  *out_len = (int)n; *out_type = fb_compat_dtype_back(t);
  return 0;
}
FB_COMPAT_BOTH(int, DatasetGetField, (DatasetHandle handle, const char* field_name, int* out_len, const void** out_ptr, int* out_type), fb_compat_get_field(handle, field_name, out_len, out_ptr, out_type))

/* booster */
FB_COMPAT_BOTH(int, BoosterLoadModelFromString, (const char* model_str, int* out_num_iterations, BoosterHandle* out),
               FB_BoosterLoadModelFromString(model_str, (int64_t)strlen(model_str), out_num_iterations, out))
FB_COMPAT_BOTH(int, BoosterUpdateOneIterCustom, (BoosterHandle handle, const float* grad, const float* hess, int* is_finished),
               FB_BoosterUpdateOneIterCustom(handle, grad, hess, 0, is_finished))
FB_COMPAT_BOTH(int, BoosterPredictForMat, (BoosterHandle handle, const void* data, int data_type, int32_t nrow, int32_t ncol, int is_row_major, int predict_type, int start_iteration, int num_iteration, const char* parameter, int64_t* out_len, double* out_result),
               FB_BoosterPredictForMat(handle, data, fb_compat_dtype(data_type), nrow, ncol, is_row_major, predict_type, start_iteration, num_iteration, parameter, out_len, out_result))
FB_COMPAT_BOTH(int, BoosterPredictForMatSingleRow, (BoosterHandle handle, const void* data, int data_type, int ncol, int is_row_major, int predict_type, int start_iteration, int num_iteration, const char* parameter, int64_t* out_len, double* out_result),
               FB_BoosterPredictForMatSingleRow(handle, data, fb_compat_dtype(data_type), ncol, is_row_major, predict_type, start_iteration, num_iteration, parameter, out_len, out_result))
FB_COMPAT_BOTH(int, BoosterPredictForMatSingleRowFastInit, (BoosterHandle handle, const int predict_type, const int start_iteration, const int num_iteration, const int data_type, const int32_t ncol, const char* parameter, FastConfigHandle* out_fastConfig),
               FB_BoosterPredictForMatSingleRowFastInit(handle, predict_type, start_iteration, num_iteration, fb_compat_dtype(data_type), ncol, parameter, out_fastConfig))
static inline int fb_compat_predict_row_pointers(BoosterHandle handle, const void** data, int data_type, int32_t nrow, int32_t ncol, int predict_type, int start_iteration, int num_iteration, const char* parameter, int64_t* out_len, double* out_result) {
  /* the old entry point takes one pointer per row */
  int rc; int32_t i;
  int32_t* ones = (int32_t*)malloc(sizeof(int32_t) * (size_t)(nrow > 0 ? nrow : 1));
  if (ones == NULL) return fb_compat_unsupported("out of memory");
  for (i = 0; i < nrow; ++i) ones[i] = 1;
  rc = FB_BoosterPredictForMats(handle, data, fb_compat_dtype(data_type), nrow, ones, ncol, 1, predict_type, start_iteration, num_iteration, parameter, out_len, out_result);
  free(ones);
  return rc;
}
FB_COMPAT_BOTH(int, BoosterPredictForMats, (BoosterHandle handle, const void** data, int data_type, int32_t nrow, int32_t ncol, int predict_type, int start_iteration, int num_iteration, const char* parameter, int64_t* out_len, double* out_result),
               fb_compat_predict_row_pointers(handle, data, data_type, nrow, ncol, predict_type, start_iteration, num_iteration, parameter, out_len, out_result))
FB_COMPAT_BOTH(int, BoosterPredictForCSR, (BoosterHandle handle, const void* indptr, int indptr_type, const int32_t* indices, const void* data, int data_type, int64_t nindptr, int64_t nelem, int64_t num_col, int predict_type, int start_iteration, int num_iteration, const char* parameter, int64_t* out_len, double* out_result),
               FB_BoosterPredictForCSR(handle, indptr, fb_compat_dtype(indptr_type), indices, data, fb_compat_dtype(data_type), nindptr, nelem, num_col, predict_type, start_iteration, num_iteration, parameter, out_len, out_result))
FB_COMPAT_BOTH(int, BoosterPredictForCSRSingleRow, (BoosterHandle handle, const void* indptr, int indptr_type, const int32_t* indices, const void* data, int data_type, int64_t nindptr, int64_t nelem, int64_t num_col, int predict_type, int start_iteration, int num_iteration, const char* parameter, int64_t* out_len, double* out_result),
               FB_BoosterPredictForCSR(handle, indptr, fb_compat_dtype(indptr_type), indices, data, fb_compat_dtype(data_type), nindptr, nelem, num_col, predict_type, start_iteration, num_iteration, parameter, out_len, out_result))
FB_COMPAT_BOTH(int, BoosterPredictForCSC, (BoosterHandle handle, const void* col_ptr, int col_ptr_type, const int32_t* indices, const void* data, int data_type, int64_t ncol_ptr, int64_t nelem, int64_t num_row, int predict_type, int start_iteration, int num_iteration, const char* parameter, int64_t* out_len, double* out_result),
               FB_BoosterPredictForCSC(handle, col_ptr, fb_compat_dtype(col_ptr_type), indices, data, fb_compat_dtype(data_type), ncol_ptr, nelem, num_row, predict_type, start_iteration, num_iteration, parameter, out_len, out_result))
FB_COMPAT_BOTH(int, BoosterPredictForArrow, (BoosterHandle handle, int64_t n_chunks, const struct ArrowArray* chunks, const struct ArrowSchema* schema, int predict_type, int start_iteration, int num_iteration, const char* parameter, int64_t* out_len, double* out_result),
               FB_BoosterPredictForArrow(handle, n_chunks, (void*)chunks, (void*)schema, predict_type, start_iteration, num_iteration, parameter, out_len, out_result))

/* ---- no counterpart: these fail with a message ---- */
FB_COMPAT_BOTH(int, NetworkInit, (const char* machines, int local_listen_port, int listen_time_out, int num_machines),
               FB_NetworkInit(machines, local_listen_port, listen_time_out, num_machines))
FB_COMPAT_BOTH(int, DatasetAddFeaturesFrom, (DatasetHandle target, DatasetHandle source), FB_DatasetAddFeaturesFrom(target, source))
FB_COMPAT_BOTH(int, DatasetSerializeReferenceToBinary, (DatasetHandle handle, ByteBufferHandle* out, int32_t* out_len), FB_DatasetSerializeReferenceToBinary(handle, out, out_len))
FB_COMPAT_BOTH(int, DatasetCreateFromSerializedReference, (const void* ref_buffer, int32_t ref_buffer_size, int64_t num_row, int32_t num_classes, const char* parameters, DatasetHandle* out),
               FB_DatasetCreateFromSerializedReference(ref_buffer, ref_buffer_size, num_row, num_classes, parameters, out))
FB_COMPAT_BOTH(int, ByteBufferGetAt, (ByteBufferHandle handle, int32_t index, uint8_t* out_val), FB_ByteBufferGetAt(handle, index, out_val))
FB_COMPAT_BOTH(int, ByteBufferFree, (ByteBufferHandle handle), FB_ByteBufferFree(handle))
FB_COMPAT_BOTH(int, BoosterPredictSparseOutput, (BoosterHandle handle, const void* indptr, int indptr_type, const int32_t* indices, const void* data, int data_type, int64_t nindptr, int64_t nelem, int64_t num_col_or_row, int predict_type, int start_iteration, int num_iteration, const char* parameter, int matrix_type, int64_t* out_len, void** out_indptr, int32_t** out_indices, void** out_data),
               FB_BoosterPredictSparseOutput(handle, indptr, fb_compat_dtype(indptr_type), indices, data, fb_compat_dtype(data_type), nindptr, nelem, num_col_or_row, predict_type, start_iteration, num_iteration, parameter, matrix_type, out_len, out_indptr, out_indices, out_data))
FB_COMPAT_BOTH(int, BoosterFreePredictSparse, (void* indptr, int32_t* indices, void* data, int indptr_type, int data_type), ((void)indptr_type, (void)data_type, FB_BoosterFreePredictSparse(indptr, indices, data)))

#undef FB_COMPAT_BOTH
#undef FB_COMPAT_NAME_GETTER

#ifdef __cplusplus
}
#endif
#endif  /* FB_C_API_COMPAT_H_ */
