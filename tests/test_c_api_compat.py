"""The `FLC_*` / `LGBM_*` names of fb/c_api_compat.h: a C program and a C++ program written against the old argument
lists compile, link against the library and train, predict and read names through them."""
import os
import shutil
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
INC = ROOT / "falcata_b200" / "csrc" / "include"

PROGRAM = r"""
#include <stdio.h>
#include <stdlib.h>
#include <math.h>
#include "fb/c_api_compat.h"
#ifdef __cplusplus
#include <functional>
#include <utility>
#include <vector>
#endif

#define CHECK(x) do { if ((x) != 0) { printf("FAILED %s: %s\n", #x, PFX(GetLastError)()); return 1; } } while (0)

int main(void) {
  enum { N = 600, F = 4 };
  static double X[N * F]; static float y[N];
  unsigned s = 12345u; int i, j;
  DatasetHandle ds = NULL, ds2 = NULL; BoosterHandle bst = NULL, loaded = NULL;
  int fin = 0, n = 0, niter = 0, nnames = 0, flen = 0, ftype = -1; int64_t out_len = 0; size_t need = 0;
  double pred[N]; double single[1]; char* names[8]; char namebuf[8][64]; const void* fptr = NULL;
  const char* feature_names[F] = {"alpha", "beta", "gamma", "delta"};
  for (i = 0; i < N; ++i) { double t = 0; for (j = 0; j < F; ++j) { s = s * 1664525u + 1013904223u; X[i * F + j] = (double)(s >> 8) / 16777216.0 - 0.5; } t = X[i * F] + 0.5 * X[i * F + 1]; y[i] = (float)t; }
  CHECK(PFX(DatasetCreateFromMat)(X, C_API_DTYPE_FLOAT64, N, F, 1, "max_bin=63 min_data_in_bin=1", NULL, &ds));
  CHECK(PFX(DatasetSetField)(ds, "label", y, N, C_API_DTYPE_FLOAT32));
  CHECK(PFX(DatasetSetFeatureNames)(ds, feature_names, F));
  CHECK(PFX(DatasetGetNumData)(ds, &n)); if (n != N) { printf("rows %d\n", n); return 1; }
  CHECK(PFX(DatasetGetField)(ds, "label", &flen, &fptr, &ftype)); if (flen != N || ftype != C_API_DTYPE_FLOAT32) { printf("field %d %d\n", flen, ftype); return 1; }
  for (i = 0; i < 8; ++i) names[i] = namebuf[i];
  CHECK(PFX(DatasetGetFeatureNames)(ds, 8, &nnames, 64, &need, names)); if (nnames != F || strcmp(names[2], "gamma") != 0) { printf("names %d %s\n", nnames, names[2]); return 1; }
  CHECK(PFX(BoosterCreate)(ds, "objective=regression num_leaves=7 min_data_in_leaf=5 verbosity=-1 metric=l2", &bst));
  for (i = 0; i < 20; ++i) CHECK(PFX(BoosterUpdateOneIter)(bst, &fin));
  CHECK(PFX(BoosterGetEvalNames)(bst, 8, &nnames, 64, &need, names)); if (nnames != 1 || strcmp(names[0], "l2") != 0) { printf("eval names %d %s\n", nnames, names[0]); return 1; }
  CHECK(PFX(BoosterPredictForMat)(bst, X, C_API_DTYPE_FLOAT64, N, F, 1, C_API_PREDICT_NORMAL, 0, -1, "", &out_len, pred)); if (out_len != N) return 1;
  { double err = 0; for (i = 0; i < N; ++i) err += (pred[i] - y[i]) * (pred[i] - y[i]); if (err / N > 0.01) { printf("mse %g\n", err / N); return 1; } }
  CHECK(PFX(BoosterPredictForMatSingleRow)(bst, X + 5 * F, C_API_DTYPE_FLOAT64, F, 1, C_API_PREDICT_NORMAL, 0, -1, "", &out_len, single)); if (fabs(single[0] - pred[5]) > 1e-12) return 1;
  {
    const void* rows[3]; double three[3];
    rows[0] = X; rows[1] = X + F; rows[2] = X + 2 * F;
    CHECK(PFX(BoosterPredictForMats)(bst, rows, C_API_DTYPE_FLOAT64, 3, F, C_API_PREDICT_NORMAL, 0, -1, "", &out_len, three)); if (out_len != 3 || fabs(three[2] - pred[2]) > 1e-12) return 1;
  }
  {
    /* two rows as CSR with 32-bit and 64-bit row pointers */
    int32_t ip32[3] = {0, 2, 4}; int64_t ip64[3] = {0, 2, 4}; int32_t idx[4] = {0, 1, 0, 1}; double val[4]; double two[2], dense[2 * F] = {0}; double want[2];
    val[0] = 0.25; val[1] = -0.125; val[2] = -0.3; val[3] = 0.2;
    dense[0] = 0.25; dense[1] = -0.125; dense[F] = -0.3; dense[F + 1] = 0.2;
    CHECK(PFX(BoosterPredictForMat)(bst, dense, C_API_DTYPE_FLOAT64, 2, F, 1, C_API_PREDICT_NORMAL, 0, -1, "", &out_len, want));
    CHECK(PFX(BoosterPredictForCSR)(bst, ip32, C_API_DTYPE_INT32, idx, val, C_API_DTYPE_FLOAT64, 3, 4, F, C_API_PREDICT_NORMAL, 0, -1, "", &out_len, two)); if (fabs(two[0] - want[0]) + fabs(two[1] - want[1]) > 1e-12) return 1;
    CHECK(PFX(BoosterPredictForCSR)(bst, ip64, C_API_DTYPE_INT64, idx, val, C_API_DTYPE_FLOAT64, 3, 4, F, C_API_PREDICT_NORMAL, 0, -1, "", &out_len, two)); if (fabs(two[0] - want[0]) + fabs(two[1] - want[1]) > 1e-12) return 1;
  }
  {
    int64_t len = 0; char* model;
    CHECK(PFX(BoosterSaveModelToString)(bst, 0, -1, C_API_FEATURE_IMPORTANCE_SPLIT, 0, &len, NULL));
    model = (char*)malloc((size_t)len); CHECK(PFX(BoosterSaveModelToString)(bst, 0, -1, C_API_FEATURE_IMPORTANCE_SPLIT, len, &len, model));
    CHECK(PFX(BoosterLoadModelFromString)(model, &niter, &loaded)); if (niter != 20) { printf("iterations %d\n", niter); return 1; }
    free(model);
  }
  /* streaming: a dataset by reference, rows pushed in two blocks */
  CHECK(PFX(DatasetCreateByReference)(ds, N, &ds2));
  CHECK(PFX(DatasetInitStreaming)(ds2, 0, 0, 0, 1, 1, 1));
  CHECK(PFX(DatasetPushRows)(ds2, X, C_API_DTYPE_FLOAT64, N / 2, F, 0));
  CHECK(PFX(DatasetPushRows)(ds2, X + (N / 2) * F, C_API_DTYPE_FLOAT64, N - N / 2, F, N / 2));
  CHECK(PFX(DatasetMarkFinished)(ds2));
  CHECK(PFX(DatasetGetNumData)(ds2, &n)); if (n != N) return 1;
  {
    /* prepared single-row prediction from a CSR row, a dataset from per-column samples with CSR rows and metadata pushed into it */
    void* fast = NULL; int32_t ip[2] = {0, 2}; int32_t idx[2] = {0, 1}; double val[2] = {0.25, -0.125}; double one[1], dense[F] = {0}, want[1];
    DatasetHandle ds3 = NULL; double* cols[F]; int* rows_of[F]; int per_col[F]; static double cv[F][N]; static int cr[F][N];
    static int32_t sip[N + 1]; static int32_t sidx[N * F]; static double sval[N * F]; const void* lptr = NULL;
    dense[0] = 0.25; dense[1] = -0.125;
    CHECK(PFX(BoosterPredictForMat)(bst, dense, C_API_DTYPE_FLOAT64, 1, F, 1, C_API_PREDICT_NORMAL, 0, -1, "", &out_len, want));
    CHECK(PFX(BoosterPredictForCSRSingleRowFastInit)(bst, C_API_PREDICT_NORMAL, 0, -1, C_API_DTYPE_FLOAT64, F, "", &fast));
    CHECK(PFX(BoosterPredictForCSRSingleRowFast)(fast, ip, C_API_DTYPE_INT32, idx, val, 2, 2, &out_len, one)); if (out_len != 1 || fabs(one[0] - want[0]) > 1e-12) { printf("csr fast %g %g\n", one[0], want[0]); return 1; }
    CHECK(FB_FastConfigFree(fast));
    for (j = 0; j < F; ++j) { per_col[j] = N; cols[j] = cv[j]; rows_of[j] = cr[j]; for (i = 0; i < N; ++i) { cv[j][i] = X[i * F + j]; cr[j][i] = i; } }
    CHECK(PFX(DatasetCreateFromSampledColumn)(cols, rows_of, F, per_col, N, N, N, "max_bin=63 min_data_in_bin=1", &ds3));
    CHECK(PFX(DatasetInitStreaming)(ds3, 0, 0, 0, 1, 1, 1));
    for (i = 0; i < N; ++i) { sip[i] = i * F; for (j = 0; j < F; ++j) { sidx[i * F + j] = j; sval[i * F + j] = X[i * F + j]; } }
    sip[N] = N * F;
    CHECK(PFX(DatasetPushRowsByCSRWithMetadata)(ds3, sip, C_API_DTYPE_INT32, sidx, sval, C_API_DTYPE_FLOAT64, N + 1, N * F, 0, y, NULL, NULL, NULL, 0));
    CHECK(PFX(DatasetMarkFinished)(ds3));
    CHECK(PFX(DatasetGetField)(ds3, "label", &flen, &lptr, &ftype)); if (flen != N || ((const float*)lptr)[7] != y[7]) { printf("streamed label\n"); return 1; }
    {
      /* the streamed dataset trains to the same model as the one-shot dataset (same bins, same rows) */
      BoosterHandle b3 = NULL; double p3[N];
      CHECK(PFX(BoosterCreate)(ds3, "objective=regression num_leaves=7 min_data_in_leaf=5 verbosity=-1 metric=l2", &b3));
      for (i = 0; i < 20; ++i) CHECK(PFX(BoosterUpdateOneIter)(b3, &fin));
      CHECK(PFX(BoosterPredictForMat)(b3, X, C_API_DTYPE_FLOAT64, N, F, 1, C_API_PREDICT_NORMAL, 0, -1, "", &out_len, p3));
      for (i = 0; i < N; ++i) if (fabs(p3[i] - pred[i]) > 1e-12) { printf("streamed model differs at %d: %g %g\n", i, p3[i], pred[i]); return 1; }
      CHECK(PFX(BoosterFree)(b3));
    }
    CHECK(PFX(DatasetFree)(ds3));
#ifdef __cplusplus
    {
      /* rows from a callback (C++ callers): the same bins and rows as the dense matrix */
      DatasetHandle ds4 = NULL; int n4 = 0;
      std::function<void(int, std::vector<std::pair<int, double>>&)> get_row = [&](int r, std::vector<std::pair<int, double>>& out) {
        out.clear(); for (int c = 0; c < F; ++c) out.emplace_back(c, X[r * F + c]); };
      CHECK(PFX(DatasetCreateFromCSRFunc)(&get_row, N, F, "max_bin=63 min_data_in_bin=1", ds, &ds4));
      CHECK(PFX(DatasetGetNumData)(ds4, &n4)); if (n4 != N) { printf("callback rows %d\n", n4); return 1; }
      CHECK(PFX(DatasetFree)(ds4));
    }
#endif
    {
      /* a serialized reference read back byte by byte gives an empty dataset with the same bins; rows are then pushed */
      ByteBufferHandle bb = NULL; int32_t blen = 0; uint8_t* copy; DatasetHandle ds5 = NULL; int n5 = 0, nf5 = 0;
      CHECK(PFX(DatasetSerializeReferenceToBinary)(ds, &bb, &blen)); if (blen <= 0) { printf("empty reference\n"); return 1; }
      copy = (uint8_t*)malloc((size_t)blen);
      for (i = 0; i < blen; ++i) CHECK(PFX(ByteBufferGetAt)(bb, i, &copy[i]));
      CHECK(PFX(ByteBufferFree)(bb));
      CHECK(PFX(DatasetCreateFromSerializedReference)(copy, blen, N, 1, "max_bin=63", &ds5));
      free(copy);
      CHECK(PFX(DatasetInitStreaming)(ds5, 0, 0, 0, 1, 1, 1));
      CHECK(PFX(DatasetPushRowsWithMetadata)(ds5, X, C_API_DTYPE_FLOAT64, N, F, 0, y, NULL, NULL, NULL, 0));
      CHECK(PFX(DatasetMarkFinished)(ds5));
      CHECK(PFX(DatasetGetNumData)(ds5, &n5)); CHECK(PFX(DatasetGetNumFeature)(ds5, &nf5)); if (n5 != N || nf5 != F) { printf("reference dataset %d x %d\n", n5, nf5); return 1; }
      CHECK(PFX(DatasetFree)(ds5));
    }
    {
      /* feature contributions of two CSR rows as CSR: the stored values add up to the raw prediction of each row */
      int32_t ip[3] = {0, 2, 4}; int32_t idx[4] = {0, 1, 0, 1}; double val[4] = {0.25, -0.125, -0.3, 0.2}; double dense[2 * F] = {0}, raw[2];
      int64_t lens[2] = {0, 0}; void* optr = NULL; int32_t* oidx = NULL; void* odat = NULL; double sum0 = 0, sum1 = 0; int64_t k;
      dense[0] = 0.25; dense[1] = -0.125; dense[F] = -0.3; dense[F + 1] = 0.2;
      CHECK(PFX(BoosterPredictForMat)(bst, dense, C_API_DTYPE_FLOAT64, 2, F, 1, C_API_PREDICT_RAW_SCORE, 0, -1, "", &out_len, raw));
      CHECK(PFX(BoosterPredictSparseOutput)(bst, ip, C_API_DTYPE_INT32, idx, val, C_API_DTYPE_FLOAT64, 3, 4, F, C_API_PREDICT_CONTRIB, 0, -1, "", C_API_MATRIX_TYPE_CSR, lens, &optr, &oidx, &odat));
      if (lens[1] != 3 || lens[0] <= 0 || ((int32_t*)optr)[2] != lens[0]) { printf("sparse output shape %lld %lld\n", (long long)lens[0], (long long)lens[1]); return 1; }
      for (k = ((int32_t*)optr)[0]; k < ((int32_t*)optr)[1]; ++k) sum0 += ((double*)odat)[k];
      for (k = ((int32_t*)optr)[1]; k < ((int32_t*)optr)[2]; ++k) { if (oidx[k] < 0 || oidx[k] > F) return 1; sum1 += ((double*)odat)[k]; }
      if (fabs(sum0 - raw[0]) > 1e-9 || fabs(sum1 - raw[1]) > 1e-9) { printf("contributions %g %g against %g %g\n", sum0, sum1, raw[0], raw[1]); return 1; }
      CHECK(PFX(BoosterFreePredictSparse)(optr, oidx, odat, C_API_DTYPE_INT32, C_API_DTYPE_FLOAT64));
      {
        /* the same two rows as CSC, contributions back as CSC: F + 1 output columns, row indices below 2, the same total */
        int32_t cp[F + 1] = {0, 2, 4, 4, 4}; int32_t ridx[4] = {0, 1, 0, 1}; double cval[4] = {0.25, -0.3, -0.125, 0.2}; double total = 0;
        CHECK(PFX(BoosterPredictSparseOutput)(bst, cp, C_API_DTYPE_INT32, ridx, cval, C_API_DTYPE_FLOAT64, F + 1, 4, 2, C_API_PREDICT_CONTRIB, 0, -1, "", C_API_MATRIX_TYPE_CSC, lens, &optr, &oidx, &odat));
        if (lens[1] != F + 2) { printf("csc pointer length %lld\n", (long long)lens[1]); return 1; }
        for (k = 0; k < lens[0]; ++k) { if (oidx[k] < 0 || oidx[k] > 1) return 1; total += ((double*)odat)[k]; }
        if (fabs(total - raw[0] - raw[1]) > 1e-9) { printf("csc contributions %g against %g\n", total, raw[0] + raw[1]); return 1; }
        CHECK(PFX(BoosterFreePredictSparse)(optr, oidx, odat, C_API_DTYPE_INT32, C_API_DTYPE_FLOAT64));
      }
      if (PFX(BoosterPredictSparseOutput)(bst, ip, C_API_DTYPE_INT32, idx, val, C_API_DTYPE_FLOAT64, 3, 4, F, C_API_PREDICT_NORMAL, 0, -1, "", C_API_MATRIX_TYPE_CSR, lens, &optr, &oidx, &odat) == 0) { printf("sparse output of plain predictions should be refused\n"); return 1; }
    }
    PFX(SetLastError)("set by the caller"); if (strcmp(PFX(GetLastError)(), "set by the caller") != 0) { printf("last error\n"); return 1; }
  }
  CHECK(PFX(NetworkInit)("127.0.0.1:1", 1, 1, 1));   /* one machine: nothing to connect */
  if (PFX(NetworkInit)("127.0.0.1:1", 1, 1, 2) == 0) { printf("NetworkInit with a one-entry list for two machines should fail\n"); return 1; }
  if (PFX(DatasetUpdateParamChecking)("max_bin=63", "max_bin=15") == 0) { printf("a changed max_bin should be refused\n"); return 1; }
  CHECK(PFX(DatasetUpdateParamChecking)("max_bin=63", "max_bin=63 learning_rate=0.3"));
  CHECK(PFX(BoosterFree)(loaded)); CHECK(PFX(BoosterFree)(bst)); CHECK(PFX(DatasetFree)(ds2)); CHECK(PFX(DatasetFree)(ds));
  printf("ok\n");
  return 0;
}
"""


def _lib_path():
    sys.path.insert(0, str(ROOT))
    from falcata_b200.libpath import find_lib_path

    return Path(find_lib_path())


@pytest.mark.parametrize("prefix", ["FLC_", "LGBM_"])
@pytest.mark.parametrize("compiler,suffix", [("gcc", ".c"), ("g++", ".cpp")])
def test_old_names_compile_link_and_run(tmp_path, prefix, compiler, suffix):
    if shutil.which(compiler) is None:
        pytest.skip(f"{compiler} is not installed")
    lib = _lib_path()
    src = tmp_path / ("prog" + suffix)
    src.write_text(f"#define PFX(name) {prefix}##name\n" + PROGRAM)
    exe = tmp_path / "prog"
    cmd = [compiler, "-O1", "-Wall", "-Werror", "-Wno-unused-function", "-I", str(INC), str(src), "-o", str(exe), str(lib), "-lm", f"-Wl,-rpath,{lib.parent}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
    env = dict(os.environ, LD_LIBRARY_PATH=f"{lib.parent}:{os.environ.get('LD_LIBRARY_PATH', '')}")
    r = subprocess.run([str(exe)], capture_output=True, text=True, env=env, timeout=120)
    assert r.returncode == 0 and r.stdout.strip().endswith("ok"), r.stdout[-2000:] + r.stderr[-2000:]
