"""Model conversion CLI, plotting data helpers and the oblique projection pool (all host side)."""
import os
import subprocess
import sys

import numpy as np
import pytest

import falcata_b200 as fb
from falcata_b200 import plotting
from util import make_binary


@pytest.fixture(scope="module")
def small_model():
    X, y = make_binary(3000, 8)
    res = {}
    ds = fb.Dataset(X[:2400], y[:2400]); dv = ds.create_valid(X[2400:], y[2400:])
    bst = fb.train({"objective": "binary", "num_leaves": 15, "verbosity": -1, "device_type": "cpu", "metric": "binary_logloss,auc"}, ds, 20, valid_sets=[dv],
                   callbacks=[fb.record_evaluation(res)])
    return bst, res, X


def test_convert_cli_round_trip(tmp_path, small_model):
    bst, _, X = small_model
    txt, falb, back = tmp_path / "m.txt", tmp_path / "m.falb", tmp_path / "back.txt"
    bst.save_model(txt)
    for a, b in ((txt, falb), (falb, back)):
        r = subprocess.run([sys.executable, "-m", "falcata_b200", "convert", str(a), str(b)], capture_output=True, text=True)
        assert r.returncode == 0, r.stderr
    assert falb.stat().st_size < txt.stat().st_size
    assert falb.read_bytes()[:4] == b"FALB"
    np.testing.assert_allclose(fb.Booster(model_file=str(back)).predict(X), bst.predict(X))
    np.testing.assert_allclose(fb.Booster(model_file=str(falb)).predict(X), bst.predict(X))


def test_plot_data_helpers(small_model):
    bst, res, X = small_model
    table = plotting.importance_table(bst)
    assert table == sorted(table, key=lambda p: p[1]) and sum(v for _, v in table) == bst.feature_importance().sum()
    used = table[-1][0]
    counts, edges = plotting.split_value_histogram(bst, used)
    assert counts.sum() == dict(table)[used] and len(edges) == len(counts) + 1
    name, curves = plotting.metric_curves(res, "auc")
    assert name == "auc" and len(curves["valid_0"]) == 20
    dot = plotting.tree_to_dot(bst, 0, show_info=["split_gain", "leaf_count"], example_case=X[0])
    assert dot.startswith("digraph") and dot.count("->") == 2 * (dot.count("<=")) and "lightblue" in dot and "leaf_count" in dot
    with pytest.raises(ImportError):
        plotting.plot_importance(bst)   # matplotlib is not part of this environment


def test_oblique_pool(tmp_path):
    rng = np.random.RandomState(0)
    X = rng.randn(4000, 6)
    X[rng.rand(*X.shape) < 0.02] = np.nan
    y = ((np.nan_to_num(X[:, 0]) + np.nan_to_num(X[:, 1]) - np.nan_to_num(X[:, 2])) > 0).astype(np.float64)   # oblique boundary
    pool = fb.ObliquePool(num_projections=64, density=3, seed=17)
    Xa = pool.fit_transform(X)
    assert Xa.shape == (4000, 6 + 64) and not np.isnan(Xa[:, 6:]).any() and len(pool.feature_names()) == 70
    pool.save(tmp_path / "pool.json")
    again = fb.ObliquePool.load(tmp_path / "pool.json")
    np.testing.assert_allclose(again.transform(X), Xa)
    p = {"objective": "binary", "num_leaves": 7, "verbosity": -1, "device_type": "cpu"}
    acc = lambda b, M: float(((b.predict(M[3000:]) > 0.5) == y[3000:]).mean())
    plain = fb.train(p, fb.Dataset(X[:3000], y[:3000]), 15)
    aug = fb.train(p, fb.Dataset(Xa[:3000], y[:3000]), 15)
    assert acc(aug, Xa) >= acc(plain, X) - 0.01


def test_dataset_and_booster_helper_methods():
    rng = np.random.default_rng(0)
    X = rng.normal(size=(600, 4)).astype(np.float32)
    X[:, 3] = 1.0                       # constant column: dropped
    y = (X[:, 0] + X[:, 1] > 0).astype(np.float32)
    ds = fb.Dataset(X, y, params={"max_bin": 15}, free_raw_data=False)
    ds.set_field("weight", np.ones(600, dtype=np.float32)).set_position(np.arange(600) % 5)
    ds.construct()
    assert ds.get_data() is X and ds.get_params() == {"max_bin": 15}
    assert 2 <= ds.feature_num_bin(0) <= 15 and ds.feature_num_bin(3) == 0
    assert ds.get_position().shape == (600,) and ds in ds.get_ref_chain()
    assert ds.get_field("weight").shape == (600,)
    other = fb.Dataset(rng.normal(size=(600, 2)).astype(np.float32), free_raw_data=False)
    ds.add_features_from(other)
    assert ds.construct().num_feature() == 6
    b = fb.train({"objective": "binary", "num_leaves": 7, "verbose": -1, "min_data_in_leaf": 5}, ds, 5)
    hist, edges = b.get_split_value_histogram(0)
    assert hist.sum() >= 1 and len(edges) == len(hist) + 1
    clone = fb.Booster(model_str=fb.train({"objective": "binary", "num_leaves": 3, "verbose": -1}, fb.Dataset(X, y), 1).model_to_string())
    clone.model_from_binary(b.model_to_binary())
    A = np.concatenate([X, rng.normal(size=(600, 2)).astype(np.float32)], axis=1)
    assert np.allclose(clone.predict(A), b.predict(A))


def test_pickle_formats_sequence_input_and_sklearn_extras():
    import pickle
    rng = np.random.default_rng(1)
    X = rng.normal(size=(900, 5)).astype(np.float32)
    y = (X[:, 0] - X[:, 2] > 0).astype(np.float32)

    class Rows(fb.Sequence):
        batch_size = 256

        def __init__(self, a):
            self.a = a

        def __getitem__(self, idx):
            return self.a[idx]

        def __len__(self):
            return len(self.a)

    p = {"objective": "binary", "num_leaves": 7, "verbose": -1, "min_data_in_leaf": 5}
    b_seq = fb.train(p, fb.Dataset([Rows(X[:500]), Rows(X[500:])], y), 5)
    b_arr = fb.train(p, fb.Dataset(X, y), 5)
    assert b_seq.model_to_string() == b_arr.model_to_string()
    assert fb.get_pickle_format() == "falb"
    blob_bin = pickle.dumps(b_arr)
    fb.set_pickle_format("text")
    try:
        blob_txt = pickle.dumps(b_arr)
    finally:
        fb.set_pickle_format("falb")
    assert len(blob_bin) < len(blob_txt)
    for blob in (blob_bin, blob_txt):
        assert np.array_equal(pickle.loads(blob).predict(X), b_arr.predict(X))
    clf = fb.LGBMClassifier(n_estimators=8, num_leaves=7, verbose=-1).fit(X, y)
    assert clf.n_estimators_ == 8 and clf.n_iter_ == 8 and len(clf.feature_names_in_) == 5
    margin = clf.decision_function(X)
    assert np.array_equal(margin > 0, clf.predict(X) == 1)


def test_arrow_table_and_array_chunks_as_input():
    import pyarrow as pa
    rng = np.random.default_rng(4)
    X = rng.normal(size=(700, 4)).astype(np.float64)
    y = (X[:, 0] > 0).astype(np.float32)
    p = {"objective": "binary", "num_leaves": 7, "verbose": -1, "min_data_in_leaf": 5}
    ref = fb.train(p, fb.Dataset(X, y), 4).model_to_string()
    table = pa.table({f"f{i}": X[:, i] for i in range(4)})
    from_arrow = fb.train(p, fb.Dataset(table, y), 4)
    assert from_arrow.feature_name() == ["f0", "f1", "f2", "f3"]
    assert np.array_equal(from_arrow.predict(X), fb.Booster(model_str=ref).predict(X))
    assert fb.train(p, fb.Dataset([X[:300], X[300:]], y), 4).model_to_string() == ref


def test_sparse_input_is_binned_in_blocks_like_the_dense_matrix():
    import scipy.sparse as sps
    rng = np.random.default_rng(6)
    X = rng.normal(size=(5000, 12)).astype(np.float64)
    X[rng.random(X.shape) < 0.8] = 0.0
    y = (X[:, 0] + X[:, 3] - X[:, 7] > 0).astype(np.float32)
    p = {"objective": "binary", "num_leaves": 15, "verbose": -1, "min_data_in_leaf": 5}
    dense = fb.train(p, fb.Dataset(X, y), 6)
    for fmt in (sps.csr_matrix, sps.csc_matrix):
        sp_ds = fb.Dataset(fmt(X), y)
        valid = fb.Dataset(fmt(X[:500]), y[:500], reference=sp_ds)
        ev = {}
        b = fb.train(p, sp_ds, 6, valid_sets=[valid], valid_names=["v"], callbacks=[fb.record_evaluation(ev)])
        assert b.model_to_string() == dense.model_to_string()
        assert len(ev["v"]["binary_logloss"]) == 6


def test_c_api_single_row_csr_and_introspection(tmp_path):
    import ctypes
    import json
    import scipy.sparse as sps
    from falcata_b200.basic import _lib, _param_str

    lib = _lib()
    rng = np.random.default_rng(8)
    X = rng.normal(size=(2000, 6)).astype(np.float64)
    X[rng.random(X.shape) < 0.6] = 0.0
    y = (X[:, 0] - X[:, 2] > 0).astype(np.float32)
    p = {"objective": "binary", "num_leaves": 7, "verbose": -1, "min_data_in_leaf": 5}
    b = fb.train(p, fb.Dataset(X, y), 5)
    ref = b.predict(X)
    # single row, plain and with a prepared configuration
    out = (ctypes.c_double * 1)(); n = ctypes.c_int64(0)
    row = np.ascontiguousarray(X[3])
    assert lib.FB_BoosterPredictForMatSingleRow(b._handle, row.ctypes.data_as(ctypes.c_void_p), 1, 6, 1, 0, 0, -1, b"", ctypes.byref(n), out) == 0
    assert n.value == 1 and abs(out[0] - ref[3]) < 1e-12
    fc = ctypes.c_void_p()
    assert lib.FB_BoosterPredictForMatSingleRowFastInit(b._handle, 0, 0, -1, 1, 6, b"", ctypes.byref(fc)) == 0
    for i in (0, 17, 1999):
        row = np.ascontiguousarray(X[i])
        assert lib.FB_BoosterPredictForMatSingleRowFast(fc, row.ctypes.data_as(ctypes.c_void_p), ctypes.byref(n), out) == 0
        assert abs(out[0] - ref[i]) < 1e-12
    assert lib.FB_FastConfigFree(fc) == 0
    # CSR predict and CSR dataset
    sp = sps.csr_matrix(X)
    indptr = sp.indptr.astype(np.int32); indices = sp.indices.astype(np.int32); data = sp.data.astype(np.float64)
    res = np.zeros(2000, dtype=np.float64)
    assert lib.FB_BoosterPredictForCSR(b._handle, indptr.ctypes.data_as(ctypes.c_void_p), 7, indices.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)),
                                       data.ctypes.data_as(ctypes.c_void_p), 1, ctypes.c_int64(len(indptr)), ctypes.c_int64(len(data)), ctypes.c_int64(6), 0, 0, -1, b"",
                                       ctypes.byref(n), res.ctypes.data_as(ctypes.POINTER(ctypes.c_double))) == 0
    assert n.value == 2000 and np.allclose(res, ref, atol=1e-12)
    h = ctypes.c_void_p()
    assert lib.FB_DatasetCreateFromCSR(indptr.ctypes.data_as(ctypes.c_void_p), 7, indices.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)), data.ctypes.data_as(ctypes.c_void_p), 1,
                                       ctypes.c_int64(len(indptr)), ctypes.c_int64(len(data)), ctypes.c_int64(6), _param_str({}), None, ctypes.byref(h)) == 0
    nb = ctypes.c_int(0)
    assert lib.FB_DatasetGetFeatureNumBin(h, 0, ctypes.byref(nb)) == 0 and nb.value == fb.Dataset(X, y).feature_num_bin(0)
    dump = tmp_path / "ds.txt"
    assert lib.FB_DatasetDumpText(h, str(dump).encode()) == 0 and "num_data: 2000" in dump.read_text()
    lib.FB_DatasetFree(h)
    # CSC forms and row blocks
    sc = sps.csc_matrix(X)
    cptr = sc.indptr.astype(np.int32); cidx = sc.indices.astype(np.int32); cval = sc.data.astype(np.float64)
    res2 = np.zeros(2000, dtype=np.float64)
    assert lib.FB_BoosterPredictForCSC(b._handle, cptr.ctypes.data_as(ctypes.c_void_p), 7, cidx.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)),
                                       cval.ctypes.data_as(ctypes.c_void_p), 1, ctypes.c_int64(len(cptr)), ctypes.c_int64(len(cval)), ctypes.c_int64(2000), 0, 0, -1, b"",
                                       ctypes.byref(n), res2.ctypes.data_as(ctypes.POINTER(ctypes.c_double))) == 0
    assert n.value == 2000 and np.allclose(res2, ref, atol=1e-12)
    h2 = ctypes.c_void_p()
    assert lib.FB_DatasetCreateFromCSC(cptr.ctypes.data_as(ctypes.c_void_p), 7, cidx.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)), cval.ctypes.data_as(ctypes.c_void_p), 1,
                                       ctypes.c_int64(len(cptr)), ctypes.c_int64(len(cval)), ctypes.c_int64(2000), _param_str({}), None, ctypes.byref(h2)) == 0
    nd = ctypes.c_int32(0)
    assert lib.FB_DatasetGetNumData(h2, ctypes.byref(nd)) == 0 and nd.value == 2000
    lib.FB_DatasetFree(h2)
    parts = [np.ascontiguousarray(X[:700]), np.ascontiguousarray(X[700:])]
    ptrs = (ctypes.c_void_p * 2)(parts[0].ctypes.data, parts[1].ctypes.data)
    rows = (ctypes.c_int32 * 2)(700, 1300)
    res3 = np.zeros(2000, dtype=np.float64)
    assert lib.FB_BoosterPredictForMats(b._handle, ptrs, 1, 2, rows, 6, 1, 0, 0, -1, b"", ctypes.byref(n), res3.ctypes.data_as(ctypes.POINTER(ctypes.c_double))) == 0
    assert np.allclose(res3, ref, atol=1e-12)
    h3 = ctypes.c_void_p()
    assert lib.FB_DatasetCreateFromMats(2, ptrs, 1, rows, 6, 1, _param_str({}), None, ctypes.byref(h3)) == 0
    assert lib.FB_DatasetGetNumData(h3, ctypes.byref(nd)) == 0 and nd.value == 2000
    lib.FB_DatasetFree(h3)
    # sample, aliases, feature-name check
    cnt = ctypes.c_int(0)
    assert lib.FB_GetSampleCount(5000, _param_str({"bin_construct_sample_cnt": 1000}), ctypes.byref(cnt)) == 0 and cnt.value == 1000
    idx = np.zeros(5000, dtype=np.int32); k = ctypes.c_int32(0)
    assert lib.FB_SampleIndices(5000, _param_str({"bin_construct_sample_cnt": 1000}), idx.ctypes.data_as(ctypes.c_void_p), ctypes.byref(k)) == 0
    assert 800 < k.value < 1200 and np.all(np.diff(idx[: k.value]) > 0)
    need = ctypes.c_int64(0)
    lib.FB_DumpParamAliases(ctypes.c_int64(0), ctypes.byref(need), None)
    buf = ctypes.create_string_buffer(need.value)
    assert lib.FB_DumpParamAliases(ctypes.c_int64(need.value), ctypes.byref(need), buf) == 0
    aliases = json.loads(buf.value.decode())
    assert "n_estimators" in aliases["num_iterations"] and "eta" in aliases["learning_rate"]
    names = (ctypes.c_char_p * 6)(*[f"Column_{i}".encode() for i in range(6)])
    assert lib.FB_BoosterValidateFeatureNames(b._handle, names, 6) == 0
    names[2] = b"other"
    assert lib.FB_BoosterValidateFeatureNames(b._handle, names, 6) != 0
    lin = ctypes.c_int(-1)
    assert lib.FB_BoosterGetLinear(b._handle, ctypes.byref(lin)) == 0 and lin.value == 0


def test_c_api_streaming_push_matches_one_shot_dataset():
    import ctypes
    from falcata_b200.basic import _lib

    lib = _lib()
    rng = np.random.default_rng(9)
    X = rng.normal(size=(3000, 5)).astype(np.float64)
    y = (X[:, 0] + X[:, 1] > 0).astype(np.float32)
    w = rng.uniform(0.5, 1.5, size=3000).astype(np.float32)
    p = {"objective": "binary", "num_leaves": 7, "verbose": -1, "min_data_in_leaf": 5}
    base = fb.Dataset(X, y, weight=w).construct()
    ref_model = fb.train(p, base, 4).model_to_string()
    h = ctypes.c_void_p()
    assert lib.FB_DatasetCreateByReference(base._handle, ctypes.byref(h)) == 0
    assert lib.FB_DatasetInitRows(h, 3000, ctypes.c_int64(0), ctypes.c_int64(3000), 1) == 0
    assert lib.FB_DatasetInitStreaming(h, 1, 0, 0, 1) == 0
    for a, b_ in ((2000, 3000), (0, 900), (900, 2000)):      # blocks in any order
        blk = np.ascontiguousarray(X[a:b_]); yb = np.ascontiguousarray(y[a:b_]); wb = np.ascontiguousarray(w[a:b_])
        assert lib.FB_DatasetPushRowsWithMetadata(h, blk.ctypes.data_as(ctypes.c_void_p), 1, b_ - a, 5, a, yb.ctypes.data_as(ctypes.POINTER(ctypes.c_float)),
                                                  wb.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), None, None) == 0
    assert lib.FB_DatasetMarkFinished(h) == 0
    streamed = fb.Dataset.__new__(fb.Dataset)
    fb.Dataset.__init__(streamed, None)
    streamed._handle = h
    assert fb.train(p, streamed, 4).model_to_string() == ref_model


def test_update_on_new_training_data_continues_the_model():
    rng = np.random.default_rng(10)
    Xa = rng.normal(size=(3000, 5)).astype(np.float32); ya = (Xa[:, 0] + 0.5 * Xa[:, 1]).astype(np.float32)
    Xb = rng.normal(size=(2500, 5)).astype(np.float32); yb = (Xb[:, 0] + 0.5 * Xb[:, 1]).astype(np.float32)
    p = {"objective": "regression", "num_leaves": 15, "verbose": -1, "metric": "l2", "learning_rate": 0.2}
    da = fb.Dataset(Xa, ya)
    b = fb.Booster(p, da)
    for _ in range(5):
        b.update()
    db = fb.Dataset(Xb, yb, reference=da)
    b.update(train_set=db)                 # scores of the 5 trees are replayed on the new rows, then round 6 is trained on them
    for _ in range(4):
        b.update()
    assert b.current_iteration() == 10
    l2_reported = b.eval_train()[0][2]
    l2_predict = float(np.mean((b.predict(Xb) - yb) ** 2))
    assert abs(l2_reported - l2_predict) < 1e-9
    assert l2_predict < 0.3 * float(np.var(yb))


def test_c_api_arrow_record_batches():
    import ctypes
    import pyarrow as pa
    from falcata_b200.basic import _lib, _param_str

    class ArrowArray(ctypes.Structure):
        _fields_ = [("length", ctypes.c_int64), ("null_count", ctypes.c_int64), ("offset", ctypes.c_int64), ("n_buffers", ctypes.c_int64), ("n_children", ctypes.c_int64),
                    ("buffers", ctypes.c_void_p), ("children", ctypes.c_void_p), ("dictionary", ctypes.c_void_p), ("release", ctypes.c_void_p), ("private_data", ctypes.c_void_p)]

    class ArrowSchema(ctypes.Structure):
        _fields_ = [("format", ctypes.c_char_p), ("name", ctypes.c_char_p), ("metadata", ctypes.c_char_p), ("flags", ctypes.c_int64), ("n_children", ctypes.c_int64),
                    ("children", ctypes.c_void_p), ("dictionary", ctypes.c_void_p), ("release", ctypes.c_void_p), ("private_data", ctypes.c_void_p)]

    def export(table):
        batches = table.to_batches(max_chunksize=400)
        arrays = (ArrowArray * len(batches))()
        schema = ArrowSchema()
        for i, bt in enumerate(batches):
            bt._export_to_c(ctypes.addressof(arrays[i]))
        table.schema._export_to_c(ctypes.addressof(schema))
        return len(batches), arrays, schema

    lib = _lib()
    rng = np.random.default_rng(11)
    X = rng.normal(size=(1000, 4))
    y = (X[:, 0] > 0).astype(np.float32)
    b = fb.train({"objective": "binary", "num_leaves": 7, "verbose": -1, "min_data_in_leaf": 5}, fb.Dataset(X, y), 4)
    table = pa.table({"a": X[:, 0], "b": X[:, 1].astype(np.float32), "c": X[:, 2], "d": X[:, 3]})
    Xt = np.column_stack([X[:, 0], X[:, 1].astype(np.float32).astype(np.float64), X[:, 2], X[:, 3]])
    n_chunks, arrays, schema = export(table)
    assert n_chunks == 3
    out = np.zeros(1000, dtype=np.float64); n = ctypes.c_int64(0)
    assert lib.FB_BoosterPredictForArrow(b._handle, ctypes.c_int64(n_chunks), ctypes.byref(arrays), ctypes.byref(schema), 0, 0, -1, b"", ctypes.byref(n),
                                         out.ctypes.data_as(ctypes.POINTER(ctypes.c_double))) == 0
    assert n.value == 1000 and np.allclose(out, b.predict(Xt), atol=1e-12)
    assert not schema.release       # the consumer released what it was given
    n_chunks, arrays, schema = export(table)
    h = ctypes.c_void_p()
    assert lib.FB_DatasetCreateFromArrow(ctypes.c_int64(n_chunks), ctypes.byref(arrays), ctypes.byref(schema), _param_str({}), None, ctypes.byref(h)) == 0
    nd = ctypes.c_int32(0); nf = ctypes.c_int32(0)
    assert lib.FB_DatasetGetNumData(h, ctypes.byref(nd)) == 0 and nd.value == 1000
    assert lib.FB_DatasetGetNumFeature(h, ctypes.byref(nf)) == 0 and nf.value == 4
    lib.FB_DatasetFree(h)


def test_c_api_arrow_streams():
    """ArrowArrayStream inputs: dataset creation, label from a stream, prediction; the stream is drained and released."""
    import ctypes
    import pyarrow as pa
    from falcata_b200.basic import _lib, _param_str

    class ArrowArrayStream(ctypes.Structure):
        _fields_ = [("get_schema", ctypes.c_void_p), ("get_next", ctypes.c_void_p), ("get_last_error", ctypes.c_void_p), ("release", ctypes.c_void_p),
                    ("private_data", ctypes.c_void_p)]

    def stream_of(table, chunk=300):
        st = ArrowArrayStream()
        pa.RecordBatchReader.from_batches(table.schema, table.to_batches(max_chunksize=chunk))._export_to_c(ctypes.addressof(st))
        return st

    lib = _lib()
    rng = np.random.default_rng(12)
    X = rng.normal(size=(1000, 3))
    y = (X[:, 0] + X[:, 1] > 0).astype(np.float32)
    table = pa.table({"a": X[:, 0], "b": X[:, 1], "c": X[:, 2]})
    st = stream_of(table)
    h = ctypes.c_void_p()
    assert lib.FB_DatasetCreateFromArrowStream(ctypes.byref(st), _param_str({"min_data_in_bin": 1}), None, ctypes.byref(h)) == 0
    assert not st.release
    nd = ctypes.c_int32(0)
    assert lib.FB_DatasetGetNumData(h, ctypes.byref(nd)) == 0 and nd.value == 1000
    lab = stream_of(pa.table({"label": y}), chunk=450)
    assert lib.FB_DatasetSetFieldFromArrowStream(h, b"label", ctypes.byref(lab)) == 0
    ln = ctypes.c_int64(0); ptr = ctypes.c_void_p(); tp = ctypes.c_int(0)
    assert lib.FB_DatasetGetField(h, b"label", ctypes.byref(ln), ctypes.byref(ptr), ctypes.byref(tp)) == 0 and ln.value == 1000
    got = np.ctypeslib.as_array(ctypes.cast(ptr, ctypes.POINTER(ctypes.c_float)), shape=(1000,))
    assert np.array_equal(got, y)
    bh = ctypes.c_void_p()
    assert lib.FB_BoosterCreate(h, _param_str({"objective": "binary", "num_leaves": 7, "verbose": -1, "min_data_in_leaf": 5}), ctypes.byref(bh)) == 0
    fin = ctypes.c_int(0)
    for _ in range(5):
        assert lib.FB_BoosterUpdateOneIter(bh, ctypes.byref(fin)) == 0
    out = np.zeros(1000); n = ctypes.c_int64(0)
    st = stream_of(table, chunk=128)
    assert lib.FB_BoosterPredictForArrowStream(bh, ctypes.byref(st), 0, 0, -1, b"", ctypes.byref(n), out.ctypes.data_as(ctypes.POINTER(ctypes.c_double))) == 0
    ref = np.zeros(1000)
    Xc = np.ascontiguousarray(X)
    assert lib.FB_BoosterPredictForMat(bh, Xc.ctypes.data_as(ctypes.c_void_p), 1, 1000, 3, 1, 0, 0, -1, b"", ctypes.byref(n), ref.ctypes.data_as(ctypes.POINTER(ctypes.c_double))) == 0
    assert np.array_equal(out, ref) and ((out > 0.5) == (y > 0.5)).mean() > 0.9
    lib.FB_BoosterFree(bh); lib.FB_DatasetFree(h)


def test_sklearn_custom_objective_metric_and_class_weight():
    """sklearn-style callables: objective f(y_true, y_pred) and metric f(y_true, y_pred[, weight]); class weights
    multiply the sample weights; the fitted check and the tags exist."""
    from sklearn.utils.validation import check_is_fitted
    from falcata_b200.sklearn import LGBMClassifier, LGBMRegressor

    rng = np.random.default_rng(21)
    X = rng.normal(size=(1500, 6)); y = X[:, 0] * 2 - X[:, 1] + 0.1 * rng.normal(size=1500)
    w = rng.uniform(0.5, 1.5, size=1500)

    def l2_obj(y_true, y_pred):
        return y_pred - y_true, np.ones_like(y_true)

    def mae(y_true, y_pred, weight):
        assert weight is not None and len(weight) == len(y_true)
        return "wmae", float(np.average(np.abs(y_true - y_pred), weights=weight)), False

    custom = LGBMRegressor(n_estimators=15, num_leaves=7, objective=l2_obj, min_child_samples=5)
    with pytest.raises(Exception):
        check_is_fitted(custom)
    custom.fit(X, y, sample_weight=w, eval_set=[(X, y)], eval_sample_weight=[w], eval_metric=mae)
    check_is_fitted(custom)
    builtin = LGBMRegressor(n_estimators=15, num_leaves=7, objective="regression", min_child_samples=5, boost_from_average=False).fit(X, y, sample_weight=w)
    assert np.allclose(custom.predict(X), builtin.predict(X), atol=1e-6)
    series = custom.evals_result_["training"]["wmae"]
    assert len(series) == 15 and series[-1] < series[0]
    assert custom._more_tags()["allow_nan"]

    yc = (X[:, 0] + 0.3 * rng.normal(size=1500) > 1.0).astype(int)      # about 17 % positives
    plain = LGBMClassifier(n_estimators=10, num_leaves=7).fit(X, yc)
    balanced = LGBMClassifier(n_estimators=10, num_leaves=7, class_weight="balanced").fit(X, yc)
    by_hand = LGBMClassifier(n_estimators=10, num_leaves=7).fit(X, yc, sample_weight=len(yc) / (2 * np.bincount(yc))[yc])
    assert np.allclose(balanced.predict_proba(X), by_hand.predict_proba(X))
    assert balanced.predict(X).mean() > plain.predict(X).mean()          # the rare class is predicted more often
    both = LGBMClassifier(n_estimators=10, num_leaves=7, class_weight={0: 1.0, 1: 3.0}).fit(X, yc, sample_weight=w)
    manual = LGBMClassifier(n_estimators=10, num_leaves=7).fit(X, yc, sample_weight=w * np.where(yc == 1, 3.0, 1.0))
    assert np.allclose(both.predict_proba(X), manual.predict_proba(X))


def test_plan_tuner_and_wisdom_file(tmp_path, monkeypatch):
    """The tuner flips the plan switches one at a time, keeps the flips that a timer calls faster by more than the
    margin, stores the plan under the workload's key, and cuda_plan="wisdom" picks it up."""
    from falcata_b200 import tuner

    monkeypatch.setenv("FALCATA_WISDOM", str(tmp_path / "w" / "wisdom.json"))
    rng = np.random.default_rng(81)
    X = rng.normal(size=(3000, 6)); y = (X[:, 0] > 0).astype(np.float64)
    ds = fb.Dataset(X, y)
    params = {"objective": "binary", "num_leaves": 15, "verbosity": -1, "quant_mode": "stochastic", "quant_bins": 4}
    seen = []

    def fake_timer(plan):
        seen.append(plan)
        ms = 10.0
        if "fused_scan:off" in plan:
            ms -= 2.0            # a real gain
        if "bulk_root:off" in plan:
            ms -= 0.05           # inside the noise margin: not kept
        if "gh_in_row:on" in plan:
            ms += 3.0
        return ms
    best = tuner.tune(params, ds, timer=fake_timer)
    assert best == "auto,fused_scan:off"
    assert seen[0] == "auto" and len(seen) == 1 + len(tuner.TUNABLE)
    assert all(p.startswith("auto") for p in seen)
    stored = tuner.load_wisdom()
    key = tuner.wisdom_key(params, 3000, 6)
    assert stored[key]["plan"] == best and abs(stored[key]["ms_per_round"] - 8.0) < 1e-9
    assert tuner.lookup(params, 3000, 6) == best
    assert tuner.lookup(params, 3100, 6) == best            # a few more rows: the same entry
    assert tuner.lookup(params, 300000, 6) == "auto"        # another size: nothing stored
    # the booster resolves "wisdom" through the same file; the plan never changes the model
    a = fb.train(dict(params, cuda_plan="wisdom"), fb.Dataset(X, y), 5)
    b = fb.train(dict(params), fb.Dataset(X, y), 5)
    assert a.model_to_string().split("\nparameters:")[0] == b.model_to_string().split("\nparameters:")[0]
    assert "fused_scan:off" in a.model_to_string()           # the resolved plan is what the model records
    # the built-in measurement runs on the host learner too
    quick = tuner.tune(params, fb.Dataset(X, y), rounds=2, warmup=1, switches=["fused_scan"], store=False)
    assert quick in ("auto", "auto,fused_scan:off")


def test_debug_environment_switches_dump_splits_and_cap_the_tree():
    """FALCATA_DEBUG=dump prints every split of every tree, FALCATA_DEBUG_SPLITS the host learner's splits as they are
    applied, FALCATA_DEBUG=maxsplits=N stops trees after N splits (reference: src/treelearner/cuda/plan.h:L286-322,
    src/treelearner/serial_tree_learner.cpp:L238-244)."""
    code = (
        "import numpy as np, falcata_b200 as fb\n"
        "rng = np.random.default_rng(0); X = rng.normal(size=(2000, 5)); y = (X[:, 0] + X[:, 1] > 0).astype(float)\n"
        "b = fb.train({'objective': 'binary', 'num_leaves': 15, 'verbosity': 1, 'device_type': 'cpu'}, fb.Dataset(X, y), 2)\n"
        "print('LEAVES', [t['num_leaves'] for t in b.dump_model()['tree_info']])\n")
    env = dict(os.environ, FALCATA_DEBUG="dump,maxsplits=3", FALCATA_DEBUG_SPLITS="1", PYTHONPATH=str(__import__("pathlib").Path(__file__).resolve().parents[1]))
    out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=300)
    text = out.stdout + out.stderr
    assert out.returncode == 0, text
    assert "LEAVES [4, 4]" in text                      # three splits per tree
    assert text.count("[split] leaf") == 6               # the host learner's own lines
    assert text.count("[dump] tree") == 2 and text.count("[dump]   node") == 6 and text.count("[dump]   leaf") == 8
    assert "maxsplits=3: num_leaves lowered from 15 to 4" in text


def test_add_features_from_merges_binned_datasets():
    """Dataset.add_features_from on two constructed datasets concatenates mappers, feature groups and bin columns without
    binning again (reference: Dataset::AddFeaturesFrom); training on the merged dataset gives the model of a dataset built
    from the concatenated matrix."""
    rng = np.random.default_rng(8)
    X = rng.normal(size=(3000, 9)).astype(np.float32)
    X[::17, 5] = np.nan
    y = (X[:, 0] + X[:, 6] * X[:, 7] > 0).astype(np.float32)
    p = {"objective": "binary", "num_leaves": 15, "verbosity": -1, "device_type": "cpu", "max_bin": 63, "min_data_in_leaf": 5}
    a = fb.Dataset(X[:, :4], y, params=p, free_raw_data=True).construct()
    b = fb.Dataset(X[:, 4:], params=p, free_raw_data=True).construct()
    a.add_features_from(b)
    assert a.num_feature() == 9 and a.num_data() == 3000
    merged = fb.train(p, a, 8)
    whole = fb.train(p, fb.Dataset(X, y, params=p), 8)
    np.testing.assert_allclose(merged.predict(X), whole.predict(X), rtol=0, atol=1e-12)
    assert merged.feature_name() == whole.feature_name()


def test_sparse_input_predicts_through_csr_and_returns_sparse_contributions():
    """A scipy sparse matrix is predicted through the CSR entry points (densified in blocks inside the library); feature
    contributions come back as a sparse matrix whose rows add up to the raw scores, equal to the dense route."""
    import scipy.sparse as sp

    rng = np.random.default_rng(4)
    dense = rng.normal(size=(1500, 12)) * (rng.random(size=(1500, 12)) < 0.3)
    y = (dense[:, 0] - dense[:, 3] + 0.5 * dense[:, 7] > 0).astype(np.float32)
    bst = fb.train({"objective": "binary", "num_leaves": 15, "verbosity": -1, "device_type": "cpu", "min_data_in_leaf": 5}, fb.Dataset(dense, y), 10)
    for make in (sp.csr_matrix, sp.csc_matrix, sp.coo_matrix):
        m = make(dense)
        np.testing.assert_allclose(bst.predict(m), bst.predict(dense), rtol=0, atol=1e-12)
        np.testing.assert_array_equal(bst.predict(m, pred_leaf=True), bst.predict(dense, pred_leaf=True))
    contrib = bst.predict(sp.csr_matrix(dense), pred_contrib=True)
    assert sp.issparse(contrib) and contrib.shape == (1500, 13)
    np.testing.assert_allclose(contrib.toarray(), bst.predict(dense, pred_contrib=True), rtol=0, atol=1e-12)
    np.testing.assert_allclose(np.asarray(contrib.sum(axis=1)).ravel(), bst.predict(dense, raw_score=True), atol=1e-9)
    assert contrib.nnz < 1500 * 13   # unused features have no entries


def test_eval_freq_fpreproc_and_the_remaining_reference_signatures():
    """train(eval_freq=k) evaluates every k-th iteration (early stopping then counts evaluations), cv(fpreproc=...) edits
    every fold, and get_field / dump_model / model_from_binary take the reference's argument names."""
    rng = np.random.default_rng(0)
    X = rng.normal(size=(3000, 6)); y = (X[:, 0] + X[:, 1] * X[:, 2] + rng.normal(size=3000) > 0).astype(float)
    tr = fb.Dataset(X[:2000], y[:2000]); va = fb.Dataset(X[2000:], y[2000:], reference=tr)
    p = {"objective": "binary", "verbosity": -1, "device_type": "cpu", "learning_rate": 0.3}
    every, sparse = {}, {}
    fb.train(p, tr, 60, valid_sets=[va], callbacks=[fb.record_evaluation(every)])
    b = fb.train(p, tr, 60, valid_sets=[va], callbacks=[fb.record_evaluation(sparse), fb.early_stopping(3, verbose=False)], eval_freq=5)
    got = sparse["valid_0"]["binary_logloss"]
    assert got == every["valid_0"]["binary_logloss"][4::5][: len(got)]          # iterations 5, 10, ...
    assert b.best_iteration % 5 == 0 and b.best_iteration == 5 * (1 + int(np.argmin(got)))
    assert len(got) == int(np.argmin(got)) + 1 + 3                               # three evaluations without improvement
    with pytest.raises(ValueError):
        fb.train(p, tr, 5, eval_freq=0)
    seen = []

    def shrink(dtrain, dvalid, params):
        seen.append((dtrain.num_data(), dvalid.num_data()))
        return dtrain, dvalid, dict(params, num_leaves=4)

    res = fb.cv(p, fb.Dataset(X, y), 5, nfold=3, fpreproc=shrink, return_cvbooster=True, stratified=False)
    assert len(seen) == 3 and all(a + v == 3000 for a, v in seen)
    assert all(t["num_leaves"] <= 4 for bst in res["cvbooster"].boosters for t in bst.dump_model()["tree_info"])
    assert tr.get_field(field_name="label").shape == (2000,)
    counted = []
    b.dump_model(object_hook=lambda d: counted.append(1) or d)
    assert len(counted) > 10
    clone = fb.Booster(model_str=b.model_to_string())
    clone.model_from_binary(model_bin=b.model_to_binary())
    np.testing.assert_allclose(clone.predict(X[:50]), b.predict(X[:50]))
