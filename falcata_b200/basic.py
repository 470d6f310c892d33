"""ctypes layer over the native core: ``Dataset`` and ``Booster``.

Parity: python-package/falcata/basic.py (Dataset L1782, numpy ingest L2362, device-array ingest
L2390-2447, Booster L3713, update L4268, save_model L4638, model_to_string L4895, predict
L5165-5265, refit L5267). torch is used only for device tensors (ingest, custom gradients,
device predict output) and for rank bootstrap; all training state lives in the C++/CUDA core.
"""
from __future__ import annotations

import ctypes
import json
import os
from pathlib import Path
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple, Union

import numpy as np

from .libpath import load_lib

_LIB = None


def _lib():
    global _LIB
    if _LIB is None:
        _LIB = load_lib()
        _LIB.FB_GetLastError.restype = ctypes.c_char_p
        _register_default_logger()
    return _LIB


class FalcataError(Exception):
    """Error raised by the native core."""


LightGBMError = FalcataError


def network_init(machines: Any, local_listen_port: int = 12400, listen_time_out: int = 120, num_machines: int = 1) -> None:
    """Open the TCP mesh between the processes of a distributed CPU training. Call it in every process BEFORE its Dataset
    is constructed: the processes then exchange their bin samples, find the same bin boundaries and number their rows in
    machine-list order. ``listen_time_out`` is in minutes."""
    if isinstance(machines, (list, tuple, set)):
        machines = ",".join(str(m) for m in machines)
    _safe_call(_lib().FB_NetworkInit(str(machines).encode("utf-8"), ctypes.c_int(int(local_listen_port)), ctypes.c_int(int(listen_time_out)), ctypes.c_int(int(num_machines))))


def network_free() -> None:
    _safe_call(_lib().FB_NetworkFree())


class FalcataDeprecationWarning(FutureWarning):
    """Deprecation notices of this package. A FutureWarning subclass: Python hides plain DeprecationWarning outside of
    ``__main__`` by default, and users should see these."""


def _safe_call(ret: int) -> None:
    if ret != 0:
        raise FalcataError(_lib().FB_GetLastError().decode("utf-8"))


# ------------------------------------------------------------------ logging ----
_LOGGER_FN: Optional[Callable[[str], None]] = None
_LOG_CB = ctypes.CFUNCTYPE(None, ctypes.c_char_p)


def _log_trampoline(msg: bytes) -> None:
    text = msg.decode("utf-8", "replace").rstrip("\n")
    if _LOGGER_FN is not None:
        _LOGGER_FN(text)
    else:
        print(text, flush=True)


_log_cb_holder = _LOG_CB(_log_trampoline)


def _register_default_logger() -> None:
    _LIB.FB_RegisterLogCallback(_log_cb_holder)


def register_logger(logger: Any, info_method_name: str = "info", warning_method_name: str = "warning") -> None:
    """Route native log lines to ``logger`` (a ``logging.Logger``-like object)."""
    global _LOGGER_FN
    info = getattr(logger, info_method_name)
    warn = getattr(logger, warning_method_name)

    def fn(text: str) -> None:
        (warn if "[Warning]" in text else info)(text)

    _LOGGER_FN = fn
    _lib()


# ------------------------------------------------------------------ helpers ----
_DTYPE_CODE = {np.dtype("float32"): 0, np.dtype("float64"): 1, np.dtype("int8"): 2, np.dtype("int16"): 3,
               np.dtype("uint8"): 4, np.dtype("uint16"): 5, np.dtype("float16"): 6, np.dtype("int32"): 7}

_PARAM_ALIASES_NUM_ROUNDS = ("num_iterations", "num_iteration", "n_iter", "num_tree", "num_trees", "num_round", "num_rounds",
                             "nrounds", "num_boost_round", "n_estimators", "max_iter")
_EARLY_STOP_ALIASES = ("early_stopping_round", "early_stopping_rounds", "early_stopping", "n_iter_no_change")


def _param_str(params: Optional[Dict[str, Any]]) -> bytes:
    if not params:
        return b""
    parts = []
    for k, v in params.items():
        if v is None or k == "keep_host_bins":   # keep_host_bins is a note between Booster and Dataset of this layer, not a native parameter
            continue
        if isinstance(v, (list, tuple, set)):
            # a list of lists (interaction_constraints) is written as [a,b],[c,d]: no blanks, which separate parameters
            v = ",".join("[" + ",".join(str(y) for y in x) + "]" if isinstance(x, (list, tuple, set)) else str(x) for x in v)
        elif isinstance(v, bool):
            v = "true" if v else "false"
        parts.append(f"{k}={v}")
    return " ".join(parts).encode("utf-8")


def _is_torch_tensor(x: Any) -> bool:
    return type(x).__module__.startswith("torch") and hasattr(x, "data_ptr")


def _is_cuda_array(x: Any) -> bool:
    if _is_torch_tensor(x):
        return x.is_cuda
    return hasattr(x, "__cuda_array_interface__")


def _to_numpy_2d(data: Any) -> np.ndarray:
    if isinstance(data, DataSequence) or (isinstance(data, list) and len(data) > 0 and all(isinstance(d, DataSequence) for d in data)):
        data = _materialize_sequences(data)
    if _is_torch_tensor(data):
        data = data.detach().cpu().numpy()
    if type(data).__module__.startswith("pyarrow") and hasattr(data, "column_names"):   # pyarrow Table / RecordBatch
        data = np.column_stack([np.asarray(data.column(i).to_numpy(zero_copy_only=False) if hasattr(data.column(i), "to_numpy") else data.column(i)) for i in range(data.num_columns)])
    if isinstance(data, list) and len(data) > 0 and all(isinstance(d, np.ndarray) and d.ndim == 2 for d in data):   # row chunks
        data = np.concatenate(data, axis=0)
    if hasattr(data, "values") and not isinstance(data, np.ndarray):   # pandas
        data = data.values
    if hasattr(data, "toarray"):                                       # scipy sparse -> dense (device path is dense)
        data = data.toarray()
    arr = np.asarray(data)
    if arr.ndim == 1:
        arr = arr.reshape(-1, 1) if arr.dtype != object else np.stack(arr)
    if arr.ndim != 2:
        raise ValueError("Input data must be 2-dimensional")
    if arr.dtype not in _DTYPE_CODE:
        arr = arr.astype(np.float64 if arr.dtype == np.float64 else np.float32)
    if not (arr.flags.c_contiguous or arr.flags.f_contiguous):
        arr = np.ascontiguousarray(arr)
    return arr


def _dump_pandas_categorical(pandas_categorical: Optional[List[List[Any]]]) -> str:
    """Trailer line of a text model: the category lists of the pandas categorical columns the model was trained on (JSON)."""
    import json

    def _default(o: Any) -> Any:
        if isinstance(o, np.generic):
            return o.item()
        raise TypeError(f"cannot serialise a category of type {type(o).__name__}")
    return "\npandas_categorical:" + json.dumps(pandas_categorical, default=_default) + "\n"


def _load_pandas_categorical(model_str: str) -> Optional[List[List[Any]]]:
    import json

    pos = model_str.rfind("\npandas_categorical:")
    if pos < 0:
        return None
    line = model_str[pos + len("\npandas_categorical:"):].strip().split("\n", 1)[0]
    try:
        return json.loads(line)
    except ValueError:
        return None


def _with_split_search(params: Dict[str, Any], ds: Any) -> Dict[str, Any]:
    """Several ranks that hold the same (gathered or replicated) bin sample split the bin search by feature."""
    from .parallel import bootstrap

    _, ws = bootstrap.world()
    if ws > 1 and (ds._global_rows is not None or ds._replicated) and "distributed_bin_finding" not in params:
        return dict(params, distributed_bin_finding=True)
    return params


def _get_string(fn: Callable, *args: Any) -> str:
    out_len = ctypes.c_int64(0)
    buf_len = 1 << 16
    buf = ctypes.create_string_buffer(buf_len)
    _safe_call(fn(*args, ctypes.c_int64(buf_len), ctypes.byref(out_len), buf))
    if out_len.value > buf_len:
        buf_len = out_len.value
        buf = ctypes.create_string_buffer(buf_len)
        _safe_call(fn(*args, ctypes.c_int64(buf_len), ctypes.byref(out_len), buf))
    return buf.value.decode("utf-8")


def _get_bytes(fn: Callable, *args: Any) -> bytes:
    out_len = ctypes.c_int64(0)
    _safe_call(fn(*args, ctypes.c_int64(0), ctypes.byref(out_len), None))
    buf = ctypes.create_string_buffer(out_len.value)
    _safe_call(fn(*args, ctypes.c_int64(out_len.value), ctypes.byref(out_len), buf))
    return buf.raw[: out_len.value]


def _resolved_int(params: Dict[str, Any], name: str) -> int:
    """An integer parameter as the native config resolves it (aliases, defaults, values derived from ``seed``)."""
    out = ctypes.c_int(0)
    _safe_call(_lib().FB_ResolveParamInt(_param_str(params), name.encode(), ctypes.byref(out)))
    return out.value


def cuda_available() -> bool:
    out = ctypes.c_int(0)
    _safe_call(_lib().FB_CudaAvailable(ctypes.byref(out)))
    return bool(out.value)


def set_num_threads(n: int) -> None:
    """Host worker threads of the native library's parallel loops (bin finding, label scans, host learners)."""
    _safe_call(_lib().FB_SetNumThreads(ctypes.c_int(int(n))))


def get_num_threads() -> int:
    out = ctypes.c_int(0)
    _safe_call(_lib().FB_GetNumThreads(ctypes.byref(out)))
    return out.value


_PY_TAGS: Dict[str, List[float]] = {}
_PY_TAGS_ON = False


class _tag:
    """Wall-clock span of a Python-side stage, accumulated under ``name`` while time tags are on."""

    def __init__(self, name: str) -> None:
        self.name = name

    def __enter__(self) -> "_tag":
        if _PY_TAGS_ON:
            import time

            self.t0 = time.perf_counter()
        return self

    def __exit__(self, *a: Any) -> None:
        if _PY_TAGS_ON:
            import time

            e = _PY_TAGS.setdefault(self.name, [0.0, 0])
            e[0] += time.perf_counter() - self.t0; e[1] += 1


def set_time_tag(enabled: bool) -> None:
    """Switch the host-side stage timers (native library and Python layer) on or off (off clears them)."""
    global _PY_TAGS_ON
    _PY_TAGS_ON = bool(enabled)
    if not enabled:
        _PY_TAGS.clear()
    _safe_call(_lib().FB_SetTimeTag(ctypes.c_int(1 if enabled else 0)))


def time_tag_report() -> str:
    """Accumulated host-side stage times, one line per stage (native stages first, then the Python layer's)."""
    out = _get_string(_lib().FB_GetTimeTagReport)
    for name in sorted(_PY_TAGS):
        out += f"py::{name} costs:\t {_PY_TAGS[name][0]:.6g} s ({int(_PY_TAGS[name][1])} calls)\n"
    return out


# ------------------------------------------------------------------ Dataset ----
_PICKLE_FORMAT = os.environ.get("FALCATA_PICKLE_FORMAT", "falb").strip().lower()
if _PICKLE_FORMAT not in ("falb", "text"):
    _PICKLE_FORMAT = "falb"


def set_pickle_format(fmt: str) -> None:
    """Payload that pickle writes for a Booster: "falb" (compact binary model, the default) or "text" (the LightGBM
    model text, for readers that only know that format). Unpickling accepts both.
    Parity: python-package/falcata/basic.py (set_pickle_format / get_pickle_format)."""
    global _PICKLE_FORMAT
    fmt = fmt.strip().lower()
    if fmt not in ("falb", "text"):
        raise ValueError(f'pickle format must be "falb" or "text", got "{fmt}"')
    _PICKLE_FORMAT = fmt


def get_pickle_format() -> str:
    return _PICKLE_FORMAT


class DataSequence:
    """Generic row access for building a Dataset without one big array: len(seq), seq[i] (one row), seq[a:b]
    (a batch of rows) and an optional batch_size. Exported as ``Sequence``.
    Parity: python-package/falcata/basic.py (class Sequence)."""

    batch_size = 4096

    def __getitem__(self, idx: Any) -> np.ndarray:
        raise NotImplementedError("Sub-classes of Sequence must implement __getitem__()")

    def __len__(self) -> int:
        raise NotImplementedError("Sub-classes of Sequence must implement __len__()")


def _materialize_sequences(data: Any) -> np.ndarray:
    seqs = [data] if isinstance(data, DataSequence) else list(data)
    parts = []
    for seq in seqs:
        bs = int(getattr(seq, "batch_size", None) or DataSequence.batch_size)
        n = len(seq)
        for start in range(0, n, bs):
            parts.append(np.asarray(seq[start:min(start + bs, n)]))
    return np.concatenate(parts, axis=0) if parts else np.zeros((0, 0), dtype=np.float32)


def _trains_on_host(params: Dict[str, Any]) -> bool:
    """Parameters with which a device booster hands the training to the host learner (the native side warns)."""
    def text(*names: str) -> str:
        for k in names:
            if params.get(k) is not None:
                return str(params[k]).lower()
        return ""
    if text("boosting", "boosting_type", "boost") in ("rf", "random_forest") and text("objective", "objective_type", "app", "application", "loss") in (
            "regression_l1", "l1", "mae", "mean_absolute_error", "quantile", "mape", "mean_absolute_percentage_error"):
        return True   # a forest whose objective renews its leaf outputs trains on the host learner
    if text("forcedsplits_filename", "fs", "forced_splits_filename", "forced_splits_file", "forced_splits"):
        return True
    for k in ("cegb_penalty_feature_coupled", "cegb_penalty_feature_lazy"):
        v = params.get(k)
        if v is not None and len(v) > 0:
            return True
    if text("monotone_constraints_method", "monotone_constraining_method", "mc_method") in ("intermediate", "advanced"):
        return True
    return False


def _wants_linear(params: Dict[str, Any], reference: Any = None) -> bool:
    """linear_tree keeps the raw feature values beside the bins, which only the host construction does."""
    for k in ("linear_tree", "linear_trees"):
        v = params.get(k)
        if v is not None and str(v).lower() in ("1", "true", "+"):
            return True
    return reference is not None and _wants_linear(getattr(reference, "params", {}) or {})


class Dataset:
    """Binned training / validation data.

    ``data`` may be a numpy array, pandas frame, scipy sparse matrix (densified), a path to a
    CSV/TSV/LibSVM/binary file, or a **CUDA tensor / ``__cuda_array_interface__`` object**: in that
    case the rows are binned on the GPU and never leave it.
    """

    def __init__(self, data: Any, label: Any = None, reference: Optional["Dataset"] = None, weight: Any = None,
                 group: Any = None, init_score: Any = None, feature_name: Union[str, List[str]] = "auto",
                 categorical_feature: Union[str, List[int], List[str]] = "auto", params: Optional[Dict[str, Any]] = None,
                 free_raw_data: bool = True, position: Any = None) -> None:
        self.data = data
        self.label = label
        self.reference = reference
        self.weight = weight
        self.group = group
        self.init_score = init_score
        self.feature_name = feature_name
        self.categorical_feature = categorical_feature
        self.params = dict(params) if params else {}
        self.free_raw_data = free_raw_data
        self._handle: Optional[ctypes.c_void_p] = None
        self.used_indices: Optional[np.ndarray] = None
        self._predictor = None
        self._keep: List[Any] = []   # arrays whose memory the native side points into
        self._global_rows: Optional[Tuple[int, int]] = None   # (offset, total) when rows are one shard of many
        self._replicated = False                               # every rank holds all rows (feature-parallel training)

    # -- construction ---------------------------------------------------------------
    def _merged_params(self) -> Dict[str, Any]:
        p = dict(self.params)
        cf = self.categorical_feature
        if cf != "auto" and cf is not None and len(cf) > 0 and all(isinstance(c, (int, np.integer)) for c in cf):
            p["categorical_feature"] = ",".join(str(int(c)) for c in cf)
        return p

    def construct(self) -> "Dataset":
        if self._handle is not None:
            return self
        lib = _lib()
        ref_handle = None
        if self.reference is not None:
            ref_handle = self.reference.construct()._handle
        params = self._merged_params()
        handle = ctypes.c_void_p()
        if self.used_indices is not None and self.reference is not None and self.data is None:
            idx = np.ascontiguousarray(self.used_indices, dtype=np.int32)
            _safe_call(lib.FB_DatasetGetSubset(ref_handle, idx.ctypes.data_as(ctypes.c_void_p), ctypes.c_int32(len(idx)), ctypes.byref(handle)))
            self._handle = handle
        elif isinstance(self.data, (str, os.PathLike)):
            _safe_call(lib.FB_DatasetCreateFromFile(str(self.data).encode(), _param_str(params), ref_handle, ctypes.byref(handle)))
            self._handle = handle
        elif _is_cuda_array(self.data) and not _wants_linear(params, self.reference):
            self._construct_from_device(self.data, params, ref_handle)
        elif hasattr(self.data, "tocsr") and not _wants_linear(params, self.reference) and self._global_rows is None:
            self._construct_sparse_host(self.data, params, ref_handle)
        elif self._host_matrix_for_device(params, ref_handle):
            self._construct_host_via_device(params)
        elif self._global_rows is not None and ref_handle is None:
            self._construct_sharded_host(_to_numpy_2d(self.data), params)
        else:
            arr = _to_numpy_2d(self.data)
            row_major = 1 if arr.flags.c_contiguous else 0
            _safe_call(lib.FB_DatasetCreateFromMat(arr.ctypes.data_as(ctypes.c_void_p), _DTYPE_CODE[arr.dtype], ctypes.c_int32(arr.shape[0]),
                                                   ctypes.c_int32(arr.shape[1]), row_major, _param_str(params), ref_handle, ctypes.byref(handle)))
            self._handle = handle
            if hasattr(self.data, "column_names") and self.feature_name == "auto":     # pyarrow
                self.feature_name = [str(c) for c in self.data.column_names]
            elif hasattr(self.data, "columns") and self.feature_name == "auto":        # pandas
                self.feature_name = [str(c) for c in self.data.columns]
        if self.feature_name != "auto" and self.feature_name is not None:
            self.set_feature_name(self.feature_name)
        if not getattr(self, "_early_fields", False):
            if self.label is not None:
                self.set_label(self.label)
            if self.weight is not None:
                self.set_weight(self.weight)
            if self.group is not None:
                self.set_group(self.group)
        if self.init_score is not None:
            self.set_init_score(self.init_score)
        elif self._predictor is not None and self.data is not None:
            init = self._predictor.predict(self.data, raw_score=True)
            self.set_init_score(np.asarray(init, dtype=np.float64).T.reshape(-1))
        if self.free_raw_data:
            self.data = None
        return self

    def _host_matrix_for_device(self, params: Dict[str, Any], ref_handle: Any) -> bool:
        """A dense host matrix that will train on the device is binned there too (unless host bins are asked for)."""
        if ref_handle is not None or str(params.get("device_type", "")).lower() not in ("cuda", "gpu") or params.get("keep_host_bins"):
            return False
        if _wants_linear(params, self.reference):
            return False   # linear leaves are fitted on the host from the raw values
        try:
            if int(params.get("max_bin", 255)) > 255:
                return False   # more than one byte per feature group: binned and trained on the host
        except (TypeError, ValueError):
            pass
        if not cuda_available():
            return False
        d = self.data
        if _is_torch_tensor(d):
            return (not d.is_cuda) and d.dim() == 2 and d.is_contiguous()
        return isinstance(d, np.ndarray) and d.ndim == 2 and d.flags.c_contiguous and d.dtype in _DTYPE_CODE and d.dtype != np.dtype("uint16")

    def _construct_host_via_device(self, params: Dict[str, Any]) -> None:
        """Host matrix -> device bins without binning on the host: the raw matrix goes to the device on a side stream
        (in one piece when it fits a quarter of the free memory, else chunk by chunk through a reused buffer) while
        the host draws the bin sample from its own copy and finds the bin boundaries; the device then bins the rows.
        Parity: src/io/cuda/cuda_dense_binner.cu:L85-170 (chunked H2D -> kernel ring for host matrices)."""
        import torch

        from .parallel import bootstrap

        lib = _lib()
        t = self.data if _is_torch_tensor(self.data) else torch.from_numpy(self.data)
        nrow, ncol = t.shape
        dev = torch.device("cuda", torch.cuda.current_device())
        free_bytes, _ = torch.cuda.mem_get_info(dev)
        nbytes = t.numel() * t.element_size()
        whole = nbytes <= free_bytes // 4
        staged: Dict[str, Any] = {}

        def _stage_matrix() -> None:
            # a helper thread pays for the side stream, the device allocation (tens of milliseconds for hundreds of
            # megabytes) and the copy's enqueue while this thread draws the sample and finds the bin boundaries
            try:
                with _tag("ingest: device buffer + copy enqueue (helper thread)"):
                    torch.cuda.set_device(dev)
                    side = torch.cuda.Stream(device=dev)
                    staged["side"] = side
                    with torch.cuda.stream(side):
                        Xd = torch.empty(t.shape, dtype=t.dtype, device=dev)
                        Xd.copy_(t, non_blocking=True)   # asynchronous when the matrix is pinned
                    staged["Xd"] = Xd
            except BaseException as e:   # re-raised by the caller after join()
                staged["error"] = e

        import threading

        stager = threading.Thread(target=_stage_matrix, daemon=True) if whole else None
        Xd = None
        goff, gtot = self._global_rows if self._global_rows is not None else (0, 0)
        with _tag("ingest: bin sample (draw + gather over ranks)"):
            # the helper starts once the row draw (a small kernel of its own) is through: device allocations of two
            # threads at the same time wait on each other
            sample, total = bootstrap.gather_bin_sample(t, _resolved_int(params, "bin_construct_sample_cnt"), _resolved_int(params, "data_random_seed"), goff, gtot,
                                                        replicated=self._replicated, after_draw=stager.start if stager is not None else None)
            sample = np.ascontiguousarray(sample)
            if sample.dtype not in _DTYPE_CODE:
                sample = sample.astype(np.float64)
        handle = ctypes.c_void_p()
        with _tag("ingest: bin boundaries"):
            _safe_call(lib.FB_DatasetCreateFromSampleTyped(sample.ctypes.data_as(ctypes.c_void_p), _DTYPE_CODE[sample.dtype], ctypes.c_int32(sample.shape[0]),
                                                           ctypes.c_int32(ncol), ctypes.c_int64(total), _param_str(_with_split_search(params, self)), None, 0, ctypes.byref(handle)))
        self._handle = handle
        off, tot = self._global_rows if self._global_rows is not None else (0, nrow)
        _safe_call(lib.FB_DatasetInitRows(handle, ctypes.c_int32(nrow), ctypes.c_int64(off), ctypes.c_int64(tot), 0))
        code = {torch.float32: 0, torch.float64: 1, torch.int8: 2, torch.int16: 3, torch.uint8: 4, torch.float16: 6, torch.int32: 7}[t.dtype]
        if whole:
            # label / weight / group go into the dataset now: tens of milliseconds of host copies for millions of rows,
            # hidden behind the matrix copy that is still in flight
            with _tag("ingest: label / weight / group"):
                self._set_early_fields()
            with _tag("ingest: wait for the matrix copy"):
                stager.join()
                if "error" in staged:
                    raise staged["error"]
                Xd = staged.pop("Xd")
                staged.pop("side").synchronize()
            with _tag("ingest: bin rows on the device"):
                _safe_call(lib.FB_DatasetBinDeviceChunk(handle, ctypes.c_void_p(Xd.data_ptr()), code, ctypes.c_int32(nrow), ctypes.c_int32(ncol), 0, ctypes.c_int32(nrow)))
                torch.cuda.synchronize()
        else:
            rows_per_chunk = max(1, int((free_bytes // 16) // max(1, ncol * t.element_size())))
            for a in range(0, nrow, rows_per_chunk):
                b = min(nrow, a + rows_per_chunk)
                chunk = t[a:b].to(dev)
                _safe_call(lib.FB_DatasetBinDeviceChunk(handle, ctypes.c_void_p(chunk.data_ptr()), code, ctypes.c_int32(b - a), ctypes.c_int32(ncol), ctypes.c_int32(a),
                                                        ctypes.c_int32(nrow)))
                del chunk
        del Xd
        torch.cuda.synchronize()

    def _construct_sparse_host(self, sp: Any, params: Dict[str, Any], ref_handle: Any) -> None:
        """scipy sparse matrix -> host bins without a dense copy of the whole matrix: the bin sample (the same draw by
        row id as for a dense matrix) is densified on its own, then the rows are binned block by block.
        Parity: src/c_api.cpp (dataset creation from CSR / CSC: sampled rows first, then pushed row blocks)."""
        import torch

        from .parallel import bootstrap

        lib = _lib()
        sp = sp.tocsr()
        nrow, ncol = sp.shape
        dt = np.float32 if sp.dtype == np.float32 else np.float64
        handle = ctypes.c_void_p()
        if ref_handle is not None:
            _safe_call(lib.FB_DatasetCreateByReference(ref_handle, ctypes.byref(handle)))
        else:
            cnt = _resolved_int(params, "bin_construct_sample_cnt")
            p = min(1.0, cnt / max(1, nrow))
            idx = bootstrap._bernoulli_rows(torch.empty(0), nrow, 0, _resolved_int(params, "data_random_seed"), p).numpy()
            if idx.size == 0:
                idx = np.arange(min(nrow, 1))
            sample = np.ascontiguousarray(sp[idx].toarray().astype(dt, copy=False))
            _safe_call(lib.FB_DatasetCreateFromSampleTyped(sample.ctypes.data_as(ctypes.c_void_p), _DTYPE_CODE[sample.dtype], ctypes.c_int32(sample.shape[0]),
                                                           ctypes.c_int32(ncol), ctypes.c_int64(nrow), _param_str(params), None, 0, ctypes.byref(handle)))
        self._handle = handle
        _safe_call(lib.FB_DatasetInitRows(handle, ctypes.c_int32(nrow), ctypes.c_int64(0), ctypes.c_int64(nrow), 1))
        block = max(1, min(nrow, (64 << 20) // max(1, ncol * np.dtype(dt).itemsize)))   # about 64 MB of dense rows at a time
        for a in range(0, nrow, block):
            b = min(nrow, a + block)
            dense = np.ascontiguousarray(sp[a:b].toarray().astype(dt, copy=False))
            _safe_call(lib.FB_DatasetPushRows(handle, dense.ctypes.data_as(ctypes.c_void_p), _DTYPE_CODE[dense.dtype], ctypes.c_int32(b - a), ctypes.c_int32(ncol), 1,
                                              ctypes.c_int32(a)))

    def _set_early_fields(self) -> None:
        """Set label, weight and group on the native dataset ahead of the end of construct(), which then skips them."""
        if self.label is not None:
            self.set_label(self.label)
        if self.weight is not None:
            self.set_weight(self.weight)
        if self.group is not None:
            self.set_group(self.group)
        self._early_fields = True

    def _construct_sharded_host(self, arr: np.ndarray, params: Dict[str, Any]) -> None:
        """Host ingest of one row shard: the bin sample is drawn by GLOBAL row id and gathered over all
        ranks, so every rank derives the same bin boundaries; the local rows are then binned on the host.
        Parity: src/io/dataset_loader.cpp:L672-759 (distributed bin finding)."""
        import torch

        from .parallel import bootstrap

        lib = _lib()
        if not arr.flags.c_contiguous:
            arr = np.ascontiguousarray(arr)
        nrow, ncol = arr.shape
        goff, gtot = self._global_rows
        sample, total = bootstrap.gather_bin_sample(torch.from_numpy(arr), _resolved_int(params, "bin_construct_sample_cnt"),
                                                    _resolved_int(params, "data_random_seed"), goff, gtot, replicated=self._replicated)
        sample = np.ascontiguousarray(sample)
        if sample.dtype not in _DTYPE_CODE:
            sample = sample.astype(np.float64)
        handle = ctypes.c_void_p()
        _safe_call(lib.FB_DatasetCreateFromSampleTyped(sample.ctypes.data_as(ctypes.c_void_p), _DTYPE_CODE[sample.dtype], ctypes.c_int32(sample.shape[0]),
                                                       ctypes.c_int32(ncol), ctypes.c_int64(total), _param_str(_with_split_search(params, self)), None, 0, ctypes.byref(handle)))
        self._handle = handle
        _safe_call(lib.FB_DatasetInitRows(handle, ctypes.c_int32(nrow), ctypes.c_int64(goff), ctypes.c_int64(total), 1))
        _safe_call(lib.FB_DatasetPushRows(handle, arr.ctypes.data_as(ctypes.c_void_p), _DTYPE_CODE[arr.dtype], ctypes.c_int32(nrow), ctypes.c_int32(ncol), 1, 0))

    def _construct_from_device(self, data: Any, params: Dict[str, Any], ref_handle: Any) -> None:
        """Device ingest: sample rows on the GPU, find bins on the host from the sample, bin on the GPU."""
        import torch

        lib = _lib()
        t = data if _is_torch_tensor(data) else torch.as_tensor(data, device="cuda")
        if t.dim() != 2:
            raise ValueError("Input data must be 2-dimensional")
        if t.dtype == torch.float64 or t.dtype == torch.float32 or t.dtype == torch.float16:
            pass
        elif t.dtype in (torch.int8, torch.int16, torch.uint8, torch.int32):
            pass
        else:
            t = t.float()
        if not t.is_contiguous():
            t = t.contiguous()
        nrow, ncol = t.shape
        handle = ctypes.c_void_p()
        if ref_handle is not None:
            _safe_call(lib.FB_DatasetCreateByReference(ref_handle, ctypes.byref(handle)))
        else:
            from .parallel import bootstrap

            goff, gtot = self._global_rows if self._global_rows is not None else (0, 0)
            sample, total = bootstrap.gather_bin_sample(t, _resolved_int(params, "bin_construct_sample_cnt"), _resolved_int(params, "data_random_seed"), goff, gtot,
                                                        replicated=self._replicated)
            sample = np.ascontiguousarray(sample)
            if sample.dtype not in _DTYPE_CODE:
                sample = sample.astype(np.float64)
            _safe_call(lib.FB_DatasetCreateFromSampleTyped(sample.ctypes.data_as(ctypes.c_void_p), _DTYPE_CODE[sample.dtype], ctypes.c_int32(sample.shape[0]),
                                                           ctypes.c_int32(ncol), ctypes.c_int64(total), _param_str(_with_split_search(params, self)), None, 0, ctypes.byref(handle)))
        self._handle = handle
        off, total = self._global_rows if self._global_rows is not None else (0, nrow)
        keep_host = 1 if str(params.get("device_type", "")).lower() == "cpu" or params.get("keep_host_bins") else 0
        _safe_call(lib.FB_DatasetInitRows(handle, ctypes.c_int32(nrow), ctypes.c_int64(off), ctypes.c_int64(total), 0))
        code = {torch.float32: 0, torch.float64: 1, torch.int8: 2, torch.int16: 3, torch.uint8: 4, torch.float16: 6, torch.int32: 7}[t.dtype]
        _safe_call(lib.FB_DatasetBinDeviceMat(handle, ctypes.c_void_p(t.data_ptr()), code, ctypes.c_int32(nrow), ctypes.c_int32(ncol), 1, keep_host))
        torch.cuda.synchronize()

    def set_replicated(self) -> "Dataset":
        """Declare that every rank holds ALL rows (``tree_learner=feature``): bins are found locally, nothing is gathered."""
        self._replicated = True
        return self

    def set_global_rows(self, offset: int, total: int) -> "Dataset":
        """Declare that this dataset holds rows [offset, offset + n) of a ``total``-row data set sharded over ranks."""
        self._global_rows = (int(offset), int(total))
        return self

    @property
    def handle(self) -> ctypes.c_void_p:
        return self.construct()._handle

    def create_valid(self, data: Any, label: Any = None, weight: Any = None, group: Any = None, init_score: Any = None,
                     params: Optional[Dict[str, Any]] = None, position: Any = None) -> "Dataset":
        ret = Dataset(data, label=label, reference=self, weight=weight, group=group, init_score=init_score, params=params or self.params,
                      free_raw_data=self.free_raw_data)
        ret._predictor = self._predictor
        return ret

    def subset(self, used_indices: Sequence[int], params: Optional[Dict[str, Any]] = None) -> "Dataset":
        ret = Dataset(None, reference=self, params=params or self.params, free_raw_data=self.free_raw_data)
        ret.used_indices = np.sort(np.asarray(used_indices, dtype=np.int32))
        ret._predictor = self._predictor
        return ret

    # -- fields -----------------------------------------------------------------------
    def _set_field(self, name: str, data: Any, dtype: Any) -> None:
        lib = _lib()
        if data is None:
            _safe_call(lib.FB_DatasetSetField(self._handle, name.encode(), None, ctypes.c_int64(0), 0))
            return
        if _is_torch_tensor(data):
            data = data.detach().cpu().numpy()
        if hasattr(data, "values") and not isinstance(data, np.ndarray):
            data = data.values
        arr = np.asarray(data)
        if name == "label" and arr.ndim == 2 and arr.shape[1] > 1:
            arr = arr.T          # several regression targets: the library keeps them [target][row]
        arr = np.ascontiguousarray(arr.reshape(-1), dtype=dtype)
        _safe_call(lib.FB_DatasetSetField(self._handle, name.encode(), arr.ctypes.data_as(ctypes.c_void_p), ctypes.c_int64(arr.size), _DTYPE_CODE[arr.dtype]))

    def get_field(self, field_name: Optional[str] = None, name: Optional[str] = None) -> Optional[np.ndarray]:
        name = field_name if field_name is not None else name
        if name is None:
            raise TypeError("get_field() needs field_name")
        lib = _lib()
        n = ctypes.c_int64(0); ptr = ctypes.c_void_p(); typ = ctypes.c_int(0)
        _safe_call(lib.FB_DatasetGetField(self.handle, name.encode(), ctypes.byref(n), ctypes.byref(ptr), ctypes.byref(typ)))
        if n.value == 0 or not ptr.value:
            return None
        ct = {0: ctypes.c_float, 1: ctypes.c_double, 7: ctypes.c_int32}[typ.value]
        return np.ctypeslib.as_array(ctypes.cast(ptr, ctypes.POINTER(ct)), shape=(n.value,)).copy()

    def set_field(self, field_name: str, data: Any) -> "Dataset":
        """Set label / weight / init_score / group (alias: query) / position by name (python-package/falcata/basic.py: Dataset.set_field)."""
        if field_name == "label":
            return self.set_label(data)
        if field_name == "weight":
            return self.set_weight(data)
        if field_name == "init_score":
            return self.set_init_score(data)
        if field_name in ("group", "query"):
            return self.set_group(data)
        if field_name == "position":
            return self.set_position(data)
        raise ValueError(f"Unknown field name: {field_name}")

    def set_position(self, position: Any) -> "Dataset":
        """Result positions for position-debiased ranking; kept with the dataset (the ranking objectives here do not use them)."""
        self.position = None if position is None else np.asarray(position, dtype=np.int32)
        return self

    def get_position(self) -> Optional[np.ndarray]:
        return getattr(self, "position", None)

    def get_data(self) -> Any:
        """The raw data this Dataset was built from (needs free_raw_data=False once constructed)."""
        if self._handle is not None and self.data is None:
            raise RuntimeError("Cannot call get_data after the raw data was freed; build the Dataset with free_raw_data=False")
        if self.used_indices is not None and self.reference is not None and self.data is None:
            ref = self.reference.get_data()
            return ref[self.used_indices] if not hasattr(ref, "iloc") else ref.iloc[self.used_indices]
        return self.data

    def get_params(self) -> Dict[str, Any]:
        """The dataset-related parameters this Dataset was given."""
        keys = ("max_bin", "max_bin_by_feature", "min_data_in_bin", "bin_construct_sample_cnt", "use_missing", "zero_as_missing", "enable_bundle",
                "categorical_feature", "feature_pre_filter", "data_random_seed", "linear_tree", "two_round", "header", "label_column", "weight_column",
                "group_column", "ignore_column", "precise_float_parser", "max_cat_to_onehot", "min_data_per_group")
        return {k: v for k, v in self.params.items() if k in keys}

    def get_ref_chain(self, ref_limit: int = 100) -> set:
        """This Dataset and the chain of its references."""
        head, chain = self, set()
        while len(chain) < ref_limit and isinstance(head, Dataset) and head not in chain:
            chain.add(head)
            head = head.reference
        return chain

    def set_categorical_feature(self, categorical_feature: Union[str, List[int], List[str]]) -> "Dataset":
        if self.categorical_feature == categorical_feature:
            return self
        if self._handle is not None:
            if self.data is None:
                raise RuntimeError("Cannot change categorical_feature after the raw data was freed; build the Dataset with free_raw_data=False")
            self._free()
        self.categorical_feature = categorical_feature
        return self

    def _free(self) -> None:
        if self._handle is not None:
            _lib().FB_DatasetFree(self._handle)
            self._handle = None

    def feature_num_bin(self, feature: Union[int, str]) -> int:
        """Number of bins of one feature (0 for a feature dropped as constant)."""
        if isinstance(feature, str):
            feature = self.get_feature_name().index(feature)
        out = ctypes.c_int(0)
        _safe_call(_lib().FB_DatasetFeatureNumBin(self.construct()._handle, ctypes.c_int(int(feature)), ctypes.byref(out)))
        return int(out.value)

    def add_features_from(self, other: "Dataset") -> "Dataset":
        """Append the columns of `other` (same rows). Two constructed datasets with host-resident bins are merged as they
        are binned (mappers, feature groups and bin columns are concatenated); otherwise both need their raw data and the
        result is binned again."""
        if self._handle is not None and other._handle is not None:
            try:
                _safe_call(_lib().FB_DatasetAddFeaturesFrom(self._handle, other._handle))
                if self.data is not None and other.data is not None and not _is_cuda_array(self.data) and not _is_cuda_array(other.data):
                    self.data = np.concatenate([_to_numpy_2d(self.data).astype(np.float64), _to_numpy_2d(other.data).astype(np.float64)], axis=1)
                else:
                    self.data = None
                self.feature_name = "auto"
                return self
            except FalcataError:
                if self.data is None or other.data is None:
                    raise
        if self.data is None or other.data is None:
            raise RuntimeError("add_features_from needs the raw data of both datasets (free_raw_data=False)")
        a, b = _to_numpy_2d(self.data), _to_numpy_2d(other.data)
        if a.shape[0] != b.shape[0]:
            raise ValueError("Both datasets must have the same number of rows")
        names = None
        if self._handle is not None and other._handle is not None:
            names = self.get_feature_name() + other.get_feature_name()
        self._free()
        self.data = np.concatenate([a.astype(np.float64), b.astype(np.float64)], axis=1)
        if names is not None and len(set(names)) == len(names):
            self.feature_name = names
        return self

    def set_label(self, label: Any) -> "Dataset":
        self.label = label
        if self._handle is not None and label is not None:
            self._set_field("label", label, np.float32)
        return self

    def set_weight(self, weight: Any) -> "Dataset":
        self.weight = weight
        if self._handle is not None:
            self._set_field("weight", weight, np.float32)
        return self

    def set_group(self, group: Any) -> "Dataset":
        self.group = group
        if self._handle is not None and group is not None:
            self._set_field("group", group, np.int32)
        return self

    def set_init_score(self, init_score: Any) -> "Dataset":
        self.init_score = init_score
        if self._handle is not None and init_score is not None:
            arr = np.asarray(init_score.detach().cpu().numpy() if _is_torch_tensor(init_score) else init_score, dtype=np.float64)
            if arr.ndim == 2:
                arr = arr.T   # class-major
            self._set_field("init_score", arr.reshape(-1), np.float64)
        return self

    def set_feature_name(self, feature_name: List[str]) -> "Dataset":
        self.feature_name = feature_name
        if self._handle is not None and feature_name != "auto" and feature_name is not None:
            arr = (ctypes.c_char_p * len(feature_name))(*[str(s).encode() for s in feature_name])
            _safe_call(_lib().FB_DatasetSetFeatureNames(self._handle, arr, len(feature_name)))
        return self

    def set_reference(self, reference: "Dataset") -> "Dataset":
        self.reference = reference
        return self

    def get_label(self) -> Optional[np.ndarray]:
        return self.get_field("label")

    def get_weight(self) -> Optional[np.ndarray]:
        return self.get_field("weight")

    def get_init_score(self) -> Optional[np.ndarray]:
        return self.get_field("init_score")

    def get_group(self) -> Optional[np.ndarray]:
        b = self.get_field("group")
        return None if b is None else np.diff(b)

    def get_feature_name(self) -> List[str]:
        return _get_string(_lib().FB_DatasetGetFeatureNames, self.handle).split("\n")

    def num_data(self) -> int:
        out = ctypes.c_int32(0)
        _safe_call(_lib().FB_DatasetGetNumData(self.handle, ctypes.byref(out)))
        return out.value

    def num_feature(self) -> int:
        out = ctypes.c_int32(0)
        _safe_call(_lib().FB_DatasetGetNumFeature(self.handle, ctypes.byref(out)))
        return out.value

    def info(self) -> Dict[str, int]:
        out = (ctypes.c_int32 * 6)()
        _safe_call(_lib().FB_DatasetGetInfo(self.handle, out))
        keys = ["num_used_features", "num_groups", "num_total_bin", "max_group_bin", "has_device", "has_host"]
        return dict(zip(keys, list(out)))

    def binned_row(self, row: int) -> np.ndarray:
        n = self.info()["num_used_features"]
        out = (ctypes.c_int32 * n)()
        _safe_call(_lib().FB_DatasetGetBinnedRow(self.handle, ctypes.c_int32(row), out))
        return np.array(out[:], dtype=np.int32)

    def save_binary(self, filename: Union[str, Path]) -> "Dataset":
        _safe_call(_lib().FB_DatasetSaveBinary(self.handle, str(filename).encode()))
        return self

    def free_device_data(self) -> "Dataset":
        if self._handle is not None:
            _safe_call(_lib().FB_DatasetFreeDeviceData(self._handle))
        return self

    def _set_predictor(self, predictor: Any) -> "Dataset":
        self._predictor = predictor
        return self

    def __del__(self) -> None:
        try:
            if self._handle is not None and _LIB is not None:
                _LIB.FB_DatasetFree(self._handle)
                self._handle = None
        except Exception:
            pass


# ------------------------------------------------------------------ Booster ----
class Booster:
    """Gradient boosting model: train with :meth:`update`, evaluate, predict, save / load."""

    def __init__(self, params: Optional[Dict[str, Any]] = None, train_set: Optional[Dataset] = None, model_file: Optional[Union[str, Path]] = None,
                 model_str: Optional[Union[str, bytes]] = None) -> None:
        lib = _lib()
        self._handle = ctypes.c_void_p()
        self.params = dict(params) if params else {}
        self.train_set = train_set
        self.valid_sets: List[Dataset] = []
        self.name_valid_sets: List[str] = []
        self.best_iteration = -1
        self.best_score: Dict[str, Dict[str, float]] = {}
        self._train_data_name = "training"
        self._network = False
        self.pandas_categorical = None
        n_iter = ctypes.c_int(0)
        if train_set is not None:
            if not isinstance(train_set, Dataset):
                raise TypeError(f"Training data should be Dataset instance, met {type(train_set).__name__}")
            merged = dict(train_set.params); merged.update(self.params)
            train_set.params = {**train_set.params, **{k: v for k, v in self.params.items() if k in _DATASET_PARAMS}}
            if _trains_on_host(self.params):
                train_set.params["keep_host_bins"] = True   # the host learner will do the training: it needs host-resident bins
            # a machine list in the parameters: join the TCP mesh before the Dataset is binned (the processes exchange their bin samples)
            nm = self.params.get("num_machines", self.params.get("num_machine"))
            machines = self.params.get("machines", self.params.get("workers", self.params.get("nodes")))
            if nm is not None and int(nm) > 1 and machines:
                if train_set._handle is not None:
                    raise FalcataError("The training Dataset was constructed before the machines were connected, so its bins were found on this "
                                       "process's rows alone. Leave the Dataset unconstructed (the Booster constructs it after joining the network) "
                                       "or call falcata_b200.network_init(...) before constructing it and drop the machine list from the parameters.")
                learner = self.params.get("tree_learner", self.params.get("tree", self.params.get("tree_type", self.params.get("tree_learner_type"))))
                if learner is not None:
                    train_set.params["tree_learner"] = learner   # feature-parallel: every process holds all rows, nothing is exchanged at binning
                self.set_network(machines, int(self.params.get("local_listen_port", self.params.get("local_port", self.params.get("port", 12400)))),
                                 int(self.params.get("time_out", 120)), int(nm))
            with _tag("booster: dataset construct"):
                train_set.construct()
            if str(self.params.get("cuda_plan", "")).strip().lower() == "wisdom":
                # the plan that tuner.tune() stored for this shape of workload on this kind of device ("auto" when none)
                from . import tuner
                from .parallel import bootstrap

                self.params = dict(self.params, cuda_plan=tuner.lookup(self.params, train_set.num_data(), train_set.num_feature(), bootstrap.world()[1]))
            with _tag("booster: native create (objective, metrics, device engine)"):
                _safe_call(lib.FB_BoosterCreate(train_set._handle, _param_str(self.params), ctypes.byref(self._handle)))
        elif model_file is not None:
            _safe_call(lib.FB_BoosterCreateFromModelfile(str(model_file).encode(), ctypes.byref(n_iter), ctypes.byref(self._handle)))
            with open(model_file, "rb") as f:   # a model file (text or binary) may end with the pandas categories trailer
                f.seek(max(0, os.path.getsize(model_file) - (1 << 20)))
                self.pandas_categorical = _load_pandas_categorical(f.read().decode("utf-8", errors="replace"))
        elif model_str is not None:
            raw = model_str if isinstance(model_str, bytes) else model_str.encode("utf-8")
            _safe_call(lib.FB_BoosterLoadModelFromString(raw, ctypes.c_int64(len(raw)), ctypes.byref(n_iter), ctypes.byref(self._handle)))
            if raw[:4] != b"FALB":
                self.pandas_categorical = _load_pandas_categorical(raw[-(1 << 20):].decode("utf-8", errors="replace"))
        else:
            raise TypeError("Need at least one training dataset or model file or model string to create Booster instance")
        self._eval_names: Optional[List[str]] = None
        self._eval_higher: Optional[List[bool]] = None

    def __del__(self) -> None:
        try:
            if self._handle and _LIB is not None:
                _LIB.FB_BoosterFree(self._handle)
                self._handle = None
        except Exception:
            pass

    # pickling goes through the text model
    def __getstate__(self) -> Dict[str, Any]:
        st = {k: v for k, v in self.__dict__.items() if k not in ("_handle", "train_set", "valid_sets")}
        if _PICKLE_FORMAT == "falb":
            try:   # statistics and diagnostics ride along: an unpickled booster is the same model in every respect
                st["_model_bin"] = self.model_to_binary(num_iteration=-1, with_stats=True, with_diagnostics=True)
            except FalcataError:   # linear trees have no binary form
                st["_model_str"] = self.model_to_string(num_iteration=-1)
        else:
            st["_model_str"] = self.model_to_string(num_iteration=-1)
        return st

    def __setstate__(self, state: Dict[str, Any]) -> None:
        # both payloads load, whatever the current setting is
        model_str = state.pop("_model_str", None)
        model_bin = state.pop("_model_bin", None)
        self.__dict__.update(state)
        self.train_set = None; self.valid_sets = []
        self._handle = ctypes.c_void_p(); n_iter = ctypes.c_int(0)
        if model_bin is not None:
            _safe_call(_lib().FB_BoosterCreateFromBinary(model_bin, ctypes.c_int64(len(model_bin)), ctypes.byref(n_iter), ctypes.byref(self._handle)))
        else:
            raw = model_str.encode("utf-8")
            _safe_call(_lib().FB_BoosterLoadModelFromString(raw, ctypes.c_int64(len(raw)), ctypes.byref(n_iter), ctypes.byref(self._handle)))

    def __copy__(self) -> "Booster":
        return self.__deepcopy__(None)

    def __deepcopy__(self, _: Any) -> "Booster":
        return Booster(model_str=self.model_to_string(num_iteration=-1))

    # -- training ---------------------------------------------------------------------
    def add_valid(self, data: Dataset, name: str) -> "Booster":
        if data.reference is None and data is not self.train_set:
            data.reference = self.train_set
        data.construct()
        _safe_call(_lib().FB_BoosterAddValidData(self._handle, data._handle))
        self.valid_sets.append(data); self.name_valid_sets.append(name)
        return self

    def set_train_data_name(self, name: str) -> "Booster":
        self._train_data_name = name
        return self

    def reset_parameter(self, params: Dict[str, Any]) -> "Booster":
        _safe_call(_lib().FB_BoosterResetParameter(self._handle, _param_str(params)))
        self.params.update(params)
        return self

    def update(self, train_set: Optional[Dataset] = None, fobj: Optional[Callable] = None) -> bool:
        """One boosting iteration. Returns True when no further split is possible."""
        lib = _lib()
        fin = ctypes.c_int(0)
        from .parallel import bootstrap as _bs

        if _bs.peer_check_enabled():
            _bs.assert_peers_alive()   # multi-rank: never enqueue a round that would wait for a rank that has left
        if train_set is not None and train_set is not self.train_set:
            if not isinstance(train_set, Dataset):
                raise TypeError(f"Training data should be Dataset instance, met {type(train_set).__name__}")
            if train_set.reference is None and self.train_set is not None:
                train_set.reference = self.train_set   # same bin mappers as the data the trees were grown on
            _safe_call(lib.FB_BoosterResetTrainingData(self._handle, train_set.construct()._handle))
            self.train_set = train_set
            self.valid_sets = []; self.name_valid_sets = []
        if fobj is None:
            _safe_call(lib.FB_BoosterUpdateOneIter(self._handle, ctypes.byref(fin)))
            return fin.value == 1
        grad, hess = fobj(self._inner_predict_raw(0), self.train_set)
        return self.__boost(grad, hess)

    def __boost(self, grad: Any, hess: Any) -> bool:
        lib = _lib()
        fin = ctypes.c_int(0)
        if _is_torch_tensor(grad) and grad.is_cuda:
            import torch

            g = grad.detach().to(torch.float32).contiguous().reshape(-1)
            h = hess.detach().to(torch.float32).contiguous().reshape(-1)
            _safe_call(lib.FB_BoosterUpdateOneIterCustom(self._handle, ctypes.c_void_p(g.data_ptr()), ctypes.c_void_p(h.data_ptr()), 1, ctypes.byref(fin)))
            torch.cuda.synchronize()
        else:
            if _is_torch_tensor(grad):
                grad = grad.detach().cpu().numpy(); hess = hess.detach().cpu().numpy()
            g = np.asarray(grad, dtype=np.float32); h = np.asarray(hess, dtype=np.float32)
            if g.ndim == 2:
                g = g.T; h = h.T   # class-major
            g = np.ascontiguousarray(g.reshape(-1)); h = np.ascontiguousarray(h.reshape(-1))
            n_pred = self.__num_predict(0)
            if g.size != n_pred or h.size != n_pred:
                raise ValueError(f"Lengths of gradient ({g.size}) and Hessian ({h.size}) don't match training data length ({n_pred})")
            if self._on_device():
                import torch

                gt = torch.from_numpy(g).cuda(); ht = torch.from_numpy(h).cuda()
                _safe_call(lib.FB_BoosterUpdateOneIterCustom(self._handle, ctypes.c_void_p(gt.data_ptr()), ctypes.c_void_p(ht.data_ptr()), 1, ctypes.byref(fin)))
                torch.cuda.synchronize()
            else:
                _safe_call(lib.FB_BoosterUpdateOneIterCustom(self._handle, g.ctypes.data_as(ctypes.c_void_p), h.ctypes.data_as(ctypes.c_void_p), 0, ctypes.byref(fin)))
        return fin.value == 1

    def _on_device(self) -> bool:
        p = ctypes.c_void_p()
        _safe_call(_lib().FB_BoosterGetTrainScoreDevicePtr(self._handle, ctypes.byref(p)))
        return bool(p.value)

    def train_score_tensor(self) -> Any:
        """Raw training scores as a torch CUDA tensor view (class-major ``[k, n]``); CUDA boosters only."""
        import torch

        p = ctypes.c_void_p()
        _safe_call(_lib().FB_BoosterGetTrainScoreDevicePtr(self._handle, ctypes.byref(p)))
        if not p.value:
            raise FalcataError("Booster is not device-resident")
        n = self.train_set.num_data(); k = self.num_model_per_iteration()
        from .utils.interop import tensor_from_ptr

        return tensor_from_ptr(p.value, (k, n), torch.float32)

    def rollback_one_iter(self) -> "Booster":
        _safe_call(_lib().FB_BoosterRollbackOneIter(self._handle))
        return self

    def current_iteration(self) -> int:
        out = ctypes.c_int(0)
        _safe_call(_lib().FB_BoosterGetCurrentIteration(self._handle, ctypes.byref(out)))
        return out.value

    def num_model_per_iteration(self) -> int:
        out = ctypes.c_int(0)
        _safe_call(_lib().FB_BoosterNumModelPerIteration(self._handle, ctypes.byref(out)))
        return out.value

    def num_trees(self) -> int:
        out = ctypes.c_int(0)
        _safe_call(_lib().FB_BoosterNumberOfTotalModel(self._handle, ctypes.byref(out)))
        return out.value

    def num_feature(self) -> int:
        out = ctypes.c_int(0)
        _safe_call(_lib().FB_BoosterGetNumFeature(self._handle, ctypes.byref(out)))
        return out.value

    def feature_name(self) -> List[str]:
        s = _get_string(_lib().FB_BoosterGetFeatureNames, self._handle)
        return s.split("\n") if s else []

    def upper_bound(self) -> float:
        out = ctypes.c_double(0)
        _safe_call(_lib().FB_BoosterGetUpperBoundValue(self._handle, ctypes.byref(out)))
        return out.value

    def lower_bound(self) -> float:
        out = ctypes.c_double(0)
        _safe_call(_lib().FB_BoosterGetLowerBoundValue(self._handle, ctypes.byref(out)))
        return out.value

    # -- evaluation -------------------------------------------------------------------
    def __get_eval_info(self) -> None:
        if self._eval_names is None:
            s = _get_string(_lib().FB_BoosterGetEvalNames, self._handle)
            items = [x for x in s.split("\n") if x]
            self._eval_names = [x[1:] for x in items]
            self._eval_higher = [x[0] == "+" for x in items]

    def __num_predict(self, data_idx: int) -> int:
        out = ctypes.c_int64(0)
        _safe_call(_lib().FB_BoosterGetNumPredict(self._handle, data_idx, ctypes.byref(out)))
        return out.value

    def _inner_predict_raw(self, data_idx: int) -> Any:
        """Raw scores of the training (0) or a validation set for custom objectives / metrics."""
        if data_idx == 0 and self._on_device():
            t = self.train_score_tensor()
            return t[0] if t.shape[0] == 1 else t.t()
        return self._inner_predict(data_idx, raw=True)

    def _inner_predict(self, data_idx: int, raw: bool = False) -> np.ndarray:
        n = self.__num_predict(data_idx)
        out = np.empty(n, dtype=np.float64)
        ln = ctypes.c_int64(0)
        _safe_call(_lib().FB_BoosterGetPredict(self._handle, data_idx, ctypes.byref(ln), out.ctypes.data_as(ctypes.c_void_p)))
        k = self.num_model_per_iteration()
        return out if k == 1 else out.reshape(k, -1).T

    def __inner_eval(self, data_name: str, data_idx: int, feval: Optional[Union[Callable, List[Callable]]] = None) -> List[Tuple[str, str, float, bool]]:
        self.__get_eval_info()
        ret: List[Tuple[str, str, float, bool]] = []
        if self._eval_names:
            res = (ctypes.c_double * len(self._eval_names))()
            ln = ctypes.c_int(0)
            _safe_call(_lib().FB_BoosterGetEval(self._handle, data_idx, ctypes.byref(ln), res))
            for i in range(ln.value):
                ret.append((data_name, self._eval_names[i], res[i], self._eval_higher[i]))
        if feval is not None:
            fevals = feval if isinstance(feval, (list, tuple)) else [feval]
            ds = self.train_set if data_idx == 0 else self.valid_sets[data_idx - 1]
            for f in fevals:
                if f is None:
                    continue
                out = f(self._inner_predict(data_idx), ds)
                outs = out if isinstance(out, list) else [out]
                for name, val, hib in outs:
                    ret.append((data_name, name, val, hib))
        return ret

    def eval_train(self, feval: Any = None) -> List[Tuple[str, str, float, bool]]:
        return self.__inner_eval(self._train_data_name, 0, feval)

    def eval_valid(self, feval: Any = None) -> List[Tuple[str, str, float, bool]]:
        out: List[Tuple[str, str, float, bool]] = []
        for i, name in enumerate(self.name_valid_sets):
            out.extend(self.__inner_eval(name, i + 1, feval))
        return out

    def eval(self, data: Dataset, name: str, feval: Any = None) -> List[Tuple[str, str, float, bool]]:
        if data is self.train_set:
            return self.__inner_eval(name, 0, feval)
        for i, v in enumerate(self.valid_sets):
            if data is v:
                return self.__inner_eval(name, i + 1, feval)
        self.add_valid(data, name)
        return self.__inner_eval(name, len(self.valid_sets), feval)

    # -- prediction -------------------------------------------------------------------
    def predict(self, data: Any, start_iteration: int = 0, num_iteration: Optional[int] = None, raw_score: bool = False, pred_leaf: bool = False,
                pred_contrib: bool = False, data_has_header: bool = False, validate_features: bool = False, **kwargs: Any) -> Any:
        """Predict for a numpy / pandas / scipy matrix (host traversal) or a CUDA tensor (device traversal kernel).

        A CUDA tensor input returns a CUDA tensor; everything else returns numpy.
        """
        lib = _lib()
        if isinstance(data, Dataset):
            raise TypeError("Cannot use Dataset instance for prediction, please use raw data instead")
        if num_iteration is None:
            num_iteration = self.best_iteration if start_iteration <= 0 and self.best_iteration > 0 else -1
        ptype = 1 if raw_score else 0
        if pred_leaf:
            ptype = 2
        if pred_contrib:
            ptype = 3
        k = self.num_model_per_iteration()
        if _is_cuda_array(data) and ptype in (0, 1) and cuda_available() and self._has_linear_trees():
            # the traversal kernel has constant leaves only: linear leaves are evaluated on the host, the result goes back
            import torch

            t = data if _is_torch_tensor(data) else torch.as_tensor(data, device="cuda")
            host = self.predict(t.detach().cpu().numpy(), start_iteration=start_iteration, num_iteration=num_iteration, raw_score=raw_score)
            return torch.as_tensor(np.asarray(host, dtype=np.float32), device=t.device)
        if _is_cuda_array(data) and ptype == 2 and cuda_available() and not self._has_linear_trees():
            # leaf indices on the device: int32 [rows, trees]; forests the kernel does not cover go through the host
            import torch

            t = data if _is_torch_tensor(data) else torch.as_tensor(data, device="cuda")
            if t.dtype not in (torch.float32, torch.float64, torch.float16):
                t = t.float()
            t = t.contiguous()
            nrow, ncol = t.shape
            per_row = ctypes.c_int64(0)
            _safe_call(lib.FB_BoosterCalcNumPredict(self._handle, 1, 2, start_iteration, num_iteration, ctypes.byref(per_row)))
            out = torch.zeros((nrow, max(1, per_row.value)), dtype=torch.int32, device=t.device)
            code = {torch.float32: 0, torch.float64: 1, torch.float16: 6}[t.dtype]
            rc = lib.FB_BoosterPredictForDeviceMat(self._handle, ctypes.c_void_p(t.data_ptr()), code, ctypes.c_int32(nrow), ctypes.c_int32(ncol), 1,
                                                   2, start_iteration, num_iteration, ctypes.c_void_p(out.data_ptr()))
            if rc == 0:
                return out
            host = self.predict(t.detach().cpu().numpy(), start_iteration=start_iteration, num_iteration=num_iteration, pred_leaf=True)
            return torch.as_tensor(np.asarray(host, dtype=np.int32), device=t.device)
        if _is_cuda_array(data) and ptype in (0, 1) and cuda_available():
            import torch

            t = data if _is_torch_tensor(data) else torch.as_tensor(data, device="cuda")
            if t.dtype not in (torch.float32, torch.float64, torch.float16):
                t = t.float()
            t = t.contiguous()
            nrow, ncol = t.shape
            out = torch.empty((k, nrow), dtype=torch.float32, device=t.device)
            code = {torch.float32: 0, torch.float64: 1, torch.float16: 6}[t.dtype]
            _safe_call(lib.FB_BoosterPredictForDeviceMat(self._handle, ctypes.c_void_p(t.data_ptr()), code, ctypes.c_int32(nrow), ctypes.c_int32(ncol), 1,
                                                         ptype, start_iteration, num_iteration, ctypes.c_void_p(out.data_ptr())))
            return out[0] if k == 1 else out.t().contiguous()
        if hasattr(data, "tocsr") and not isinstance(data, np.ndarray):
            # scipy sparse input: the rows are densified in blocks inside the library, never as one matrix; contributions
            # come back sparse as well
            return self._predict_csr(data.tocsr(), ptype, start_iteration, num_iteration, pred_leaf, pred_contrib, kwargs)
        if isinstance(data, (str, os.PathLike)):
            arr = np.loadtxt(str(data), delimiter="," if str(data).endswith(".csv") else None, skiprows=1 if data_has_header else 0, ndmin=2)[:, 1:]
        else:
            arr = _to_numpy_2d(data)
        nrow, ncol = arr.shape
        n_out = ctypes.c_int64(0)
        _safe_call(lib.FB_BoosterCalcNumPredict(self._handle, nrow, ptype, start_iteration, num_iteration, ctypes.byref(n_out)))
        out = np.empty(n_out.value, dtype=np.float64)
        ln = ctypes.c_int64(0)
        _safe_call(lib.FB_BoosterPredictForMat(self._handle, arr.ctypes.data_as(ctypes.c_void_p), _DTYPE_CODE[arr.dtype], ctypes.c_int32(nrow), ctypes.c_int32(ncol),
                                               1 if arr.flags.c_contiguous else 0, ptype, start_iteration, num_iteration, _param_str(kwargs),
                                               ctypes.byref(ln), out.ctypes.data_as(ctypes.c_void_p)))
        if pred_leaf:
            return out.astype(np.int32).reshape(nrow, -1)
        if out.size != nrow:
            return out.reshape(nrow, -1)
        return out

    def _predict_csr(self, csr: Any, ptype: int, start_iteration: int, num_iteration: int, pred_leaf: bool, pred_contrib: bool, kwargs: Dict[str, Any]) -> Any:
        lib = _lib()
        nrow, ncol = csr.shape
        indptr = np.ascontiguousarray(csr.indptr, dtype=np.int64 if csr.indptr.dtype == np.int64 else np.int32)
        indices = np.ascontiguousarray(csr.indices, dtype=np.int32)
        values = np.ascontiguousarray(csr.data, dtype=np.float32 if csr.data.dtype == np.float32 else np.float64)
        ptr_code = 8 if indptr.dtype == np.int64 else 7
        val_code = 0 if values.dtype == np.float32 else 1
        if pred_contrib:
            import scipy.sparse as sp

            lens = (ctypes.c_int64 * 2)(0, 0)
            optr, oidx, odat = ctypes.c_void_p(), ctypes.POINTER(ctypes.c_int32)(), ctypes.c_void_p()
            _safe_call(lib.FB_BoosterPredictSparseOutput(self._handle, indptr.ctypes.data_as(ctypes.c_void_p), ptr_code, indices.ctypes.data_as(ctypes.c_void_p),
                                                         values.ctypes.data_as(ctypes.c_void_p), val_code, ctypes.c_int64(len(indptr)), ctypes.c_int64(len(values)),
                                                         ctypes.c_int64(ncol), 3, start_iteration, num_iteration, _param_str(kwargs), 0, lens,
                                                         ctypes.byref(optr), ctypes.byref(oidx), ctypes.byref(odat)))
            nnz, nptr = int(lens[0]), int(lens[1])
            try:
                out_ptr = np.ctypeslib.as_array(ctypes.cast(optr, ctypes.POINTER(ctypes.c_int64 if ptr_code == 8 else ctypes.c_int32)), shape=(nptr,)).copy()
                out_idx = np.ctypeslib.as_array(oidx, shape=(max(nnz, 1),))[:nnz].copy()
                out_val = np.ctypeslib.as_array(ctypes.cast(odat, ctypes.POINTER(ctypes.c_float if val_code == 0 else ctypes.c_double)), shape=(max(nnz, 1),))[:nnz].copy()
            finally:
                _safe_call(lib.FB_BoosterFreePredictSparse(optr, oidx, odat))
            per_row = ctypes.c_int64(0)
            _safe_call(lib.FB_BoosterCalcNumPredict(self._handle, 1, 3, start_iteration, num_iteration, ctypes.byref(per_row)))
            return sp.csr_matrix((out_val, out_idx, out_ptr), shape=(nrow, int(per_row.value)))
        n_out = ctypes.c_int64(0)
        _safe_call(lib.FB_BoosterCalcNumPredict(self._handle, nrow, ptype, start_iteration, num_iteration, ctypes.byref(n_out)))
        out = np.empty(n_out.value, dtype=np.float64)
        ln = ctypes.c_int64(0)
        _safe_call(lib.FB_BoosterPredictForCSR(self._handle, indptr.ctypes.data_as(ctypes.c_void_p), ptr_code, indices.ctypes.data_as(ctypes.c_void_p),
                                               values.ctypes.data_as(ctypes.c_void_p), val_code, ctypes.c_int64(len(indptr)), ctypes.c_int64(len(values)), ctypes.c_int64(ncol),
                                               ptype, start_iteration, num_iteration, _param_str(kwargs), ctypes.byref(ln), out.ctypes.data_as(ctypes.c_void_p)))
        if pred_leaf:
            return out.astype(np.int32).reshape(nrow, -1)
        return out.reshape(nrow, -1) if out.size != nrow else out

    def _has_linear_trees(self) -> bool:
        if self.train_set is not None:   # a training booster knows from its parameters
            return _wants_linear(self.params or {})
        cached = getattr(self, "_linear_cache", None)
        n = self.num_trees()
        if cached is None or cached[0] != n:
            cached = (n, "is_linear=1" in self.model_to_string(num_iteration=-1))
            self._linear_cache = cached
        return cached[1]

    def refit(self, data: Any, label: Any, decay_rate: float = 0.9, **kwargs: Any) -> "Booster":
        leaf_preds = self.predict(data, pred_leaf=True).astype(np.int32)
        params = dict(self.params); params["refit_decay_rate"] = decay_rate; params["device_type"] = "cpu"
        params.setdefault("objective", self._objective_from_model())
        train = Dataset(data, label=label, params=params, **kwargs)
        new = Booster(params, train)
        new_handle = new._handle
        # move the trees of this model into the new booster, then refit leaf values on the new data
        _safe_call(_lib().FB_BoosterMerge(new_handle, self._handle))
        lp = np.ascontiguousarray(leaf_preds)
        _safe_call(_lib().FB_BoosterRefit(new_handle, lp.ctypes.data_as(ctypes.c_void_p), ctypes.c_int32(lp.shape[0]), ctypes.c_int32(lp.shape[1])))
        return new

    def _objective_from_model(self) -> str:
        for line in self.model_to_string(num_iteration=1).split("\n"):
            if line.startswith("objective="):
                return line[len("objective="):].split(" ")[0]
        return "regression"

    # -- model IO ---------------------------------------------------------------------
    def save_model(self, filename: Union[str, Path], num_iteration: Optional[int] = None, start_iteration: int = 0, importance_type: str = "split",
                   format: str = "txt", f32_leaves: bool = False, **_ignored: Any) -> "Booster":
        """Write the model as LightGBM-compatible text (``format="txt"``) or as compressed binary FALB (``format="falb"``)."""
        if num_iteration is None:
            num_iteration = self.best_iteration
        if format == "falb":
            Path(filename).write_bytes(self.model_to_binary(num_iteration, start_iteration, importance_type=importance_type, f32_leaves=f32_leaves,
                                                            **{k: v for k, v in _ignored.items() if k in ("with_stats", "with_diagnostics", "compress_level")})
                                       + _dump_pandas_categorical(self.pandas_categorical).encode("utf-8"))
            return self
        if format not in ("txt", "text"):
            raise ValueError("format must be 'txt' or 'falb'")
        _safe_call(_lib().FB_BoosterSaveModel(self._handle, start_iteration, num_iteration, 0 if importance_type == "split" else 1, str(filename).encode()))
        with open(filename, "a") as f:
            f.write(_dump_pandas_categorical(self.pandas_categorical))
        return self

    def model_to_string(self, num_iteration: Optional[int] = None, start_iteration: int = 0, importance_type: str = "split") -> str:
        if num_iteration is None:
            num_iteration = self.best_iteration
        return _get_string(_lib().FB_BoosterSaveModelToString, self._handle, start_iteration, num_iteration, 0 if importance_type == "split" else 1) + \
            _dump_pandas_categorical(self.pandas_categorical)

    def model_to_binary(self, num_iteration: Optional[int] = None, start_iteration: int = 0, importance_type: str = "split", with_stats: bool = False,
                        with_diagnostics: bool = False, f32_leaves: bool = False, compress_level: int = 6) -> bytes:
        """The model in the sectioned binary ``FALB`` container (readable by, and reading, the reference's files).

        ``with_stats`` adds per-node counts and weights (needed by ``pred_contrib``, ``trees_to_dataframe`` and
        ``dump_model``), ``with_diagnostics`` adds split gains and internal values (needed by gain importance);
        ``f32_leaves`` stores leaf values as float32 (lossy); ``compress_level`` is the zlib level, 0 = raw sections."""
        if num_iteration is None:
            num_iteration = self.best_iteration
        return _get_bytes(_lib().FB_BoosterSaveModelToBinary, self._handle, start_iteration, num_iteration, 0 if importance_type == "split" else 1,
                          1 if with_stats else 0, 1 if with_diagnostics else 0, 1 if f32_leaves else 0, int(compress_level))

    @classmethod
    def from_binary(cls, data: bytes) -> "Booster":
        self = cls.__new__(cls)
        self.params = {}; self.train_set = None; self.valid_sets = []; self.name_valid_sets = []; self.best_iteration = -1; self.best_score = {}
        self._train_data_name = "training"; self._network = False; self.pandas_categorical = None; self._eval_names = None; self._eval_higher = None
        self._handle = ctypes.c_void_p(); n_iter = ctypes.c_int(0)
        _safe_call(_lib().FB_BoosterCreateFromBinary(data, ctypes.c_int64(len(data)), ctypes.byref(n_iter), ctypes.byref(self._handle)))
        return self

    def model_from_string(self, model_str: str) -> "Booster":
        _lib().FB_BoosterFree(self._handle)
        self._handle = ctypes.c_void_p(); n_iter = ctypes.c_int(0)
        raw = model_str.encode("utf-8")
        _safe_call(_lib().FB_BoosterLoadModelFromString(raw, ctypes.c_int64(len(raw)), ctypes.byref(n_iter), ctypes.byref(self._handle)))
        return self

    def dump_model(self, num_iteration: Optional[int] = None, start_iteration: int = 0, importance_type: str = "split",
                   object_hook: Optional[Callable[[Dict[str, Any]], Dict[str, Any]]] = None) -> Dict[str, Any]:
        """The model as nested dicts; ``object_hook`` is handed to the JSON decoder (called on every decoded object)."""
        if num_iteration is None:
            num_iteration = self.best_iteration
        s = _get_string(_lib().FB_BoosterDumpModel, self._handle, start_iteration, num_iteration, 0 if importance_type == "split" else 1)
        return json.loads(s, object_hook=object_hook)

    def model_to_if_else(self, num_iteration: int = -1) -> str:
        return _get_string(_lib().FB_BoosterModelToIfElse, self._handle, num_iteration)

    def feature_importance(self, importance_type: str = "split", iteration: Optional[int] = None) -> np.ndarray:
        if iteration is None:
            iteration = self.best_iteration
        out = np.zeros(self.num_feature(), dtype=np.float64)
        _safe_call(_lib().FB_BoosterFeatureImportance(self._handle, iteration, 0 if importance_type == "split" else 1, out.ctypes.data_as(ctypes.c_void_p)))
        return out.astype(np.int32) if importance_type == "split" else out

    def get_leaf_output(self, tree_id: int, leaf_id: int) -> float:
        out = ctypes.c_double(0)
        _safe_call(_lib().FB_BoosterGetLeafValue(self._handle, tree_id, leaf_id, ctypes.byref(out)))
        return out.value

    def set_leaf_output(self, tree_id: int, leaf_id: int, value: float) -> "Booster":
        _safe_call(_lib().FB_BoosterSetLeafValue(self._handle, tree_id, leaf_id, ctypes.c_double(value)))
        return self

    def get_split_value_histogram(self, feature: Union[int, str], bins: Any = None, xgboost_style: bool = False) -> Any:
        """Histogram of the thresholds the model uses for one numerical feature (python-package/falcata/basic.py: Booster.get_split_value_histogram)."""
        names = self.feature_name()
        fidx = names.index(feature) if isinstance(feature, str) else int(feature)
        values: List[float] = []

        def walk(node: Dict[str, Any]) -> None:
            if "split_feature" not in node:
                return
            if int(node["split_feature"]) == fidx:
                if node.get("decision_type", "<=") != "<=":
                    raise ValueError("Cannot compute a split value histogram for a categorical feature")
                values.append(float(node["threshold"]))
            walk(node["left_child"])
            walk(node["right_child"])

        for t in self.dump_model()["tree_info"]:
            walk(t["tree_structure"])
        if bins is None or (isinstance(bins, int) and xgboost_style):
            n_unique = len(np.unique(values))
            bins = max(min(n_unique, bins) if bins is not None else n_unique, 1)
        hist, edges = np.histogram(values, bins=bins)
        if not xgboost_style:
            return hist, edges
        ret = np.column_stack((edges[1:], hist))
        ret = ret[ret[:, 1] > 0]
        try:
            import pandas as pd
            return pd.DataFrame(ret, columns=["SplitValue", "Count"])
        except ImportError:
            return ret

    def set_network(self, machines: Any, local_listen_port: int = 12400, listen_time_out: int = 120, num_machines: int = 1) -> "Booster":
        """Join the TCP mesh of a distributed CPU training (host learner): ``machines`` is "host:port,host:port,..." or a
        list of such strings, this process is the local entry that listens on ``local_listen_port``. Multi-GPU training
        does not use it: its ranks are torch.distributed processes set up by ``falcata_b200.parallel.init()``."""
        network_init(machines, local_listen_port, listen_time_out, num_machines)
        self._network = True
        return self

    def free_network(self) -> "Booster":
        _safe_call(_lib().FB_NetworkFree())
        self._network = False
        return self

    def model_from_binary(self, model_bin: Optional[bytes] = None, data: Optional[bytes] = None) -> "Booster":
        """Replace this Booster's model by one serialised with model_to_binary()."""
        other = Booster.from_binary(model_bin if model_bin is not None else data)
        return self.model_from_string(other.model_to_string())

    def shuffle_models(self, start_iteration: int = 0, end_iteration: int = -1) -> "Booster":
        _safe_call(_lib().FB_BoosterShuffleModels(self._handle, start_iteration, end_iteration))
        return self

    def trees_to_dataframe(self) -> Any:
        import pandas as pd

        model = self.dump_model()
        rows: List[Dict[str, Any]] = []

        def walk(tree_idx: int, node: Dict[str, Any], depth: int, parent: Optional[str]) -> None:
            if "split_index" in node:
                idx = f"{tree_idx}-S{node['split_index']}"
                rows.append({"tree_index": tree_idx, "node_depth": depth, "node_index": idx, "parent_index": parent,
                             "split_feature": model["feature_names"][node["split_feature"]], "split_gain": node["split_gain"],
                             "threshold": node["threshold"], "decision_type": node["decision_type"], "missing_type": node["missing_type"],
                             "value": node["internal_value"], "weight": node["internal_weight"], "count": node["internal_count"]})
                walk(tree_idx, node["left_child"], depth + 1, idx); walk(tree_idx, node["right_child"], depth + 1, idx)
            else:
                idx = f"{tree_idx}-L{node.get('leaf_index', 0)}"
                rows.append({"tree_index": tree_idx, "node_depth": depth, "node_index": idx, "parent_index": parent, "split_feature": None,
                             "split_gain": None, "threshold": None, "decision_type": None, "missing_type": None, "value": node["leaf_value"],
                             "weight": node.get("leaf_weight"), "count": node.get("leaf_count")})

        for t in model["tree_info"]:
            walk(t["tree_index"], t["tree_structure"], 1, None)
        return pd.DataFrame(rows)

    def gpu_launches(self) -> int:
        """Number of kernels this booster's device engine has launched so far."""
        out = ctypes.c_int64(0)
        _safe_call(_lib().FB_BoosterGpuLaunches(self._handle, ctypes.byref(out)))
        return out.value

    def stage_report(self) -> str:
        """Per-stage device time (CUDA events) accumulated by the device engine."""
        return _get_string(_lib().FB_BoosterStageReport, self._handle)

    def free_dataset(self) -> "Booster":
        self.train_set = None; self.valid_sets = []
        return self


_DATASET_PARAMS = {"max_bin", "min_data_in_bin", "bin_construct_sample_cnt", "data_random_seed", "enable_bundle", "use_missing", "zero_as_missing",
                   "feature_pre_filter", "categorical_feature", "max_bin_by_feature", "min_data_in_leaf", "device_type", "keep_host_bins"}
