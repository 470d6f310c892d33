"""Sparse oblique projection pool: random linear combinations of a few features, appended as columns.

Axis-aligned splits approximate ``y ~ f(w1*x1 + w2*x2)`` by staircases. A pool of K sparse projections drawn
once, evaluated on the raw matrix (on the GPU when the matrix is a CUDA tensor) and appended before binning
lets ordinary threshold splits act on such combinations; ``feature_fraction`` then gives per-tree diversity.
The pool has to be applied again at predict time, so it saves itself as JSON next to the model.

Choices: weights uniform in [-1, 1]; each projection takes ``density`` distinct features on average (at
least 2); features are centred by their median and scaled by their inter-quartile range (from a row sample)
so weights are comparable; inside a projection NaN is replaced by the feature's median (the original
columns keep their NaN).

Parity: python-package/falcata/oblique.py (ObliquePool L66: fit L107, transform L148, save L185, load L207).
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Any, List, Optional

import numpy as np

__all__ = ["ObliquePool"]


def _is_torch(x: Any) -> bool:
    return type(x).__module__.startswith("torch")


class ObliquePool:
    def __init__(self, num_projections: int = 256, density: float = 3.0, seed: int = 0, sample_rows: int = 100_000) -> None:
        if num_projections <= 0:
            raise ValueError("num_projections must be positive")
        if density < 1:
            raise ValueError("density must be >= 1")
        self.num_projections = int(num_projections); self.density = float(density); self.seed = int(seed); self.sample_rows = int(sample_rows)
        self.feature_idx_: Optional[List[np.ndarray]] = None
        self.weights_: Optional[List[np.ndarray]] = None
        self.center_: Optional[np.ndarray] = None
        self.scale_: Optional[np.ndarray] = None
        self.num_features_: Optional[int] = None

    # ---- fitting ----
    def fit(self, X: Any) -> "ObliquePool":
        """Draw the pool for a raw feature matrix (rows x features)."""
        n, p = X.shape
        if p < 2:
            raise ValueError("oblique projections need at least 2 features")
        rng = np.random.RandomState(self.seed)
        take = np.sort(rng.choice(n, size=min(n, self.sample_rows), replace=False))
        sample = X[take]
        sample = sample.detach().double().cpu().numpy() if _is_torch(sample) else np.asarray(sample, dtype=np.float64)
        q25, med, q75 = np.nanpercentile(sample, [25, 50, 75], axis=0)
        med = np.where(np.isnan(med), 0.0, med)
        iqr = np.where(np.isnan(q75 - q25) | ((q75 - q25) <= 0), 1.0, q75 - q25)
        self.center_, self.scale_, self.num_features_ = med, iqr, int(p)
        self.feature_idx_, self.weights_ = [], []
        for _ in range(self.num_projections):
            k = int(min(p, max(2, rng.geometric(1.0 / self.density))))
            idx = np.sort(rng.choice(p, size=k, replace=False))
            self.feature_idx_.append(idx.astype(np.int64)); self.weights_.append(rng.uniform(-1.0, 1.0, size=k))
        return self

    # ---- applying ----
    def _dense_weights(self) -> np.ndarray:
        W = np.zeros((self.num_features_, self.num_projections), dtype=np.float64)
        for j, (idx, w) in enumerate(zip(self.feature_idx_, self.weights_)):
            W[idx, j] = w
        return W

    def transform(self, X: Any, dtype: Any = None) -> Any:
        """X with the K projection columns appended (same container type and device as X)."""
        if self.feature_idx_ is None:
            raise RuntimeError("fit() the pool first")
        if X.shape[1] != self.num_features_:
            raise ValueError(f"the pool was fitted on {self.num_features_} features, got {X.shape[1]}")
        W = self._dense_weights() / self.scale_[:, None]
        if _is_torch(X):
            import torch

            dt = dtype or X.dtype
            c = torch.as_tensor(self.center_, device=X.device, dtype=torch.float32)
            Z = torch.where(torch.isnan(X), c, X.float()) - c
            z = Z @ torch.as_tensor(W, device=X.device, dtype=torch.float32)
            return torch.cat([X.to(dt), z.to(dt)], dim=1)
        Xn = np.asarray(X)
        dt = dtype or (Xn.dtype if Xn.dtype.kind == "f" else np.float64)
        Z = np.where(np.isnan(Xn), self.center_, Xn).astype(np.float64) - self.center_
        return np.concatenate([Xn.astype(dt), (Z @ W).astype(dt)], axis=1)

    def fit_transform(self, X: Any, dtype: Any = None) -> Any:
        return self.fit(X).transform(X, dtype)

    def feature_names(self, base_names: Optional[List[str]] = None) -> List[str]:
        base = list(base_names) if base_names else [f"Column_{i}" for i in range(self.num_features_)]
        return base + [f"oblique_{j}" for j in range(self.num_projections)]

    # ---- persistence ----
    def save(self, path: Any) -> None:
        blob = {"version": 1, "num_projections": self.num_projections, "density": self.density, "seed": self.seed, "sample_rows": self.sample_rows,
                "num_features": self.num_features_, "center": self.center_.tolist(), "scale": self.scale_.tolist(),
                "feature_idx": [i.tolist() for i in self.feature_idx_], "weights": [w.tolist() for w in self.weights_]}
        Path(path).write_text(json.dumps(blob))

    @classmethod
    def load(cls, path: Any) -> "ObliquePool":
        b = json.loads(Path(path).read_text())
        self = cls(b["num_projections"], b["density"], b["seed"], b["sample_rows"])
        self.num_features_ = int(b["num_features"]); self.center_ = np.asarray(b["center"], dtype=np.float64); self.scale_ = np.asarray(b["scale"], dtype=np.float64)
        self.feature_idx_ = [np.asarray(i, dtype=np.int64) for i in b["feature_idx"]]; self.weights_ = [np.asarray(w, dtype=np.float64) for w in b["weights"]]
        return self
