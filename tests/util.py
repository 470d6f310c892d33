import numpy as np


def make_binary(n=10000, f=28, seed=0):
    rng = np.random.RandomState(seed)
    X = rng.randn(n, f).astype(np.float32)
    w = rng.randn(f)
    y = ((X @ w + 0.5 * rng.randn(n)) > 0).astype(np.float32)
    return X, y


def make_regression(n=5000, f=10, seed=0):
    rng = np.random.RandomState(seed)
    X = rng.randn(n, f).astype(np.float32)
    y = (np.sin(X[:, 0]) * 2 + X[:, 1] * X[:, 2] + 0.1 * rng.randn(n)).astype(np.float32)
    return X, y


def make_multiclass(n=6000, f=12, k=4, seed=0):
    rng = np.random.RandomState(seed)
    X = rng.randn(n, f).astype(np.float32)
    W = rng.randn(f, k)
    y = np.argmax(X @ W + rng.gumbel(size=(n, k)), axis=1).astype(np.float32)
    return X, y


def make_ranking(nq=200, docs=20, f=10, seed=0):
    rng = np.random.RandomState(seed)
    X = rng.rand(nq * docs, f).astype(np.float32)
    w = rng.randn(f)
    s = (X @ w + 0.3 * rng.randn(nq * docs)).reshape(nq, docs)
    rank = s.argsort(1).argsort(1)
    y = (rank * 5 // docs).astype(np.float32).reshape(-1)
    return X, y, np.full(nq, docs, dtype=np.int32)


def auc(y, p):
    order = np.argsort(p, kind="stable")
    r = np.empty(len(p)); r[order] = np.arange(1, len(p) + 1)
    pos = y > 0
    return (r[pos].sum() - pos.sum() * (pos.sum() + 1) / 2) / (pos.sum() * (~pos).sum())


def model_body(s):
    """Model text up to the parameter dump (device_type and friends differ between arms)."""
    return s.split("\nparameters:")[0]
