"""Train, evaluate, save and reload a model through the Python API.

    python examples/quickstart.py                  # device engine when a GPU is visible, host learner otherwise
    python examples/quickstart.py --device cpu

Synthetic binary data (20 features, two interacting signals); prints the validation AUC per 10 rounds, the ten most
used features and checks that the reloaded model predicts like the trained one.
"""
from __future__ import annotations

import argparse
import os
import sys
import tempfile

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import falcata_b200 as fb   # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cuda" if fb.cuda_available() else "cpu", choices=["cuda", "cpu"])
    ap.add_argument("--rows", type=int, default=50_000)
    ap.add_argument("--rounds", type=int, default=50)
    args = ap.parse_args()

    rng = np.random.default_rng(0)
    X = rng.normal(size=(args.rows, 20)).astype(np.float32)
    logit = 1.5 * X[:, 0] - X[:, 1] * X[:, 2] + 0.5 * np.abs(X[:, 3])
    y = (rng.uniform(size=args.rows) < 1.0 / (1.0 + np.exp(-logit))).astype(np.float32)
    cut = args.rows * 4 // 5
    params = {"objective": "binary", "metric": "auc", "num_leaves": 63, "max_bin": 63, "learning_rate": 0.1, "device_type": args.device, "verbosity": -1}
    if args.device == "cuda":
        import torch

        params["quant_mode"] = "stochastic"                      # packed integer gradients: the fastest device path
        train = fb.Dataset(torch.as_tensor(X[:cut], device="cuda"), y[:cut])   # a CUDA tensor is binned on the device
    else:
        train = fb.Dataset(X[:cut], y[:cut])
    valid = fb.Dataset(X[cut:], y[cut:], reference=train)
    history: dict = {}
    booster = fb.train(params, train, args.rounds, valid_sets=[valid], valid_names=["valid"],
                       callbacks=[fb.log_evaluation(10), fb.record_evaluation(history), fb.early_stopping(20, verbose=False)])
    print(f"best iteration {booster.best_iteration}, validation AUC {history['valid']['auc'][booster.best_iteration - 1]:.4f}")
    order = np.argsort(-booster.feature_importance())[:10]
    print("most used features:", [int(i) for i in order])

    pred = np.asarray(booster.predict(X[cut:]))
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "model.txt")
        booster.save_model(path)
        again = np.asarray(fb.Booster(model_file=path).predict(X[cut:]))
    assert np.allclose(pred, again, atol=1e-7), "the reloaded model predicts differently"
    print("saved, reloaded, same predictions on", len(pred), "rows")


if __name__ == "__main__":
    main()
