"""Writes the tab-separated files used by the command-line examples (label in the first column)."""
import os

import numpy as np

here = os.path.dirname(os.path.abspath(__file__))
rng = np.random.default_rng(1)
X = rng.normal(size=(20000, 10))
y = (X[:, 0] + X[:, 1] * X[:, 2] + 0.3 * rng.normal(size=len(X)) > 0).astype(int)
data = np.column_stack([y, X])
np.savetxt(os.path.join(here, "train.tsv"), data[:16000], delimiter="\t", fmt="%.9g")
np.savetxt(os.path.join(here, "valid.tsv"), data[16000:], delimiter="\t", fmt="%.9g")
print("wrote train.tsv (16000 rows) and valid.tsv (4000 rows) to", here)
