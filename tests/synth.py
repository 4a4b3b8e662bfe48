"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations
(they stand in for a real checkpoint: no dataset or evaluation suite is involved)."""
from __future__ import annotations

import numpy as np


def activations(rows: int, cols: int, seed: int, outlier_fraction: float = 0.005, outlier_scale: float = 20.0,
                outlier_columns: int | None = None, student_t: float | None = None) -> np.ndarray:
    """fp32 [rows, cols]: N(0,1) (or Student-t) with a few seeded outlier channels scaled up."""
    rng = np.random.default_rng(seed)
    x = rng.standard_t(student_t, size=(rows, cols)) if student_t else rng.standard_normal((rows, cols))
    count = outlier_columns if outlier_columns is not None else max(1, int(round(cols * outlier_fraction)))
    columns = rng.choice(cols, size=min(count, cols), replace=False)
    x[:, columns] *= outlier_scale
    return x.astype(np.float32)


def weights(rows: int, cols: int, seed: int, std: float = 0.02) -> np.ndarray:
    rng = np.random.default_rng(seed)
    return (rng.standard_normal((rows, cols)) * std).astype(np.float32)
