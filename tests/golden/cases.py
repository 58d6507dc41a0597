"""Seeded parity cases shared by the golden-fixture generator and the tests.

Each case is ``(X, y, era, config-dict, num_rounds, X_holdout)``.  The generator
(`make_golden.py`) feeds them to the unmodified reference; the tests feed the
same inputs to the oracle and to the CUDA path.
"""

from __future__ import annotations

import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from packboost_b200 import workloads  # noqa: E402


def _linear(seed, n_rows, n_features, n_eras, shuffle_eras=True):
    rng = np.random.default_rng(seed)
    X = rng.normal(size=(n_rows, n_features)).astype(np.float32)
    coefs = rng.normal(size=n_features).astype(np.float32)
    y = (X @ coefs + 0.1 * rng.standard_normal(n_rows)).astype(np.float32)
    eras = np.arange(n_rows, dtype=np.int16) % n_eras
    if shuffle_eras:
        rng.shuffle(eras)
    Xh = rng.normal(size=(64, n_features)).astype(np.float32)
    return X, y, eras, Xh


def case_config1():
    w = workloads.config1()
    rng = np.random.default_rng(1001)
    Xh = rng.standard_normal((512, w.X.shape[1])).astype(np.float32)
    return w.X, w.y, w.era, w.config, w.num_rounds, Xh


def case_interleaved():
    X, y, eras, Xh = _linear(123, 320, 12, 8)
    cfg = dict(pack_size=2, max_depth=4, learning_rate=0.15, min_samples_leaf=8, max_bins=63, random_state=3)
    return X, y, eras, cfg, 3, Xh


def case_dro_direction():
    X, y, eras, Xh = _linear(5, 600, 6, 10)
    cfg = dict(pack_size=3, max_depth=4, learning_rate=0.1, lambda_l2=0.5, lambda_dro=0.3,
               direction_weight=0.2, era_alpha=1.5, min_samples_leaf=5, max_bins=31,
               layer_feature_fraction=0.6, random_state=11)
    return X, y, eras, cfg, 4, Xh


def case_kcuts_even():
    X, y, eras, Xh = _linear(77, 800, 10, 6)
    cfg = dict(pack_size=2, max_depth=3, learning_rate=0.1, lambda_l2=1e-3, lambda_dro=0.2,
               min_samples_leaf=6, max_bins=63, k_cuts=7, cut_selection="even", random_state=2)
    return X, y, eras, cfg, 3, Xh


# ``k_cuts > 0`` with ``cut_selection="mass"`` has no case: the reference's torch
# frontier raises "Index tensor must have the same number of dimensions as input
# tensor" when it maps the winner back to a threshold (``packboost/booster.py:1940``),
# so there is no reference behaviour to pin.


def case_prebinned5():
    """Small stand-in for the era-heavy five-level table (96 features, 40 eras,
    10 % of the features sampled per depth -> several 32-feature blocks do not
    arise, so the fraction is raised to 0.5 to exercise two blocks)."""
    w = workloads.config3(seed=9, n_rows=20_000, n_features=96, n_eras=40, num_rounds=4)
    cfg = dict(w.config)
    cfg.update(pack_size=4, learning_rate=0.1, layer_feature_fraction=0.5)
    rng = np.random.default_rng(1002)
    Xh = rng.integers(0, 5, size=(256, 96), dtype=np.uint8)
    return w.X, w.y, w.era, cfg, 4, Xh


def case_fallthrough():
    """No candidate satisfies ``min_samples_leaf``: every score is -inf and the
    reference still splits on the largest left count (possibly leaving an empty
    child)."""
    rng = np.random.default_rng(31)
    X = rng.integers(0, 5, size=(100, 2), dtype=np.uint8)
    X[:, 0] = np.where(np.arange(100) < 97, 1, 3)
    X[:, 1] = np.where(np.arange(100) < 3, 0, 3)
    y = rng.normal(size=100).astype(np.float32)
    eras = (np.arange(100) % 4).astype(np.int16)
    cfg = dict(pack_size=2, max_depth=2, learning_rate=0.1, lambda_l2=1e-3, min_samples_leaf=50,
               max_bins=5, prebinned=True, random_state=1)
    Xh = rng.integers(0, 5, size=(32, 2), dtype=np.uint8)
    return X, y, eras, cfg, 2, Xh


def case_era_none():
    X, y, _, Xh = _linear(41, 500, 8, 1)
    cfg = dict(pack_size=2, max_depth=3, learning_rate=0.2, lambda_l2=1e-3, min_samples_leaf=10,
               max_bins=16, random_state=4)
    return X, y, None, cfg, 3, Xh


def case_ragged_eras():
    """Unequal, non-contiguous eras with gaps in the era ids and one tiny era."""
    rng = np.random.default_rng(99)
    n = 1500
    X = rng.normal(size=(n, 9)).astype(np.float32)
    y = (np.tanh(X[:, 0]) - X[:, 4] * X[:, 5] + 0.2 * rng.standard_normal(n)).astype(np.float32)
    eras = rng.choice(np.array([3, 4, 9, 17, 40, 41], dtype=np.int16), size=n,
                      p=[0.4, 0.25, 0.2, 0.1, 0.048, 0.002])
    cfg = dict(pack_size=2, max_depth=5, learning_rate=0.1, lambda_l2=0.1, lambda_dro=0.5,
               min_samples_leaf=7, max_bins=128, layer_feature_fraction=0.7, random_state=8)
    Xh = rng.normal(size=(64, 9)).astype(np.float32)
    return X, y, eras, cfg, 4, Xh


def case_config3_wide():
    """The era-heavy five-level table at its full width (2 376 features, 10 % sampled per depth =
    238 features = eight 32-feature blocks, pack of 32) with a tenth of the rows and eras."""
    w = workloads.config3(seed=3, n_rows=270_000, n_features=2376, n_eras=57, num_rounds=2)
    rng = np.random.default_rng(1003)
    Xh = rng.integers(0, 5, size=(256, 2376), dtype=np.uint8)
    return w.X, w.y, w.era, dict(w.config), 2, Xh


def case_config2_full():
    """The mixed-column configuration at full size (500 000 x 256, 128 bins, 100 eras, pack of 16)."""
    w = workloads.config2()
    rng = np.random.default_rng(1004)
    Xh = w.X[rng.choice(w.X.shape[0], size=512, replace=False)] + 0.0
    return w.X, w.y, w.era, dict(w.config), 2, Xh


def case_config4_deep():
    """Deep frontier at the real width: 500 features, depth 10 (up to 512 live nodes), 128 bins;
    rows and eras cut so that the CPU path finishes in minutes."""
    w = workloads.config4(seed=11, n_rows=100_000, n_features=500, n_eras=10, num_rounds=2, max_bins=128)
    cfg = dict(w.config)
    cfg.update(pack_size=8, learning_rate=0.05)
    rng = np.random.default_rng(1005)
    Xh = rng.standard_normal((256, 500)).astype(np.float32)
    return w.X, w.y, w.era, cfg, 2, Xh


CASES = {
    "config1": case_config1,
    "interleaved": case_interleaved,
    "dro_direction": case_dro_direction,
    "kcuts_even": case_kcuts_even,
    "prebinned5": case_prebinned5,
    "fallthrough": case_fallthrough,
    "era_none": case_era_none,
    "ragged_eras": case_ragged_eras,
}


# Cases at the widths of the benchmark configurations.  The reference needs minutes for them, so
# only the CUDA path is compared with their fixtures (and the oracle with the first one).
WIDE_CASES = {
    "config3_wide": case_config3_wide,
    "config2_full": case_config2_full,
    "config4_deep": case_config4_deep,
}


def des_known_answer_inputs():
    """The six-row, one-feature, two-era node of the reference's DES test
    (general hessians, four bins)."""
    grad = np.array([0.5, -0.2, 0.1, -0.3, 0.4, -0.1], dtype=np.float32)
    hess = np.array([1.0, 0.8, 1.2, 1.0, 0.9, 1.1], dtype=np.float32)
    codes = np.array([[0], [1], [1], [2], [2], [3]], dtype=np.int64)
    era_rows = [np.array([0, 1], dtype=np.int64), np.array([2, 3, 4, 5], dtype=np.int64)]
    cfg = dict(max_bins=4, min_samples_leaf=1, lambda_l2=0.5, lambda_dro=0.1, direction_weight=0.2)
    return grad, hess, codes, era_rows, cfg


def inference_case():
    """Small stand-in for the inference-only configuration."""
    w = workloads.config5(seed=5, n_rows=3000, n_features=2376, n_rounds=3, pack_size=16, depth=6)
    return w
