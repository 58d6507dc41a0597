"""Helpers shared by the GPU parity tests."""

import ctypes as C

import numpy as np
import torch

from packboost_b200 import backends as B
from packboost_b200.booster import PackBoost, _DeviceTrainer
from packboost_b200.config import PackBoostConfig
from packboost_b200.data import pack_feature_major


def flatten_trees(trees):
    off = [0]
    cols = {k: [] for k in ("feature", "threshold", "left", "right", "value", "is_leaf")}
    for t in trees:
        for n in t.nodes:
            cols["feature"].append(n.feature)
            cols["threshold"].append(n.threshold)
            cols["left"].append(n.left)
            cols["right"].append(n.right)
            cols["value"].append(n.value)
            cols["is_leaf"].append(n.is_leaf)
        off.append(len(cols["feature"]))
    return np.asarray(off), {
        "feature": np.asarray(cols["feature"], np.int32), "threshold": np.asarray(cols["threshold"], np.int32),
        "left": np.asarray(cols["left"], np.int32), "right": np.asarray(cols["right"], np.int32),
        "value": np.asarray(cols["value"], np.float64), "is_leaf": np.asarray(cols["is_leaf"], np.bool_)}


def flatten_oracle(trees):
    off = [0]
    cols = {k: [] for k in ("feature", "threshold", "left", "right", "value", "is_leaf")}
    for t in trees:
        for k in cols:
            cols[k].append(t[k])
        off.append(off[-1] + t["feature"].shape[0])
    return np.asarray(off), {k: np.concatenate(v) for k, v in cols.items()}


# Leaf values: float32 sums of ~N gradients carry a relative rounding noise of ~1e-6 in the CPU
# path (sequential float32 accumulation), while the GPU sums exactly in fixed point.  A value is
# -G/(H+lambda); when G nearly cancels, the noise is relative to sum|g|, not to |G|, hence the
# absolute term.  Tolerance: 1e-5 relative plus 1e-5 of the value scale of the tree.
def assert_values_close(got, want, is_leaf, scale=None):
    got = np.asarray(got, np.float64)[is_leaf]
    want = np.asarray(want, np.float64)[is_leaf]
    finite = np.isfinite(want) & (np.abs(want) < 1e30)
    s = np.abs(want[finite]).max() if scale is None and finite.any() else (scale or 1.0)
    np.testing.assert_allclose(got[finite], want[finite], rtol=1e-5, atol=1e-5 * s)
