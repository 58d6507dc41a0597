"""Seeded synthetic workloads with the shapes of the five benchmark configurations.

The reference measures on the Numerai training table, which is not shipped; the
generators below stand in for it (same shapes, bin counts, era structure and
signal strength).  All of them are driven by ``np.random.default_rng(seed)`` so
that tests, the golden-fixture script and the benchmark see identical inputs.
Every generator takes scale arguments so that tests can use reduced sizes.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import numpy as np


@dataclass
class Workload:
    name: str
    X: np.ndarray
    y: np.ndarray
    era: np.ndarray | None
    config: dict[str, Any]
    num_rounds: int
    notes: str = ""
    extra: dict[str, Any] = field(default_factory=dict)


def config1(seed: int = 42, n_rows: int = 20_000, n_features: int = 64, n_eras: int = 20,
            num_rounds: int = 20) -> Workload:
    """CPU-runnable regression: N(0,1) features, smooth non-linear target,
    contiguous eras, 128 quantile bins."""
    rng = np.random.default_rng(seed)
    X = rng.standard_normal((n_rows, n_features)).astype(np.float32)
    y = (np.sin(X[:, 0]) + 0.5 * X[:, 1] * X[:, 2] + 0.3 * X[:, 3] ** 2
         + rng.normal(0.0, 0.1, n_rows)).astype(np.float32)
    era = np.repeat(np.arange(n_eras, dtype=np.int16), n_rows // n_eras)
    era = np.concatenate([era, np.full(n_rows - era.shape[0], n_eras - 1, dtype=np.int16)])
    cfg = dict(pack_size=8, max_depth=5, learning_rate=0.05, lambda_l2=1.0, lambda_dro=0.5,
               min_samples_leaf=20, max_bins=128, random_state=42)
    return Workload("config1", X, y, era, cfg, num_rounds)


def config2(seed: int = 7, n_rows: int = 500_000, n_features: int = 256, n_eras: int = 100,
            num_rounds: int = 100) -> Workload:
    """Mixed Gaussian / log-normal / integer-valued columns; sparse linear target
    with pairwise interactions whose sign flips on 30 % of the eras."""
    rng = np.random.default_rng(seed)
    n_gauss = n_features // 2
    n_int = max(1, int(round(0.1 * n_features)))
    n_logn = n_features - n_gauss - n_int
    X = np.empty((n_rows, n_features), dtype=np.float32)
    X[:, :n_gauss] = rng.standard_normal((n_rows, n_gauss), dtype=np.float32)
    X[:, n_gauss:n_gauss + n_logn] = np.exp(rng.standard_normal((n_rows, n_logn), dtype=np.float32))
    X[:, n_gauss + n_logn:] = rng.integers(0, 10, size=(n_rows, n_int)).astype(np.float32)
    per_era = n_rows // n_eras
    era = np.minimum(np.arange(n_rows) // max(per_era, 1), n_eras - 1).astype(np.int16)
    lin_idx = rng.choice(n_features, size=min(16, n_features), replace=False)
    lin_w = rng.normal(0.0, 1.0, lin_idx.shape[0]).astype(np.float32)
    pairs = rng.choice(n_features, size=(4, 2), replace=True)
    pair_w = rng.normal(0.0, 0.5, 4).astype(np.float32)
    sign = np.where(rng.random(n_eras) < 0.3, -1.0, 1.0).astype(np.float32)
    Xs = (X - X.mean(0, keepdims=True)) / (X.std(0, keepdims=True) + 1e-6)
    signal = Xs[:, lin_idx] @ lin_w
    for (a, b), w in zip(pairs, pair_w):
        signal = signal + w * Xs[:, a] * Xs[:, b]
    y = (sign[era] * signal + rng.normal(0.0, 0.5, n_rows)).astype(np.float32)
    cfg = dict(pack_size=16, max_depth=6, learning_rate=0.4 / 16, lambda_l2=1e-6, lambda_dro=0.5,
               min_samples_leaf=20, max_bins=128, random_state=42)
    return Workload("config2", X, y, era, cfg, num_rounds,
                    notes="learning_rate fixed at 0.4/pack_size: the pack is summed, not averaged")


def config3_target(codes_sel: np.ndarray, era: np.ndarray, n_eras: int, rng: np.random.Generator) -> np.ndarray:
    """Five-level target from a weak per-era linear latent (correlation ~0.02)."""
    w = rng.normal(0.02, 0.02, size=(n_eras, codes_sel.shape[1])).astype(np.float32)
    centred = codes_sel.astype(np.float32) - 2.0
    latent = np.einsum("nf,nf->n", centred, w[era])
    latent = latent + rng.normal(0.0, 1.0, codes_sel.shape[0]).astype(np.float32) * (
        np.std(latent) / 0.02 if np.std(latent) > 0 else 1.0)
    ranks = np.argsort(np.argsort(latent, kind="stable"), kind="stable")
    return (np.floor(ranks * 5.0 / codes_sel.shape[0]).clip(0, 4) * 0.25).astype(np.float32)


def config3(seed: int = 3, n_rows: int = 2_700_000, n_features: int = 2376, n_eras: int = 574,
            num_rounds: int = 1000) -> Workload:
    """Era-heavy wide table: uint8 codes in {0..4}, ~4 700 rows per era, weak
    signal.  At full size the matrix is 6.4 GB; callers that only need the shape
    on a GPU should use ``config3_device`` instead."""
    rng = np.random.default_rng(seed)
    X = rng.integers(0, 5, size=(n_rows, n_features), dtype=np.uint8)
    era = (np.arange(n_rows, dtype=np.int64) * n_eras // n_rows).astype(np.int16)
    sel = rng.choice(n_features, size=min(50, n_features), replace=False)
    y = config3_target(X[:, sel], era, n_eras, rng)
    cfg = dict(pack_size=32, max_depth=6, learning_rate=0.4 / 32, lambda_l2=1e-6, lambda_dro=0.5,
               min_samples_leaf=20, max_bins=5, layer_feature_fraction=0.1, prebinned=True,
               random_state=42)
    return Workload("config3", X, y, era, cfg, num_rounds,
                    notes="learning_rate fixed at 0.4/pack_size: the pack is summed, not averaged")


def config3_device(n_rows: int = 2_700_000, n_features: int = 2376, n_eras: int = 574, device=None, seed: int = 3):
    """The config-3 table generated on a GPU (same shape, bin count, era structure and signal
    strength as :func:`config3`, from the device generator): ``(X uint8 [n, F], y float32 [n],
    era int16 [n])`` as device tensors."""
    import torch
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    X = torch.empty((n_rows, n_features), dtype=torch.uint8, device=device)
    step = 1 << 18
    for a in range(0, n_rows, step):
        b = min(n_rows, a + step)
        X[a:b] = torch.randint(0, 5, (b - a, n_features), generator=g, device=device, dtype=torch.uint8)
    era = (torch.arange(n_rows, device=device, dtype=torch.int64) * n_eras // n_rows)
    sel = torch.randperm(n_features, generator=g, device=device)[:50]
    w = 0.02 + 0.02 * torch.randn((n_eras, 50), generator=g, device=device)
    latent = ((X[:, sel].float() - 2.0) * w[era]).sum(1)
    latent = latent + torch.randn(n_rows, generator=g, device=device) * (latent.std() / 0.02)
    ranks = torch.argsort(torch.argsort(latent))
    y = (torch.floor(ranks.float() * 5.0 / n_rows).clamp_(0, 4) * 0.25).float()
    return X, y, era.to(torch.int16)


def config4(seed: int = 11, n_rows: int = 1_000_000, n_features: int = 500, n_eras: int = 200,
            num_rounds: int = 200, max_bins: int = 128, tree_depth: int = 8) -> Workload:
    """Deep frontier: target is a seeded random depth-8 tree over the features."""
    rng = np.random.default_rng(seed)
    X = rng.standard_normal((n_rows, n_features), dtype=np.float32)
    per_era = max(n_rows // n_eras, 1)
    era = np.minimum(np.arange(n_rows) // per_era, n_eras - 1).astype(np.int16)
    n_internal = (1 << tree_depth) - 1
    t_feat = rng.integers(0, n_features, n_internal)
    t_thr = rng.normal(0.0, 0.7, n_internal).astype(np.float32)
    leaf_val = rng.normal(0.0, 1.0, 1 << tree_depth).astype(np.float32)
    node = np.zeros(n_rows, dtype=np.int64)
    for _ in range(tree_depth):
        go_right = X[np.arange(n_rows), t_feat[node]] > t_thr[node]
        node = 2 * node + 1 + go_right
    y = (leaf_val[node - n_internal] + rng.normal(0.0, 0.2, n_rows)).astype(np.float32)
    cfg = dict(pack_size=64, max_depth=10, learning_rate=0.4 / 64, lambda_l2=1e-6, lambda_dro=0.5,
               min_samples_leaf=20, max_bins=max_bins, random_state=42)
    return Workload("config4", X, y, era, cfg, num_rounds,
                    notes="max_bins=128 is the reference's limit; 255 needs the widened oracle")


def config5(seed: int = 5, n_rows: int = 5_000_000, n_features: int = 2376, n_rounds: int = 2000,
            pack_size: int = 32, depth: int = 6) -> Workload:
    """Inference only: complete random trees over 5-level codes.

    ``extra`` holds the ensemble as heap-ordered arrays ``feature [T, 2^d-1]``,
    ``threshold [T, 2^d-1]`` and ``leaf [T, 2^d]``."""
    rng = np.random.default_rng(seed)
    n_trees = n_rounds * pack_size
    n_int = (1 << depth) - 1
    feature = rng.integers(0, n_features, size=(n_trees, n_int), dtype=np.int32)
    threshold = rng.integers(0, 4, size=(n_trees, n_int), dtype=np.int32)
    leaf = rng.normal(0.0, 0.01, size=(n_trees, 1 << depth)).astype(np.float32)
    X = rng.integers(0, 5, size=(n_rows, n_features), dtype=np.uint8)
    cfg = dict(pack_size=pack_size, max_depth=depth, max_bins=5, prebinned=True, learning_rate=1.0)
    return Workload("config5", X, np.zeros(n_rows, dtype=np.float32), None, cfg, 0,
                    extra=dict(feature=feature, threshold=threshold, leaf=leaf, depth=depth))


def heap_ensemble_to_trees(feature: np.ndarray, threshold: np.ndarray, leaf: np.ndarray) -> list[dict[str, np.ndarray]]:
    """Complete heap-ordered trees -> the per-tree array dictionaries used by the
    predictor (node i has children 2i+1 and 2i+2; the last level holds leaves)."""
    n_trees, n_int = feature.shape
    n_leaf = leaf.shape[1]
    total = n_int + n_leaf
    idx = np.arange(n_int, dtype=np.int32)
    out = []
    for t in range(n_trees):
        out.append({
            "feature": np.concatenate([feature[t], np.full(n_leaf, -1, np.int32)]).astype(np.int32),
            "threshold": np.concatenate([threshold[t], np.zeros(n_leaf, np.int32)]).astype(np.int32),
            "left": np.concatenate([2 * idx + 1, np.full(n_leaf, -1, np.int32)]).astype(np.int32),
            "right": np.concatenate([2 * idx + 2, np.full(n_leaf, -1, np.int32)]).astype(np.int32),
            "value": np.concatenate([np.zeros(n_int), leaf[t].astype(np.float64)]),
            "is_leaf": np.concatenate([np.zeros(n_int, bool), np.ones(n_leaf, bool)]),
        })
        assert out[-1]["feature"].shape[0] == total
    return out
