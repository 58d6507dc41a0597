"""scikit-learn style wrapper and a standalone predictor.

``PackBoostRegressor(pack_size=..., max_depth=..., ...).fit(X, y, era=...)`` and
``.predict(X)`` follow the usage shown in the reference's README
(``README.md:93-101``); the reference tree ships no implementation of them, so
these are thin layers over ``PackBoost``.  ``PackBoostPredictor`` holds only what
inference needs (trees, bin edges, tree weight) and can be saved to / loaded
from a single ``.npz`` file.
"""

from __future__ import annotations

import dataclasses
from typing import Any, Iterable, Sequence

import numpy as np

from .config import PackBoostConfig
from .forest import validate_forest

_CONFIG_FIELDS = [f.name for f in dataclasses.fields(PackBoostConfig)]


class PackBoostRegressor:
    """Estimator with ``get_params`` / ``set_params`` / ``fit`` / ``predict`` / ``score``."""

    def __init__(self, num_rounds: int = 100, **config: Any) -> None:
        unknown = set(config) - set(_CONFIG_FIELDS)
        if unknown:
            raise TypeError(f"unknown PackBoost parameters: {sorted(unknown)}")
        self.num_rounds = int(num_rounds)
        self._params = dict(config)
        self.booster_ = None

    # -- scikit-learn parameter protocol --
    def get_params(self, deep: bool = True) -> dict[str, Any]:
        out = {"num_rounds": self.num_rounds}
        out.update(self._params)
        return out

    def set_params(self, **params: Any) -> "PackBoostRegressor":
        if "num_rounds" in params:
            self.num_rounds = int(params.pop("num_rounds"))
        unknown = set(params) - set(_CONFIG_FIELDS)
        if unknown:
            raise TypeError(f"unknown PackBoost parameters: {sorted(unknown)}")
        self._params.update(params)
        return self

    def fit(self, X, y, era: Iterable[int] | None = None, *, eval_set=None, log_evaluation: int | None = None,
            round_callback=None) -> "PackBoostRegressor":
        """``eval_set=(X_valid, y_valid, era_valid)`` adds a ``valid_corr`` entry to
        ``booster_.round_metrics``; ``log_evaluation=n`` prints it every ``n`` rounds."""
        from .booster import PackBoost
        self.booster_ = PackBoost(PackBoostConfig(**self._params))
        eval_sets = None
        if eval_set is not None:
            Xv, yv, ev = eval_set
            eval_sets = [("valid", Xv, yv, ev)]

        def cb(round_idx: int, metrics: dict[str, float]) -> None:
            if log_evaluation and (round_idx % int(log_evaluation) == 0):
                print({k: (round(v, 6) if isinstance(v, float) else v) for k, v in metrics.items()})
            if round_callback is not None:
                round_callback(round_idx, metrics)

        use_cb = cb if (log_evaluation or round_callback is not None) else None
        self.booster_.fit(X, y, era, num_rounds=self.num_rounds, eval_sets=eval_sets, round_callback=use_cb)
        return self

    def predict(self, X) -> np.ndarray:
        if self.booster_ is None:
            raise RuntimeError("Model must be fitted before predict()")
        return self.booster_.predict(X)

    def score(self, X, y) -> float:
        """Coefficient of determination R^2."""
        y = np.asarray(y, dtype=np.float64)
        p = self.predict(X).astype(np.float64)
        ss_res = float(((y - p) ** 2).sum())
        ss_tot = float(((y - y.mean()) ** 2).sum())
        return 1.0 - ss_res / ss_tot if ss_tot > 0 else 0.0

    def to_predictor(self) -> "PackBoostPredictor":
        if self.booster_ is None:
            raise RuntimeError("Model must be fitted first")
        return PackBoostPredictor.from_booster(self.booster_)


class PackBoostPredictor:
    """Inference-only model: distinct trees with repeat counts, bin edges and tree weight."""

    def __init__(self, trees: Sequence[dict[str, np.ndarray]], repeats: Sequence[int], tree_weight: float,
                 bin_edges: np.ndarray | None, max_bins: int, pack_size: int) -> None:
        self.trees = [{k: np.asarray(v) for k, v in t.items()} for t in trees]
        for t in self.trees:  # a malformed file is refused here, on the host
            validate_forest(t["feature"], t["threshold"], t["left"], t["right"], t["is_leaf"],
                            [0, t["feature"].shape[0]])
        self.repeats = [int(r) for r in repeats]
        if len(self.repeats) != len(self.trees) or any(r < 0 for r in self.repeats):
            raise ValueError("repeats must hold one non-negative count per tree")
        self.tree_weight = float(tree_weight)
        self.bin_edges = None if bin_edges is None else np.asarray(bin_edges, dtype=np.float32)
        self.max_bins = int(max_bins)
        self.pack_size = int(pack_size)
        self._booster = None

    @classmethod
    def from_booster(cls, booster) -> "PackBoostPredictor":
        booster.trees  # makes sure the last round's trees are materialised
        trees = [t.arrays() for t, _ in booster._distinct]
        reps = [r for _, r in booster._distinct]
        edges = booster._binner.bin_edges if booster._binner is not None else None
        return cls(trees, reps, booster._tree_weight, edges, booster.config.max_bins, booster.config.pack_size)

    # -- serialisation: one .npz with concatenated node arrays --
    def save(self, path: str) -> None:
        offs = np.zeros(len(self.trees) + 1, dtype=np.int64)
        np.cumsum([t["feature"].shape[0] for t in self.trees], out=offs[1:])
        cat = {k: np.concatenate([t[k] for t in self.trees]) if self.trees else np.zeros(0)
               for k in ("feature", "threshold", "left", "right", "value", "is_leaf")}
        np.savez_compressed(
            path, tree_offsets=offs, repeats=np.asarray(self.repeats, dtype=np.int32),
            tree_weight=np.float64(self.tree_weight), max_bins=np.int64(self.max_bins),
            pack_size=np.int64(self.pack_size), has_edges=np.bool_(self.bin_edges is not None),
            bin_edges=self.bin_edges if self.bin_edges is not None else np.zeros((0, 0), np.float32), **cat)

    @classmethod
    def load(cls, path: str) -> "PackBoostPredictor":
        z = np.load(path)
        offs = z["tree_offsets"]
        trees = []
        for i in range(len(offs) - 1):
            sl = slice(int(offs[i]), int(offs[i + 1]))
            trees.append({k: z[k][sl] for k in ("feature", "threshold", "left", "right", "value", "is_leaf")})
        edges = z["bin_edges"] if bool(z["has_edges"]) else None
        return cls(trees, z["repeats"].tolist(), float(z["tree_weight"]), edges, int(z["max_bins"]), int(z["pack_size"]))

    def _ensure_booster(self):
        if self._booster is None:
            from .booster import PackBoost, Tree, TreeNode
            b = PackBoost(PackBoostConfig(device="cuda", pack_size=self.pack_size, max_bins=self.max_bins,
                                          prebinned=self.bin_edges is None))
            trees = [Tree(nodes=[TreeNode(int(f), int(t), int(l), int(r), float(v), bool(il))
                                 for f, t, l, r, v, il in zip(d["feature"], d["threshold"], d["left"], d["right"],
                                                              d["value"], d["is_leaf"])]) for d in self.trees]
            b.set_forest(trees, self.tree_weight, bin_edges=self.bin_edges, repeats=self.repeats)
            self._booster = b
        return self._booster

    def predict(self, X) -> np.ndarray:
        return self._ensure_booster().predict(X)
