"""Hyper-parameters of PackBoost training.

Field names, order and defaults follow the reference configuration object
(``packboost/config.py:68-90``) so that existing call sites construct it
unchanged.  ``era_tile_size``, ``histogram_mode`` and ``enable_node_batching``
never influence the arithmetic there either; they are accepted and ignored.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Literal


@dataclass(frozen=True, slots=True)
class PackBoostConfig:
    pack_size: int = 8
    max_depth: int = 6
    learning_rate: float = 0.1
    lambda_l2: float = 1e-6
    lambda_dro: float = 0.0
    direction_weight: float = 0.0
    min_samples_leaf: int = 20
    max_bins: int = 63
    k_cuts: int = 0
    cut_selection: Literal["even", "mass"] = "mass"
    layer_feature_fraction: float = 1.0
    era_alpha: float = 0.0
    era_tile_size: int = 32
    histogram_mode: Literal["rebuild", "subtract", "auto"] = "rebuild"
    feature_block_size: int = 32
    enable_node_batching: bool = True
    random_state: int | None = None
    device: str = "cuda"
    prebinned: bool = False
