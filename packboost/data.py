"""Alias of ``packboost_b200.data`` under the reference's module path (``packboost/data.py``)."""

from packboost_b200.data import (BinningResult, apply_bins, build_era_index, detect_prebinned,  # noqa: F401
                                 preprocess_features, quantile_bin)
