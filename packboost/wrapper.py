"""Alias of ``packboost_b200.wrapper`` (the estimator and predictor named in the reference's README)."""

from packboost_b200.wrapper import PackBoostPredictor, PackBoostRegressor  # noqa: F401
