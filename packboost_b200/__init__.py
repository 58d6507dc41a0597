"""PackBoost on B200: pack-parallel gradient boosting with DES scoring, sm_100a backend."""

from .config import PackBoostConfig

__all__ = ["PackBoost", "PackBoostConfig", "PackBoostRegressor", "PackBoostPredictor"]


def __getattr__(name):
    # booster / wrapper import torch; keep ``import packboost_b200.workloads`` light
    if name == "PackBoost":
        from .booster import PackBoost
        return PackBoost
    if name in ("PackBoostRegressor", "PackBoostPredictor"):
        from . import wrapper
        return getattr(wrapper, name)
    raise AttributeError(name)
