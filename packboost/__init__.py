"""``packboost``: the import name of the reference project, served by the B200 backend.

Code written against the reference (``from packboost import PackBoost, PackBoostConfig``,
``from packboost.booster import ...``, ``from packboost.data import apply_bins``,
``from packboost.backends import cuda_available``) imports unchanged; every name is the
object of the same name in ``packboost_b200``.
"""

from packboost_b200 import PackBoostConfig

__all__ = ["PackBoost", "PackBoostConfig", "PackBoostRegressor", "PackBoostPredictor"]


def __getattr__(name):
    import packboost_b200
    if name in __all__:
        return getattr(packboost_b200, name)
    raise AttributeError(name)
