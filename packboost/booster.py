"""Alias of ``packboost_b200.booster`` under the reference's module path (``packboost/booster.py``)."""

from packboost_b200.booster import PackBoost, Tree, TreeBuilder, TreeNode  # noqa: F401
