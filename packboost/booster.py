"""Alias of ``packboost_b200.booster`` under the reference's module path (``packboost/booster.py``)."""

from packboost_b200.booster import NodeShard, PackBoost, SplitDecision, Tree, TreeBuilder, TreeNode  # noqa: F401
