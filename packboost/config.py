"""Alias of ``packboost_b200.config`` under the reference's module path (``packboost/config.py``)."""

from packboost_b200.config import *  # noqa: F401,F403
from packboost_b200.config import PackBoostConfig  # noqa: F401
