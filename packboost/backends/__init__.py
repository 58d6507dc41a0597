"""Alias of ``packboost_b200.backends`` under the reference's module path
(``packboost/backends/__init__.py``): the same seven dispatch names."""

from packboost_b200.backends import (cpu_available, cuda_available, find_best_splits_batched,  # noqa: F401
                                     find_best_splits_batched_cuda, partition_frontier_cuda, predict_bins_cuda,
                                     predict_pack_cuda)

__all__ = [
    "cpu_available",
    "find_best_splits_batched",
    "cuda_available",
    "find_best_splits_batched_cuda",
    "partition_frontier_cuda",
    "predict_bins_cuda",
    "predict_pack_cuda",
]
