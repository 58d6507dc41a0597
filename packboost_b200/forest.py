"""Host-side checks of an ensemble before it is handed to the predictor kernels.

Trees reach the device from outside ``fit`` as well (``PackBoost.set_forest``,
``PackBoostPredictor.load``, the array-based predictor bindings).  The kernels bound
every walk on their own, but a malformed ensemble is a caller error and is reported
here, on the host, before anything is launched (the reference bounds its walks in the
kernels only, ``packboost/backends/cuda/frontier_cuda.cu:214-231, 953-966``).
"""

from __future__ import annotations

import numpy as np


def validate_forest(feature, threshold, left, right, is_leaf, offsets, *, n_features: int | None = None,
                    absolute_children: bool = False) -> int:
    """Raise ``ValueError`` unless the concatenated node arrays describe proper trees.

    ``offsets[t]`` is the first node of tree ``t`` (``len(offsets) == n_trees + 1``).  For
    every internal node both children must lie inside the node's own tree and *after* the
    node (the numbering produced by ``TreeBuilder.split``: a split appends its children),
    which also rules out cycles; ``feature`` must be in ``[0, n_features)`` and ``threshold``
    in ``[0, 256)``.  Children are tree-relative unless ``absolute_children``.

    Returns the node count of the largest tree."""
    feature = np.asarray(feature)
    threshold = np.asarray(threshold)
    left = np.asarray(left).astype(np.int64)
    right = np.asarray(right).astype(np.int64)
    internal = np.asarray(is_leaf).astype(bool) == False  # noqa: E712
    offs = np.asarray(offsets).astype(np.int64)
    n = feature.shape[0]
    if not (threshold.shape[0] == left.shape[0] == right.shape[0] == internal.shape[0] == n):
        raise ValueError("forest arrays differ in length")
    if offs.ndim != 1 or offs.shape[0] < 1 or offs[0] != 0 or offs[-1] != n or np.any(np.diff(offs) < 0):
        raise ValueError("tree offsets must start at 0, end at the node count and not decrease")
    sizes = np.diff(offs)
    if sizes.size and sizes.min() < 1:
        raise ValueError("every tree needs at least one node")
    if n == 0:
        return 0
    tree_of = np.repeat(np.arange(sizes.shape[0]), sizes)
    first = offs[:-1][tree_of]
    rel = np.arange(n, dtype=np.int64) - first
    size_of = sizes[tree_of]
    if absolute_children:
        left = left - first
        right = right - first
    bad = internal & ((left <= rel) | (right <= rel) | (left >= size_of) | (right >= size_of))
    if bad.any():
        i = int(np.flatnonzero(bad)[0])
        raise ValueError(f"node {int(rel[i])} of tree {int(tree_of[i])}: children ({int(left[i])}, {int(right[i])}) "
                         f"must lie after the node and inside its tree of {int(size_of[i])} nodes")
    f_int = feature[internal]
    if f_int.size:
        if f_int.min() < 0 or (n_features is not None and f_int.max() >= n_features):
            raise ValueError(f"split feature outside [0, {n_features if n_features is not None else 'F'})")
        t_int = threshold[internal]
        if t_int.min() < 0 or t_int.max() >= 256:
            raise ValueError("split threshold outside [0, 256)")
    return int(sizes.max())
