"""The oracle against the reference's compiled C++ split finder (``oracle/_ref``, built from the
reference's own sources by ``oracle/build_ref.py``; skipped where it was not built)."""

import numpy as np
import pytest

import cases
from oracle import native_ref
from oracle import packboost_oracle as po

pytestmark = pytest.mark.skipif(not native_ref.available(), reason="oracle/_ref is not built")


def _same_structure(a, b):
    assert len(a.trees) == len(b.trees)
    for ta, tb in zip(a.trees, b.trees):
        for k in ("feature", "threshold", "left", "right"):
            np.testing.assert_array_equal(ta[k], tb[k], err_msg=k)


@pytest.mark.parametrize("name", ["config1", "interleaved", "ragged_eras", "prebinned5"])
def test_torch_frontier_port_and_compiled_split_finder_grow_the_same_trees(name):
    """Full threshold sweep, no directional term, no fall-through case: the two implementations of
    the reference agree, and so does the oracle with both."""
    X, y, era, cfg, rounds, _ = cases.CASES[name]()
    cfg = dict(cfg)
    cfg.update(direction_weight=0.0)
    a = po.fit(X, y, era, po.OracleParams(**cfg), min(rounds, 3))
    b = native_ref.fit(X, y, era, po.OracleParams(**cfg), min(rounds, 3))
    _same_structure(a, b)
    np.testing.assert_allclose(a.train_preds, b.train_preds, rtol=1e-4, atol=1e-5 * np.abs(b.train_preds).max())


@pytest.mark.parametrize("name,k", [("config1", 4), ("prebinned5", 2), ("ragged_eras", 7), ("interleaved", 5)])
def test_mass_cut_policy_is_pinned_by_the_compiled_split_finder(name, k):
    """``cut_selection="mass"`` runs only in the compiled split finder
    (``packboost/backends/cpu/frontier_cpu.cpp:59-109``; the torch frontier raises).  The oracle's
    restatement of the policy must choose the same thresholds: same trees."""
    X, y, era, cfg, rounds, _ = cases.CASES[name]()
    cfg = dict(cfg)
    cfg.update(k_cuts=k, cut_selection="mass", direction_weight=0.0)
    a = po.fit(X, y, era, po.OracleParams(native_mass_cuts=True, **cfg), rounds)
    b = native_ref.fit(X, y, era, po.OracleParams(**cfg), rounds)
    _same_structure(a, b)


def test_mass_and_even_cut_helpers_on_hand_cases():
    assert po.even_cuts_native(5, 2) == [0, 3]
    assert po.even_cuts_native(128, 4) == [0, 42, 84, 126]
    assert po.even_cuts_native(5, 1) == [0]
    # all mass in one bin: the quantile targets collapse onto one threshold, evenly spaced ids fill up
    assert po.mass_cuts_native(np.array([0, 0, 100, 0, 0]), 5, 3) == [0, 1, 2]
    assert po.mass_cuts_native(np.array([10, 10, 10, 10, 10]), 5, 4) == [0, 1, 2, 3]
    assert po.mass_cuts_native(np.zeros(5, dtype=np.int64), 5, 2) == [0, 3]


@pytest.mark.parametrize("name", ["dro_direction", "config1", "interleaved"])
def test_helper_form_direction_term_is_pinned_by_the_compiled_split_finder(name):
    """The ``+1 / -1`` directional term (``packboost/booster.py:869-907``) runs in the reference's
    native code (``frontier_cpu.cpp:395-401``), never in its torch frontier; the oracle's
    ``direction_form="helper"`` must grow the same trees as the compiled split finder."""
    X, y, era, cfg, rounds, _ = cases.CASES[name]()
    cfg = dict(cfg)
    cfg.update(direction_weight=0.2)
    a = po.fit(X, y, era, po.OracleParams(direction_form="helper", **cfg), min(rounds, 3))
    b = native_ref.fit(X, y, era, po.OracleParams(**cfg), min(rounds, 3))
    _same_structure(a, b)
