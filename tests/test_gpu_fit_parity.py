"""End-to-end parity of the CUDA path with the reference (golden fixtures) and the oracle.

Split structure (feature, threshold, children, leaf flags) must match exactly; leaf values and
predictions within 1e-5 relative (see ``gpu_util.assert_values_close`` for the absolute term).
"""

import os

import numpy as np
import pytest
import torch

import cases
from gpu_util import (assert_values_close, flatten_oracle, flatten_trees, populated_leaves,
                      rows_avoiding_empty_leaves)
from oracle import packboost_oracle as po

pytestmark = pytest.mark.gpu

GOLD = os.path.dirname(os.path.abspath(cases.__file__))


def _fit_gpu(X, y, era, cfg, rounds):
    from packboost_b200 import PackBoost, PackBoostConfig
    booster = PackBoost(PackBoostConfig(device="cuda", **cfg))
    booster.fit(X, y, era, num_rounds=rounds)
    return booster


@pytest.mark.parametrize("name", list(cases.CASES))
def test_fit_matches_reference_golden(name):
    X, y, era, cfg, rounds, Xh = cases.CASES[name]()
    gold = np.load(os.path.join(GOLD, f"{name}.npz"))
    booster = _fit_gpu(X, y, era, cfg, rounds)
    off, cols = flatten_trees(booster.trees)
    np.testing.assert_array_equal(off, gold["tree_offsets"])
    for k in ("feature", "threshold", "left", "right", "is_leaf"):
        np.testing.assert_array_equal(cols[k], gold[k], err_msg=k)
    # children that received no training row carry float-noise values in the reference: excluded
    gcols = {k: gold[k] for k in cols}
    p = po.OracleParams(**cfg)
    codes_train, edges = po.preprocess(X, p)
    populated = populated_leaves(off, gcols, codes_train)
    assert_values_close(cols["value"], gold["value"], gold["is_leaf"] & populated)
    scale = np.abs(gold["pred_train_head"]).max() + 1e-12
    np.testing.assert_allclose(booster.predict(X[:2048]), gold["pred_train_head"], rtol=1e-5, atol=1e-5 * scale)
    ok = rows_avoiding_empty_leaves(off, gcols, populated, po.apply_bins(Xh, edges, cfg["max_bins"]))
    np.testing.assert_allclose(booster.predict(Xh)[ok], gold["pred_holdout"][ok], rtol=1e-5, atol=1e-5 * scale)
    # the prediction state kept during training equals predict() on the training rows
    np.testing.assert_allclose(booster.train_predictions()[:2048], booster.predict(X[:2048]), rtol=1e-5,
                               atol=1e-5 * scale)


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_fit_matches_oracle_fresh_seeds(seed):
    rng = np.random.default_rng(seed)
    n, f, e = 3000, 20, 12
    X = rng.normal(size=(n, f)).astype(np.float32)
    X[:, 3] = np.round(X[:, 3])            # heavy ties -> empty bins -> equal-score candidates
    X[:, 7] = (X[:, 7] > 0).astype(np.float32)
    y = (X[:, 0] * X[:, 1] + np.sin(X[:, 2]) + 0.3 * rng.standard_normal(n)).astype(np.float32)
    era = rng.integers(0, e, size=n).astype(np.int16)
    cfg = dict(pack_size=4, max_depth=5, learning_rate=0.05, lambda_l2=1.0, lambda_dro=0.5, min_samples_leaf=10,
               max_bins=64, layer_feature_fraction=0.8, random_state=seed)
    model = po.fit(X, y, era, po.OracleParams(**cfg), 5)
    booster = _fit_gpu(X, y, era, cfg, 5)
    off_o, cols_o = flatten_oracle(model.trees)
    off_g, cols_g = flatten_trees(booster.trees)
    np.testing.assert_array_equal(off_g, off_o)
    for k in ("feature", "threshold", "left", "right", "is_leaf"):
        np.testing.assert_array_equal(cols_g[k], cols_o[k], err_msg=k)
    assert_values_close(cols_g["value"], cols_o["value"], cols_o["is_leaf"])
    scale = np.abs(model.train_preds).max()
    np.testing.assert_allclose(booster.train_predictions(), model.train_preds, rtol=1e-5, atol=1e-5 * scale)


@pytest.mark.parametrize("run_ahead", ["1", "0"])
def test_rounds_that_end_early_rewind_the_generator(run_ahead, monkeypatch):
    """min_samples_leaf stops every tree after two or three levels of max_depth 6, so each round
    draws fewer feature subsets than speculated: the generator is rewound and, when the host runs
    a round ahead of the device, the round already enqueued is replaced."""
    monkeypatch.setenv("PACKBOOST_RUN_AHEAD", run_ahead)
    rng = np.random.default_rng(11)
    n, f, e = 2400, 16, 6
    X = rng.normal(size=(n, f)).astype(np.float32)
    y = (X[:, 0] - 0.5 * X[:, 4] + 0.2 * rng.standard_normal(n)).astype(np.float32)
    era = rng.integers(0, e, size=n).astype(np.int16)
    cfg = dict(pack_size=2, max_depth=6, learning_rate=0.1, lambda_l2=1.0, lambda_dro=0.25, min_samples_leaf=500,
               max_bins=32, layer_feature_fraction=0.5, random_state=3)
    rounds = 6
    model = po.fit(X, y, era, po.OracleParams(**cfg), rounds)
    def height(t, nid=0):
        return 0 if t["is_leaf"][nid] else 1 + max(height(t, t["left"][nid]), height(t, t["right"][nid]))

    heights = [height(t) for t in model.trees[:: cfg["pack_size"]]]
    assert 0 < max(heights) < cfg["max_depth"], "the case must split and still end rounds early"
    booster = _fit_gpu(X, y, era, cfg, rounds)
    off_o, cols_o = flatten_oracle(model.trees)
    off_g, cols_g = flatten_trees(booster.trees)
    np.testing.assert_array_equal(off_g, off_o)
    for k in ("feature", "threshold", "left", "right", "is_leaf"):
        np.testing.assert_array_equal(cols_g[k], cols_o[k], err_msg=k)
    assert_values_close(cols_g["value"], cols_o["value"], cols_o["is_leaf"])
    scale = np.abs(model.train_preds).max()
    np.testing.assert_allclose(booster.train_predictions(), model.train_preds, rtol=1e-5, atol=1e-5 * scale)


def test_fit_is_bitwise_deterministic():
    X, y, era, cfg, rounds, Xh = cases.CASES["prebinned5"]()
    a = _fit_gpu(X, y, era, cfg, rounds)
    b = _fit_gpu(X, y, era, cfg, rounds)
    _, ca = flatten_trees(a.trees)
    _, cb = flatten_trees(b.trees)
    for k in ca:
        if k == "value":
            np.testing.assert_array_equal(ca[k].view(np.int64), cb[k].view(np.int64))
        else:
            np.testing.assert_array_equal(ca[k], cb[k])
    np.testing.assert_array_equal(a.train_predictions().view(np.int32), b.train_predictions().view(np.int32))


def test_predict_is_bit_exact_given_the_same_trees():
    """With identical trees the GPU ensemble sum reproduces the CPU route bit for bit."""
    X, y, era, cfg, rounds, Xh = cases.CASES["config1"]()
    booster = _fit_gpu(X, y, era, cfg, 3)
    _, cols = flatten_trees(booster.trees)
    off, _ = flatten_trees(booster.trees)
    trees = []
    for i in range(len(off) - 1):
        sl = slice(off[i], off[i + 1])
        trees.append({k: v[sl] for k, v in cols.items()})
    codes = po.apply_bins(Xh, booster._binner.bin_edges, cfg["max_bins"])
    want = po.predict_codes(trees, codes, float(booster._tree_weight))
    got = booster.predict(Xh)
    np.testing.assert_array_equal(got.view(np.int32), want.view(np.int32))


def test_inference_stand_in_bit_exact():
    from packboost_b200 import PackBoost, PackBoostConfig
    from packboost_b200.booster import Tree, TreeNode
    from packboost_b200.workloads import heap_ensemble_to_trees
    w = cases.inference_case()
    tds = heap_ensemble_to_trees(w.extra["feature"], w.extra["threshold"], w.extra["leaf"])
    trees = [Tree(nodes=[TreeNode(int(f), int(t), int(l), int(r), float(v), bool(il))
                         for f, t, l, r, v, il in zip(d["feature"], d["threshold"], d["left"], d["right"], d["value"], d["is_leaf"])])
             for d in tds]
    b = PackBoost(PackBoostConfig(device="cuda", pack_size=w.config["pack_size"], max_bins=5, prebinned=True))
    b.set_forest(trees, 1.0)
    gold = np.load(os.path.join(GOLD, "inference_small.npz"))["pred"]
    np.testing.assert_array_equal(b.predict(w.X).view(np.int32), gold.view(np.int32))


def test_errors_are_loud():
    from packboost_b200 import PackBoost, PackBoostConfig
    with pytest.raises(RuntimeError):
        PackBoost(PackBoostConfig(device="cpu"))
    b = PackBoost(PackBoostConfig(device="cuda", max_bins=200))
    with pytest.raises(ValueError):
        b.fit(np.zeros((10, 2), np.float32), np.zeros(10, np.float32), None, num_rounds=1)
    with pytest.raises(RuntimeError):
        PackBoost(PackBoostConfig(device="cuda")).predict(np.zeros((4, 2), np.float32))


def test_wrapper_and_predictor_roundtrip(tmp_path):
    """README-style usage: regressor with an eval set, then a saved / reloaded predictor."""
    from packboost_b200 import PackBoostPredictor, PackBoostRegressor
    X, y, era, cfg, rounds, Xh = cases.CASES["interleaved"]()
    seen = []
    m = PackBoostRegressor(num_rounds=rounds, **cfg)
    m.fit(X, y, era=era, eval_set=(X[:100], y[:100], era[:100]), round_callback=lambda r, met: seen.append(met))
    assert len(seen) == rounds and "valid_corr" in seen[-1] and np.isfinite(seen[-1]["train_corr"])
    gold = np.load(os.path.join(GOLD, "interleaved.npz"))
    scale = np.abs(gold["pred_holdout"]).max()
    np.testing.assert_allclose(m.predict(Xh), gold["pred_holdout"], rtol=1e-5, atol=1e-5 * scale)
    path = str(tmp_path / "m.npz")
    m.to_predictor().save(path)
    p = PackBoostPredictor.load(path)
    np.testing.assert_array_equal(p.predict(Xh).view(np.int32), m.predict(Xh).view(np.int32))
    assert m.score(X, y) > 0.3


def _compare_with_oracle(X, y, era, cfg, rounds, env=None):
    model = po.fit(X, y, era, po.OracleParams(**cfg, **(env or {})), rounds)
    booster = _fit_gpu(X, y, era, cfg, rounds)
    off_o, cols_o = flatten_oracle(model.trees)
    off_g, cols_g = flatten_trees(booster.trees)
    np.testing.assert_array_equal(off_g, off_o)
    for k in ("feature", "threshold", "left", "right", "is_leaf"):
        np.testing.assert_array_equal(cols_g[k], cols_o[k], err_msg=k)
    codes_train, _ = po.preprocess(X, po.OracleParams(**cfg, **(env or {})))
    populated = populated_leaves(off_o, cols_o, codes_train)
    assert_values_close(cols_g["value"], cols_o["value"], cols_o["is_leaf"] & populated)
    scale = np.abs(model.train_preds).max()
    np.testing.assert_allclose(booster.train_predictions(), model.train_preds, rtol=1e-5, atol=1e-5 * scale)
    return booster, model


def test_deep_frontier_matches_oracle():
    """Reduced stand-in for the deep-frontier configuration: depth 9 (up to 256 live nodes),
    128 bins, all features per depth; exercises the shared-cell histogram kernel, node
    chunking and the many-bin scorer path."""
    from packboost_b200 import workloads
    w = workloads.config4(seed=11, n_rows=40_000, n_features=24, n_eras=4, num_rounds=2, max_bins=128, tree_depth=6)
    cfg = dict(w.config)
    cfg.update(pack_size=2, max_depth=9, learning_rate=0.1, min_samples_leaf=30, lambda_l2=1.0)
    # structure can only be compared where no two candidates are closer than the float32 summation
    # noise of the CPU path (see oracle.near_tie_gaps); this input keeps a 10x margin
    assert po.near_tie_gaps(w.X, w.y, w.era, po.OracleParams(**cfg), 2).min() > 1e-5
    booster, _ = _compare_with_oracle(w.X, w.y, w.era, cfg, 2)
    assert max(len(t.nodes) for t in booster.trees) > 400


def test_mixed_columns_matches_oracle():
    """Reduced stand-in for the mixed-column configuration (Gaussian / log-normal / integer-valued
    columns, era-dependent sign flips), 128 bins, depth 6."""
    from packboost_b200 import workloads
    w = workloads.config2(seed=7, n_rows=30_000, n_features=40, n_eras=15, num_rounds=3)
    cfg = dict(w.config)
    cfg.update(pack_size=4, learning_rate=0.1)
    _compare_with_oracle(w.X, w.y, w.era, cfg, 3)


def test_small_workspace_forces_feature_blocks():
    """With a workspace that holds only a few features of histogram the per-depth pass loops over
    feature blocks; the trees must not change."""
    X, y, era, cfg, rounds, Xh = cases.CASES["config1"]()
    ref = _fit_gpu(X, y, era, cfg, 2)
    os.environ["PACKBOOST_WORKSPACE_BYTES"] = str(24 << 20)
    try:
        small = _fit_gpu(X, y, era, cfg, 2)
    finally:
        del os.environ["PACKBOOST_WORKSPACE_BYTES"]
    _, ca = flatten_trees(ref.trees)
    _, cb = flatten_trees(small.trees)
    for k in ca:
        a, b = (ca[k].view(np.int64), cb[k].view(np.int64)) if k == "value" else (ca[k], cb[k])
        np.testing.assert_array_equal(a, b)


def test_wide_bins_match_widened_oracle():
    """255 bins: the reference refuses more than 128 (int8 storage); with the guard lifted on both
    sides (8-bit codes here, int16 codes in the oracle) the trees agree."""
    rng = np.random.default_rng(12)
    n = 6000
    X = rng.normal(size=(n, 6)).astype(np.float32)
    y = (np.sin(2 * X[:, 0]) + X[:, 1] * X[:, 2] + 0.1 * rng.standard_normal(n)).astype(np.float32)
    era = (np.arange(n) // 1000).astype(np.int16)
    cfg = dict(pack_size=2, max_depth=4, learning_rate=0.2, lambda_l2=1.0, lambda_dro=0.2, min_samples_leaf=10,
               max_bins=255, random_state=3)
    os.environ["PACKBOOST_ALLOW_WIDE_BINS"] = "1"
    try:
        _compare_with_oracle(X, y, era, cfg, 2, env=dict(allow_wide_bins=True))
    finally:
        del os.environ["PACKBOOST_ALLOW_WIDE_BINS"]


def test_predict_generic_node_arrays_when_children_are_not_adjacent():
    """Trees whose right child is not stored right after the left one cannot use the packed node
    form; the array-based predictor must give the same answer as the CPU router."""
    from packboost_b200 import PackBoost, PackBoostConfig
    from packboost_b200.booster import Tree, TreeNode
    rng = np.random.default_rng(8)
    codes = rng.integers(0, 5, size=(500, 7), dtype=np.uint8)
    nodes = [TreeNode(3, 1, 2, 1, 0.0, False), TreeNode(-1, 0, -1, -1, 0.7, True), TreeNode(5, 2, 4, 3, 0.0, False),
             TreeNode(-1, 0, -1, -1, -0.2, True), TreeNode(-1, 0, -1, -1, 0.4, True)]
    tree = Tree(nodes=nodes)
    b = PackBoost(PackBoostConfig(device="cuda", pack_size=1, max_bins=5, prebinned=True))
    b.set_forest([tree, tree], 0.3, repeats=[2, 1])
    arr = {k: (v.astype(np.float64) if k == "value" else v) for k, v in tree.arrays().items()}
    arr["is_leaf"] = arr["is_leaf"].astype(bool)
    want = po.predict_codes([arr] * 3, codes.astype(np.int8), 0.3)
    np.testing.assert_array_equal(b.predict(codes).view(np.int32), want.view(np.int32))
    assert "packed" not in b._forest_cache


def _check_scores(got, want, label):
    """DES scores against the reference's: within 1e-5 relative, or within 1e-4 of the largest score
    of the fit.  A per-era gain is the small difference of terms G^2 / (H + lambda) that are
    thousands of times larger (a root era of 4 700 rows: terms of ~600, gains of ~0.05), and the
    reference feeds it float32 sums taken row by row, whose rounding noise (~1e-7 of the terms)
    therefore shows up at ~1e-4 of the gain.  The CUDA path takes the same sums exactly; that its
    scores are the reference's arithmetic on exact sums is checked bit for bit in
    ``test_fit_is_bit_identical_to_the_exact_sum_oracle``.  The number of scores that needed the
    absolute term is printed."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    finite = np.isfinite(want)
    np.testing.assert_array_equal(np.isfinite(got), finite)
    np.testing.assert_array_equal(got[~finite], want[~finite])          # -inf fall-through splits
    g, w = got[finite], want[finite]
    scale = np.abs(w).max() if w.size else 1.0
    rel_ok = np.abs(g - w) <= 1e-5 * np.abs(w)
    print(f"{label}: {w.size} scores, {int((~rel_ok).sum())} outside 1e-5 relative "
          f"(max abs diff there {np.abs(g - w)[~rel_ok].max() if (~rel_ok).any() else 0:.3g}, score scale {scale:.3g})")
    np.testing.assert_allclose(g, w, rtol=1e-5, atol=1e-4 * scale)
    return int((~rel_ok).sum()), int(w.size)


@pytest.mark.parametrize("name", list(cases.CASES) + ["config3_wide"])
def test_fit_is_bit_identical_to_the_exact_sum_oracle(name):
    """The oracle's ``exact_sums`` variant is the reference's algorithm with one change: gradient
    sums are exact (the fixed-point gradients of the CUDA path) and rounded to float32 once,
    instead of float32 sums in row order.  Everything downstream is the reference's float32 /
    float64 arithmetic, operation by operation, so the CUDA path must agree with it in every bit:
    tree structure, every split's DES score (float32), every leaf value (float64) and every
    training prediction (float32)."""
    X, y, era, cfg, rounds, Xh = {**cases.CASES, **cases.WIDE_CASES}[name]()
    model = po.fit(X, y, era, po.OracleParams(exact_sums=True, **cfg), rounds, record_depths=True)
    booster = _fit_gpu(X, y, era, cfg, rounds)
    off_o, cols_o = flatten_oracle(model.trees)
    off_g, cols_g = flatten_trees(booster.trees)
    np.testing.assert_array_equal(off_g, off_o)
    for k in ("feature", "threshold", "left", "right", "is_leaf"):
        np.testing.assert_array_equal(cols_g[k], cols_o[k], err_msg=k)
    np.testing.assert_array_equal(cols_g["value"].view(np.int64), cols_o["value"].astype(np.float64).view(np.int64))
    rec = booster.split_records()
    B = cfg["pack_size"]
    want = model.depth_records
    assert len(want) == rec["node"].shape[0]
    np.testing.assert_array_equal(rec["node"], [r["node"] for r in want])
    np.testing.assert_array_equal(rec["left_count"], [r["left_count"] for r in want])
    np.testing.assert_array_equal(rec["score"].view(np.int32),
                                  np.asarray([r["score"] for r in want], dtype=np.float32).view(np.int32))
    np.testing.assert_array_equal(booster.train_predictions().view(np.int32), model.train_preds.view(np.int32))
    np.testing.assert_array_equal(booster.predict(Xh).view(np.int32), model.predict(Xh).view(np.int32))


@pytest.mark.parametrize("name", list(cases.CASES))
def test_split_scores_match_reference(name):
    """Every split the reference's frontier returned (first tree of each pack): same node,
    feature, threshold and child counts, DES score within 1e-5."""
    X, y, era, cfg, rounds, Xh = cases.CASES[name]()
    gold = np.load(os.path.join(GOLD, f"{name}.npz"))
    rec = _fit_gpu(X, y, era, cfg, rounds).split_records()
    for k in ("node", "feature", "threshold", "left_count", "right_count"):
        np.testing.assert_array_equal(rec[k], gold[f"split_{k}"], err_msg=k)
    _check_scores(rec["score"], gold["split_score"], name)


@pytest.mark.parametrize("name", list(cases.WIDE_CASES))
def test_wide_cases_match_reference(name):
    """The benchmark configurations at their real widths (238 sampled features = eight feature
    blocks; 500 000 x 256 at 128 bins; 500 features at depth 10) against fixtures written by the
    unmodified reference: split structure exact, scores, leaf values and predictions within 1e-5."""
    X, y, era, cfg, rounds, Xh = cases.WIDE_CASES[name]()
    gold = np.load(os.path.join(GOLD, f"{name}.npz"))
    booster = _fit_gpu(X, y, era, cfg, rounds)
    rec = booster.split_records()
    for k in ("node", "feature", "threshold", "left_count", "right_count"):
        np.testing.assert_array_equal(rec[k], gold[f"split_{k}"], err_msg=k)
    _check_scores(rec["score"], gold["split_score"], name)
    off, cols = flatten_trees(booster.trees)
    np.testing.assert_array_equal(off, gold["tree_offsets"])
    for k in ("feature", "threshold", "left", "right", "is_leaf"):
        np.testing.assert_array_equal(cols[k], gold[k], err_msg=k)
    gcols = {k: gold[k] for k in cols}
    codes_train, edges = po.preprocess(X, po.OracleParams(**cfg))
    # (the trees of a pack are identical: the populated-leaf mask of the first one serves all)
    B = cfg["pack_size"]
    first = np.arange(0, len(off) - 1, B)
    populated = np.zeros(cols["feature"].shape[0], dtype=bool)
    for t in first:
        sl = slice(off[t], off[t + 1])
        m = populated_leaves(np.array([0, off[t + 1] - off[t]]), {k: v[sl] for k, v in gcols.items()}, codes_train)
        for j in range(B):
            populated[off[t + j]: off[t + j + 1]] = m
    leaves = gold["is_leaf"] & populated
    n_abs = assert_values_close(cols["value"], gold["value"], leaves)
    print(f"{name}: {int(leaves.sum())} leaf values, {n_abs} outside 1e-5 relative (within 1e-5 of the largest leaf value)")
    # A prediction is tree_weight * (sum of one leaf value per tree): its tolerance is the leaf
    # tolerance carried through that sum, 1e-5 of tree_weight * sum over trees of the largest |leaf|.
    # (The reference adds up to 500 000 float32 gradients one after the other; the rounding noise of
    # that sum alone is ~2e-5 of its value, so 1e-5 of each prediction is not attainable against it.)
    per_tree = np.array([np.abs(gold["value"][off[t]: off[t + 1]][leaves[off[t]: off[t + 1]]]).max()
                         for t in range(len(off) - 1)])
    scale = float(gold["tree_weight"]) * float(per_tree.sum())
    np.testing.assert_allclose(booster.predict(X[:2048]), gold["pred_train_head"], rtol=1e-5, atol=1e-5 * scale)
    np.testing.assert_allclose(booster.train_predictions()[:2048], gold["pred_train_head"], rtol=1e-5, atol=1e-5 * scale)
    # First-round leaf values against float64 arithmetic: with zero predictions the gradients are
    # exactly -y, so the gradient sum of every node can be recomputed without summation noise.
    # The CUDA path sums exactly in fixed point and rounds a node's total and its left child's sum
    # to float32 once each; the right child's sum is their difference (packboost/booster.py:2103-2108),
    # so a child's value may be off by the float32 rounding of those two numbers and no more.
    t0 = {k: gold[k][off[0]: off[1]] for k in ("feature", "threshold", "left", "right", "is_leaf")}
    from gpu_util import leaf_index
    n0 = int(off[1] - off[0])
    where = leaf_index(t0, codes_train)
    lam = float(cfg.get("lambda_l2", 1e-6))
    sums = np.bincount(where, weights=-y.astype(np.float64), minlength=n0)
    cnts = np.bincount(where, minlength=n0).astype(np.float64)
    parent = np.full(n0, -1)
    for i in range(n0 - 1, -1, -1):            # children carry larger ids than their parent
        if not t0["is_leaf"][i]:
            l, r = int(t0["left"][i]), int(t0["right"][i])
            sums[i] = sums[l] + sums[r]
            cnts[i] = cnts[l] + cnts[r]
            parent[l] = parent[r] = i
    hit = (cnts > 0) & t0["is_leaf"] & (parent >= 0)
    idx = np.flatnonzero(hit)
    sib = np.where(t0["left"][parent[idx]] == idx, t0["right"][parent[idx]], t0["left"][parent[idx]])
    exact = -sums[idx] / (cnts[idx] + lam)
    eps = 2.0 ** -23
    bound = eps * (np.abs(sums[parent[idx]]) + np.abs(sums[sib]) + np.abs(sums[idx])) / (cnts[idx] + lam) + 1e-7 * np.abs(exact)
    # (plus the fixed-point quantum of a gradient, 2^-24 of the largest one, as a random walk over the rows)
    bound += 2.0 ** -24 * float(np.abs(y).max()) * (np.sqrt(cnts[parent[idx]]) + np.sqrt(cnts[sib]) + np.sqrt(cnts[idx])) / (cnts[idx] + lam)
    got0 = cols["value"][off[0]: off[1]][idx]
    worst = np.max(np.abs(got0 - exact) / bound)
    print(f"{name}: first-round leaves vs float64: worst error / float32 rounding bound = {worst:.3f}")
    assert worst <= 1.0


@pytest.mark.parametrize("name,k", [("config1", 4), ("prebinned5", 2), ("ragged_eras", 7), ("interleaved", 5)])
def test_mass_k_cuts_match_the_compiled_reference_and_the_oracle(name, k):
    """``k_cuts`` with ``cut_selection="mass"`` (the reference's default policy, and the one its
    published GPU run uses).  The reference's torch frontier raises on it; its compiled C++ split
    finder implements it.  The thresholds of every (depth, feature) follow the C++ definition, the
    scoring the torch frontier as always: the trees must equal those of the compiled reference
    (``oracle/_ref``, when it was built) in structure, and the oracle's restatement of the policy in
    its exact-sum variant in every bit."""
    from oracle import native_ref
    X, y, era, cfg, rounds, Xh = cases.CASES[name]()
    cfg = dict(cfg)
    cfg.update(k_cuts=k, cut_selection="mass", direction_weight=0.0)
    booster = _fit_gpu(X, y, era, cfg, rounds)
    off_g, cols_g = flatten_trees(booster.trees)
    model = po.fit(X, y, era, po.OracleParams(exact_sums=True, native_mass_cuts=True, **cfg), rounds, record_depths=True)
    off_o, cols_o = flatten_oracle(model.trees)
    np.testing.assert_array_equal(off_g, off_o)
    for key in ("feature", "threshold", "left", "right", "is_leaf"):
        np.testing.assert_array_equal(cols_g[key], cols_o[key], err_msg=key)
    np.testing.assert_array_equal(cols_g["value"].view(np.int64), cols_o["value"].astype(np.float64).view(np.int64))
    rec = booster.split_records()
    np.testing.assert_array_equal(rec["score"].view(np.int32),
                                  np.asarray([r["score"] for r in model.depth_records], dtype=np.float32).view(np.int32))
    np.testing.assert_array_equal(booster.train_predictions().view(np.int32), model.train_preds.view(np.int32))
    if native_ref.available():
        ref = native_ref.fit(X, y, era, po.OracleParams(**cfg), rounds)
        off_r, cols_r = flatten_oracle(ref.trees)
        np.testing.assert_array_equal(off_g, off_r)
        for key in ("feature", "threshold", "left", "right", "is_leaf"):
            np.testing.assert_array_equal(cols_g[key], cols_r[key], err_msg=f"compiled reference: {key}")
        scale = np.abs(ref.train_preds).max()
        np.testing.assert_allclose(booster.train_predictions(), ref.train_preds, rtol=1e-5, atol=1e-5 * scale)


@pytest.mark.parametrize("name", ["dro_direction", "interleaved"])
def test_helper_form_direction_term_matches_the_oracle(name, monkeypatch):
    """``PACKBOOST_DIRECTION_FORM=helper``: the ``+1 / -1`` directional term of the reference's helper
    and native code (``packboost/booster.py:869-907``) instead of the torch frontier's agreement
    with the parent direction; bit-identical to the oracle's restatement of that form."""
    monkeypatch.setenv("PACKBOOST_DIRECTION_FORM", "helper")
    X, y, era, cfg, rounds, Xh = cases.CASES[name]()
    cfg = dict(cfg)
    cfg.update(direction_weight=0.2)
    model = po.fit(X, y, era, po.OracleParams(exact_sums=True, direction_form="helper", **cfg), rounds, record_depths=True)
    booster = _fit_gpu(X, y, era, cfg, rounds)
    off_o, cols_o = flatten_oracle(model.trees)
    off_g, cols_g = flatten_trees(booster.trees)
    np.testing.assert_array_equal(off_g, off_o)
    for key in ("feature", "threshold", "left", "right", "is_leaf"):
        np.testing.assert_array_equal(cols_g[key], cols_o[key], err_msg=key)
    np.testing.assert_array_equal(booster.split_records()["score"].view(np.int32),
                                  np.asarray([r["score"] for r in model.depth_records], dtype=np.float32).view(np.int32))
    np.testing.assert_array_equal(booster.train_predictions().view(np.int32), model.train_preds.view(np.int32))


@pytest.mark.parametrize("shape", ["1 8 1", "2 4 1", "2 2 2", "1 2 4"])
def test_fit_is_bit_identical_in_forced_histogram_shapes(shape):
    """The fused flush of the histogram kernel reads the cells in the layout of the launch shape
    (private columns, or one column shared by two row phases).  The bit-for-bit comparison with
    the exact-sum oracle and the golden comparison run again in a child process that forces one
    shape wherever it fits (the override is read once per process)."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, PACKBOOST_HIST_SHAPE=shape)
    res = subprocess.run([sys.executable, "-m", "pytest", os.path.join(root, "tests", "test_gpu_fit_parity.py"), "-q", "-x", "-s",
                          "-m", "gpu", "-k", "exact_sum_oracle or matches_reference_golden"], env=env, cwd=root,
                         capture_output=True, text=True, timeout=1200)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-2000:]
    assert "hist_lane_kernel<%s>" % shape.replace(" ", ",") in res.stderr + res.stdout, "forced shape never launched"
