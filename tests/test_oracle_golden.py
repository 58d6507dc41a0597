"""The CPU oracle must reproduce the reference's own outputs bit for bit.

The fixtures under ``tests/golden`` were written by ``make_golden.py`` from the
unmodified reference (torch CPU frontier).  Structure (feature, threshold,
children, leaf flags) is compared exactly; leaf values and predictions are
compared as exact float bit patterns, which is what pins the oracle's
arithmetic order.
"""

import os

import numpy as np
import pytest
import torch

import cases
from oracle import packboost_oracle as po

GOLD = os.path.dirname(os.path.abspath(cases.__file__))


def _flatten(trees):
    off = [0]
    cols = {k: [] for k in ("feature", "threshold", "left", "right", "value", "is_leaf")}
    for t in trees:
        for k in cols:
            cols[k].append(t[k])
        off.append(off[-1] + t["feature"].shape[0])
    return np.asarray(off), {k: np.concatenate(v) for k, v in cols.items()}


def check_split_records(model, gold):
    """Every split the reference's frontier returned for the first tree of each pack (node,
    feature, threshold, child counts) and its DES score as a float32 bit pattern."""
    rec = model.depth_records
    assert len(rec) == gold["split_node"].shape[0]
    np.testing.assert_array_equal([r["node"] for r in rec], gold["split_node"])
    np.testing.assert_array_equal([r["feature"] for r in rec], gold["split_feature"])
    np.testing.assert_array_equal([r["threshold"] for r in rec], gold["split_threshold"])
    np.testing.assert_array_equal([r["left_count"] for r in rec], gold["split_left_count"])
    np.testing.assert_array_equal([r["right_count"] for r in rec], gold["split_right_count"])
    got = np.asarray([r["score"] for r in rec], dtype=np.float32)
    np.testing.assert_array_equal(got.view(np.int32), gold["split_score"].view(np.int32))


# the full-width five-level case pins the oracle where the tie-break crosses eight feature blocks;
# the other wide cases take the oracle minutes and are compared with the CUDA path only
@pytest.mark.parametrize("name", list(cases.CASES) + ["config3_wide"])
def test_fit_and_predict_match_reference_bitwise(name):
    X, y, era, cfg, rounds, Xh = {**cases.CASES, **cases.WIDE_CASES}[name]()
    gold = np.load(os.path.join(GOLD, f"{name}.npz"))
    model = po.fit(X, y, era, po.OracleParams(**cfg), rounds, record_depths=True)
    check_split_records(model, gold)
    off, cols = _flatten(model.trees)
    np.testing.assert_array_equal(off, gold["tree_offsets"])
    for k in ("feature", "threshold", "left", "right", "is_leaf"):
        np.testing.assert_array_equal(cols[k], gold[k], err_msg=k)
    np.testing.assert_array_equal(cols["value"].view(np.int64), gold["value"].view(np.int64))
    assert model.tree_weight == float(gold["tree_weight"])
    np.testing.assert_array_equal(model.predict(X[:2048]).view(np.int32), gold["pred_train_head"].view(np.int32))
    np.testing.assert_array_equal(model.predict(Xh).view(np.int32), gold["pred_holdout"].view(np.int32))
    # the training-time prediction state equals predict() on the training rows
    np.testing.assert_allclose(model.train_preds[:2048], gold["pred_train_head"], rtol=1e-5, atol=1e-6)
    if "edges_head" in gold.files:
        np.testing.assert_array_equal(model.bin_edges[:, : gold["edges_head"].shape[1]], gold["edges_head"])
        assert float(model.bin_edges.astype(np.float64).sum()) == float(gold["edges_sum64"])
        codes = po.apply_bins(X[:256], model.bin_edges, cfg["max_bins"])
        np.testing.assert_array_equal(codes, gold["codes_head"])


@pytest.mark.parametrize("alpha", [0.0, 1.5])
def test_des_known_answer(alpha):
    """Hand-built six-row node of the reference's DES test (general hessians)."""
    grad, hess, codes, era_rows, cfg = cases.des_known_answer_inputs()
    gold = np.load(os.path.join(GOLD, "des_known_answer.npz"))
    p = po.OracleParams(era_alpha=alpha, **cfg)
    rows = torch.from_numpy(np.concatenate(era_rows))
    eras = torch.from_numpy(np.concatenate([np.full(r.shape, i, np.int16) for i, r in enumerate(era_rows)]))
    dec = po.find_splits([rows], [eras], torch.from_numpy(grad), torch.from_numpy(hess),
                         torch.from_numpy(codes), torch.tensor([0]), len(era_rows), p)[0]
    gi, gf = gold[f"a{alpha}"], gold[f"a{alpha}_f"]
    assert [dec.feature, dec.threshold, dec.left_count, dec.right_count] == gi.tolist()
    got = np.array([dec.score, dec.left_grad, dec.left_hess, dec.right_grad, dec.right_hess])
    np.testing.assert_array_equal(got.view(np.int64), gf.view(np.int64))


def test_era_alpha_weights():
    """``era_alpha=2.5``: counts [0,3,5] -> weights [0,5.5,7.5] (reference tests/test_des.py:220-226)."""
    w = po.era_weights(torch.tensor([0.0, 3.0, 5.0]), 2.5)
    assert w.tolist() == [0.0, 5.5, 7.5]


def test_inference_stand_in_matches_reference_router():
    from packboost_b200.workloads import heap_ensemble_to_trees
    w = cases.inference_case()
    trees = heap_ensemble_to_trees(w.extra["feature"], w.extra["threshold"], w.extra["leaf"])
    pred = po.predict_codes(trees, w.X.astype(np.int8), 1.0)
    gold = np.load(os.path.join(GOLD, "inference_small.npz"))["pred"]
    np.testing.assert_array_equal(pred.view(np.int32), gold.view(np.int32))


def test_histogram_conservation():
    """left + right == total for counts and sums (reference tests/test_execution_modes.py:84-132)."""
    g = torch.Generator().manual_seed(1234)
    for _ in range(5):
        codes = torch.randint(0, 16, (128, 3), generator=g)
        gr = torch.randn(128, generator=g)
        he = torch.rand(128, generator=g) + 0.1
        er = torch.randint(0, 4, (128,), generator=g)
        cnt, gh, hh = po.block_histograms(codes, gr, he, er, torch.zeros(128, dtype=torch.int64), 1, 4, 16)
        lc = cnt[:, 0, :, :-1].cumsum(2)
        rc = cnt[:, 0, :, 1:].flip(2).cumsum(2).flip(2)
        assert torch.equal(lc + rc, cnt[:, 0].sum(2, keepdim=True).expand_as(lc))
        lg = gh[:, 0, :, :-1].cumsum(2)
        rg = gh[:, 0, :, 1:].flip(2).cumsum(2).flip(2)
        torch.testing.assert_close(lg + rg, gh[:, 0].sum(2, keepdim=True).expand_as(lg), atol=1e-5, rtol=1e-6)
