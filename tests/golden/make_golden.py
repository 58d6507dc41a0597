"""Generate the golden fixtures by running the UNMODIFIED reference on CPU.

Usage (in a container that has the reference checked out):

    python tests/golden/make_golden.py /path/to/reference [case ...]

Without case names every fixture is rewritten (the wide cases take several minutes each).
The reference is imported read-only (no bytecode is written), driven through
its public API with ``device="cpu"`` and with its optional native backend
absent, so the torch frontier is the code that runs.  Outputs are the small
``*.npz`` files beside this script; they are committed, the reference is not.
"""

from __future__ import annotations

import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.dont_write_bytecode = True


def _flatten_trees(trees):
    off = [0]
    cols = {k: [] for k in ("feature", "threshold", "left", "right", "value", "is_leaf")}
    for t in trees:
        for n in t.nodes:
            cols["feature"].append(n.feature)
            cols["threshold"].append(n.threshold)
            cols["left"].append(n.left)
            cols["right"].append(n.right)
            cols["value"].append(n.value)
            cols["is_leaf"].append(n.is_leaf)
        off.append(len(cols["feature"]))
    return dict(
        tree_offsets=np.asarray(off, dtype=np.int64),
        feature=np.asarray(cols["feature"], dtype=np.int32),
        threshold=np.asarray(cols["threshold"], dtype=np.int32),
        left=np.asarray(cols["left"], dtype=np.int32),
        right=np.asarray(cols["right"], dtype=np.int32),
        value=np.asarray(cols["value"], dtype=np.float64),
        is_leaf=np.asarray(cols["is_leaf"], dtype=np.bool_),
    )


def _record_splits(booster, log):
    """Wrap the booster's frontier call so that the decisions it returns for the first tree of the
    pack are appended to ``log`` as (call index, tree node, feature, threshold, score, left count,
    right count).  The wrapped method runs unchanged; nothing else of the reference is touched."""
    inner = booster._find_best_splits_batched
    calls = [0]

    def spy(nodes, grad, hess, bins, feature_subset):
        decisions, stats = inner(nodes, grad, hess, bins, feature_subset)
        for node, dec in zip(nodes, decisions):
            if node.tree_id != 0 or dec is None:
                continue
            log.append((calls[0], node.node_id, dec.feature, dec.threshold, float(dec.score),
                        int(dec.left_count), int(dec.right_count)))
        calls[0] += 1
        return decisions, stats

    booster._find_best_splits_batched = spy


def main(ref_root: str, only: list[str] | None = None) -> None:
    sys.path.insert(0, ref_root)
    os.environ["PACKBOOST_DISABLE_NATIVE_CPU"] = "1"
    import torch
    from packboost.booster import NodeShard, PackBoost, Tree, TreeNode
    from packboost.config import PackBoostConfig
    from packboost.data import BinningResult

    sys.path.insert(0, HERE)
    import cases

    all_cases = dict(cases.CASES)
    all_cases.update(cases.WIDE_CASES)
    for name, make in all_cases.items():
        if only and name not in only:
            continue
        X, y, era, cfg, rounds, Xh = make()
        booster = PackBoost(PackBoostConfig(device="cpu", **cfg))
        splits: list[tuple] = []
        _record_splits(booster, splits)
        booster.fit(X, y, era, num_rounds=rounds)
        out = _flatten_trees(booster.trees)
        # every split of the first tree of each pack, in the order the frontier produced them
        sp = np.asarray(splits, dtype=np.float64).reshape(-1, 7)
        out["split_call"] = sp[:, 0].astype(np.int32)
        out["split_node"] = sp[:, 1].astype(np.int32)
        out["split_feature"] = sp[:, 2].astype(np.int32)
        out["split_threshold"] = sp[:, 3].astype(np.int32)
        out["split_score"] = sp[:, 4].astype(np.float32)
        out["split_left_count"] = sp[:, 5].astype(np.int64)
        out["split_right_count"] = sp[:, 6].astype(np.int64)
        out["pred_train_head"] = booster.predict(X[:2048])
        out["pred_holdout"] = booster.predict(Xh)
        out["tree_weight"] = np.float64(booster._tree_weight)
        if booster._binner.bin_edges is not None:
            edges = booster._binner.bin_edges
            # a checksum of the edges keeps the fixture small
            out["edges_sum64"] = np.float64(edges.astype(np.float64).sum())
            out["edges_head"] = edges[:, : min(4, edges.shape[1])].copy()
            out["codes_head"] = np.asarray(booster._binner.bins[:256], dtype=np.int8)
        np.savez_compressed(os.path.join(HERE, f"{name}.npz"), **out)
        print(name, "trees", len(booster.trees), "nodes", out["feature"].shape[0])

    if only:
        return
    # frontier known answer: hand-built node of the reference's DES test
    grad, hess, codes, era_rows, cfg = cases.des_known_answer_inputs()
    res = {}
    for alpha in (0.0, 1.5):
        b = PackBoost(PackBoostConfig(device="cpu", era_alpha=alpha, **cfg))
        node = NodeShard(tree_id=0, node_id=0, depth=0, era_rows=[torch.from_numpy(r) for r in era_rows])
        dec = b._find_best_split(node, torch.from_numpy(grad), torch.from_numpy(hess),
                                 torch.from_numpy(codes), torch.tensor([0], dtype=torch.int64))
        res[f"a{alpha}"] = np.array([dec.feature, dec.threshold, dec.left_count, dec.right_count], dtype=np.int64)
        res[f"a{alpha}_f"] = np.array([dec.score, dec.left_grad, dec.left_hess, dec.right_grad, dec.right_hess],
                                      dtype=np.float64)
    np.savez_compressed(os.path.join(HERE, "des_known_answer.npz"), **res)

    # inference-only stand-in: a constructed ensemble scored by the reference router
    w = cases.inference_case()
    from packboost_b200.workloads import heap_ensemble_to_trees
    tdicts = heap_ensemble_to_trees(w.extra["feature"], w.extra["threshold"], w.extra["leaf"])
    trees = []
    for t in tdicts:
        nodes = [TreeNode(feature=int(f), threshold=int(th), left=int(l), right=int(r), value=float(v), is_leaf=bool(il))
                 for f, th, l, r, v, il in zip(t["feature"], t["threshold"], t["left"], t["right"], t["value"], t["is_leaf"])]
        trees.append(Tree(nodes=nodes))
    b = PackBoost(PackBoostConfig(device="cpu", pack_size=w.config["pack_size"], max_bins=5, prebinned=True))
    b._trees = trees
    b._tree_weight = 1.0
    b._trained_pack_size = w.config["pack_size"]
    b._binner = BinningResult(bins=None, bin_edges=None, prebinned=True)
    np.savez_compressed(os.path.join(HERE, "inference_small.npz"), pred=b.predict(w.X))
    print("inference_small done")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/reference [case ...]")
    main(sys.argv[1], sys.argv[2:] or None)
