"""Driver for the reference's compiled C++/OpenMP split finder (``oracle/_ref/_backend*.so``,
built by ``oracle/build_ref.py`` from the reference's own sources).

TEST INFRASTRUCTURE ONLY.  The split finder is the reference's second implementation of the
frontier (``packboost/backends/cpu/frontier_cpu.cpp:111-515``).  It differs from the torch
frontier the oracle restates in three documented ways — no split when no candidate passes
``min_samples_leaf`` (``frontier_cpu.cpp:404-407``), the ``+1 / -1`` direction term
(``frontier_cpu.cpp:395-401``), unit hessians (``frontier_cpu.cpp:206``) — and it is the only
place where the reference's mass-based K-cut selection actually runs
(``frontier_cpu.cpp:59-109``; the torch frontier raises on it).  Here it serves as

* the pin for mass K-cuts (``tests``), and
* the "native CPU" baseline of the benchmark, timed beside the torch-path port.

``fit`` restates the round loop the reference wraps around it (``packboost/booster.py:494-599``
with ``_find_best_splits_batched_native``, ``booster.py:1012-1160``) with the same containers as
``packboost_oracle.fit``.
"""

from __future__ import annotations

import importlib.util
import os
from time import perf_counter

import numpy as np
import torch

from . import packboost_oracle as po
from .build_ref import output_path

_MOD = None


def available() -> bool:
    return os.path.exists(output_path())


def backend():
    global _MOD
    if _MOD is None:
        path = output_path()
        if not os.path.exists(path):
            raise RuntimeError(f"{path} is missing: build it with `python oracle/build_ref.py <reference checkout>`")
        spec = importlib.util.spec_from_file_location("_backend", path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        _MOD = mod
    return _MOD


def find_splits(node_era_rows, grad_np, codes_np, subset_np, p: po.OracleParams):
    """One frontier call: ``node_era_rows[i]`` is the list of per-era int64 row arrays of node i."""
    dec, stats = backend().find_best_splits_batched_cpu(
        codes_np, grad_np, node_era_rows, subset_np, int(p.max_bins), int(p.k_cuts), str(p.cut_selection),
        float(p.lambda_l2), float(p.lambda_dro), float(p.direction_weight), float(p.era_alpha),
        int(p.min_samples_leaf))
    return list(dec), dict(stats)


def fit(X, y, era, p: po.OracleParams, num_rounds: int, *, record_depths: bool = False) -> po.OracleModel:
    """Boosting rounds with the compiled split finder; one tree per round, recorded ``pack_size``
    times (the reference de-duplicates the identical nodes of a pack before calling it,
    ``booster.py:1033-1062``)."""
    Xn = np.asarray(X)
    y32 = np.asarray(y, dtype=np.float32)
    N, F = Xn.shape
    era_codes, E = po.encode_eras(era, N)
    codes_np, edges = po.preprocess(Xn, p)
    codes_np = np.ascontiguousarray(codes_np.astype(np.int8, copy=False))
    rng = torch.Generator(device="cpu")
    if p.random_state is not None:
        rng.manual_seed(int(p.random_state))
    preds = np.zeros(N, dtype=np.float32)
    order = np.argsort(era_codes, kind="stable")
    bounds = np.concatenate([[0], np.cumsum(np.bincount(era_codes.astype(np.int64), minlength=E))])
    root = [order[bounds[e]:bounds[e + 1]].astype(np.int64) for e in range(E)]
    lam = float(p.lambda_l2)
    lr32 = np.float32(p.learning_rate)
    trees, records, seconds = [], [], []
    for rnd in range(num_rounds):
        t0 = perf_counter()
        grad = (preds - y32).astype(np.float32)
        tree = po.OracleTree()
        rows_all = np.concatenate(root) if N else np.zeros(0, np.int64)
        tree.set_leaf(0, -float(grad[rows_all].sum(dtype=np.float32)) / (float(rows_all.size) + lam) if N else 0.0)
        leaves = {0: rows_all}
        frontier = [(0, root)]
        for depth in range(p.max_depth):
            active = [(nid, er) for nid, er in frontier if sum(a.size for a in er) >= 2 * p.min_samples_leaf]
            if not active:
                break
            subset = po.sample_features(rng, F, p.layer_feature_fraction).numpy().astype(np.int32)
            decisions, _ = find_splits([er for _, er in active], grad, codes_np, subset, p)
            nxt = []
            for (nid, er), dec in zip(active, decisions):
                if dec is None:
                    rows = np.concatenate(er)
                    leaves.setdefault(nid, rows)
                    tree.set_leaf(nid, -float(grad[rows].sum(dtype=np.float32)) / (float(rows.size) + lam))
                    continue
                l_id, r_id = tree.split(nid, int(dec["feature"]), int(dec["threshold"]))
                tree.set_leaf(l_id, -float(dec["left_grad"]) / (float(dec["left_hess"]) + lam))
                tree.set_leaf(r_id, -float(dec["right_grad"]) / (float(dec["right_hess"]) + lam))
                left = [np.asarray(a, dtype=np.int64).reshape(-1) for a in dec["left_rows"]]
                right = [np.asarray(a, dtype=np.int64).reshape(-1) for a in dec["right_rows"]]
                leaves.pop(nid, None)
                leaves[l_id] = np.concatenate(left)
                leaves[r_id] = np.concatenate(right)
                nxt.append((l_id, left))
                nxt.append((r_id, right))
                if record_depths:
                    records.append({"round": rnd, "depth": depth, "node": nid, "feature": int(dec["feature"]),
                                    "threshold": int(dec["threshold"]), "score": float(dec["score"]),
                                    "left_count": int(dec["left_count"]), "right_count": int(dec["right_count"])})
            frontier = nxt
        arr = tree.arrays()
        pack_sum = np.zeros(N, dtype=np.float32)
        for _ in range(p.pack_size):
            for leaf_id, rows in leaves.items():
                if rows.size:
                    pack_sum[rows] += np.float32(arr["value"][leaf_id])
        preds = preds + lr32 * pack_sum
        trees.extend([arr] * p.pack_size)
        seconds.append(perf_counter() - t0)
    return po.OracleModel(params=p, trees=trees, bin_edges=edges, tree_weight=float(lr32), train_preds=preds.copy(),
                          depth_records=records, round_seconds=seconds, wide=False)
