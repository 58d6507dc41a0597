"""Helpers shared by the GPU parity tests."""

import ctypes as C

import numpy as np
import torch

from packboost_b200 import backends as B
from packboost_b200.booster import PackBoost, _DeviceTrainer
from packboost_b200.config import PackBoostConfig
from packboost_b200.data import pack_feature_major


def flatten_trees(trees):
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
    return np.asarray(off), {
        "feature": np.asarray(cols["feature"], np.int32), "threshold": np.asarray(cols["threshold"], np.int32),
        "left": np.asarray(cols["left"], np.int32), "right": np.asarray(cols["right"], np.int32),
        "value": np.asarray(cols["value"], np.float64), "is_leaf": np.asarray(cols["is_leaf"], np.bool_)}


def flatten_oracle(trees):
    off = [0]
    cols = {k: [] for k in ("feature", "threshold", "left", "right", "value", "is_leaf")}
    for t in trees:
        for k in cols:
            cols[k].append(t[k])
        off.append(off[-1] + t["feature"].shape[0])
    return np.asarray(off), {k: np.concatenate(v) for k, v in cols.items()}


# Leaf values: float32 sums of ~N gradients carry a relative rounding noise of ~1e-6 in the CPU
# path (sequential float32 accumulation), while the GPU sums exactly in fixed point.  A value is
# -G/(H+lambda); when G nearly cancels, the noise is relative to sum|g|, not to |G|, hence the
# absolute term.  Tolerance: 1e-5 relative plus 1e-5 of the value scale of the tree.
def assert_values_close(got, want, is_leaf, scale=None):
    got = np.asarray(got, np.float64)[is_leaf]
    want = np.asarray(want, np.float64)[is_leaf]
    finite = np.isfinite(want) & (np.abs(want) < 1e30)
    s = np.abs(want[finite]).max() if scale is None and finite.any() else (scale or 1.0)
    np.testing.assert_allclose(got[finite], want[finite], rtol=1e-5, atol=1e-5 * s)
    # how many values needed the absolute term (reported by the caller where it matters)
    return int((np.abs(got[finite] - want[finite]) > 1e-5 * np.abs(want[finite])).sum())


def leaf_index(tree, codes):
    """Index of the leaf node each row lands in (same routing rule as the oracle)."""
    n = codes.shape[0]
    node = np.zeros(n, dtype=np.int64)
    live = np.arange(n)
    while live.size:
        cur = node[live]
        keep = ~tree["is_leaf"][cur]
        live, cur = live[keep], cur[keep]
        if live.size == 0:
            break
        go_left = codes[live, tree["feature"][cur]] <= tree["threshold"][cur]
        node[live] = np.where(go_left, tree["left"][cur], tree["right"][cur])
    return node


def populated_leaves(off, cols, codes_train):
    """Boolean mask over all nodes: leaf reached by at least one training row.  A child that
    received no rows (possible after the reference's -inf fall-through split) has the value
    -eps/(0+lambda) with eps the float32 summation noise of the CPU path; such values are not
    comparable and are excluded from value checks."""
    mask = np.zeros(cols["feature"].shape[0], dtype=bool)
    for i in range(len(off) - 1):
        sl = slice(off[i], off[i + 1])
        tree = {k: v[sl] for k, v in cols.items()}
        hit = np.unique(leaf_index(tree, codes_train))
        mask[off[i] + hit] = True
    return mask


def rows_avoiding_empty_leaves(off, cols, populated, codes):
    ok = np.ones(codes.shape[0], dtype=bool)
    for i in range(len(off) - 1):
        sl = slice(off[i], off[i + 1])
        tree = {k: v[sl] for k, v in cols.items()}
        ok &= populated[off[i] + leaf_index(tree, codes)]
    return ok


def gpu_candidates_at(X, y, era, cfg, round_idx, depth):
    """Run ``round_idx`` whole rounds through the booster, then the phases of the next round up to
    the histogram + score pass of ``depth``, and return that pass's candidate table as a structured
    array ``[sampled position][frontier node]`` (score, k, left_count, flags, left_gq), the sampled
    feature list and the number of frontier nodes."""
    import os
    os.environ["PACKBOOST_RUN_AHEAD"] = "0"
    try:
        booster = PackBoost(PackBoostConfig(device="cuda", **cfg))
        booster._start(X, y, era)
        for r in range(round_idx):
            booster._boost_one_round(r, round_idx + 1)
        booster._drain()
        booster._predrawn = None
    finally:
        del os.environ["PACKBOOST_RUN_AHEAD"]
    tr = booster._trainer
    # the generator was advanced past the next round's draws by the look-ahead: rewind to the state
    # the rounds so far leave behind by replaying them on a fresh generator
    F, D, k = tr.F, tr.D, tr.n_sampled()
    rng = torch.Generator(device="cpu")
    rng.manual_seed(int(cfg["random_state"]))
    for n_ctx in booster._round_depths:
        for _ in range(n_ctx):
            torch.randperm(F, generator=rng)
    subsets = [torch.randperm(F, generator=rng)[:k].numpy().astype(np.int32) for _ in range(D)]
    lib, st = tr.lib, C.byref(tr.st)
    stream = torch.cuda.current_stream().cuda_stream
    fh = torch.zeros((D, 3, max(k, 1)), dtype=torch.int32)
    for d in range(D):
        fh[d, 0, :k] = torch.from_numpy(subsets[d])
        fh[d, 1, :k] = torch.from_numpy(subsets[d])
        fh[d, 2, :k] = torch.arange(k, dtype=torch.int32)
    tr.feat_dev.copy_(fh)
    B.check(lib.pb_round_begin(st, 1 if round_idx > 0 else 0, stream))
    for d in range(depth + 1):
        B.check(lib.pb_depth_hist_score(st, d, tr.feat_dev[d, 1].data_ptr(), tr.feat_dev[d, 2].data_ptr(), k, k, stream))
        if d < depth:
            B.check(lib.pb_depth_select(st, d, tr.feat_dev[d, 0].data_ptr(), k, stream))
            B.check(lib.pb_depth_partition(st, d, stream))
    ptr, nbytes = C.c_void_p(), C.c_int64()
    B.check(lib.pb_candidates_buffer(st, depth, k, C.byref(ptr), C.byref(nbytes)))
    off = ptr.value - tr.workspace.data_ptr()
    torch.cuda.synchronize()
    raw = tr.workspace[off: off + nbytes.value].cpu().numpy()
    cand_dt = np.dtype([("score", "<f4"), ("k", "<i4"), ("left_count", "<u4"), ("flags", "<u4"), ("left_gq", "<i8")])
    table = raw.view(cand_dt).reshape(k, 1 << depth)
    head = tr.ctl.cpu().numpy()
    n_ctx = int(np.frombuffer(head[:256].tobytes(), dtype=np.int32, offset=24, count=PB_N_CTX)[depth])
    return table, subsets[depth], n_ctx


PB_N_CTX = 14  # entries of the per-depth frontier counts in the control block head
