"""Kernel-level parity through the C ABI: binning/packing, histograms, legacy predictors."""

import ctypes as C
import os

import numpy as np
import pytest
import torch

from oracle import packboost_oracle as po

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda", 0)


@pytest.mark.parametrize("max_bins", [5, 16, 64, 128])
def test_bin_pack_matches_searchsorted(max_bins):
    from packboost_b200.data import pack_feature_major, pack_row_major, quantile_edges
    rng = np.random.default_rng(max_bins)
    X = rng.normal(size=(1537, 37)).astype(np.float32)
    X[::7, 3] = np.nan
    X[:, 5] = np.round(X[:, 5])
    edges = quantile_edges(np.nan_to_num(X), max_bins)
    want = po.bin_codes(X, edges, max_bins).astype(np.uint8)
    pm = pack_feature_major(X, edges, max_bins)
    np.testing.assert_array_equal(pm.unpack().cpu().numpy(), want.T)
    pr = pack_row_major(X, edges, max_bins)
    raw = pr.codes.cpu().numpy()
    if pr.code_bits == 4:
        got = np.stack([raw & 0xF, raw >> 4], axis=2).reshape(raw.shape[0], -1)[:, : X.shape[1]]
    else:
        got = raw[:, : X.shape[1]]
    np.testing.assert_array_equal(got, want)


def _hist_case(n, f, e, nb, n_nodes, seed, big_era=False):
    from packboost_b200 import backends as B
    from packboost_b200.data import pack_feature_major
    rng = np.random.default_rng(seed)
    codes = rng.integers(0, nb, size=(n, f), dtype=np.uint8)
    if big_era:
        cuts = np.sort(rng.choice(np.arange(1, n), size=e - 1, replace=False))
        cuts[0] = max(cuts[0], 40000) if n > 50000 else cuts[0]
        cuts = np.sort(cuts)
    else:
        cuts = np.sort(rng.choice(np.arange(1, n), size=e - 1, replace=False))
    era_off = np.concatenate([[0], cuts, [n]]).astype(np.int32)
    pm = pack_feature_major(codes, None, nb)
    npad = pm.rows_padded
    gq = np.zeros(npad, np.int32)
    slot = np.full(npad, 0xFFFF, np.uint16)
    slot[:n] = rng.integers(0, n_nodes + 1, size=n)
    slot[:n][slot[:n] == n_nodes] = 0xFFFF      # some rows sit in finished leaves
    dev = _dev()
    t = dict(gq=torch.from_numpy(gq).to(dev), slot=torch.from_numpy(slot.view(np.int16)).to(dev),
             era=torch.from_numpy(era_off).to(dev))
    st = B.TrainState()
    st.n_rows, st.n_features_total, st.n_features_local, st.n_eras = n, f, f, e
    st.max_bins, st.code_bits, st.pitch = nb, pm.code_bits, pm.pitch
    st.max_depth, st.pack_size, st.min_samples_leaf, st.n_thresholds, st.feature_block_size = 6, 1, 1, nb - 1, 32
    st.lambda_l2 = 1.0
    dummy = torch.zeros(max(npad, 4096), dtype=torch.float32, device=dev)
    ids = torch.arange(max(f, nb), dtype=torch.int32, device=dev)
    st.codes, st.era_offsets, st.thr_ids, st.feat_local = pm.codes.data_ptr(), t["era"].data_ptr(), ids.data_ptr(), ids.data_ptr()
    st.y = st.preds = dummy.data_ptr()
    st.gq, st.slot, st.leaf = t["gq"].data_ptr(), t["slot"].data_ptr(), t["slot"].data_ptr()
    ctl = torch.zeros(int(B.lib().pb_ctl_bytes()), dtype=torch.uint8, device=dev)
    ws = torch.zeros(int(B.lib().pb_workspace_min_bytes(C.byref(st))) + 1024, dtype=torch.uint8, device=dev)
    st.ctl, st.workspace, st.workspace_bytes = ctl.data_ptr(), ws.data_ptr(), ws.numel()
    B.check(B.lib().pb_train_prepare(C.byref(st), era_off.ctypes.data))
    lim = 1 << int(st.gq_bits)
    gq[:n] = rng.integers(-lim, lim + 1, size=n)     # the full range the quantiser may produce
    t["gq"].copy_(torch.from_numpy(gq))
    feat = rng.permutation(f)[: max(1, f // 2)].astype(np.int32)
    feat_t = torch.from_numpy(feat).to(dev)
    cnt = torch.full((feat.shape[0], e, n_nodes, nb), -1, dtype=torch.int32, device=dev)
    gs = torch.full((feat.shape[0], e, n_nodes, nb), -1, dtype=torch.int64, device=dev)
    B.check(B.lib().pb_hist_build(C.byref(st), feat_t.data_ptr(), feat.shape[0], n_nodes, n_nodes, cnt.data_ptr(),
                                  gs.data_ptr(), torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    # numpy reference (exact integers)
    era_of = np.repeat(np.arange(e), np.diff(era_off))
    live = slot[:n] != 0xFFFF
    want_c = np.zeros((feat.shape[0], n_nodes, e, nb), np.int64)
    want_g = np.zeros_like(want_c)
    for i, fid in enumerate(feat):
        key = (slot[:n][live].astype(np.int64) * e + era_of[live]) * nb + codes[live, fid]
        want_c[i] = np.bincount(key, minlength=n_nodes * e * nb).reshape(n_nodes, e, nb)
        pos = np.bincount(key, weights=np.maximum(gq[:n][live], 0).astype(np.float64), minlength=n_nodes * e * nb)
        # float64 bincount is not exact at this magnitude; accumulate exactly instead
        acc = np.zeros(n_nodes * e * nb, np.int64)
        np.add.at(acc, key, gq[:n][live].astype(np.int64))
        want_g[i] = acc.reshape(n_nodes, e, nb)
    # device layout is [feature][era][node][bin]
    np.testing.assert_array_equal(cnt.cpu().numpy().astype(np.int64).transpose(0, 2, 1, 3), want_c)
    np.testing.assert_array_equal(gs.cpu().numpy().transpose(0, 2, 1, 3), want_g)


@pytest.mark.parametrize("n,f,e,nb,nodes", [
    (5000, 12, 7, 5, 1), (5000, 12, 7, 5, 32), (4097, 9, 3, 16, 4), (6000, 10, 5, 128, 8),
    (3001, 6, 4, 200, 3), (20000, 5, 2, 64, 300), (1000, 3, 1, 2, 1), (16000, 4, 2, 5, 2),
    (7000, 70, 3, 5, 2), (7000, 41, 3, 5, 8), (7000, 33, 2, 5, 50), (5000, 9, 2, 16, 1), (5000, 9, 2, 3, 9),
    (5000, 20, 2, 16, 17),
])
def test_histogram_exact(n, f, e, nb, nodes):
    _hist_case(n, f, e, nb, nodes, seed=n + nb)


def test_histogram_exact_when_an_era_spans_several_tiles():
    _hist_case(120_000, 6, 3, 5, 4, seed=5, big_era=True)
    _hist_case(90_000, 4, 1, 32, 2, seed=6)
    _hist_case(30_000, 3, 2, 128, 40, seed=7)


def test_legacy_predictors_match_oracle_router():
    from packboost_b200 import backends as B
    rng = np.random.default_rng(3)
    n, f = 3000, 40
    codes = rng.integers(0, 16, size=(n, f), dtype=np.uint8)
    # three random (not complete) trees with BFS-compact numbering
    trees = []
    for t in range(3):
        tr = po.OracleTree()
        frontier = [0]
        for depth in range(4):
            nxt = []
            for nid in frontier:
                if rng.random() < 0.8:
                    l, r = tr.split(nid, int(rng.integers(0, f)), int(rng.integers(0, 15)))
                    tr.set_leaf(l, float(rng.normal()))
                    tr.set_leaf(r, float(rng.normal()))
                    nxt += [l, r]
            frontier = nxt
        trees.append(tr.arrays())
    dev = _dev()
    fm = torch.from_numpy(np.ascontiguousarray(codes.T)).to(dev)
    for tr in trees:
        got = B.predict_bins_cuda(fm, *(torch.from_numpy(tr[k].astype(np.int32)).to(dev) for k in ("feature", "threshold", "left", "right")),
                                  torch.from_numpy(tr["value"].astype(np.float32)).to(dev),
                                  torch.from_numpy(tr["is_leaf"].astype(np.uint8)).to(dev))
        np.testing.assert_array_equal(got.cpu().numpy().view(np.int32), po.route_tree(tr, codes.astype(np.int8)).view(np.int32))
    # pack: absolute child ids, out = w * sum of leaves
    off = np.cumsum([0] + [t["feature"].shape[0] for t in trees]).astype(np.int32)
    cat = {k: np.concatenate([t[k] for t in trees]) for k in trees[0]}
    la = np.concatenate([np.where(t["left"] >= 0, t["left"] + o, -1) for t, o in zip(trees, off[:-1])]).astype(np.int32)
    ra = np.concatenate([np.where(t["right"] >= 0, t["right"] + o, -1) for t, o in zip(trees, off[:-1])]).astype(np.int32)
    got = B.predict_pack_cuda(fm, torch.from_numpy(cat["feature"]).to(dev), torch.from_numpy(cat["threshold"]).to(dev),
                              torch.from_numpy(la).to(dev), torch.from_numpy(ra).to(dev),
                              torch.from_numpy(cat["value"].astype(np.float32)).to(dev),
                              torch.from_numpy(cat["is_leaf"].astype(np.uint8)).to(dev), torch.from_numpy(off).to(dev), 0.25)
    want = np.zeros(n, np.float32)
    for tr in trees:
        want = want + po.route_tree(tr, codes.astype(np.int8))
    np.testing.assert_allclose(got.cpu().numpy(), np.float32(0.25) * want, rtol=1e-6, atol=1e-7)


def test_superseded_frontier_calls_say_so():
    from packboost_b200 import backends as B
    assert B.cuda_available() and not B.cpu_available()
    for fn in (B.find_best_splits_batched_cuda, B.partition_frontier_cuda, B.find_best_splits_batched):
        with pytest.raises(RuntimeError):
            fn()


def test_era_correlation_matches_host_formula():
    """Device per-era correlation against the reference's numpy loop, with the eras it skips:
    a single-row era, an era of constant predictions and an era of constant targets."""
    import ctypes as C
    from packboost_b200 import backends as B
    from packboost_b200.booster import _era_correlation_np
    rng = np.random.default_rng(5)
    sizes = [700, 1, 333, 50, 1200, 64]
    era = np.repeat(np.arange(len(sizes)), sizes).astype(np.int16)
    n = era.shape[0]
    y = rng.integers(0, 5, size=n).astype(np.float32) / 4
    p = (0.05 * y + 0.02 * rng.standard_normal(n)).astype(np.float32)
    p[era == 3] = 0.125          # constant predictions
    y[era == 5] = 0.5            # constant targets
    offs = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int32)
    dev = torch.device("cuda", 0)
    yd, pd, od = (torch.from_numpy(a).to(dev) for a in (y, p, offs))
    out = torch.empty(len(sizes), dtype=torch.float64, device=dev)
    B.check(B.lib().pb_era_correlation(yd.data_ptr(), pd.data_ptr(), od.data_ptr(), len(sizes), out.data_ptr(),
                                       torch.cuda.current_stream().cuda_stream))
    c = out.cpu().numpy()
    assert np.isnan(c[[1, 3, 5]]).all() and np.isfinite(c[[0, 2, 4]]).all()
    want = _era_correlation_np(era, y, p)
    np.testing.assert_allclose(c[np.isfinite(c)].mean(), want, rtol=1e-5)


def test_device_quantile_edges_equal_host_quantile_edges():
    from packboost_b200.data import quantile_edges, quantile_edges_device
    rng = np.random.default_rng(3)
    X = rng.normal(size=(60_001, 33)).astype(np.float32)
    X[:, 4] = np.round(X[:, 4] * 2)
    X[:, 9] = np.exp(X[:, 9])
    for nb in (5, 128):
        want = quantile_edges(X, nb)
        assert np.array_equal(quantile_edges_device(X, nb), want)
        assert np.array_equal(quantile_edges_device(torch.from_numpy(X).cuda(), nb), want)


def _oracle_candidates(trace, K):
    """Best threshold of every (sampled position, frontier node) from the oracle's per-candidate
    scores: highest score, then largest left count, then largest threshold index
    (packboost/booster.py:1912-1919 restricted to one feature)."""
    out = {}
    pos = 0
    for blk in trace["blocks"]:
        score = blk["score"].numpy()          # [node, feature in block, K], -inf where min_samples_leaf fails
        lc = blk["left_count"].numpy()
        for j in range(score.shape[1]):
            for n in range(score.shape[0]):
                s, c = score[n, j], lc[n, j]
                best = None
                for k in range(K):
                    if np.isnan(s[k]):
                        continue
                    if best is None or s[k] > s[best] or (s[k] == s[best] and c[k] >= c[best]):
                        best = k
                out[(pos + j, n)] = (np.float32(s[best]), best, int(c[best]))
        pos += score.shape[1]
    return out


@pytest.mark.parametrize("case,round_idx,depth", [("prebinned5", 0, 0), ("prebinned5", 1, 3), ("prebinned5", 3, 4),
                                                  ("config1", 0, 2), ("config1", 4, 4), ("ragged_eras", 2, 3),
                                                  ("kcuts_even", 1, 2), ("interleaved", 2, 3)])
def test_scorer_candidates_match_oracle_bit_for_bit(case, round_idx, depth):
    """Kernel-level check of the histogram + DES scorer pass: the candidate table it writes (best
    threshold of every sampled feature at every frontier node: float32 score, threshold index,
    left count) against the oracle's per-candidate scores in its exact-sum variant, for frontiers
    of one to sixteen nodes in the first and in later rounds."""
    import cases
    from gpu_util import gpu_candidates_at
    X, y, era, cfg, rounds, _ = cases.CASES[case]()
    table, subset, n_ctx = gpu_candidates_at(X, y, era, cfg, round_idx, depth)
    model = po.fit(X, y, era, po.OracleParams(exact_sums=True, **cfg), round_idx + 1, trace_at=(round_idx, depth))
    tr = model.trace
    assert tr, "the oracle did not reach this frontier"
    np.testing.assert_array_equal(tr["subset"].numpy(), subset)
    K = tr["blocks"][0]["K"]
    want = _oracle_candidates(tr, K)
    assert n_ctx == len(tr["context_nodes"])
    bad = []
    for (p, n), (s, k, c) in want.items():
        g = table[p, n]
        if (np.float32(g["score"]).view(np.int32) != s.view(np.int32)) or int(g["k"]) != k or int(g["left_count"]) != c:
            bad.append((p, n, float(g["score"]), int(g["k"]), int(g["left_count"]), float(s), k, c))
    assert not bad, f"{len(bad)} of {len(want)} candidates differ, first: {bad[:5]}"


_SHAPE_SCRIPT = """
import sys
sys.path.insert(0, {root!r})
from tests.test_gpu_kernels import _hist_case
_hist_case(7000, 70, 3, 5, 2, seed=11)
_hist_case(5000, 40, 2, 16, 1, seed=12)
_hist_case(9000, 300, 4, 5, 4, seed=13)
_hist_case(6000, 24, 3, 3, 9, seed=14)
_hist_case(4100, 16, 2, 5, 30, seed=15)
print("ok")
"""


@pytest.mark.parametrize("shape", ["1 8 1", "1 4 2", "1 1 4", "2 4 1", "2 2 2", "2 1 4", "2 4 2", "1 8 2", "1 2 1"])
def test_histogram_exact_in_every_launch_shape(shape):
    """The launcher picks the shape <features per joint code, tuples per lane, row phases> of the
    lane kernel by a cost model, so a given test size exercises one shape only.  The tuning
    override forces each shape in turn (it is read once per process, hence the child process) and
    the same exact-integer comparison runs on several sizes; the launch log must show that the
    forced shape really ran."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, PACKBOOST_HIST_SHAPE=shape)
    res = subprocess.run([sys.executable, "-c", _SHAPE_SCRIPT.format(root=root)], env=env, capture_output=True,
                         text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    assert res.stdout.strip().endswith("ok")
    assert "hist_lane_kernel<%s>" % shape.replace(" ", ",") in res.stderr, res.stderr[-2000:]
