"""Properties that hold at any size, checked at the full sizes of the headline workloads.

The oracle cannot run 2.7 M x 2 376 in seconds, so these tests use what the domain offers
instead: conservation of counts and gradient sums in the histograms, leaf values recomputed from
the rows a tree routes to each leaf, agreement of the prediction state kept during training with
inference, run-to-run bit identity, and for the ensemble predictor exact scaling and exact
chaining of partial ensembles.
"""

import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

N_ROWS, N_FEAT, N_ERAS = 2_700_000, 2376, 574
CFG = dict(pack_size=32, max_depth=6, learning_rate=0.4 / 32, lambda_l2=1e-6, lambda_dro=0.5,
           min_samples_leaf=20, max_bins=5, layer_feature_fraction=0.1, prebinned=True, random_state=42)


def _need_memory(gib):
    free, _ = torch.cuda.mem_get_info(0)
    if free < gib * (1 << 30):
        pytest.skip(f"needs {gib} GiB of free device memory")


@pytest.fixture(scope="module")
def table():
    from packboost_b200.workloads import config3_device
    _need_memory(24)
    dev = torch.device("cuda", 0)
    n = N_ROWS // N_ERAS * N_ERAS
    X, y, era = config3_device(n, N_FEAT, N_ERAS, dev)
    yield X, y.cpu().numpy(), era.cpu().numpy()
    del X
    torch.cuda.empty_cache()


def _route(X, tree):
    """Leaf index of every row (device tensors; one gather per level of the tree)."""
    a = tree.arrays()
    dev = X.device
    feature = torch.from_numpy(a["feature"].astype(np.int64)).to(dev)
    threshold = torch.from_numpy(a["threshold"].astype(np.int64)).to(dev)
    left = torch.from_numpy(a["left"].astype(np.int64)).to(dev)
    right = torch.from_numpy(a["right"].astype(np.int64)).to(dev)
    is_leaf = torch.from_numpy(a["is_leaf"].astype(bool)).to(dev)
    node = torch.zeros(X.shape[0], dtype=torch.int64, device=dev)
    rows = torch.arange(X.shape[0], device=dev)
    for _ in range(64):
        live = ~is_leaf[node]
        if not bool(live.any()):
            break
        f = feature[node].clamp_min(0)
        code = X[rows, f].to(torch.int64)
        nxt = torch.where(code <= threshold[node], left[node], right[node])
        node = torch.where(live, nxt, node)
    return node, a


def test_first_round_leaf_values_follow_from_the_routed_rows(table):
    """Round 1 starts from predictions 0, so the gradient of a row is -y and a leaf's value is
    sum(y) / (count + lambda) over the rows the tree sends there: checks histograms, winner
    bookkeeping and the row -> node partition against one another on all 2.7 M rows."""
    from packboost_b200 import PackBoost, PackBoostConfig
    X, y, era = table
    booster = PackBoost(PackBoostConfig(device="cuda", **CFG))
    booster.fit(X, y, era, num_rounds=1)
    tree = booster.trees[0]
    node, a = _route(X, tree)
    n_nodes = a["feature"].shape[0]
    yd = torch.from_numpy(y).to(X.device).double()
    cnt = torch.bincount(node, minlength=n_nodes).cpu().numpy()
    sy = torch.bincount(node, weights=yd, minlength=n_nodes).cpu().numpy()
    leaf = a["is_leaf"].astype(bool)
    assert leaf.sum() >= 2, "the tree must have split"
    assert cnt[~leaf].sum() == 0 and cnt[leaf].sum() == X.shape[0]
    assert (cnt[leaf] >= CFG["min_samples_leaf"]).all()
    want = sy[leaf] / (cnt[leaf] + CFG["lambda_l2"])
    np.testing.assert_allclose(a["value"][leaf], want, rtol=1e-5, atol=1e-7)
    # the prediction state of training equals inference on the same rows
    p_train = booster.train_predictions()
    lr = np.float32(CFG["learning_rate"])
    want_p = (a["value"].astype(np.float32)[node.cpu().numpy()] * lr * CFG["pack_size"]).astype(np.float32)
    np.testing.assert_allclose(p_train, want_p, rtol=1e-5, atol=1e-8)
    head = slice(0, 200_000)
    np.testing.assert_allclose(booster.predict(X[head]), p_train[head], rtol=1e-5, atol=1e-8)


def test_two_fits_are_bit_identical_and_pipelining_changes_nothing(table, monkeypatch):
    """Three rounds, twice with the round graph and the host one round ahead, once with both
    switched off: the same trees and the same predictions, bit for bit."""
    from packboost_b200 import PackBoost, PackBoostConfig
    from gpu_util import flatten_trees
    X, y, era = table

    def run():
        b = PackBoost(PackBoostConfig(device="cuda", **CFG))
        b.fit(X, y, era, num_rounds=3)
        off, cols = flatten_trees(b.trees)
        return off, cols, b.train_predictions()

    first = run()
    second = run()
    monkeypatch.setenv("PACKBOOST_RUN_AHEAD", "0")
    monkeypatch.setenv("PACKBOOST_CUDA_GRAPH", "0")
    plain = run()
    for other in (second, plain):
        np.testing.assert_array_equal(first[0], other[0])
        for k in first[1]:
            x, z = first[1][k], other[1][k]
            if k == "value":
                x, z = x.view(np.int64), z.view(np.int64)
            np.testing.assert_array_equal(x, z, err_msg=k)
        np.testing.assert_array_equal(first[2].view(np.int32), other[2].view(np.int32))


def test_histograms_conserve_counts_and_gradient_sums(table):
    """Every sampled feature partitions the same rows, so for each (era, node) the counts and the
    fixed-point gradient sums added over a feature's bins must be the same for all 238 features
    and equal to a direct reduction of the row state."""
    from packboost_b200 import backends as B
    from packboost_b200.data import pack_feature_major
    X, _y, era = table
    dev = X.device
    lib = B.lib()
    n, F = X.shape
    E, NB, nodes, Fs = N_ERAS, 5, 32, 238
    pm = pack_feature_major(X, None, NB)
    npad = pm.rows_padded
    era_off = np.concatenate([[0], np.cumsum(np.bincount(era.astype(np.int64), minlength=E))]).astype(np.int32)
    g = torch.Generator(device=dev)
    g.manual_seed(9)
    st = B.TrainState()
    st.n_rows, st.n_features_total, st.n_features_local, st.n_eras = n, F, F, E
    st.max_bins, st.code_bits, st.pitch = NB, pm.code_bits, pm.pitch
    st.max_depth, st.pack_size, st.min_samples_leaf, st.n_thresholds, st.feature_block_size = 6, 1, 1, NB - 1, 32
    st.lambda_l2 = 1.0
    dummy = torch.zeros(npad, dtype=torch.float32, device=dev)
    ids = torch.arange(F, dtype=torch.int32, device=dev)
    era_t = torch.from_numpy(era_off).to(dev)
    gq = torch.zeros(npad, dtype=torch.int32, device=dev)
    slot = torch.full((npad,), -1, dtype=torch.int16, device=dev)
    st.codes, st.era_offsets, st.thr_ids, st.feat_local = pm.codes.data_ptr(), era_t.data_ptr(), ids.data_ptr(), ids.data_ptr()
    st.y = st.preds = dummy.data_ptr()
    st.gq, st.slot, st.leaf = gq.data_ptr(), slot.data_ptr(), slot.data_ptr()
    ctl = torch.zeros(int(lib.pb_ctl_bytes()), dtype=torch.uint8, device=dev)
    ws = torch.zeros(int(lib.pb_workspace_min_bytes(C.byref(st))) + 1024, dtype=torch.uint8, device=dev)
    st.ctl, st.workspace, st.workspace_bytes = ctl.data_ptr(), ws.data_ptr(), ws.numel()
    B.check(lib.pb_train_prepare(C.byref(st), era_off.ctypes.data))
    lim = 1 << int(st.gq_bits)
    gq[:n] = torch.randint(-lim, lim + 1, (n,), generator=g, device=dev, dtype=torch.int32)
    s_rows = torch.randint(0, nodes + 1, (n,), generator=g, device=dev, dtype=torch.int32)
    s_rows[s_rows == nodes] = -1                      # rows that sit in finished leaves
    slot[:n] = s_rows.to(torch.int16)
    feat = torch.randperm(F, generator=g, device=dev)[:Fs].to(torch.int32)
    cnt = torch.empty((Fs, E, nodes, NB), dtype=torch.int32, device=dev)
    gs = torch.empty((Fs, E, nodes, NB), dtype=torch.int64, device=dev)
    B.check(lib.pb_hist_build(C.byref(st), feat.data_ptr(), Fs, nodes, nodes, cnt.data_ptr(), gs.data_ptr(),
                              torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    # direct reduction of the row state per (era, node)
    live = s_rows >= 0
    key = torch.from_numpy(era.astype(np.int64)).to(dev)[live] * nodes + s_rows[live].to(torch.int64)
    want_c = torch.bincount(key, minlength=E * nodes).view(E, nodes)
    want_g = torch.zeros(E * nodes, dtype=torch.int64, device=dev).scatter_add_(0, key, gq[:n][live].to(torch.int64))
    want_g = want_g.view(E, nodes)
    got_c = cnt.to(torch.int64).sum(dim=3)            # [Fs, E, nodes]
    got_g = gs.sum(dim=3)
    assert bool((got_c == want_c.unsqueeze(0)).all())
    assert bool((got_g == want_g.unsqueeze(0)).all())
    # and one feature in full against a direct count of its codes
    f0 = int(feat[0])
    k3 = key * NB + X[:, f0][live].to(torch.int64)
    full = torch.bincount(k3, minlength=E * nodes * NB).view(E, nodes, NB)
    assert bool((cnt[0].to(torch.int64) == full).all())


def _heap_ensemble_packed(feature, threshold, leaf):
    """Heap-ordered complete trees (left = 2i+1, right = 2i+2) as 8-byte predictor nodes."""
    T, n_int = feature.shape
    n_leaf = leaf.shape[1]
    idx = np.arange(n_int, dtype=np.uint32)
    w0 = np.concatenate([(feature.astype(np.uint32) & 0xFFFF) | (threshold.astype(np.uint32) << 16),
                         np.full((T, n_leaf), 1 << 31, np.uint32)], axis=1)
    w1 = np.concatenate([np.broadcast_to(2 * idx + 1, (T, n_int)), leaf.view(np.uint32)], axis=1)
    packed = np.stack([w0, w1], axis=2).reshape(-1, 2).view(np.int32).copy()
    return packed, n_int + n_leaf


def test_ensemble_predictor_scales_and_chains_exactly():
    """Inference-only workload (2 000 rounds x 32 trees of depth 6 over 2 376 five-level features)
    on 100 000 rows: doubling the tree weight doubles every prediction exactly (a power of two
    commutes with every rounding), running the ensemble in two parts with the first part's output
    as the second part's start equals the single run bit for bit (the sum is sequential in tree
    order), and a sample of rows matches the oracle's router."""
    from oracle import packboost_oracle as po
    from packboost_b200 import backends as B, workloads
    from packboost_b200.data import pack_row_major
    _need_memory(8)
    dev = torch.device("cuda", 0)
    lib = B.lib()
    w = workloads.config5(seed=5, n_rows=1000, n_features=2376, n_rounds=2000, pack_size=32, depth=6)
    feature, threshold, leaf = w.extra["feature"], w.extra["threshold"], w.extra["leaf"]
    T = feature.shape[0]
    packed_np, per_tree = _heap_ensemble_packed(feature, threshold, leaf)
    packed = torch.from_numpy(packed_np).to(dev)
    offs = torch.arange(T + 1, dtype=torch.int32, device=dev) * per_tree
    n_rows = 100_000
    g = torch.Generator(device=dev)
    g.manual_seed(1)
    X = torch.randint(0, 5, (n_rows, 2376), generator=g, device=dev, dtype=torch.uint8)
    rows = pack_row_major(X, None, 5)
    stream = torch.cuda.current_stream().cuda_stream

    def run(t0, t1, weight, init=None):
        out = torch.empty(n_rows, dtype=torch.float32, device=dev)
        B.check(lib.pb_predict_rows_packed(rows.codes.data_ptr(), n_rows, rows.pitch_row, rows.code_bits,
                                           packed.data_ptr(), offs[t0:].data_ptr(), 0, t1 - t0, per_tree, weight,
                                           out.data_ptr(), init.data_ptr() if init is not None else 0, stream))
        return out

    whole = run(0, T, 1.0)
    twice = run(0, T, 2.0)
    assert bool((twice == 2.0 * whole).all())
    cut = 20_008                                      # not a multiple of the trees walked together
    second = run(cut, T, 1.0, init=run(0, cut, 1.0))
    assert bool((second.view(torch.int32) == whole.view(torch.int32)).all())
    assert float(whole.abs().max()) > 0.1
    sample = 48
    trees = workloads.heap_ensemble_to_trees(feature[:640], threshold[:640], leaf[:640])
    want = po.predict_codes(trees, X[:sample].cpu().numpy().astype(np.int8), 1.0)
    got = run(0, 640, 1.0)[:sample].cpu().numpy()
    np.testing.assert_array_equal(got.view(np.int32), want.view(np.int32))
