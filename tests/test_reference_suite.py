"""The reference project's own test cases, run against this backend through the reference's
import paths (``packboost.booster``, ``packboost.config``, ``packboost.data``).

Each test restates one case of the reference's suite with the same data, configuration and
assertions (cited per test).  Two of the reference's expectations are stale in the reference
itself and are parameterised here instead of copied:

* ``tests/test_config.py:4-9`` expects ``PackBoostConfig().device == "cpu"`` although
  ``packboost/config.py:89`` sets ``"cuda"``: the default is ``"cuda"`` here as well.
* ``tests/test_execution_modes.py:50-52`` expects ``tree_weight == learning_rate / pack_size``
  although ``packboost/booster.py:583,598`` sums the pack (``tree_weight == learning_rate``): the
  summed pack is what both implementations do.

The hand-built DES known answer of ``tests/test_des.py:9-217`` uses non-unit hessians and the
helper-form direction term; it pins the oracle (``tests/test_oracle_golden.py``).
"""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _linear_dataset(n_rows=200, n_features=6, n_eras=10):
    rng = np.random.default_rng(42)
    X = rng.normal(size=(n_rows, n_features)).astype(np.float32)
    coefs = rng.normal(size=n_features).astype(np.float32)
    y = X @ coefs + 0.1 * rng.standard_normal(n_rows)
    eras = np.repeat(np.arange(n_eras, dtype=np.int16), n_rows // n_eras)
    if eras.shape[0] < n_rows:
        extra = rng.integers(0, n_eras, size=n_rows - eras.shape[0], dtype=np.int16)
        eras = np.concatenate([eras, extra])
    return X, y.astype(np.float32), eras


def test_booster_fit_predict_improves_loss():
    """tests/test_booster_small.py:22-42"""
    from packboost.booster import PackBoost
    from packboost.config import PackBoostConfig
    X, y, eras = _linear_dataset()
    config = PackBoostConfig(pack_size=4, max_depth=3, learning_rate=0.2, lambda_l2=1e-3, lambda_dro=0.1,
                             direction_weight=0.05, min_samples_leaf=5, max_bins=63, layer_feature_fraction=0.6,
                             random_state=13)
    booster = PackBoost(config)
    booster.fit(X, y, eras, num_rounds=3)
    preds = booster.predict(X)
    assert preds.shape == (X.shape[0],)
    assert float(np.mean((y - preds) ** 2)) < float(np.mean((y - y.mean()) ** 2))


def test_booster_accepts_dataframe():
    """tests/test_booster_small.py:45-52"""
    import pandas as pd
    from packboost.booster import PackBoost
    from packboost.config import PackBoostConfig
    X, y, eras = _linear_dataset(n_rows=120, n_features=4, n_eras=6)
    df = pd.DataFrame(X, columns=[f"f{i}" for i in range(X.shape[1])])
    booster = PackBoost(PackBoostConfig(pack_size=2, max_depth=2, learning_rate=0.1, random_state=7))
    booster.fit(df, y, eras, num_rounds=2)
    assert booster.predict(df).shape == (df.shape[0],)


def _shuffled_dataset(seed=0, n_rows=320, n_features=12, n_eras=8):
    rng = np.random.default_rng(seed)
    X = rng.normal(size=(n_rows, n_features)).astype(np.float32)
    coefs = rng.normal(size=n_features).astype(np.float32)
    y = (X @ coefs + 0.1 * rng.standard_normal(n_rows)).astype(np.float32)
    eras = np.arange(n_rows, dtype=np.int16) % n_eras
    rng.shuffle(eras)
    return X, y, eras


def _fit_model(config, num_rounds=3):
    from packboost.booster import PackBoost
    X, y, eras = _shuffled_dataset(seed=123)
    booster = PackBoost(config)
    booster.fit(X, y, eras, num_rounds=num_rounds)
    return booster, X, y, eras


def test_predict_packwise_matches_predict():
    """tests/test_packboost_parity.py:25-38"""
    from packboost.config import PackBoostConfig
    config = PackBoostConfig(pack_size=3, max_depth=3, learning_rate=0.1, min_samples_leaf=10, max_bins=63,
                             random_state=11, histogram_mode="auto")
    booster, X, _, _ = _fit_model(config)
    np.testing.assert_allclose(booster.predict(X), booster.predict_packwise(X, block_size_trees=2), atol=1e-7, rtol=0.0)


@pytest.mark.parametrize("seed", [3, 7, 19])
def test_split_determinism(seed):
    """tests/test_packboost_parity.py:41-64"""
    from packboost.booster import PackBoost
    from packboost.config import PackBoostConfig
    config = PackBoostConfig(pack_size=2, max_depth=4, learning_rate=0.15, min_samples_leaf=8, max_bins=63,
                             histogram_mode="auto", random_state=seed)
    booster1, X, y, eras = _fit_model(config)
    booster2 = PackBoost(config)
    booster2.fit(X, y, eras, num_rounds=3)
    assert len(booster1.trees) == len(booster2.trees)
    for tree_a, tree_b in zip(booster1.trees, booster2.trees):
        assert len(tree_a.nodes) == len(tree_b.nodes)
        for node_a, node_b in zip(tree_a.nodes, tree_b.nodes):
            assert node_a.feature == node_b.feature
            assert node_a.threshold == node_b.threshold
            assert node_a.is_leaf == node_b.is_leaf
            if node_a.is_leaf:
                assert np.isclose(node_a.value, node_b.value, atol=1e-9)


@pytest.mark.parametrize("hist_mode", ["auto", "subtract", "rebuild"])
def test_validator_accounting(hist_mode):
    """tests/test_packboost_parity.py:67-87"""
    from packboost.config import PackBoostConfig
    config = PackBoostConfig(pack_size=2, max_depth=3, learning_rate=0.1, min_samples_leaf=6, max_bins=63,
                             histogram_mode=hist_mode, random_state=5)
    booster, _, _, _ = _fit_model(config, num_rounds=2)
    assert booster._depth_logs
    for depth_log in booster._depth_logs:
        nodes_processed = depth_log["nodes_processed"]
        assert depth_log["nodes_subtract_ok"] + depth_log["nodes_rebuild"] == nodes_processed
        if hist_mode == "rebuild":
            assert depth_log["nodes_subtract_ok"] == 0
        else:
            assert depth_log["nodes_subtract_ok"] >= 0
            assert depth_log["nodes_subtract_fallback"] <= depth_log["nodes_rebuild"]


def _random_regression(seed=42):
    rng = np.random.default_rng(seed)
    X = rng.normal(size=(256, 6)).astype(np.float32)
    coefs = rng.normal(size=6).astype(np.float32)
    y = X @ coefs + 0.1 * rng.standard_normal(X.shape[0])
    eras = rng.integers(0, 4, size=X.shape[0], dtype=np.int32)
    return X, y.astype(np.float32), eras


def _tree_signature(booster):
    return [(node.feature, node.threshold, node.is_leaf) for tree in booster.trees for node in tree.nodes]


def test_pack_weight_applied_and_manual_sum_equals_predict():
    """tests/test_execution_modes.py:31-57 (the weight expectation is the summed pack, see the
    module docstring)."""
    from packboost.booster import PackBoost
    from packboost.config import PackBoostConfig
    from packboost.data import apply_bins
    X, y, eras = _random_regression()
    config = PackBoostConfig(pack_size=4, max_depth=2, learning_rate=0.2, lambda_l2=1e-3, min_samples_leaf=5,
                             max_bins=63, random_state=7, histogram_mode="rebuild")
    booster = PackBoost(config)
    booster.fit(X, y, eras, num_rounds=2)
    assert booster._tree_weight is not None
    assert pytest.approx(config.learning_rate) == booster._tree_weight
    assert booster._binner is not None
    bins = apply_bins(X, booster._binner.bin_edges, booster.config.max_bins)
    bins_tensor = torch.from_numpy(bins).to(device=booster._device)
    manual = np.zeros(X.shape[0], dtype=np.float32)
    for tree in booster.trees:
        manual += booster._tree_weight * tree.predict_bins(bins_tensor).cpu().numpy()
    np.testing.assert_allclose(booster.predict(X), manual, rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("mode", ["subtract", "auto"])
def test_histogram_modes_match_rebuild(mode):
    """tests/test_execution_modes.py:60-81"""
    from packboost.booster import PackBoost
    from packboost.config import PackBoostConfig
    X, y, eras = _random_regression(seed=202)
    base = dict(pack_size=1, max_depth=3, learning_rate=0.1, lambda_l2=1e-3, min_samples_leaf=5, max_bins=31,
                random_state=11, enable_node_batching=True)
    rebuild = PackBoost(PackBoostConfig(histogram_mode="rebuild", **base))
    rebuild.fit(X, y, eras, num_rounds=2)
    other = PackBoost(PackBoostConfig(histogram_mode=mode, **base))
    other.fit(X, y, eras, num_rounds=2)
    np.testing.assert_allclose(rebuild.predict(X), other.predict(X), rtol=1e-6, atol=1e-6)
    assert _tree_signature(rebuild) == _tree_signature(other)


def test_histogram_subtraction_invariants_random():
    """tests/test_execution_modes.py:84-132: left + right == total for counts, gradient and
    hessian sums of ``_batched_histograms_nodes`` (general hessians)."""
    from packboost.booster import PackBoost
    from packboost.config import PackBoostConfig
    config = PackBoostConfig(max_bins=16)
    booster = PackBoost(config)
    device = booster._device
    rng = torch.Generator(device=device)
    rng.manual_seed(1234)
    for _ in range(20):
        rows, features, num_eras = 128, 3, 4
        bins_matrix = torch.randint(0, config.max_bins, (rows, features), generator=rng, dtype=torch.int64, device=device)
        grad_rows = torch.randn(rows, generator=rng, dtype=torch.float32, device=device)
        hess_rows = torch.rand(rows, generator=rng, dtype=torch.float32, device=device) + 0.1
        era_ids = torch.randint(0, num_eras, (rows,), generator=rng, dtype=torch.int64, device=device)
        node_ids = torch.zeros(rows, dtype=torch.int64, device=device)
        counts, grad_hist, hess_hist = booster._batched_histograms_nodes(
            bins_matrix, grad_rows, hess_rows, era_ids, node_ids, num_nodes=1, num_eras=num_eras,
            num_bins=config.max_bins)
        assert counts.shape == (features, 1, num_eras, config.max_bins)
        counts, grad_hist, hess_hist = counts[:, 0], grad_hist[:, 0], hess_hist[:, 0]
        left_count = counts[:, :, :-1].cumsum(dim=2)
        left_grad = grad_hist[:, :, :-1].cumsum(dim=2)
        left_hess = hess_hist[:, :, :-1].cumsum(dim=2)
        total_count = counts.sum(dim=2, keepdim=True)
        total_grad = grad_hist.sum(dim=2, keepdim=True)
        total_hess = hess_hist.sum(dim=2, keepdim=True)
        right_count_sub = total_count - left_count
        right_grad_sub = total_grad - left_grad
        right_hess_sub = total_hess - left_hess
        right_count_rebuild = counts[:, :, 1:].flip(2).cumsum(2).flip(2)
        right_grad_rebuild = grad_hist[:, :, 1:].flip(2).cumsum(2).flip(2)
        right_hess_rebuild = hess_hist[:, :, 1:].flip(2).cumsum(2).flip(2)
        torch.testing.assert_close(right_count_sub, right_count_rebuild, atol=0, rtol=0)
        torch.testing.assert_close(right_grad_sub, right_grad_rebuild, atol=1e-5, rtol=1e-6)
        torch.testing.assert_close(right_hess_sub, right_hess_rebuild, atol=1e-5, rtol=1e-6)
        assert torch.all(right_count_sub >= 0)
        assert torch.all(right_hess_sub >= -1e-5)
        # and against a direct reduction of the inputs
        for f in range(features):
            for e in range(num_eras):
                m = era_ids == e
                want_c = torch.bincount(bins_matrix[m, f], minlength=config.max_bins)
                assert torch.equal(counts[f, e], want_c)
                want_h = torch.zeros(config.max_bins, device=device).index_add_(0, bins_matrix[m, f], hess_rows[m])
                torch.testing.assert_close(hess_hist[f, e], want_h, atol=1e-5, rtol=1e-5)


def test_node_batching_matches_sequential():
    """tests/test_execution_modes.py:135-155"""
    from packboost.booster import PackBoost
    from packboost.config import PackBoostConfig
    X, y, eras = _random_regression(seed=99)
    common = dict(pack_size=1, max_depth=3, learning_rate=0.1, lambda_l2=1e-3, min_samples_leaf=4, max_bins=31,
                  random_state=5, histogram_mode="rebuild")
    batched = PackBoost(PackBoostConfig(enable_node_batching=True, **common))
    batched.fit(X, y, eras, num_rounds=3)
    sequential = PackBoost(PackBoostConfig(enable_node_batching=False, **common))
    sequential.fit(X, y, eras, num_rounds=3)
    np.testing.assert_allclose(batched.predict(X), sequential.predict(X), rtol=1e-6, atol=1e-6)
    assert _tree_signature(batched) == _tree_signature(sequential)


def test_era_alpha_weighting():
    """tests/test_des.py:220-226"""
    from packboost.booster import PackBoost
    from packboost.config import PackBoostConfig
    booster = PackBoost(PackBoostConfig(era_alpha=2.5))
    counts = torch.tensor([0.0, 3.0, 5.0], dtype=torch.float32, device=booster._device)
    expected = torch.tensor([0.0, 5.5, 7.5], dtype=torch.float32, device=booster._device)
    torch.testing.assert_close(booster._compute_era_weights(counts), expected)


def test_config_defaults():
    """tests/test_config.py:4-9 (device default: see the module docstring)."""
    from packboost.config import PackBoostConfig
    cfg = PackBoostConfig()
    assert cfg.pack_size == 8
    assert cfg.max_depth == 6
    assert cfg.device == "cuda"
    assert cfg.max_bins <= 256
