"""Host-side behaviour of the wrapper layer (no GPU): parameters and serialisation."""

import numpy as np
import pytest

from packboost_b200.wrapper import PackBoostPredictor, PackBoostRegressor


def test_regressor_params_roundtrip():
    m = PackBoostRegressor(num_rounds=7, pack_size=4, max_depth=3, learning_rate=0.2)
    p = m.get_params()
    assert p["num_rounds"] == 7 and p["pack_size"] == 4 and p["max_depth"] == 3
    m.set_params(max_depth=5, num_rounds=9)
    assert m.get_params()["max_depth"] == 5 and m.num_rounds == 9
    with pytest.raises(TypeError):
        PackBoostRegressor(not_a_param=1)
    with pytest.raises(RuntimeError):
        m.predict(np.zeros((2, 2), np.float32))


def test_predictor_npz_roundtrip(tmp_path):
    rng = np.random.default_rng(0)
    trees = []
    for n in (1, 3, 7):  # complete trees in heap order: node i has children 2i+1 and 2i+2
        inner = np.arange(n) < n // 2
        idx = np.arange(n)
        trees.append({"feature": np.where(inner, rng.integers(0, 5, n), -1).astype(np.int32),
                      "threshold": np.where(inner, rng.integers(0, 4, n), 0).astype(np.int32),
                      "left": np.where(inner, 2 * idx + 1, -1).astype(np.int32),
                      "right": np.where(inner, 2 * idx + 2, -1).astype(np.int32),
                      "value": rng.normal(size=n).astype(np.float32), "is_leaf": (~inner).astype(np.uint8)})
    edges = rng.normal(size=(4, 6)).astype(np.float32)
    p = PackBoostPredictor(trees, [2, 1, 5], 0.05, edges, 5, 8)
    path = str(tmp_path / "model.npz")
    p.save(path)
    q = PackBoostPredictor.load(path)
    assert q.repeats == [2, 1, 5] and q.tree_weight == 0.05 and q.max_bins == 5 and q.pack_size == 8
    np.testing.assert_array_equal(q.bin_edges, edges)
    for a, b in zip(p.trees, q.trees):
        for k in a:
            np.testing.assert_array_equal(a[k], b[k])
    p2 = PackBoostPredictor(trees, [1, 1, 1], 1.0, None, 5, 1)
    p2.save(path)
    assert PackBoostPredictor.load(path).bin_edges is None
