"""Instrumentation: per-depth phase times in the depth logs, and the debug build whose kernels check
the indices they are handed (it records a violation and skips the index; nothing traps)."""

import os
import subprocess
import sys

import numpy as np
import pytest

import cases

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_depth_logs_carry_device_phase_times_when_metrics_are_requested():
    from packboost_b200 import PackBoost, PackBoostConfig
    X, y, era, cfg, rounds, _ = cases.CASES["prebinned5"]()
    seen = []
    b = PackBoost(PackBoostConfig(device="cuda", **cfg))
    b.fit(X, y, era, num_rounds=2, round_callback=lambda r, m: seen.append(m))
    assert len(seen) == 2 and np.isfinite(seen[-1]["train_corr"])
    logs = b._depth_logs
    assert len(logs) == 2 * cfg["max_depth"]
    for entry in logs:
        assert entry["hist_ms"] > 0.0 and entry["score_ms"] > 0.0 and entry["partition_ms"] > 0.0
        assert entry["hist_ms"] < 1000.0
    # without a per-round consumer the fast path runs (round graph, no events): the fields stay 0
    b2 = PackBoost(PackBoostConfig(device="cuda", **cfg))
    b2.fit(X, y, era, num_rounds=2)
    assert all(e["hist_ms"] == 0.0 for e in b2._depth_logs)
    # same trees either way
    for ta, tb in zip(b.trees, b2.trees):
        assert [(n.feature, n.threshold, n.value) for n in ta.nodes] == [(n.feature, n.threshold, n.value) for n in tb.nodes]


_SCRIPT = r"""
import ctypes as C, sys
import numpy as np, torch
sys.path.insert(0, %(root)r)
from packboost_b200 import backends as B, workloads
from packboost_b200.booster import _DeviceTrainer
from packboost_b200.config import PackBoostConfig
from packboost_b200.data import pack_feature_major
from packboost_b200.sharding import feature_map
lib = B.lib()
assert lib.pb_debug_bounds_enabled() == 1
w = workloads.config3(seed=17, n_rows=6000, n_features=8, n_eras=4, num_rounds=1)
X = w.X.copy()
X[1234, 3] = 9                                   # not a bin of a five-level feature
cfg = dict(w.config); cfg.update(pack_size=1, layer_feature_fraction=1.0, max_depth=2)
config = PackBoostConfig(device="cuda", **cfg)
matrix = pack_feature_major(X, None, config.max_bins)           # (no validation on this path)
counts = np.bincount(w.era.astype(np.int64), minlength=4)
eo = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
tr = _DeviceTrainer(config, matrix, w.y, eo, 8, feature_map(8, 0, 1), 0, 1)
st = C.byref(tr.st)
stream = torch.cuda.current_stream().cuda_stream
B.check(lib.pb_round_begin(st, 0, stream))
feats = torch.arange(8, dtype=torch.int32, device="cuda")
cnt = torch.zeros((8, 4, 1, 5), dtype=torch.int32, device="cuda")
gs = torch.zeros((8, 4, 1, 5), dtype=torch.int64, device="cuda")
B.check(lib.pb_hist_build(st, feats.data_ptr(), 8, 1, 1, cnt.data_ptr(), gs.data_ptr(), stream))
flags = C.c_uint32(0)
B.check(lib.pb_debug_flags(st, C.byref(flags)))
per_feature = cnt.sum(dim=(1, 2, 3)).cpu().tolist()
print("FLAGS", flags.value, "ROWS", per_feature)
"""


def test_debug_build_records_a_bad_bin_code_and_skips_it():
    """The row with the impossible code is left out of that feature's histogram, the violation is
    reported through pb_debug_flags, and the process carries on."""
    env = dict(os.environ, PACKBOOST_DEBUG_LIB="1")
    if not os.path.exists(os.path.join(ROOT, "packboost_b200", "libpackboost_b200_dbg.so")):
        pytest.skip("the debug library is not built")
    res = subprocess.run([sys.executable, "-c", _SCRIPT % {"root": ROOT}], capture_output=True, text=True, env=env, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    line = [l for l in res.stdout.splitlines() if l.startswith("FLAGS")][-1]
    parts = line.split()
    flags = int(parts[1])
    rows = eval(line.split("ROWS", 1)[1])
    assert flags & 2, line
    assert rows[3] == 5999 and all(r == 6000 for i, r in enumerate(rows) if i != 3), line
