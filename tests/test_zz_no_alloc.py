"""pb_depth_hist_score_static: the histogram + score phase for hosts that cannot allocate.

Some callers of the library run where device allocation is not available to them (all device
memory pre-reserved by another component's pool, or a no-allocation-after-start policy), so they
cannot supply the workspace that pb_depth_hist_score needs.  The static variant keeps its
histogram scratch in a fixed 64 MiB array inside the library.  This test drives it through the C
ABI and requires byte-identical candidate tables to the workspace-based entry point, on two
consecutive calls with different feature subsets (the second call sees the first call's
leftovers in the shared array), and checks that an oversized shape is refused.
"""

import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _trainer():
    from packboost_b200 import workloads
    from packboost_b200.booster import _DeviceTrainer
    from packboost_b200.config import PackBoostConfig
    from packboost_b200.data import pack_feature_major
    from packboost_b200.sharding import feature_map
    w = workloads.config3(seed=17, n_rows=30_000, n_features=80, n_eras=12, num_rounds=1)
    cfg = dict(w.config)
    cfg.update(pack_size=2, layer_feature_fraction=0.5, max_depth=4)
    config = PackBoostConfig(device="cuda", **cfg)
    matrix = pack_feature_major(w.X, None, config.max_bins)
    counts = np.bincount(w.era.astype(np.int64), minlength=12)
    era_offsets = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    return _DeviceTrainer(config, matrix, w.y, era_offsets, 80, feature_map(80, 0, 1), 0, 1)


def _candidates_workspace(tr, depth, rows, pos, k):
    from packboost_b200 import backends as B
    st = C.byref(tr.st)
    stream = torch.cuda.current_stream().cuda_stream
    B.check(tr.lib.pb_depth_clear_candidates(st, depth, k, stream))
    B.check(tr.lib.pb_depth_hist_score(st, depth, rows.data_ptr(), pos.data_ptr(), rows.numel(), k, stream))
    ptr, nbytes = C.c_void_p(), C.c_int64()
    B.check(tr.lib.pb_candidates_buffer(st, depth, k, C.byref(ptr), C.byref(nbytes)))
    off = ptr.value - tr.workspace.data_ptr()
    torch.cuda.synchronize()
    return tr.workspace[off: off + nbytes.value].clone()


def test_static_scratch_variant_matches_workspace_variant_twice():
    from packboost_b200 import backends as B
    tr = _trainer()
    lib, st = tr.lib, C.byref(tr.st)
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.pb_static_scratch_bytes() == 64 << 20
    B.check(lib.pb_round_begin(st, 0, stream))
    rng = np.random.default_rng(4)
    depth = 0
    for call, k in enumerate((40, 23)):
        subset = rng.permutation(80)[:k].astype(np.int32)
        rows = torch.from_numpy(subset).cuda()
        pos = torch.arange(k, dtype=torch.int32, device="cuda")
        want = _candidates_workspace(tr, depth, rows, pos, k)
        got = torch.zeros_like(want)            # output buffer owned by the caller
        B.check(lib.pb_depth_hist_score_static(st, depth, rows.data_ptr(), pos.data_ptr(), k, k, got.data_ptr(), stream))
        torch.cuda.synchronize()
        assert want.numel() == 24 * k
        assert torch.equal(got, want), f"call {call}"
        rec = got.cpu().numpy().view(np.int32).reshape(k, 6)
        assert (rec[:, 1] >= 0).all()           # every feature produced a threshold index


def test_static_scratch_variant_refuses_oversized_shapes():
    from packboost_b200 import backends as B
    tr = _trainer()
    lib = tr.lib
    st = B.TrainState.from_buffer_copy(tr.st)
    st.n_eras = 20_000                           # 8 nodes * 20 000 eras * 5 bins * 12 B = 9.6 MB at depth 3 ...
    st.max_bins = 16                             # ... * 16/5 and 8-bit era counts push one feature past 64 MiB
    st.n_thresholds = 15
    st.max_depth = 12
    out = torch.zeros(24 * 4096, dtype=torch.uint8, device="cuda")
    rows = torch.zeros(1, dtype=torch.int32, device="cuda")
    with pytest.raises(ValueError, match="static scratch too small"):
        B.check(lib.pb_depth_hist_score_static(C.byref(st), 11, rows.data_ptr(), rows.data_ptr(), 1, 1,
                                               out.data_ptr(), torch.cuda.current_stream().cuda_stream))
