"""pb_depth_hist_score_static: the histogram + score phase for hosts that cannot allocate.

Some callers of the library run where device allocation is not available to them (all device
memory pre-reserved by another component's pool, or a no-allocation-after-start policy), so they
cannot supply the workspace that pb_depth_hist_score needs.  The static variant keeps its
histogram scratch in a fixed 64 MiB array inside the library.  This test drives it through the C
ABI and requires byte-identical candidate tables to the workspace-based entry point, on two
consecutive calls with different feature subsets (the second call sees the first call's
leftovers in the shared array), checks that an oversized shape is refused, and grows three levels
of a tree on a training state that has no workspace at all (static histogram + score, winner
selection from the caller's candidate buffer, partition) against the workspace-based phases.
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


def test_three_levels_without_any_workspace_match_the_workspace_phases():
    """A host with no workspace: `workspace` NULL, `workspace_bytes` 0.  pb_train_prepare accepts
    the state, pb_depth_hist_score_static writes the candidates to a caller buffer,
    pb_depth_select_cand reads them from there, and pb_depth_partition never needed a workspace.
    Winners, the row -> node map and the leaf ids must equal those of the workspace-based phases,
    also after an earlier, larger call left other contents in the shared array."""
    from packboost_b200 import backends as B
    ref = _trainer()
    alt = _trainer()
    lib = ref.lib
    stream = torch.cuda.current_stream().cuda_stream
    bare = B.TrainState.from_buffer_copy(alt.st)
    bare.workspace = None
    bare.workspace_bytes = 0
    eo = alt.era_offsets.cpu().numpy().astype(np.int32)
    B.check(lib.pb_train_prepare(C.byref(bare), eo.ctypes.data))
    with pytest.raises(ValueError, match="needs pb_train_state.workspace"):
        B.check(lib.pb_depth_hist_score(C.byref(bare), 0, 0, 0, 0, 1, stream))

    rng = np.random.default_rng(9)
    # an earlier, larger call fills the shared array with something else
    B.check(lib.pb_round_begin(C.byref(bare), 0, stream))
    big = torch.arange(80, dtype=torch.int32, device="cuda")
    scratch_out = torch.zeros(24 * 80 * 8, dtype=torch.uint8, device="cuda")
    B.check(lib.pb_depth_hist_score_static(C.byref(bare), 0, big.data_ptr(), big.data_ptr(), 80, 80,
                                           scratch_out.data_ptr(), stream))

    B.check(lib.pb_round_begin(C.byref(ref.st), 0, stream))
    B.check(lib.pb_round_begin(C.byref(bare), 0, stream))
    for depth in range(3):
        k = 40
        subset = rng.permutation(80)[:k].astype(np.int32)
        feats = torch.from_numpy(subset).cuda()
        pos = torch.arange(k, dtype=torch.int32, device="cuda")
        B.check(lib.pb_depth_hist_score(C.byref(ref.st), depth, feats.data_ptr(), pos.data_ptr(), k, k, stream))
        B.check(lib.pb_depth_select(C.byref(ref.st), depth, feats.data_ptr(), k, stream))
        B.check(lib.pb_depth_partition(C.byref(ref.st), depth, stream))
        cand = torch.zeros(24 * k * (1 << depth), dtype=torch.uint8, device="cuda")
        B.check(lib.pb_depth_hist_score_static(C.byref(bare), depth, feats.data_ptr(), pos.data_ptr(), k, k,
                                               cand.data_ptr(), stream))
        B.check(lib.pb_depth_select_cand(C.byref(bare), depth, feats.data_ptr(), k, cand.data_ptr(), stream))
        B.check(lib.pb_depth_partition(C.byref(bare), depth, stream))
    torch.cuda.synchronize()
    assert torch.equal(ref.log_dev, alt.log_dev)
    assert torch.equal(ref.slot, alt.slot) and torch.equal(ref.leaf, alt.leaf)
    head = ref.log_dev.cpu().numpy()[:88].view(np.uint8)
    n_ctx = np.frombuffer(head.tobytes(), dtype=np.int32, offset=24, count=4)
    assert n_ctx[2] >= 2, "the case must reach a frontier of several nodes"
