"""Host-side refusals that keep malformed input away from the GPU (no device needed)."""

import ctypes as C

import numpy as np
import pytest

from packboost_b200.forest import validate_forest


def _tree(left, right, is_leaf, feature=None, threshold=None):
    n = len(left)
    feature = feature if feature is not None else [0 if not l else -1 for l in is_leaf]
    threshold = threshold if threshold is not None else [1] * n
    return (np.asarray(feature, np.int32), np.asarray(threshold, np.int32), np.asarray(left, np.int32),
            np.asarray(right, np.int32), np.asarray(is_leaf, np.uint8))


def test_well_formed_trees_pass_and_report_the_largest_tree():
    f, t, l, r, il = _tree([1, -1, 3, -1, -1], [2, -1, 4, -1, -1], [0, 1, 0, 1, 1])
    assert validate_forest(f, t, l, r, il, [0, 5]) == 5
    # two trees back to back, the second a single leaf
    f2 = np.concatenate([f, [-1]]).astype(np.int32)
    assert validate_forest(f2, np.append(t, 0), np.append(l, -1), np.append(r, -1), np.append(il, 1), [0, 5, 6]) == 5
    # children need not be adjacent, only later than their parent
    f, t, l, r, il = _tree([2, -1, 4, -1, -1], [1, -1, 3, -1, -1], [0, 1, 0, 1, 1])
    assert validate_forest(f, t, l, r, il, [0, 5]) == 5


@pytest.mark.parametrize("left,right,why", [
    ([0, -1, -1], [2, -1, -1], "a node that is its own child (cycle)"),
    ([1, 0, -1], [2, 2, -1], "a child that points back to the root (cycle)"),
    ([1, -1, -1], [7, -1, -1], "a child outside the tree"),
    ([1, -1, -1], [-3, -1, -1], "a negative child of an internal node"),
])
def test_cyclic_and_out_of_range_children_are_refused(left, right, why):
    is_leaf = [0, 1 if left[1] < 0 else 0, 1]
    f, t, l, r, il = _tree(left, right, is_leaf)
    with pytest.raises(ValueError, match="children"):
        validate_forest(f, t, l, r, il, [0, 3])


def test_children_must_stay_inside_their_own_tree():
    # tree 0 = nodes 0..2, tree 1 = nodes 3..5; node 0 points at relative index 4 (a node of tree 1)
    f, t, l, r, il = _tree([1, -1, -1, 1, -1, -1], [4, -1, -1, 2, -1, -1], [0, 1, 1, 0, 1, 1])
    with pytest.raises(ValueError, match="children"):
        validate_forest(f, t, l, r, il, [0, 3, 6])
    # the same ensemble with absolute child ids is fine when they stay in range ...
    f, t, l, r, il = _tree([1, -1, -1, 4, -1, -1], [2, -1, -1, 5, -1, -1], [0, 1, 1, 0, 1, 1])
    assert validate_forest(f, t, l, r, il, [0, 3, 6], absolute_children=True) == 3
    # ... and refused when a child crosses into the other tree
    f, t, l, r, il = _tree([1, -1, -1, 4, -1, -1], [3, -1, -1, 5, -1, -1], [0, 1, 1, 0, 1, 1])
    with pytest.raises(ValueError, match="children"):
        validate_forest(f, t, l, r, il, [0, 3, 6], absolute_children=True)


def test_feature_threshold_and_offset_ranges():
    f, t, l, r, il = _tree([1, -1, -1], [2, -1, -1], [0, 1, 1], feature=[9, -1, -1])
    assert validate_forest(f, t, l, r, il, [0, 3], n_features=10) == 3
    with pytest.raises(ValueError, match="feature"):
        validate_forest(f, t, l, r, il, [0, 3], n_features=9)
    f, t, l, r, il = _tree([1, -1, -1], [2, -1, -1], [0, 1, 1], feature=[-1, -1, -1])
    with pytest.raises(ValueError, match="feature"):
        validate_forest(f, t, l, r, il, [0, 3])
    f, t, l, r, il = _tree([1, -1, -1], [2, -1, -1], [0, 1, 1], threshold=[300, 0, 0])
    with pytest.raises(ValueError, match="threshold"):
        validate_forest(f, t, l, r, il, [0, 3])
    f, t, l, r, il = _tree([1, -1, -1], [2, -1, -1], [0, 1, 1])
    for offs in ([1, 3], [0, 2], [0, 3, 2, 3], [0, 0, 3]):
        with pytest.raises(ValueError):
            validate_forest(f, t, l, r, il, offs)


def test_predictor_refuses_a_malformed_file_before_touching_the_device(tmp_path):
    from packboost_b200.wrapper import PackBoostPredictor
    path = str(tmp_path / "bad.npz")
    np.savez(path, tree_offsets=np.array([0, 3]), repeats=np.array([1], np.int32), tree_weight=np.float64(1.0),
             max_bins=np.int64(5), pack_size=np.int64(1), has_edges=np.bool_(False),
             bin_edges=np.zeros((0, 0), np.float32), feature=np.array([0, -1, -1], np.int32),
             threshold=np.array([1, 0, 0], np.int32), left=np.array([0, -1, -1], np.int32),
             right=np.array([2, -1, -1], np.int32), value=np.zeros(3), is_leaf=np.array([0, 1, 1], np.uint8))
    with pytest.raises(ValueError, match="children"):
        PackBoostPredictor.load(path)


# ---- training state: alignment and the no-workspace mode, through the C ABI ------------------------

@pytest.fixture(scope="module")
def lib():
    from packboost_b200 import build
    build.build()
    from packboost_b200 import backends as B
    return B.lib()


def _state(B, base=1 << 20):
    """A shape-valid training state over made-up addresses (never dereferenced: pb_train_prepare
    does no device work)."""
    st = B.TrainState()
    st.n_rows, st.n_features_total, st.n_features_local, st.n_eras = 1000, 4, 4, 2
    st.max_bins, st.code_bits, st.pitch = 5, 4, 512
    st.max_depth, st.pack_size, st.min_samples_leaf, st.n_thresholds, st.feature_block_size = 3, 2, 5, 4, 32
    st.lambda_l2, st.learning_rate = 1e-3, 0.1
    for i, name in enumerate(("codes", "era_offsets", "thr_ids", "feat_local", "y", "preds", "gq", "slot", "leaf", "ctl")):
        setattr(st, name, base * (i + 1))
    st.workspace = base * 20
    st.workspace_bytes = 1 << 30
    return st


def test_codes_must_be_32_byte_aligned(lib):
    from packboost_b200 import backends as B
    eo = np.array([0, 600, 1000], np.int32)
    st = _state(B)
    B.check(lib.pb_train_prepare(C.byref(st), eo.ctypes.data))
    st.codes = (1 << 20) + 16          # 16-byte aligned only: the 256-bit code loads would fault
    with pytest.raises(ValueError, match="32-byte"):
        B.check(lib.pb_train_prepare(C.byref(st), eo.ctypes.data))


def test_a_state_without_workspace_is_accepted_and_workspace_entries_say_so(lib):
    from packboost_b200 import backends as B
    eo = np.array([0, 600, 1000], np.int32)
    st = _state(B)
    st.workspace = None
    st.workspace_bytes = 0
    B.check(lib.pb_train_prepare(C.byref(st), eo.ctypes.data))
    with pytest.raises(ValueError, match="needs pb_train_state.workspace"):
        B.check(lib.pb_depth_hist_score(C.byref(st), 0, None, None, 0, 1, None))
    with pytest.raises(ValueError, match="needs pb_train_state.workspace"):
        B.check(lib.pb_depth_select(C.byref(st), 0, None, 1, None))
    ptr, nbytes = C.c_void_p(), C.c_int64()
    with pytest.raises(ValueError, match="needs pb_train_state.workspace"):
        B.check(lib.pb_candidates_buffer(C.byref(st), 0, 1, C.byref(ptr), C.byref(nbytes)))
    st.workspace_bytes = 64            # a size without a pointer is a caller error
    with pytest.raises(ValueError, match="workspace is null"):
        B.check(lib.pb_train_prepare(C.byref(st), eo.ctypes.data))
    st = _state(B)
    st.workspace_bytes = 16            # a pointer with too few bytes still is, too
    with pytest.raises(ValueError, match="workspace too small"):
        B.check(lib.pb_train_prepare(C.byref(st), eo.ctypes.data))


def test_comm_entries_validate_their_arguments_without_a_gpu(lib):
    """The NCCL-backed exchange entries refuse bad arguments before touching NCCL or a device."""
    from packboost_b200 import backends as B
    comm = C.c_void_p()
    ident = (C.c_ubyte * 128)()
    for n_ranks, rank in ((0, 0), (2, 2), (2, -1)):
        with pytest.raises(ValueError, match="out of range"):
            B.check(lib.pb_comm_init(C.byref(comm), ident, n_ranks, rank))
    with pytest.raises(ValueError, match="null"):
        B.check(lib.pb_comm_init(None, ident, 2, 0))
    with pytest.raises(ValueError, match="null"):
        B.check(lib.pb_comm_unique_id(None))
    with pytest.raises(ValueError, match="communicator is null"):
        B.check(lib.pb_comm_allreduce_mask(None, 1 << 20, 16, None))
    st = _state(B)
    with pytest.raises(ValueError, match="communicator is null"):
        B.check(lib.pb_comm_allreduce_candidates(None, C.byref(st), 0, 4, None))
    assert lib.pb_comm_destroy(None) == 0
