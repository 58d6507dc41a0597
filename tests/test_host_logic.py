"""Host-side logic that needs no GPU: log replay, threshold lists, feature sharding (gloo)."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import packboost_oracle as po
from packboost_b200 import sharding
from packboost_b200.booster import _HEADER_DT, _WINNER_DT, _tree_from_log, even_cut_ids


def test_log_dtypes_match_the_c_structs():
    assert _WINNER_DT.itemsize == 80 and _HEADER_DT.itemsize == 88


def test_even_cuts_match_oracle():
    for nb in (4, 5, 16, 63, 128):
        for k in (1, 2, 3, 7, 15, 200):
            np.testing.assert_array_equal(even_cut_ids(nb, k), po.even_cuts(nb, k).numpy())


def _log(rows, n_ctx, root=0.5, n_nodes=None, depth=3):
    head = np.zeros(1, dtype=_HEADER_DT)[0]
    head["root_value"] = root
    for d, c in enumerate(n_ctx):
        head["n_ctx"][d] = c
    win = np.zeros((1 << depth) - 1, dtype=_WINNER_DT)
    for (d, i), r in rows.items():
        w = win[(1 << d) - 1 + i]
        for k, v in r.items():
            w[k] = v
    head["n_tree_nodes"] = n_nodes
    return head, win


def test_tree_replay_numbers_children_like_the_reference():
    # depth 0 splits the root; depth 1: first child splits, second has no usable candidate
    rows = {
        (0, 0): dict(feature=3, threshold=1, tree_node=0, left_id=1, right_id=2, left_value=-0.1, right_value=0.2),
        (1, 0): dict(feature=5, threshold=0, tree_node=1, left_id=3, right_id=4, left_value=-0.3, right_value=0.4),
        (1, 1): dict(feature=-1, threshold=-1, tree_node=2, left_id=-1, right_id=-1, left_value=0.25, right_value=0.25),
    }
    head, win = _log(rows, [1, 2, 0], n_nodes=5)
    tree, n_ctx = _tree_from_log(head, win, 3)
    assert n_ctx[:3] == [1, 2, 0]
    sig = [(n.feature, n.threshold, n.left, n.right, n.is_leaf) for n in tree.nodes]
    assert sig == [(3, 1, 1, 2, False), (5, 0, 3, 4, False), (-1, 0, -1, -1, True), (-1, 0, -1, -1, True),
                   (-1, 0, -1, -1, True)]
    assert [n.value for n in tree.nodes][2:] == [0.25, -0.3, 0.4]


def test_tree_replay_detects_numbering_mismatch():
    rows = {(0, 0): dict(feature=3, threshold=1, tree_node=0, left_id=2, right_id=3, left_value=0.0, right_value=0.0)}
    head, win = _log(rows, [1, 0, 0], n_nodes=3)
    with pytest.raises(RuntimeError):
        _tree_from_log(head, win, 3)


def test_root_only_tree():
    head, win = _log({}, [0, 0, 0], root=-1.5, n_nodes=1)
    tree, n_ctx = _tree_from_log(head, win, 3)
    assert len(tree.nodes) == 1 and tree.nodes[0].is_leaf and tree.nodes[0].value == -1.5


def test_feature_map_and_local_part_partition_the_features():
    F, world = 37, 4
    seen = np.zeros(F, dtype=int)
    for r in range(world):
        m = sharding.feature_map(F, r, world)
        own = np.nonzero(m >= 0)[0]
        c0, c1 = sharding.owned_range(F, r, world)
        assert np.array_equal(own, np.arange(c0, c1))          # one contiguous strip of columns
        assert np.array_equal(m[own], own - c0)
        assert c1 - c0 <= sharding.block_size(F, world)
        seen[own] += 1
    assert np.all(seen == 1)
    subset = np.random.default_rng(0).permutation(F)[:11].astype(np.int32)
    pos_all = []
    for r in range(world):
        rows, pos = sharding.local_part(subset, r, world, F)
        c0, c1 = sharding.owned_range(F, r, world)
        assert np.array_equal(rows, subset[pos] - c0) and np.all((subset[pos] >= c0) & (subset[pos] < c1))
        pos_all.append(pos)
    assert np.array_equal(np.sort(np.concatenate(pos_all)), np.arange(11))
    # more ranks than features: the surplus ranks hold nothing
    assert [sharding.owned_range(3, r, 8) for r in range(8)] == [(0, 1), (1, 2), (2, 3)] + [(3, 3)] * 5


def test_edges_from_sorted_columns_equal_numpy_quantile():
    """The interpolation that follows the device sort of the binning step against
    ``np.quantile(method="linear")``: ties, a binary column, a column with NaNs, tiny inputs."""
    import torch
    from packboost_b200.data import edges_from_sorted
    rng = np.random.default_rng(0)
    for n, f, nb in [(1000, 7, 128), (1537, 5, 64), (20000, 9, 128), (17, 4, 5), (2, 2, 16), (1, 2, 4), (5000, 6, 255)]:
        X = rng.normal(size=(n, f)).astype(np.float32)
        if f > 2:
            X[:, 1] = np.round(X[:, 1])
            X[:, 2] = X[:, 2] > 0
        if f > 3:
            X[::7, 3] = np.nan
        with np.errstate(all="ignore"):
            want = np.quantile(X, np.linspace(0.0, 1.0, nb + 1, dtype=np.float64)[1:-1], axis=0, method="linear")
        got = edges_from_sorted(torch.sort(torch.from_numpy(X), dim=0).values, nb)
        assert got.dtype == np.float64 and got.shape == want.shape
        assert np.array_equal(got, want, equal_nan=True)


def test_dealt_part_gives_equal_disjoint_shares():
    """Replicated-codes layout: the sampled list is dealt by position; shares are disjoint, cover
    the list, differ by at most one feature and do not depend on which features were drawn."""
    F, k = 2376, 238
    for world in (2, 4, 8):
        sizes = None
        for seed in range(3):
            subset = np.random.default_rng(seed).permutation(F)[:k].astype(np.int32)
            parts = [sharding.dealt_part(subset, r, world) for r in range(world)]
            pos = np.concatenate([p for _, p in parts])
            assert np.array_equal(np.sort(pos), np.arange(k))
            for rows, p in parts:
                assert rows.dtype == np.int32 and p.dtype == np.int32
                assert np.array_equal(rows, subset[p])
            now = [len(p) for _, p in parts]
            assert max(now) - min(now) <= 1
            assert sizes is None or sizes == now   # the same in every round: a fixed launch shape
            sizes = now


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(5)                       # same seed on every rank
    F, nodes, n_rows = 23, 4, 1000
    subset = rng.permutation(F)[:9].astype(np.int32)
    full = rng.integers(1, 1 << 30, size=(subset.shape[0], nodes, 6)).astype(np.int32)   # 24-byte records
    # each rank fills the records of the features it holds; the others stay zero
    table = np.zeros_like(full)
    _, pos = sharding.local_part(subset, rank, world, F)
    table[pos] = full[pos]
    t = torch.from_numpy(table)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    ok1 = np.array_equal(t.numpy(), full)
    # go-left bits: the owner of each node's winning feature sets the bits of that node's rows
    node_of = rng.integers(0, nodes, size=n_rows)
    win_feat = subset[rng.integers(0, subset.shape[0], size=nodes)]
    go_left = rng.integers(0, 2, size=n_rows).astype(bool)
    c0, c1 = sharding.owned_range(F, rank, world)
    mine = (win_feat[node_of] >= c0) & (win_feat[node_of] < c1) & go_left
    bits = np.packbits(mine, bitorder="little")
    bits = np.pad(bits, (0, (-len(bits)) % 4)).view(np.int32).copy()
    tb = torch.from_numpy(bits)
    dist.all_reduce(tb, op=dist.ReduceOp.SUM)
    want = np.packbits(go_left, bitorder="little")
    want = np.pad(want, (0, (-len(want)) % 4)).view(np.int32)
    ok2 = np.array_equal(tb.numpy(), want)
    out[rank] = int(ok1 and ok2)
    dist.destroy_process_group()


def test_two_rank_exchange_merges_disjoint_tables_and_bitmasks():
    """The per-depth exchange of the feature-sharded path on CPU ranks (gloo, world size 2):
    a SUM all-reduce over int32 words merges disjoint candidate records exactly, and a SUM of
    disjoint go-left bit words equals their OR."""
    world = 2
    out = mp.get_context("spawn").Manager().dict()   # (no fork of this multi-threaded process)
    mp.spawn(_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    assert [out[r] for r in range(world)] == [1, 1]


def _layout_worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    packed = 3 << 30
    # rank 1's GPU is nearly full: alone it would shard, rank 0 alone would replicate
    free = (100 << 30) if rank == 0 else (4 << 30)
    mixed = sharding.choose_replicated(packed, free, world, False, device="cpu")
    roomy = sharding.choose_replicated(packed, 100 << 30, world, False, device="cpu")
    forced = sharding.choose_replicated(packed, 100 << 30, world, rank == 1, device="cpu")
    out[rank] = (mixed, roomy, forced)
    dist.destroy_process_group()


def test_ranks_with_different_free_memory_agree_on_one_layout():
    """The replicated / sharded choice is collective: one rank short of memory (or one rank with
    the sharding override set) moves every rank to the sharded layout."""
    world = 2
    out = mp.get_context("spawn").Manager().dict()
    mp.spawn(_layout_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    assert out[0] == out[1] == (False, True, False)
    assert sharding.choose_replicated(1, 1 << 40, 1, False) is False   # one GPU: nothing to replicate


# ---- the round loop of the booster against a scripted device ----------------------------------

class _ScriptedTrainer:
    """Stands in for the device: round r (counted by accepted enqueues) has live nodes at the first
    ``used[r]`` depths, every live node splits, and the log is delivered when asked for."""

    def __init__(self, depth, k, used):
        self.D, self.k, self.used = depth, k, used
        self.attempts = []          # (round index, subsets, redo)
        self.round_of_ticket = {}
        self.next_round = 0

    def n_sampled(self):
        return self.k

    def run_round(self, subsets, redo=False):
        if redo:
            self.next_round -= 1
        ticket = len(self.attempts)
        self.attempts.append((self.next_round, [s.copy() for s in subsets], redo))
        self.round_of_ticket[ticket] = self.next_round
        self.next_round += 1
        return ticket

    def read_log(self, ticket):
        used = self.used[self.round_of_ticket[ticket]]
        n_ctx = [(1 << d) if d < used else 0 for d in range(self.D + 1)]
        rows = {}
        nid = 0
        for d in range(used):
            for i in range(1 << d):
                node = (1 << d) - 1 + i
                rows[(d, i)] = dict(feature=d, threshold=1, tree_node=node, left_id=2 * node + 1, right_id=2 * node + 2,
                                    left_value=0.25, right_value=-0.25)
                nid = max(nid, 2 * node + 2)
        return _log(rows, n_ctx, n_nodes=nid + 1, depth=self.D)

    def flush_predictions(self):
        pass

    def release_graph(self):
        pass


def _scripted_booster(monkeypatch, trainer, seed, n_features):
    from packboost_b200 import booster as bm
    from packboost_b200.config import PackBoostConfig
    monkeypatch.setattr(bm.B, "cuda_available", lambda: True)
    monkeypatch.setattr(torch.cuda, "current_device", lambda: 0)
    b = bm.PackBoost(PackBoostConfig(device="cuda", max_depth=trainer.D, pack_size=2, random_state=seed,
                                     layer_feature_fraction=trainer.k / n_features))
    b._trainer = trainer
    b._fit_ctx = {"F": n_features, "era_sorted": None, "y_sorted": None}
    return b


@pytest.mark.parametrize("run_ahead", ["1", "0"])
def test_round_loop_draws_features_like_the_reference_when_rounds_end_early(run_ahead, monkeypatch):
    """The reference draws one feature subset per depth and only while nodes are live.  The round
    loop draws all depths up front (and, running ahead, the next round too), so after a round that
    ends early it must rewind the generator and enqueue the following round again: the subsets of
    the rounds that count must be exactly the reference's draws, in both loop modes."""
    monkeypatch.setenv("PACKBOOST_RUN_AHEAD", run_ahead)
    D, F, k, seed = 3, 40, 9, 123
    used = [3, 1, 3, 2, 0, 3, 3, 1]            # live depths per round; 0: even the root has no split
    trainer = _ScriptedTrainer(D, k, used)
    b = _scripted_booster(monkeypatch, trainer, seed, F)
    for r in range(len(used)):
        b._boost_one_round(r, len(used))
    b._drain()                                 # (what _finish does, without the device synchronisation)
    b._flush_pending_tree()
    # reference order of draws
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    want = []
    for r, u in enumerate(used):
        want.append([torch.randperm(F, generator=g)[:k].numpy().astype(np.int32) for _ in range(u)])
    accepted = {}
    for rnd, subsets, _redo in trainer.attempts:
        accepted[rnd] = subsets                   # the last attempt of a round is the one that counts
    assert sorted(accepted) == list(range(len(used)))
    for r, u in enumerate(used):
        for d in range(u):
            np.testing.assert_array_equal(accepted[r][d], want[r][d], err_msg=f"round {r} depth {d}")
    # one tree per round, recorded pack_size times, with the scripted shape
    assert len(b.trees) == 2 * len(used)
    sizes = [len(t.nodes) for t in b.trees[::2]]
    assert sizes == [(1 << (u + 1)) - 1 for u in used]
    if run_ahead == "1":
        assert any(redo for _, _, redo in trainer.attempts)
    else:
        assert not any(redo for _, _, redo in trainer.attempts)


def test_row_split_upload_reassembles_the_single_gpu_layout():
    """Every rank packs 1/world of the rows of all features into a slab ``[F_pad][seg]``; an
    all-gather (replicated layout) or an all-to-all (sharded layout) followed by one strided copy
    must give exactly the feature-major matrix one GPU would have packed.  The exchange is emulated
    on CPU tensors: this pins the index algebra of ``pack_feature_major_distributed``."""
    from packboost_b200.data import rows_per_rank
    from packboost_b200.sharding import block_size
    for world, F, n_rows, bits in [(2, 7, 1000, 4), (3, 10, 5000, 8), (4, 96, 20_000, 4), (8, 2376, 9_000, 4)]:
        per = rows_per_rank(n_rows, world)
        assert per % 256 == 0 and per * world >= n_rows and per * (world - 1) < n_rows + 256 * world
        seg = per * bits // 8
        assert seg % 128 == 0
        blk = block_size(F, world)
        f_pad = blk * world
        full = torch.randint(0, 256, (f_pad, world * seg), dtype=torch.uint8,
                             generator=torch.Generator().manual_seed(world))
        slabs = [full[:, r * seg:(r + 1) * seg].contiguous() for r in range(world)]   # what each rank packs
        # replicated layout: all_gather_into_tensor(parts, slab) on every rank
        parts = torch.stack(slabs)                                                    # [world, f_pad, seg]
        rebuilt = torch.empty_like(full)
        rebuilt.view(f_pad, world, seg).copy_(parts.permute(1, 0, 2))
        assert torch.equal(rebuilt, full)
        # sharded layout: all_to_all_single(parts, slab.view(world, blk, seg)) -> rank dst receives
        # from every source the feature block it owns
        for dst in range(world):
            recv = torch.stack([slabs[src].view(world, blk, seg)[dst] for src in range(world)])   # [world, blk, seg]
            mine = torch.empty((blk, world * seg), dtype=torch.uint8)
            mine.view(blk, world, seg).copy_(recv.permute(1, 0, 2))
            assert torch.equal(mine, full[dst * blk:(dst + 1) * blk])
