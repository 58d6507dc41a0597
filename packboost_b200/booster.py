"""PackBoost host orchestration for the B200 backend.

The public surface follows the reference booster (``packboost/booster.py``):
``PackBoost(config).fit(X, y, era, num_rounds=..., feature_names=...,
eval_sets=..., round_callback=...)``, ``predict``, ``predict_packwise``,
``trees`` and ``round_metrics``, with ``Tree`` / ``TreeNode`` / ``TreeBuilder``
as the model containers.  What changed is everything below the round loop:

* the feature matrix lives on the device as feature-major packed bin codes with
  rows ordered by era;
* frontier bookkeeping is a per-row ``slot`` / ``leaf`` map on the device, not
  Python lists of row-index tensors;
* histograms, DES scores, winner selection, child numbering, leaf values,
  partition and the prediction update are CUDA kernels reached through the C
  ABI (``include/packboost_b200.h``); the host only draws the per-depth feature
  subset, launches the phases and reads one small decision log per round.

All ``pack_size`` trees of a round are identical in the reference (it has no
per-tree randomness and de-duplicates identical frontier nodes,
``packboost/booster.py:1670-1682``); this implementation grows the tree once and
records it ``pack_size`` times, keeping the summed (not averaged) pack update of
``packboost/booster.py:582-597``.

With ``torch.distributed`` initialised (one process per GPU) the features are
sharded ``feature % world_size == rank``; each depth exchanges the candidate
table and a go-left bitmask with two all-reduces.
"""

from __future__ import annotations

import ctypes as C
import logging
import json
import math
import os
import sys
from dataclasses import dataclass, field
from time import perf_counter
from typing import Callable, Iterable, List, Sequence, Tuple

import numpy as np
import torch

from . import backends as B
from .config import PackBoostConfig
from .forest import validate_forest
from .sharding import agree_all, block_size, choose_replicated, dealt_part, feature_map, local_part, owned_range
from .data import (BinningResult, PackedMatrix, PackedRows, code_bits_for, detect_prebinned, pack_feature_major,
                   pack_feature_major_distributed, pack_row_major, quantile_edges_device)

# ------------------------------ tree containers ------------------------------


@dataclass(slots=True)
class TreeNode:
    feature: int = -1
    threshold: int = 0
    left: int = -1
    right: int = -1
    value: float = 0.0
    is_leaf: bool = True


@dataclass(slots=True)
class Tree:
    nodes: List[TreeNode]
    _arrays: dict | None = field(init=False, repr=False, default=None)

    def arrays(self) -> dict[str, np.ndarray]:
        if self._arrays is None:
            self._arrays = {
                "feature": np.asarray([n.feature for n in self.nodes], dtype=np.int32),
                "threshold": np.asarray([n.threshold for n in self.nodes], dtype=np.int32),
                "left": np.asarray([n.left for n in self.nodes], dtype=np.int32),
                "right": np.asarray([n.right for n in self.nodes], dtype=np.int32),
                "value": np.asarray([n.value for n in self.nodes], dtype=np.float32),
                "is_leaf": np.asarray([n.is_leaf for n in self.nodes], dtype=np.uint8),
            }
        return self._arrays

    def predict_bins(self, bins: torch.Tensor) -> torch.Tensor:
        """Leaf value per row for integer-binned features ``[N, F]``
        (``packboost/booster.py:66-128``).  Always routed on the GPU; the result is
        returned on the input's device."""
        n = bins.shape[0]
        if n == 0:
            return torch.empty(0, dtype=torch.float32, device=bins.device)
        dev = torch.device("cuda", torch.cuda.current_device())
        a = self.arrays()
        fm = bins.to(device=dev, dtype=torch.uint8).t().contiguous()
        t = {k: torch.from_numpy(v).to(dev) for k, v in a.items()}
        out = B.predict_bins_cuda(fm, t["feature"], t["threshold"], t["left"], t["right"], t["value"], t["is_leaf"])
        return out.to(bins.device)


class TreeBuilder:
    """BFS-compact node numbering (``packboost/booster.py:172-190``)."""

    def __init__(self) -> None:
        self.nodes: List[TreeNode] = [TreeNode()]

    def set_leaf(self, node_id: int, value: float) -> None:
        n = self.nodes[node_id]
        n.value = float(value)
        n.is_leaf = True
        n.feature = -1
        n.threshold = 0
        n.left = -1
        n.right = -1

    def split(self, node_id: int, feature: int, threshold: int) -> Tuple[int, int]:
        n = self.nodes[node_id]
        n.feature = int(feature)
        n.threshold = int(threshold)
        n.is_leaf = False
        l = len(self.nodes)
        n.left = l
        n.right = l + 1
        self.nodes.append(TreeNode())
        self.nodes.append(TreeNode())
        return l, l + 1

    def build(self) -> Tree:
        return Tree(nodes=self.nodes)


@dataclass(slots=True)
class NodeShard:
    """A frontier node as the reference passes it to its single-node helpers: per-era row-id tensors
    (``packboost/booster.py:197-203``).  The training loop here keeps a row -> node map instead."""

    tree_id: int
    node_id: int
    depth: int
    era_rows: list


@dataclass(slots=True)
class SplitDecision:
    """``packboost/booster.py:205-217`` (the row lists are filled by ``_find_best_split`` only)."""

    feature: int
    threshold: int
    score: float
    left_grad: float
    left_hess: float
    right_grad: float
    right_hess: float
    left_count: int
    right_count: int
    left_rows: list = field(default_factory=list)
    right_rows: list = field(default_factory=list)


# ------------------------------ decision log ------------------------------

_WINNER_DT = np.dtype({
    "names": ["feature", "threshold", "score", "tree_node", "left_count", "total_count", "left_gq", "total_gq",
              "left_id", "right_id", "left_value", "right_value", "left_grad", "total_grad"],
    "formats": ["<i4", "<i4", "<f4", "<i4", "<i8", "<i8", "<i8", "<i8", "<i4", "<i4", "<f8", "<f8", "<f4", "<f4"],
    "offsets": [0, 4, 8, 12, 16, 24, 32, 40, 48, 52, 56, 64, 72, 76],
    "itemsize": 80,
})
_HEADER_DT = np.dtype({
    "names": ["root_value", "scale", "max_abs_grad", "root_gq", "n_ctx", "n_tree_nodes"],
    "formats": ["<f8", "<f4", "<f4", "<i8", ("<i4", (B.PB_MAX_DEPTH + 1,)), "<i4"],
    "offsets": [0, 8, 12, 16, 24, 24 + 4 * (B.PB_MAX_DEPTH + 1)],
    "itemsize": 88,
})


def even_cut_ids(num_bins: int, k: int) -> np.ndarray:
    """Evenly spaced threshold ids (``packboost/booster.py:1006-1010``)."""
    k = max(1, min(k, max(1, num_bins - 1)))
    idx = torch.round(torch.linspace(0, num_bins - 2, k)).to(torch.int64)
    return torch.unique(idx, sorted=True).clamp_(0, num_bins - 2).numpy().astype(np.int32)


def _era_correlation_np(era_ids: np.ndarray, target: np.ndarray, preds: np.ndarray) -> float:
    """Mean per-era Pearson correlation (``packboost/booster.py:909-929``)."""
    if era_ids.shape[0] == 0:
        return float("nan")
    cors: list[float] = []
    for era in np.unique(era_ids):
        m = era_ids == era
        y = target[m]
        p = preds[m]
        if y.size < 2:
            continue
        sy = y.std(ddof=0)
        sp = p.std(ddof=0)
        if sy <= 1e-12 or sp <= 1e-12:
            continue
        corr = float(((y - y.mean()) * (p - p.mean())).mean()) / (sy * sp)
        if math.isfinite(corr):
            cors.append(corr)
    return float(np.mean(cors)) if cors else float("nan")


# ------------------------------ device training state ------------------------------


_RING = 4  # staging slots: at most three rounds are in flight (previous, a discarded one, its redo)


class _DeviceTrainer:
    """Owns the device buffers of one fit and launches the round phases."""

    def __init__(self, cfg: PackBoostConfig, matrix: PackedMatrix, y_sorted: np.ndarray, era_offsets: np.ndarray,
                 n_features_total: int, feat_local: np.ndarray, rank: int, world: int,
                 workspace_bytes: int | None = None, replicated: bool = False):
        self.cfg = cfg
        self.lib = B.lib()
        self.dev = matrix.codes.device
        self.rank, self.world = rank, world
        self.replicated = bool(replicated)  # every rank holds all feature rows (see PackBoost._start)
        self.matrix = matrix
        n = matrix.n_rows
        npad = matrix.rows_padded
        self.n_rows = n
        self.F = n_features_total
        self.E = int(era_offsets.shape[0] - 1)
        nb = int(cfg.max_bins)
        k_user = int(cfg.k_cuts)
        self.cut_mass = False
        if 0 < k_user < nb - 1:
            # "mass": per depth and feature, thresholds at the quantiles of the bin masses of the frontier
            # rows (the policy of the reference's compiled split finder; its torch frontier raises on
            # it); the evenly spaced ids below are what the device falls back to for an empty frontier
            self.cut_mass = cfg.cut_selection == "mass"
            thr = even_cut_ids(nb, k_user)
            if self.cut_mass and thr.shape[0] != k_user:
                thr = np.arange(k_user, dtype=np.int32)
        else:
            thr = np.arange(nb - 1, dtype=np.int32)
        self.thr_ids = torch.from_numpy(thr).to(self.dev)
        self.era_offsets = torch.from_numpy(np.ascontiguousarray(era_offsets, dtype=np.int32)).to(self.dev)
        self.feat_local = torch.from_numpy(np.ascontiguousarray(feat_local, dtype=np.int32)).to(self.dev)
        self.y = torch.from_numpy(np.ascontiguousarray(y_sorted, dtype=np.float32)).to(self.dev)
        self.preds = torch.zeros(n, dtype=torch.float32, device=self.dev)
        self.gq = torch.zeros(npad, dtype=torch.int32, device=self.dev)
        self.slot = torch.full((npad,), -1, dtype=torch.int16, device=self.dev)  # 0xFFFF: no slot
        self.leaf = torch.zeros(npad, dtype=torch.int16, device=self.dev)
        self.bits = (torch.zeros(npad // 32, dtype=torch.int32, device=self.dev)
                     if (world > 1 and not replicated) else None)
        self.ctl = torch.zeros(int(self.lib.pb_ctl_bytes()), dtype=torch.uint8, device=self.dev)

        st = B.TrainState()
        st.n_rows = n
        st.n_features_total = n_features_total
        st.n_features_local = matrix.n_features_local
        st.n_eras = self.E
        st.max_bins = nb
        st.code_bits = matrix.code_bits
        st.pitch = matrix.pitch
        st.max_depth = int(cfg.max_depth)
        st.pack_size = int(cfg.pack_size)
        st.min_samples_leaf = int(cfg.min_samples_leaf)
        st.n_thresholds = int(thr.shape[0])
        st.feature_block_size = int(cfg.feature_block_size)
        st.cut_mass = 1 if self.cut_mass else 0
        # PACKBOOST_DIRECTION_FORM=helper: the +1 / -1 directional term of the reference's helper and
        # native code instead of the torch frontier's agreement with the parent direction
        st.direction_form = 1 if os.getenv("PACKBOOST_DIRECTION_FORM") == "helper" else 0
        st.lambda_l2 = float(cfg.lambda_l2)
        st.lambda_dro = float(cfg.lambda_dro)
        st.direction_weight = float(cfg.direction_weight)
        st.era_alpha = float(cfg.era_alpha)
        st.learning_rate = float(cfg.learning_rate)
        st.codes = matrix.codes.data_ptr()
        st.era_offsets = self.era_offsets.data_ptr()
        st.thr_ids = self.thr_ids.data_ptr()
        st.feat_local = self.feat_local.data_ptr()
        st.y = self.y.data_ptr()
        st.preds = self.preds.data_ptr()
        st.gq = self.gq.data_ptr()
        st.slot = self.slot.data_ptr()
        st.leaf = self.leaf.data_ptr()
        st.ctl = self.ctl.data_ptr()
        self.st = st

        # workspace: candidate table + as many features of histogram as fit the budget
        k_sampled = self.n_sampled()
        stride = 1 << (int(cfg.max_depth) - 1)
        per_feat = stride * self.E * (nb * 12 + int(thr.shape[0]) * 8) + stride * int(thr.shape[0]) * 12
        local_sampled = (k_sampled + world - 1) // world + 1
        want = 24 * self.F * stride + per_feat * min(local_sampled, max(matrix.n_features_local, 1)) + (1 << 20)
        min_bytes = int(self.lib.pb_workspace_min_bytes(C.byref(st)))
        if workspace_bytes is None:
            free, _total = torch.cuda.mem_get_info(self.dev)
            cap = int(os.getenv("PACKBOOST_WORKSPACE_BYTES", str(min(8 << 30, int(free * 0.6)))))
            workspace_bytes = max(min_bytes, min(want, cap))
        self.workspace = torch.empty(int(workspace_bytes), dtype=torch.uint8, device=self.dev)
        st.workspace = self.workspace.data_ptr()
        st.workspace_bytes = int(workspace_bytes)
        eo = np.ascontiguousarray(era_offsets, dtype=np.int32)
        B.check(self.lib.pb_train_prepare(C.byref(st), eo.ctypes.data))

        # pinned staging for the per-round feature lists and the decision log
        D = int(cfg.max_depth)
        self.D = D
        ptr, nbytes = C.c_void_p(), C.c_int64()
        B.check(self.lib.pb_round_log_buffer(C.byref(st), C.byref(ptr), C.byref(nbytes)))
        self.log_bytes = int(nbytes.value)
        off = ptr.value - self.ctl.data_ptr()
        self.log_dev = self.ctl[off: off + self.log_bytes]
        # Rounds are enqueued ahead of the host's bookkeeping, so the pinned staging buffers form a
        # ring: a slot is reused only after the round that used it has delivered its log.
        self.log_host = [torch.empty(self.log_bytes, dtype=torch.uint8).pin_memory() for _ in range(_RING)]
        self.feat_host = [torch.empty((D, 3, max(k_sampled, 1)), dtype=torch.int32).pin_memory() for _ in range(_RING)]
        self.log_event = [torch.cuda.Event() for _ in range(_RING)]
        self.feat_dev = torch.empty((D, 3, max(k_sampled, 1)), dtype=torch.int32, device=self.dev)
        self.corr_dev = None
        self.enqueued = 0
        self.rounds_done = 0
        # CUDA graph of one round (PACKBOOST_CUDA_GRAPH=0 disables it).  With the memory-sharded
        # layout the local feature counts change from round to round, so it stays off there.
        self.use_graph = os.getenv("PACKBOOST_CUDA_GRAPH") != "0" and (world == 1 or self.replicated)
        self.graph = None
        self.graph_signature = None
        self.graph_launches = 0
        self.graph_replays = 0
        self.pending_delta = False
        self.prof = None
        # PACKBOOST_COMM=native: the per-depth exchanges go through the library's own NCCL entry
        # points (pb_comm_*) instead of torch.distributed; the communicator id is handed round once
        self.comm = None
        if world > 1 and os.getenv("PACKBOOST_COMM") == "native":
            ident = torch.zeros(128, dtype=torch.uint8, device=self.dev)
            if rank == 0:
                raw = (C.c_ubyte * 128)()
                B.check(self.lib.pb_comm_unique_id(raw))
                ident.copy_(torch.tensor(list(raw), dtype=torch.uint8))
            torch.distributed.broadcast(ident, src=0)
            raw = (C.c_ubyte * 128)(*ident.cpu().tolist())
            comm = C.c_void_p()
            B.check(self.lib.pb_comm_init(C.byref(comm), raw, world, rank))
            self.comm = comm
        self._prof_ms, self._prof_n = [0.0] * 5, [0] * 5
        self._prof_queue: list[tuple[int, float]] = []

    # -- per-phase timing (the reference fills hist_ms / score_ms / partition_ms of its depth logs
    #    with perf_counter buckets, packboost/booster.py:220-270) --------------------------------
    def enable_profile(self) -> None:
        """Bracket every kernel family launch of this trainer with CUDA events.  Events cannot time
        kernels inside a graph replay, so rounds are launched eagerly while this is on."""
        if self.prof is None:
            self.prof = self.lib.pb_profile_create()
            self.st.profile = self.prof
            self.use_graph = False
            self.release_graph()

    def disable_profile(self) -> None:
        if self.prof is not None:
            torch.cuda.current_stream().synchronize()
            self.st.profile = None
            self.lib.pb_profile_destroy(self.prof)
            self.prof = None

    def __del__(self):
        if sys is None or sys.is_finalizing():   # (the CUDA context may be gone already; the process is ending anyway)
            return
        try:
            self.disable_profile()
        except Exception:
            pass

    def profile_totals(self) -> tuple[list[float], list[int]]:
        """Summed milliseconds and launch counts per kernel family since the last collection
        (0 histogram, 1 scorer, 2 select, 3 partition, 4 round begin); synchronise first."""
        ms5, n5 = (C.c_double * 5)(), (C.c_int64 * 5)()
        B.check(self.lib.pb_profile_collect(self.prof, ms5, n5))
        tot_ms = [a + b for a, b in zip(self._prof_ms, ms5)]
        tot_n = [a + b for a, b in zip(self._prof_n, n5)]
        self._prof_ms, self._prof_n = [0.0] * 5, [0] * 5
        return tot_ms, tot_n

    def profile_by_depth(self) -> list[dict[str, float]]:
        """Milliseconds per depth of the oldest round whose launches have not been handed out yet.
        The library returns finished launches in issue order; a round opens with its round-begin
        bracket, and within it a histogram launch after a select launch opens the next depth.  The
        host may be enqueuing a round ahead: launches of later rounds stay queued here."""
        cap = 4096
        kinds, ms, n = (C.c_int32 * cap)(), (C.c_float * cap)(), C.c_int64()
        B.check(self.lib.pb_profile_collect_launches(self.prof, kinds, ms, cap, C.byref(n)))
        for i in range(min(int(n.value), cap)):
            k = int(kinds[i])
            self._prof_ms[k] += float(ms[i])   # (kept for profile_totals)
            self._prof_n[k] += 1
            self._prof_queue.append((k, float(ms[i])))
        q = self._prof_queue
        while q and q[0][0] != 4:              # leftovers of a round that was handed out already
            q.pop(0)
        if not q:
            return []
        end = next((i for i in range(1, len(q)) if q[i][0] == 4), len(q))
        mine, self._prof_queue = q[1:end], q[end:]
        out: list[dict[str, float]] = []
        cur = None
        seen_select = True
        names = {0: "hist_ms", 1: "score_ms", 2: "select_ms", 3: "partition_ms"}
        for k, t in mine:
            if k == 0 and seen_select:
                cur = {"hist_ms": 0.0, "score_ms": 0.0, "select_ms": 0.0, "partition_ms": 0.0}
                out.append(cur)
                seen_select = False
            if cur is None:
                continue
            cur[names[k]] += t
            if k == 2:
                seen_select = True
        return out

    def n_sampled(self) -> int:
        frac = float(self.cfg.layer_feature_fraction)
        k = max(1, int(round(frac * self.F)))
        return min(k, self.F)

    # -- one round ---------------------------------------------------------
    def run_round(self, subsets: list[np.ndarray], redo: bool = False) -> int:
        """Enqueue every phase of one round; ``subsets[d]`` is the sampled feature list of depth d.

        Returns the ticket to pass to :meth:`read_log`.  ``redo=True`` replaces the round enqueued
        last (its leaf deltas are dropped, the predictions it started from are kept)."""
        lib, st = self.lib, C.byref(self.st)
        stream = torch.cuda.current_stream().cuda_stream
        D = self.D
        k = subsets[0].shape[0]
        ticket = self.enqueued
        slot = ticket % _RING
        if ticket >= _RING:
            self.log_event[slot].synchronize()  # the slot's previous round has long finished
        fh = self.feat_host[slot]
        n_local = []
        for d in range(D):
            s = subsets[d]
            fh[d, 0, :k] = torch.from_numpy(s)
            if self.replicated and self.world > 1:
                rows, pos = dealt_part(s, self.rank, self.world)
            else:
                rows, pos = local_part(s, self.rank, self.world, self.F)
            n_local.append(int(pos.shape[0]))
            fh[d, 1, : pos.shape[0]] = torch.from_numpy(rows)
            fh[d, 2, : pos.shape[0]] = torch.from_numpy(pos)
        self.feat_dev.copy_(fh, non_blocking=True)
        apply_previous = 1 if (self.pending_delta and not redo) else 0
        # The phases of a round are the same launches every round (the feature lists change only as
        # data in feat_dev), so from the second round on they are replayed as one CUDA graph.  The
        # graph is tied to the per-depth local feature counts; any other round runs eagerly.
        signature = (k, tuple(n_local))
        if self.use_graph and apply_previous == 1:
            if self.graph is None:
                try:
                    self._capture(k, n_local, signature)
                except RuntimeError as exc:  # e.g. a collective that cannot be captured: launch eagerly
                    logging.getLogger(__name__).warning("round graph capture failed (%s); launching eagerly", exc)
                    self.use_graph = False
            if self.graph_signature == signature:
                self.graph.replay()
                self.graph_replays += 1
                return self._round_enqueued(slot, redo)
        self._enqueue_phases(k, n_local, apply_previous)
        return self._round_enqueued(slot, redo)

    def _capture(self, k: int, n_local: list[int], signature) -> None:
        """Capture the launches of one round into a CUDA graph.  The capture is driven directly
        (``capture_begin`` / ``capture_end`` on a side stream) rather than through the
        ``torch.cuda.graph`` context, whose entry collects garbage and empties the allocator caches —
        tens of milliseconds per fit, and far more when a large page-locked buffer of the caller
        happens to be waiting in the host cache; nothing is allocated while these launches are
        recorded, so the private pool that step prepares is not needed."""
        before = int(self.lib.pb_launch_count())
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream(device=self.dev)
        cur = torch.cuda.current_stream()
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            graph.capture_begin(capture_error_mode="thread_local")
            try:
                self._enqueue_phases(k, n_local, 1)
            finally:
                graph.capture_end()
        cur.wait_stream(side)
        self.graph, self.graph_signature = graph, signature
        self.graph_launches = int(self.lib.pb_launch_count()) - before  # kernels per replay

    def close_comm(self) -> None:
        if self.comm is not None:
            torch.cuda.current_stream().synchronize()
            B.check(self.lib.pb_comm_destroy(self.comm))
            self.comm = None

    def release_graph(self) -> None:
        """Drop the captured round graph (it is captured again if more rounds are enqueued)."""
        if self.graph is not None:
            torch.cuda.current_stream().synchronize()
            self.graph = None
            self.graph_signature = None

    def _round_enqueued(self, slot: int, redo: bool) -> int:
        self.pending_delta = True
        self.log_host[slot].copy_(self.log_dev, non_blocking=True)
        self.log_event[slot].record()
        self.enqueued += 1
        if not redo:
            self.rounds_done += 1
        return self.enqueued - 1

    def _enqueue_phases(self, k: int, n_local: list[int], apply_previous: int) -> None:
        lib, st = self.lib, C.byref(self.st)
        stream = torch.cuda.current_stream().cuda_stream
        D = self.D
        B.check(lib.pb_round_begin(st, apply_previous, stream))
        for d in range(D):
            sampled = self.feat_dev[d, 0].data_ptr()
            rows = self.feat_dev[d, 1].data_ptr()
            pos = self.feat_dev[d, 2].data_ptr()
            if self.world > 1:
                B.check(lib.pb_depth_clear_candidates(st, d, k, stream))
            B.check(lib.pb_depth_hist_score(st, d, rows, pos, n_local[d], k, stream))
            if self.world > 1:
                self._allreduce_candidates(d, k)
            B.check(lib.pb_depth_select(st, d, sampled, k, stream))
            if self.world > 1 and not self.replicated:
                B.check(lib.pb_depth_goleft_bits(st, d, self.bits.data_ptr(), stream))
                if self.comm is not None:
                    B.check(lib.pb_comm_allreduce_mask(self.comm, self.bits.data_ptr(), self.bits.numel(), stream))
                else:
                    torch.distributed.all_reduce(self.bits, op=torch.distributed.ReduceOp.SUM)
                B.check(lib.pb_depth_apply_bits(st, d, self.bits.data_ptr(), stream))
            else:
                B.check(lib.pb_depth_partition(st, d, stream))
        B.check(lib.pb_round_end(st, stream))

    def _allreduce_candidates(self, depth: int, k: int) -> None:
        if self.comm is not None:
            B.check(self.lib.pb_comm_allreduce_candidates(self.comm, C.byref(self.st), depth, k,
                                                          torch.cuda.current_stream().cuda_stream))
            return
        ptr, nbytes = C.c_void_p(), C.c_int64()
        B.check(self.lib.pb_candidates_buffer(C.byref(self.st), depth, k, C.byref(ptr), C.byref(nbytes)))
        off = ptr.value - self.workspace.data_ptr()
        view = self.workspace[off: off + int(nbytes.value)].view(torch.int32)
        torch.distributed.all_reduce(view, op=torch.distributed.ReduceOp.SUM)

    def flush_predictions(self) -> None:
        """Apply the last round's leaf deltas to ``preds`` now (metrics, end of fit)."""
        if self.pending_delta:
            B.check(self.lib.pb_apply_leaf_delta(C.byref(self.st), torch.cuda.current_stream().cuda_stream))
            self.pending_delta = False

    def era_correlation(self) -> float:
        """Mean per-era correlation of the training predictions with the targets, computed on the
        device (``packboost/booster.py:909-929``); only ``n_eras`` doubles travel to the host."""
        if self.corr_dev is None:
            self.corr_dev = torch.empty(self.E, dtype=torch.float64, device=self.dev)
        B.check(self.lib.pb_era_correlation(self.y.data_ptr(), self.preds.data_ptr(), self.era_offsets.data_ptr(),
                                            self.E, self.corr_dev.data_ptr(),
                                            torch.cuda.current_stream().cuda_stream))
        c = self.corr_dev.cpu().numpy()
        c = c[np.isfinite(c)]
        return float(c.mean()) if c.size else float("nan")

    def read_log(self, ticket: int) -> tuple[np.ndarray, np.ndarray]:
        """Wait for the round behind ``ticket`` and return its decision log (views of pinned memory)."""
        if not 0 <= self.enqueued - 1 - ticket < _RING:
            raise RuntimeError("round log is no longer held")
        slot = ticket % _RING
        self.log_event[slot].synchronize()
        raw = self.log_host[slot].numpy()
        head = raw[:88].view(_HEADER_DT)[0]
        winners = raw[88:].view(_WINNER_DT)
        return head, winners


def _tree_from_log(head, winners, max_depth: int) -> tuple[Tree, list[int]]:
    """Replay the device's decisions into a ``Tree`` (``packboost/booster.py:527-563``)."""
    tb = TreeBuilder()
    tb.set_leaf(0, float(head["root_value"]))
    n_ctx = [int(v) for v in head["n_ctx"][: max_depth + 1]]
    for d in range(max_depth):
        if n_ctx[d] == 0:
            break
        base = (1 << d) - 1
        sl = winners[base: base + n_ctx[d]]
        # (field columns as plain lists: element access on structured records is what costs here)
        for nid, feat, thr, lid, rid, lv, rv in zip(sl["tree_node"].tolist(), sl["feature"].tolist(),
                                                    sl["threshold"].tolist(), sl["left_id"].tolist(),
                                                    sl["right_id"].tolist(), sl["left_value"].tolist(),
                                                    sl["right_value"].tolist()):
            if feat < 0:
                tb.set_leaf(nid, lv)
                continue
            l, r = tb.split(nid, feat, thr)
            if l != lid or r != rid:
                raise RuntimeError("device and host child numbering disagree")
            tb.set_leaf(l, lv)
            tb.set_leaf(r, rv)
    if len(tb.nodes) != int(head["n_tree_nodes"]):
        raise RuntimeError("device and host tree sizes disagree")
    return tb.build(), n_ctx


# ------------------------------ the booster ------------------------------


class PackBoost:
    """Pack-parallel gradient booster with DES scoring on the B200 backend."""

    def __init__(self, config: PackBoostConfig) -> None:
        self.config = config
        if torch.device(config.device).type != "cuda":
            raise RuntimeError("packboost_b200 has no CPU path: PackBoostConfig.device must be 'cuda'")
        if not B.cuda_available():
            raise RuntimeError("packboost_b200: libpackboost_b200.so is not built or no sm_100 device is visible")
        self._device = torch.device("cuda", torch.cuda.current_device())
        self._rng = torch.Generator(device="cpu")
        if config.random_state is not None:
            self._rng.manual_seed(int(config.random_state))
        mode = (os.getenv("PACKBOOST_HIST_MODE") or config.histogram_mode).lower()
        if mode not in {"rebuild", "subtract", "auto"}:
            raise ValueError(f"Unsupported histogram_mode: {mode}")
        self._histogram_mode = mode
        self._logger = logging.getLogger(__name__)
        self._depth_logs: list[dict[str, object]] = []
        self._binner: BinningResult | None = None
        self._trees: list[Tree] = []
        self._distinct: list[tuple[Tree, int]] = []  # (tree, repeat) per round
        self._era_unique: np.ndarray | None = None
        self._feature_names: list[str] | None = None
        self._tree_weight: float | None = None
        self._trained_pack_size: int | None = None
        self._round_metrics: list[dict[str, float]] = []
        self._use_native_cuda = True
        self._cuda_backend = B
        self._forest_cache: dict | None = None
        self._train_preds: np.ndarray | None = None
        self._trainer: _DeviceTrainer | None = None
        self._row_order: np.ndarray | None = None
        self._fit_ctx: dict | None = None
        self._eval_states: list = []
        self._last_n_ctx: list[int] = []
        self._round_depths: list[int] = []   # depths with live nodes (= feature draws consumed) per round
        self._split_log: list[np.ndarray] = []
        self._pending_log = None
        self._predrawn = None
        self._inflight = None  # (log ticket, generator state at the round's start) of the enqueued round

    # Public -------------------------------------------------------------

    @property
    def trees(self) -> Sequence[Tree]:
        self._drain()
        self._flush_pending_tree()
        return self._trees

    @property
    def round_metrics(self) -> Sequence[dict[str, float]]:
        return self._round_metrics

    def fit(
        self,
        X: np.ndarray,
        y: np.ndarray,
        era: Iterable[int] | None,
        *,
        num_rounds: int,
        feature_names: Sequence[str] | None = None,
        eval_sets: Sequence[tuple[str, np.ndarray, np.ndarray, Iterable[int] | None]] | None = None,
        round_callback: Callable[[int, dict[str, float]], None] | None = None,
    ) -> "PackBoost":
        """Squared-loss boosting with pack-synchronous growth and DES (``packboost/booster.py:375-656``)."""
        self._start(X, y, era, feature_names=feature_names, eval_sets=eval_sets)
        for round_idx in range(num_rounds):
            metrics = self._boost_one_round(round_idx, num_rounds, round_callback is not None)
            if round_callback is not None:
                round_callback(round_idx + 1, metrics)
        self._finish()
        return self

    # -- fit, step by step (the benchmark times _boost_one_round) -------------
    def _start(self, X, y, era, *, feature_names=None, eval_sets=None) -> None:
        """Validate, bin, pack and upload the data; allocate the device state."""
        cfg = self.config
        # torch tensors (device-resident, or pinned host memory) are consumed without conversion
        on_device = isinstance(X, torch.Tensor)
        X_np = X.detach() if on_device else np.asarray(X)
        y_np = np.asarray(y.detach().cpu().numpy() if isinstance(y, torch.Tensor) else y, dtype=np.float32)
        if y_np.ndim != 1:
            raise ValueError("y must be 1-D")
        N, F = X_np.shape
        if N != y_np.shape[0]:
            raise ValueError("X and y row mismatch")
        wide = os.getenv("PACKBOOST_ALLOW_WIDE_BINS") == "1"
        if cfg.max_bins > 128 and not wide:
            raise ValueError("max_bins must be ≤ 128 when using int8 bin storage")
        if cfg.max_bins > 256:
            raise ValueError("max_bins must be ≤ 256")
        if era is None:
            era_encoded = np.zeros(N, dtype=np.int16)
            uniq = np.array([0], dtype=np.int16)
        else:
            era_np = np.asarray(era, dtype=np.int16)
            if era_np.shape[0] != N:
                raise ValueError("era must align with X rows")
            if N > 1 and np.all(era_np[1:] >= era_np[:-1]):
                # eras already contiguous and ascending: their runs give the unique values directly
                starts = np.concatenate([[0], np.flatnonzero(era_np[1:] != era_np[:-1]) + 1])
                uniq = era_np[starts]
                era_encoded = np.repeat(np.arange(starts.shape[0], dtype=np.int16),
                                        np.diff(np.concatenate([starts, [N]])))
            else:
                uniq, inv = np.unique(era_np, return_inverse=True)
                era_encoded = inv.astype(np.int16)
        self._era_unique = uniq
        E = int(uniq.shape[0])
        self._feature_names = list(feature_names) if feature_names is not None else [f"f{i}" for i in range(F)]

        # rows ordered by (era, row); identity when eras are already contiguous and ascending
        if N <= 1 or np.all(era_encoded[1:] >= era_encoded[:-1]):
            order = None
            era_sorted = era_encoded
        else:
            order = np.argsort(era_encoded, kind="stable")
            era_sorted = era_encoded[order]
        counts = np.bincount(era_sorted.astype(np.int64), minlength=E)
        era_offsets = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)

        # binning (packboost/data.py:61-93)
        small_int = X_np.dtype in (torch.uint8, torch.int8, np.dtype(np.uint8), np.dtype(np.int8))
        validate_on_device = bool(cfg.prebinned) and small_int
        if validate_on_device:
            is_binned = True   # declared by the caller; the range is checked on the device while packing
        elif on_device:
            host_view = X_np.cpu().numpy() if X_np.is_cuda else X_np.numpy()
            is_binned = detect_prebinned(host_view, cfg.max_bins)
        else:
            is_binned = detect_prebinned(X_np, cfg.max_bins)
        if bool(cfg.prebinned) and not is_binned:
            raise ValueError("prebinned=True requires X to contain integer bins within [0, max_bins).")
        rank, world = 0, 1
        if torch.distributed.is_available() and torch.distributed.is_initialized():
            rank, world = torch.distributed.get_rank(), torch.distributed.get_world_size()
        # With several GPUs every rank histograms and scores only a share of the sampled features,
        # and brings to its device only the strip of columns it owns (a contiguous block of
        # ceil(F / world) features).
        c0, c1 = owned_range(F, rank, world)
        blk = block_size(F, world)
        if is_binned:
            edges = None
            self._binner = BinningResult(bins=None, bin_edges=None, prebinned=True)
            if on_device:
                X_src = X_np.view(torch.uint8) if X_np.dtype == torch.int8 else X_np.to(torch.uint8)
            else:
                X_src = X_np if X_np.dtype in (np.uint8, np.int8) else X_np.astype(np.uint8)
                X_src = X_src.view(np.uint8)
        else:
            X_src = X_np.to(torch.float32) if on_device else X_np.astype(np.float32, copy=False)
            if world > 1:
                # each rank sorts its own columns; the edge tables are exchanged
                own = np.zeros((cfg.max_bins - 1, blk), dtype=np.float32)
                if c1 > c0:
                    own[:, : c1 - c0] = quantile_edges_device(X_src[:, c0:c1], cfg.max_bins)
                parts = torch.empty((world, cfg.max_bins - 1, blk), dtype=torch.float32, device=self._device)
                torch.distributed.all_gather_into_tensor(parts, torch.from_numpy(own).to(self._device))
                edges = np.ascontiguousarray(parts.permute(1, 0, 2).reshape(cfg.max_bins - 1, world * blk)[:, :F].cpu().numpy())
            else:
                edges = quantile_edges_device(X_src, cfg.max_bins)
            self._binner = BinningResult(bins=None, bin_edges=edges, prebinned=False)

        # When the whole packed matrix fits comfortably in one GPU's memory it is kept on every rank
        # anyway (each rank packs its strip, an all-gather over NVLink completes the copies): each
        # rank can then route rows itself and the per-depth go-left bitmask exchange disappears (one
        # exchange per depth instead of two).  PACKBOOST_SHARD_CODES=1 forces the memory-sharded
        # layout.  The choice is agreed by all ranks (their GPUs may have different amounts of free
        # memory, and the two layouts issue different collectives).
        replicate = False
        bits = code_bits_for(cfg.max_bins)
        if world > 1:
            free, _tot = torch.cuda.mem_get_info(self._device)
            replicate = choose_replicated(N * F * bits // 8, free, world,
                                          os.getenv("PACKBOOST_SHARD_CODES") == "1", self._device)
        if world > 1:
            # every rank brings over and packs 1 / world of the rows; the packed pieces are exchanged
            # between the GPUs (all-gather for the replicated layout, all-to-all for the sharded one)
            feat_local = feature_map(F, 0, 1) if replicate else feature_map(F, rank, world)
            matrix = pack_feature_major_distributed(X_src, edges, cfg.max_bins, row_order=order, rank=rank, world=world,
                                                    n_features=F, keep=None if replicate else (c0, c1),
                                                    validate_codes=validate_on_device)
        else:
            feat_local = feature_map(F, 0, 1)
            matrix = pack_feature_major(X_src, edges, cfg.max_bins, row_order=order, validate_codes=validate_on_device,
                                        defer_validation=True)
        if validate_on_device and not agree_all(matrix.max_code < min(cfg.max_bins, 128), self._device):
            raise ValueError("prebinned=True requires X to contain integer bins within [0, max_bins).")
        y_sorted = y_np if order is None else y_np[order]
        self._trainer = _DeviceTrainer(cfg, matrix, y_sorted, era_offsets, F, feat_local, rank, world,
                                       replicated=replicate)
        self._row_order = order
        self._fit_ctx = {"era_sorted": era_sorted, "y_sorted": y_sorted, "F": F}

        self._depth_logs = []
        self._round_depths = []
        self._split_log = []
        self._round_metrics = []
        self._trees = []
        self._distinct = []
        self._forest_cache = None
        self._tree_weight = float(cfg.learning_rate)
        self._trained_pack_size = int(cfg.pack_size)
        self._eval_states = self._prepare_eval_sets(eval_sets)
        self._pending_log = None
        self._predrawn = None
        self._inflight = None

    def _boost_one_round(self, round_idx: int, num_rounds: int, want_callback: bool = False) -> dict[str, float]:
        """One boosting round (``packboost/booster.py:494-655``)."""
        cfg, trainer, ctx = self.config, self._trainer, self._fit_ctx
        F, D, k = ctx["F"], int(cfg.max_depth), trainer.n_sampled()
        t0 = perf_counter()
        # One draw per depth, speculating that every depth has active nodes; when the device
        # reports an empty frontier at depth d the reference would not have drawn for d or any
        # later depth of this round (packboost/booster.py:516-519), so the generator is rewound to
        # the round's start and the first d draws are replayed.
        def draw():
            st0 = self._rng.get_state()
            return st0, [torch.randperm(F, generator=self._rng)[:k].numpy().astype(np.int32) for _ in range(D)]

        eval_states = self._eval_states
        want_metrics = want_callback or bool(eval_states) or os.getenv("PACKBOOST_TRAIN_METRICS") == "1"
        # Without per-round consumers the host runs one round ahead of the device: round r is
        # enqueued before the log of round r - 1 is read, so the device never waits for the host.
        run_ahead = not want_metrics and os.getenv("PACKBOOST_RUN_AHEAD") != "0"
        if want_metrics and os.getenv("PACKBOOST_PHASE_TIMERS", "1") != "0":
            trainer.enable_profile()   # fills hist_ms / score_ms / partition_ms of the depth logs

        state0, subsets = self._predrawn if self._predrawn is not None else draw()
        self._predrawn = None
        ticket = trainer.run_round(subsets)
        previous, self._inflight = self._inflight, (ticket, state0)
        # while the device works on this round: finish the host bookkeeping of earlier rounds and
        # draw the next round's subsets (discarded if a round turns out to rewind the generator)
        self._flush_pending_tree()
        if previous is not None and not self._retire(previous):
            # round r - 1 ended early and the generator was rewound, so this round's subsets came
            # from the wrong state.  Enqueue it again with the right ones; the first attempt is dropped.
            state0, subsets = draw()
            ticket = trainer.run_round(subsets, redo=True)
            self._inflight = (ticket, state0)
        if round_idx + 1 < num_rounds:
            self._predrawn = draw()
        if not run_ahead:
            self._drain()
        if want_metrics:
            self._flush_pending_tree()  # callbacks and evaluation sets see this round's trees
        metrics: dict[str, float] = {"round": round_idx + 1}
        if want_metrics:
            trainer.flush_predictions()
            metrics["train_corr"] = trainer.era_correlation()
        else:
            metrics["train_corr"] = float("nan")
        try:
            eval_every = int(os.getenv("PACKBOOST_EVAL_EVERY", "1"))
        except Exception:
            eval_every = 1
        if eval_states and eval_every > 0 and (((round_idx + 1) % eval_every == 0) or round_idx + 1 == num_rounds):
            self._update_eval_sets(eval_states)
        dt = perf_counter() - t0
        metrics["trees_per_second"] = (cfg.pack_size / dt) if dt > 0 else float("inf")
        metrics["round_seconds"] = dt
        for stt in eval_states:
            metrics[f"{stt['name']}_corr"] = _era_correlation_np(stt["era"], stt["y"], stt["preds"].cpu().numpy())
        self._round_metrics.append(metrics)
        return metrics

    def _flush_pending_tree(self) -> None:
        """Replay the stored decision log of the last finished round into ``Tree`` objects."""
        if self._pending_log is None:
            return
        head, winners = self._pending_log
        self._pending_log = None
        tree, _ = _tree_from_log(head, winners, int(self.config.max_depth))
        self._distinct.append((tree, int(self.config.pack_size)))
        self._trees.extend([tree] * int(self.config.pack_size))

    def _retire(self, inflight) -> bool:
        """Take in the decision log of an enqueued round.  Returns False when the round ended before
        ``max_depth``: the reference would not have drawn feature subsets for the unused depths
        (``packboost/booster.py:516-519``), so the generator is rewound to the round's start, the
        used draws are replayed and every later draw is invalid."""
        ticket, state0 = inflight
        D = int(self.config.max_depth)
        head, winners = self._trainer.read_log(ticket)
        n_ctx = [int(v) for v in head["n_ctx"][: D + 1]]
        self._last_n_ctx = n_ctx
        used = next((d for d in range(D) if n_ctx[d] == 0), D)
        self._round_depths.append(used)
        if used < D:
            self._rng.set_state(state0)
            for _ in range(used):
                torch.randperm(self._fit_ctx["F"], generator=self._rng)
            self._predrawn = None
        k = self._trainer.n_sampled()
        phase_ms = self._trainer.profile_by_depth() if getattr(self._trainer, "prof", None) is not None else []
        for d in range(used):
            self._depth_logs.append(self._depth_log(d, n_ctx[d], k, phase_ms[d] if d < len(phase_ms) else None))
            w = winners[(1 << d) - 1: (1 << d) - 1 + n_ctx[d]]
            self._split_log.append(w[w["feature"] >= 0].copy())
        self._flush_pending_tree()
        self._pending_log = (head.copy(), winners[: (1 << D) - 1].copy())
        return used == D

    def _drain(self) -> None:
        """Wait for the round in flight, if any, and take in its log."""
        if self._inflight is not None:
            inflight, self._inflight = self._inflight, None
            self._retire(inflight)

    def _finish(self) -> None:
        self._drain()
        self._flush_pending_tree()
        # a graph that holds captured collectives must be gone before the process group is torn
        # down (communicator destruction waits for it otherwise)
        self._trainer.release_graph()
        self._trainer.flush_predictions()
        torch.cuda.current_stream().synchronize()
        self._trainer.close_comm()

    def train_predictions(self) -> np.ndarray:
        """Predictions of the training rows as maintained during ``fit`` (original row order)."""
        if self._trainer is None:
            raise RuntimeError("Model must be fitted first")
        self._trainer.flush_predictions()
        p = self._trainer.preds.cpu().numpy()
        if self._row_order is None:
            return p
        out = np.empty_like(p)
        out[self._row_order] = p
        return out

    # -- helpers the reference exposes on the booster (its own tests call them) ----------------
    def _compute_era_weights(self, counts: torch.Tensor) -> torch.Tensor:
        """Era weights from per-era row counts (``packboost/booster.py:815-826``): 0 for an absent
        era, else 1, or ``count + era_alpha`` when ``era_alpha > 0``."""
        counts = counts.to(torch.float32)
        alpha = float(self.config.era_alpha)
        present = counts > 0
        w = counts + alpha if alpha > 0.0 else torch.ones_like(counts)
        return torch.where(present, w, torch.zeros_like(counts))

    def _batched_histograms_nodes(self, bins_matrix, grad_rows, hess_rows, era_ids, node_ids, num_nodes, num_eras,
                                  num_bins):
        """Counts and gradient / hessian sums ``[feature, node, era, bin]`` of the given rows
        (``packboost/booster.py:933-977``), built by the histogram kernel."""
        from .kernels import histograms_nodes
        return histograms_nodes(bins_matrix, grad_rows, hess_rows, era_ids, node_ids, int(num_nodes), int(num_eras),
                                int(num_bins))

    def _stack_node_rows(self, era_rows: Sequence[torch.Tensor]) -> tuple[torch.Tensor, torch.Tensor]:
        """Concatenated row ids of a node and their era index (``packboost/booster.py:2156-2170``)."""
        rows = [r for r in era_rows if r.numel() > 0]
        if not rows:
            return (torch.empty(0, dtype=torch.int64, device=self._device),
                    torch.empty(0, dtype=torch.int16, device=self._device))
        eras = [torch.full((r.numel(),), e, dtype=torch.int16, device=r.device)
                for e, r in enumerate(era_rows) if r.numel() > 0]
        return torch.cat(rows, 0), torch.cat(eras, 0)

    def _compute_histograms(self, feature_values, grad_rows, hess_rows, era_ids, *, num_eras: int, num_bins: int):
        """Counts, gradient and hessian sums ``[era, bin]`` of one feature of one node
        (``packboost/booster.py:979-1002``), built by the histogram kernel."""
        if num_bins <= 0:
            raise ValueError("num_bins must be positive")
        dev = self._device
        if feature_values.numel() == 0:
            z = torch.zeros((num_eras, num_bins), dtype=torch.int64, device=dev)
            return z, z.to(torch.float32), z.to(torch.float32)
        hess = torch.ones_like(grad_rows) if hess_rows is None else hess_rows
        node = torch.zeros(feature_values.numel(), dtype=torch.int64, device=dev)
        c, g, h = self._batched_histograms_nodes(feature_values.view(-1, 1), grad_rows, hess, era_ids, node, 1,
                                                 num_eras, num_bins)
        return c[0, 0], g[0, 0], h[0, 0]

    def _weighted_welford(self, values: torch.Tensor, valid: torch.Tensor, weights: torch.Tensor):
        """Streaming weighted mean / std over the eras of ``values [E, T]`` with invalid entries
        masked: ``(mean, std, weight sum)`` (``packboost/booster.py:828-867``)."""
        if values.ndim != 2:
            raise ValueError("values must be 2D [E, T]")
        values, valid, weights = values.to(torch.float32), valid.to(torch.bool), weights.to(torch.float32)
        mean = torch.zeros(values.shape[1], dtype=torch.float32, device=values.device)
        m2, wsum = torch.zeros_like(mean), torch.zeros_like(mean)
        for e in range(values.shape[0]):
            w = torch.where(valid[e], weights[e].clamp_min(0.0), torch.zeros((), device=values.device))
            wsum_new = wsum + w
            factor = torch.where(wsum_new > 0, w / wsum_new.clamp_min(1e-38), torch.zeros_like(w))
            delta = values[e] - mean
            mean = mean + factor * delta
            m2 = m2 + w * delta * (values[e] - mean)
            wsum = wsum_new
        std = torch.sqrt(torch.clamp_min(m2 / torch.clamp_min(wsum, 1e-12), 0.0))
        return mean, std, wsum

    def _directional_agreement(self, left_values, right_values, valid, weights, weight_sum) -> torch.Tensor:
        """Weighted mean over valid eras of ``+1`` where the left leaf value exceeds the right one,
        else ``-1`` (``packboost/booster.py:869-907``)."""
        left, right = left_values.to(torch.float32), right_values.to(torch.float32)
        w = weights.to(torch.float32).clamp_min(0.0).view(-1, 1) * valid.to(torch.float32)
        direction = torch.where(left > right, 1.0, -1.0)
        accum = (w * direction).sum(0)
        denom = torch.clamp_min(weight_sum.to(torch.float32), 1e-12)
        return accum / denom

    def _find_best_split(self, node: NodeShard, grad: torch.Tensor, hess: torch.Tensor, bins: torch.Tensor,
                         feature_subset: torch.Tensor) -> SplitDecision | None:
        """Best split of one node given as per-era row lists, with arbitrary per-row hessians
        (``packboost/booster.py:1010-1290``): histograms and scores on the device.  The directional
        term follows ``PACKBOOST_DIRECTION_FORM`` (default: the torch frontier's form)."""
        from .kernels import best_split_one_node
        cfg = self.config
        dev = self._device
        eras = [r.to(dev).to(torch.int64) for r in node.era_rows]
        rows = torch.cat(eras) if eras else torch.zeros(0, dtype=torch.int64, device=dev)
        era_ids = torch.cat([torch.full((int(r.numel()),), e, dtype=torch.int64, device=dev) for e, r in enumerate(eras)]) \
            if eras else rows
        feats = feature_subset.to(torch.int64).cpu().numpy()
        nb, k_user = int(cfg.max_bins), int(cfg.k_cuts)
        if 0 < k_user < nb - 1:
            if cfg.cut_selection == "mass":
                raise RuntimeError("_find_best_split supports the full sweep and even k_cuts only")
            thr = even_cut_ids(nb, k_user)
        else:
            thr = np.arange(nb - 1, dtype=np.int32)
        codes = bins.to(dev).index_select(0, rows).index_select(1, torch.from_numpy(feats).to(dev))
        res = best_split_one_node(
            codes, grad.to(dev).index_select(0, rows), hess.to(dev).index_select(0, rows), era_ids, feats, len(eras),
            max_bins=nb, thr_ids=thr, lambda_l2=cfg.lambda_l2, lambda_dro=cfg.lambda_dro,
            direction_weight=cfg.direction_weight, era_alpha=cfg.era_alpha,
            direction_form=1 if os.getenv("PACKBOOST_DIRECTION_FORM") == "helper" else 0,
            min_samples_leaf=int(cfg.min_samples_leaf), feature_block_size=int(cfg.feature_block_size))
        if res is None:
            return None
        col = bins.to(dev)[:, res["feature"]]
        left_rows = [r[col.index_select(0, r) <= res["threshold"]] for r in eras]
        right_rows = [r[col.index_select(0, r) > res["threshold"]] for r in eras]
        return SplitDecision(left_rows=left_rows, right_rows=right_rows, **res)

    def split_records(self) -> dict[str, np.ndarray]:
        """Every split of the fit in the order the frontier produced it (round, depth, frontier
        position): tree node, feature, threshold, DES score (the ``SplitDecision.score`` of
        ``packboost/booster.py:206-217``), rows sent left and rows of the node."""
        self._drain()
        rec = (np.concatenate(self._split_log) if self._split_log else np.zeros(0, dtype=_WINNER_DT))
        return {"node": rec["tree_node"].astype(np.int32), "feature": rec["feature"].astype(np.int32),
                "threshold": rec["threshold"].astype(np.int32), "score": rec["score"].astype(np.float32),
                "left_count": rec["left_count"].astype(np.int64),
                "right_count": (rec["total_count"] - rec["left_count"]).astype(np.int64)}

    def _depth_log(self, depth: int, n_nodes: int, k: int, ms: dict | None = None) -> dict[str, object]:
        """Depth record with the reference's field names (``packboost/booster.py:220-270, 565-579``).
        The millisecond fields are device times of the depth's kernels (CUDA events) when per-round
        metrics were asked for, else 0: timing needs eager launches, which the fast path avoids.
        ``scan_ms`` stays 0 (the prefix scan is part of the scorer kernels)."""
        blk = int(self.config.feature_block_size)
        blk = k if (blk <= 0 or blk > k) else blk
        ms = ms or {}
        return {
            "nodes_processed": n_nodes, "nodes_skipped": 0, "rows_total": 0,
            "feature_blocks": (k + blk - 1) // blk, "bincount_calls": 0,
            "hist_ms": ms.get("hist_ms", 0.0), "scan_ms": 0.0,
            "score_ms": ms.get("score_ms", 0.0) + ms.get("select_ms", 0.0), "partition_ms": ms.get("partition_ms", 0.0),
            "nodes_subtract_ok": 0, "nodes_rebuild": n_nodes, "nodes_subtract_fallback": 0,
            "nodes_collapsed": n_nodes * (int(self.config.pack_size) - 1), "feature_block_size": blk,
            "depth": depth, "feature_subset_size": k, "pack_size": int(self.config.pack_size),
            "layer_feature_fraction": float(self.config.layer_feature_fraction),
            "histogram_mode": self._histogram_mode, "seed": self.config.random_state,
            "torch_threads": torch.get_num_threads(),
        }

    # -- evaluation sets -----------------------------------------------------
    def _prepare_eval_sets(self, eval_sets):
        states = []
        if not eval_sets:
            return states
        for name, X_eval, y_eval, era_eval in eval_sets:
            if y_eval is None:
                raise ValueError(f"eval set '{name}' requires y values for correlation logging")
            Xe = np.asarray(X_eval)
            rows = self._pack_rows(Xe)
            era_e = np.zeros(Xe.shape[0], dtype=np.int16) if era_eval is None else np.asarray(era_eval, dtype=np.int16)
            if era_e.shape[0] != Xe.shape[0]:
                raise ValueError(f"eval set '{name}' era ids must align with X rows")
            states.append({"name": name, "rows": rows, "y": np.asarray(y_eval, dtype=np.float32), "era": era_e,
                           "preds": torch.zeros(Xe.shape[0], dtype=torch.float32, device=self._device), "done": 0})
        return states

    def _update_eval_sets(self, states) -> None:
        # predictions accumulate in tree order, so adding only the new rounds reproduces a
        # from-scratch evaluation bit for bit
        for stt in states:
            new = self._distinct[stt["done"]:]
            if not new:
                continue
            forest = self._pack_forest(new)
            stt["preds"] = self._predict_packed(stt["rows"], forest, init=stt["preds"])
            stt["done"] = len(self._distinct)

    # -- prediction -------------------------------------------------------------
    def _pack_rows(self, X: np.ndarray) -> PackedRows:
        if self._binner is None:
            raise RuntimeError("Model must be fitted before predict()")
        if isinstance(X, torch.Tensor) and X.is_cuda:
            # device input is consumed where it is (codes: range-checked on the device)
            Xd = X.detach()
            if self._binner.bin_edges is None:
                if Xd.dtype not in (torch.uint8, torch.int8):
                    raise ValueError("Input must already be prebinned when no edges are provided")
                Xd = Xd.view(torch.uint8)
                if Xd.numel() and int(Xd.max()) >= int(self.config.max_bins):
                    raise ValueError("Input must already be prebinned when no edges are provided")
                return pack_row_major(Xd, None, self.config.max_bins)
            return pack_row_major(Xd.to(torch.float32), self._binner.bin_edges, self.config.max_bins)
        X_np = X.detach().cpu().numpy() if isinstance(X, torch.Tensor) else np.asarray(X)
        if self._binner.bin_edges is None:
            if not detect_prebinned(X_np, self.config.max_bins):
                raise ValueError("Input must already be prebinned when no edges are provided")
            src = X_np if X_np.dtype in (np.uint8, np.int8) else X_np.astype(np.uint8)
            return pack_row_major(src.view(np.uint8), None, self.config.max_bins)
        return pack_row_major(X_np.astype(np.float32, copy=False), self._binner.bin_edges, self.config.max_bins)

    def _pack_forest(self, distinct: Sequence[tuple[Tree, int]]) -> dict[str, torch.Tensor]:
        arrs = [t.arrays() for t, _ in distinct]
        offs = np.zeros(len(arrs) + 1, dtype=np.int32)
        np.cumsum([a["feature"].shape[0] for a in arrs], out=offs[1:])
        cat = {k: np.concatenate([a[k] for a in arrs]) for k in ("feature", "threshold", "left", "right", "value", "is_leaf")}
        # nothing malformed reaches the device: children inside their tree and after their parent
        validate_forest(cat["feature"], cat["threshold"], cat["left"], cat["right"], cat["is_leaf"], offs)
        out = {k: torch.from_numpy(v).to(self._device) for k, v in cat.items()}
        out["offsets"] = torch.from_numpy(offs).to(self._device)
        out["repeat"] = torch.tensor([r for _, r in distinct], dtype=torch.int32, device=self._device)
        out["n_trees"] = len(arrs)
        out["max_feature"] = int(cat["feature"][cat["is_leaf"] == 0].max(initial=-1))
        # packed 8-byte nodes when the trees allow it (right child == left child + 1, small ids)
        internal = cat["is_leaf"] == 0
        ok = (bool(np.all(cat["right"][internal] == cat["left"][internal] + 1))
              and (cat["feature"][internal].max(initial=0) < 65536) and (cat["threshold"][internal].max(initial=0) < 256)
              and (cat["threshold"][internal].min(initial=0) >= 0))
        if ok:
            w0 = np.where(internal, (cat["feature"].astype(np.int64) & 0xFFFF) | ((cat["threshold"].astype(np.int64) & 0xFF) << 16),
                          1 << 31).astype(np.uint32)
            w1 = np.where(internal, cat["left"].astype(np.int64) & 0xFFFFFFFF,
                          cat["value"].astype(np.float32).view(np.uint32).astype(np.int64)).astype(np.uint32)
            out["packed"] = torch.from_numpy(np.stack([w0, w1], axis=1).view(np.int32).copy()).to(self._device)
            out["max_tree_nodes"] = int(np.diff(offs).max()) if len(arrs) else 1
        return out

    def _predict_packed(self, rows: PackedRows, forest: dict, init: torch.Tensor | None = None) -> torch.Tensor:
        out = torch.empty(rows.n_rows, dtype=torch.float32, device=self._device)
        if rows.n_rows == 0:
            return out
        f = forest
        if f["max_feature"] >= rows.n_features:
            raise ValueError(f"the ensemble splits on feature {f['max_feature']} but the input has {rows.n_features} columns")
        if "packed" in f:
            B.check(B.lib().pb_predict_rows_packed(
                rows.codes.data_ptr(), rows.n_rows, rows.pitch_row, rows.code_bits, f["packed"].data_ptr(),
                f["offsets"].data_ptr(), f["repeat"].data_ptr(), f["n_trees"], f["max_tree_nodes"],
                float(self._tree_weight),
                out.data_ptr(), B._ptr(init) if init is not None else 0, torch.cuda.current_stream().cuda_stream))
            return out
        B.check(B.lib().pb_predict_rows(
            rows.codes.data_ptr(), rows.n_rows, rows.pitch_row, rows.code_bits, f["feature"].data_ptr(),
            f["threshold"].data_ptr(), f["left"].data_ptr(), f["right"].data_ptr(), f["value"].data_ptr(),
            f["is_leaf"].data_ptr(), f["offsets"].data_ptr(), f["repeat"].data_ptr(), f["n_trees"],
            float(self._tree_weight), out.data_ptr(), B._ptr(init) if init is not None else 0,
            torch.cuda.current_stream().cuda_stream))
        return out

    def predict(self, X: np.ndarray) -> np.ndarray:
        """``pred = sum over trees of tree_weight * tree(X)`` accumulated in tree order, float32
        (``packboost/booster.py:658-712``)."""
        if self._binner is None:
            raise RuntimeError("Model must be fitted before predict()")
        self._drain()
        self._flush_pending_tree()
        rows = self._pack_rows(X)
        if not self._trees:
            return np.zeros(rows.n_rows, dtype=np.float32)
        if self._tree_weight is None:
            raise RuntimeError("Missing _tree_weight; call fit() first.")
        if self._trained_pack_size is not None and int(self.config.pack_size) != self._trained_pack_size:
            raise RuntimeError("pack_size differs from training; keep it constant.")
        if self._forest_cache is None or self._forest_cache["n_distinct"] != len(self._distinct):
            self._forest_cache = self._pack_forest(self._distinct)
            self._forest_cache["n_distinct"] = len(self._distinct)
        return self._predict_packed(rows, self._forest_cache).cpu().numpy()

    def predict_packwise(self, X: np.ndarray, block_size_trees: int = 8) -> np.ndarray:
        if block_size_trees <= 0:
            raise ValueError("block_size_trees must be positive")
        if self._binner is None:
            raise RuntimeError("Model must be fitted before predict_packwise()")
        return self.predict(X)

    def set_forest(self, trees: Sequence[Tree], tree_weight: float, *, bin_edges: np.ndarray | None = None,
                   repeats: Sequence[int] | None = None) -> "PackBoost":
        """Install an externally built ensemble (inference-only use)."""
        reps = list(repeats) if repeats is not None else [1] * len(trees)
        if len(reps) != len(trees) or any(int(r) < 0 for r in reps):
            raise ValueError("repeats must hold one non-negative count per tree")
        for t in trees:  # checked on the host, before any launch
            a = t.arrays()
            validate_forest(a["feature"], a["threshold"], a["left"], a["right"], a["is_leaf"],
                            [0, a["feature"].shape[0]])
        self._distinct = list(zip(trees, reps))
        self._trees = [t for t, r in self._distinct for _ in range(r)]
        self._tree_weight = float(tree_weight)
        self._trained_pack_size = int(self.config.pack_size)
        self._binner = BinningResult(bins=None, bin_edges=bin_edges, prebinned=bin_edges is None)
        self._forest_cache = None
        return self
