#!/usr/bin/env python
"""Benchmark: boosting rounds/s and histogram-kernel HBM GB/s on the era-heavy wide workload.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--scale S]

One "step" is one boosting round (pack of 32 identical trees, depth 6, 10 % of the 2 376
features sampled per depth, 574 eras) over a seeded synthetic stand-in for the 2.7 M-row
five-level table.  With N > 1 (launched by torchrun, one rank per GPU) the features are
sharded over the ranks and the same data set is trained, i.e. strong scaling.

Own arm: `value` is rounds/s with the packed matrix resident in HBM, timed with CUDA events
around exactly K rounds (barrier + synchronize on both sides, max over ranks); `e2e` is
rounds/s of the public `PackBoost.fit` call on HOST buffers for K rounds, including binning,
packing and the host->device copy of the matrix and the device->host read of each round's
decision log.  `roofline` is the histogram kernel: algorithmic bytes of its launches divided
by their event-timed duration inside the timed region.  `cpu_baseline` (N=1 only) and
`--impl reference` time the CPU port of the reference's torch frontier (oracle/) on two bounded
era-subsamples of the same workload on this box's host cores; `cpu_baseline_native` is the
reference's own compiled C++/OpenMP split finder (oracle/_ref) on the same samples.
`e2e_numpy` repeats the end-to-end fit on a pageable numpy array, `e2e_sharded` /
`value_sharded` (N > 1) with every rank holding only its own feature columns, and
`model_digest*` is a hash of the trees and training predictions of each end-to-end fit: equal
digests at every N and in every layout mean the same model bit for bit.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_ROWS, N_FEAT, N_ERAS = 2_700_000, 2376, 574
CFG = dict(pack_size=32, max_depth=6, learning_rate=0.4 / 32, lambda_l2=1e-6, lambda_dro=0.5,
           min_samples_leaf=20, max_bins=5, layer_feature_fraction=0.1, prebinned=True, random_state=42)
METRIC = "boosting_rounds_per_sec"
UNIT = "rounds/s"


def workload_name(n_rows, n_feat, n_eras):
    return (f"config3 era-heavy wide: {n_rows} rows x {n_feat} uint8 features in {{0..4}} (4-bit packed), "
            f"{n_eras} eras, pack_size=32, max_depth=6, feature fraction 0.1, lambda_dro=0.5, lr=0.4/32")


# ---------------------------------------------------------------------------------------------
# synthetic data (seeded, generated on the device; same shape and value distribution as
# packboost_b200.workloads.config3)
# ---------------------------------------------------------------------------------------------

def make_device_data(n_rows, n_feat, n_eras, device, seed=3):
    from packboost_b200.workloads import config3_device
    return config3_device(n_rows, n_feat, n_eras, device, seed)


# ---------------------------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------------------------

class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self._stop = threading.Event()
        self._t = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5).stdout
                parts = [p.strip() for p in out.strip().split(",")]
                if len(parts) >= 6:
                    self.samples.append(parts)
            except Exception:
                pass
            self._stop.wait(0.2)

    def start(self):
        self._t.start()

    def stop(self):
        self._stop.set()
        self._t.join(timeout=6)
        sm = [int(float(s[0])) for s in self.samples if s[0].replace(".", "").isdigit()]
        mx = [int(float(s[1])) for s in self.samples if s[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": int(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(self.samples)}


# ---------------------------------------------------------------------------------------------
# CPU port of the reference on a bounded era-subsample
# ---------------------------------------------------------------------------------------------

def cpu_rounds_per_sec(n_rows, n_feat, n_eras, sample_eras, rounds, warmup, kind="port"):
    """Time a CPU implementation of the path on the first `sample_eras` eras of a host-generated
    table of the same shape: `kind="port"` is the oracle's restatement of the reference's torch
    frontier, `kind="native"` the reference's own compiled C++/OpenMP split finder
    (oracle/_ref).  Histogram and scoring cost are linear in the number of whole eras, so rounds/s of
    the full workload is the sample's rounds/s times sample_eras / n_eras."""
    import torch
    from oracle import packboost_oracle as po
    from packboost_b200 import workloads
    torch.set_num_threads(os.cpu_count() or 1)
    rows_per_era = n_rows // n_eras
    w = workloads.config3(seed=3, n_rows=rows_per_era * sample_eras, n_features=n_feat, n_eras=sample_eras)
    p = po.OracleParams(**CFG)
    if kind == "native":
        from oracle import native_ref
        model = native_ref.fit(w.X, w.y, w.era, p, warmup + rounds)
    else:
        model = po.fit(w.X, w.y, w.era, p, warmup + rounds)
    secs = float(np.sum(model.round_seconds[warmup:]))
    sample_rps = rounds / secs
    return sample_rps * sample_eras / n_eras, secs, w.X.shape[0]


def cpu_baseline_two_sizes(n_rows, n_feat, n_eras, big_eras, rounds, warmup, kind="port"):
    """The CPU arm at two sample sizes (half and full): the two extrapolations to the whole workload
    are printed side by side, which shows inside the record how linear the cost is in the eras."""
    out = []
    for se in sorted({max(2, big_eras // 2), big_eras}):
        rps, secs, srows = cpu_rounds_per_sec(n_rows, n_feat, n_eras, min(se, n_eras), rounds, warmup, kind)
        out.append({"eras": min(se, n_eras), "rows": srows, "seconds": round(secs, 3), "extrapolated_rounds_per_sec": rps})
    return out


def pick_sample_eras(steps, warmup, n_eras, budget_s=60.0, per_era_round_s=0.2):
    e = int(budget_s / max(1, steps + warmup) / per_era_round_s / 1.5)   # 1.5: the half-size sample runs too
    return max(2, min(e, 24, n_eras))


def predict_bench(n_rows, n_rounds, steps, warmup):
    """Side benchmark of the ensemble predictor (one GPU): a seeded random ensemble in the
    8-byte node format scored through pb_predict_rows_packed; prints one JSON line."""
    import numpy as np
    import torch
    from packboost_b200 import backends as B, workloads
    from packboost_b200.data import pack_row_major
    steps, warmup = max(1, min(steps, 10)), max(1, min(warmup, 3))
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    w = workloads.config5(seed=5, n_rows=8, n_features=N_FEAT, n_rounds=n_rounds, pack_size=32, depth=6)
    feature, threshold, leaf = w.extra["feature"], w.extra["threshold"], w.extra["leaf"]
    T, n_int = feature.shape
    idx = np.arange(n_int, dtype=np.uint32)   # heap order: children of node i are 2i+1 and 2i+2
    w0 = np.concatenate([(feature.astype(np.uint32) & 0xFFFF) | (threshold.astype(np.uint32) << 16),
                         np.full(leaf.shape, 1 << 31, np.uint32)], axis=1)
    w1 = np.concatenate([np.broadcast_to(2 * idx + 1, (T, n_int)), leaf.view(np.uint32)], axis=1)
    per_tree = w0.shape[1]
    packed = torch.from_numpy(np.stack([w0, w1], axis=2).reshape(-1, 2).view(np.int32).copy()).to(dev)
    offs = torch.arange(T + 1, dtype=torch.int32, device=dev) * per_tree
    g = torch.Generator(device=dev)
    g.manual_seed(1)
    X = torch.randint(0, 5, (n_rows, N_FEAT), generator=g, device=dev, dtype=torch.uint8)
    rows = pack_row_major(X, None, 5)
    out = torch.empty(n_rows, dtype=torch.float32, device=dev)
    lib = B.lib()

    def run():
        B.check(lib.pb_predict_rows_packed(rows.codes.data_ptr(), n_rows, rows.pitch_row, rows.code_bits,
                                           packed.data_ptr(), offs.data_ptr(), 0, T, per_tree, 1.0, out.data_ptr(), 0,
                                           torch.cuda.current_stream().cuda_stream))
    for _ in range(warmup):
        run()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        run()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    print(json.dumps({"metric": "predictor_node_visits_per_sec", "value": n_rows * T * 6 / (ms / 1000.0), "unit": "visits/s",
                      "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True,
                      "dtype": "f32", "data": "synthetic",
                      "config": {"workload": f"ensemble inference: {n_rows} rows x {N_FEAT} five-level features, "
                                             f"{T} complete depth-6 trees"},
                      "rows_per_sec": n_rows / (ms / 1000.0)}))


# ---------------------------------------------------------------------------------------------

def model_digest(booster, preds):
    """sha256 over the distinct trees' (feature, threshold, left, right) arrays and the raw bytes of
    the training predictions: equal digests mean the same model bit for bit."""
    import hashlib
    h = hashlib.sha256()
    booster.trees  # materialise the last round
    for tree, _rep in booster._distinct:
        a = tree.arrays()
        for k in ("feature", "threshold", "left", "right"):
            h.update(np.ascontiguousarray(a[k]).tobytes())
    h.update(np.ascontiguousarray(preds).tobytes())
    return h.hexdigest()[:24]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="packboost_b200", choices=["packboost_b200", "reference"])
    ap.add_argument("--scale", type=float, default=1.0, help="row/era scale of the workload (profiling captures use < 1)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--predict", type=int, nargs=2, metavar=("ROWS", "ROUNDS"),
                    help="time the ensemble predictor instead: ROWS rows x 2376 five-level features scored by "
                         "ROUNDS x 32 complete depth-6 trees (the inference-only workload is 5 000 000 x 2000)")
    args = ap.parse_args()
    if args.predict:
        predict_bench(args.predict[0], args.predict[1], args.steps, args.warmup)
        return

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    n_eras = max(2, int(round(N_ERAS * args.scale)))
    n_rows = int(N_ROWS * args.scale) // n_eras * n_eras
    n_feat = N_FEAT
    config = {"workload": workload_name(n_rows, n_feat, n_eras), "parallelism": f"feature-sharded x{world}",
              "trees": "the 32 trees of a pack are identical in the reference (no per-tree randomness; it de-duplicates "
                       "the nodes): one tree is grown per round and recorded 32 times, on both arms",
              "l2": "inputs larger than L2 (packed matrix 3.2 GB at full size); no flush needed",
              "scale": args.scale}

    if args.impl == "reference":
        if rank != 0:
            return
        from oracle import native_ref
        cores = os.cpu_count() or 1
        se = pick_sample_eras(args.steps, args.warmup, n_eras)
        sizes = cpu_baseline_two_sizes(n_rows, n_feat, n_eras, se, args.steps, args.warmup, "port")
        rps = sizes[-1]["extrapolated_rounds_per_sec"]
        sample = (f"CPU port of the reference torch frontier (oracle/): {args.steps} timed rounds on the first "
                  f"{sizes[-1]['eras']} of {n_eras} eras ({sizes[-1]['rows']} rows x {n_feat} features), rounds/s scaled "
                  f"by eras; the half-size sample is timed too (samples)")
        native = None
        if native_ref.available():
            nsz = cpu_baseline_two_sizes(n_rows, n_feat, n_eras, se, min(args.steps, 3), 1, "native")
            native = {"value": nsz[-1]["extrapolated_rounds_per_sec"], "unit": UNIT, "cores": cores, "kind": "reference",
                      "sample": "the reference's compiled C++/OpenMP split finder (oracle/_ref) on the same era samples",
                      "samples": nsz}
        line = {"impl": "reference", "metric": METRIC, "value": rps, "unit": UNIT, "n_gpus": args.gpus,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1000.0 / rps, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config,
                "cpu_baseline": {"value": rps, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample,
                                 "samples": sizes},
                "cpu_baseline_native": native,
                "e2e": {"value": rps, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return

    import torch
    import torch.distributed as dist
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    from packboost_b200 import PackBoost, PackBoostConfig
    from packboost_b200 import backends as B
    lib = B.lib()

    X, y, era = make_device_data(n_rows, n_feat, n_eras, dev)
    y_host = y.cpu().numpy()
    era_host = era.cpu().numpy()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v):
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def set_layout(sharded):
        if sharded:
            os.environ["PACKBOOST_SHARD_CODES"] = "1"
        else:
            os.environ.pop("PACKBOOST_SHARD_CODES", None)

    # ---- device-resident leg ------------------------------------------------------------------
    def resident_leg(sharded, profile):
        """K rounds of the device-resident loop exactly as fit() runs it (CUDA events, max over
        ranks); with `profile` a second pass of K rounds with the round graph off and CUDA events
        around every launch of a kernel family."""
        set_layout(sharded)
        booster = PackBoost(PackBoostConfig(device="cuda", **CFG))
        booster._start(X, y_host, era_host)
        trainer = booster._trainer
        total = args.warmup + 2 * args.steps
        for r in range(args.warmup):
            booster._boost_one_round(r, total)
        booster._drain()
        barrier()
        sampler = ClockSampler(local_rank)
        if rank == 0 and profile:
            sampler.start()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        launches0 = int(lib.pb_launch_count())
        replays0 = trainer.graph_replays
        barrier()
        ev0.record()
        for r in range(args.warmup, args.warmup + args.steps):
            booster._boost_one_round(r, total)   # enqueues round r, takes in the log of round r - 1
        booster._drain()                         # waits for the last round and its log
        ev1.record()
        barrier()
        ms = max_over_ranks(ev0.elapsed_time(ev1))
        out = {"ms": ms, "value": args.steps / (ms / 1000.0)}
        if not profile:
            set_layout(False)
            return out
        out["clocks"] = sampler.stop() if rank == 0 else None
        # kernels of the timed region: eager launches are counted by the library as they are issued,
        # a replayed round graph holds the number counted while it was captured
        out["launches"] = (int(lib.pb_launch_count()) - launches0
                           + (trainer.graph_replays - replays0) * trainer.graph_launches)
        trainer.enable_profile()    # eager launches, every kernel family bracketed by CUDA events
        logs0 = len(booster._depth_logs)
        barrier()
        for r in range(args.warmup + args.steps, total):
            booster._boost_one_round(r, total)
        booster._drain()
        barrier()
        ms5, n5 = trainer.profile_totals()
        trainer.disable_profile()
        F_s = trainer.n_sampled()
        f_loc = F_s / world
        K = CFG["max_bins"] - 1
        in_bytes = out_bytes = 0.0
        for entry in booster._depth_logs[logs0:]:
            in_bytes += n_rows * f_loc * 0.5 + n_rows * (4 + 2) + (n_eras + 1) * 4
            out_bytes += int(entry["nodes_processed"]) * f_loc * n_eras * K * 8
        out.update(hist_ms=float(ms5[0]), hist_launches=int(n5[0]), in_bytes=in_bytes, out_bytes=out_bytes, F_s=F_s,
                   phases={"hist_ms_per_step": float(ms5[0]) / args.steps, "score_ms_per_step": float(ms5[1]) / args.steps,
                           "select_ms_per_step": float(ms5[2]) / args.steps,
                           "partition_ms_per_step": float(ms5[3]) / args.steps,
                           "round_begin_ms_per_step": float(ms5[4]) / args.steps},
                   log_bytes=trainer.log_bytes)
        set_layout(False)
        return out

    res = resident_leg(False, True)
    res_sharded = resident_leg(True, False) if world > 1 else None
    torch.cuda.empty_cache()

    value, ms = res["value"], res["ms"]
    hist_ms, hist_launches = res["hist_ms"], res["hist_launches"]
    achieved = res["in_bytes"] / (hist_ms / 1000.0) / 1e9 if hist_ms > 0 else 0.0
    achieved_out = (res["in_bytes"] + res["out_bytes"]) / (hist_ms / 1000.0) / 1e9 if hist_ms > 0 else 0.0
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak = float(json.load(open(peaks_path))["hbm_gbs"])
        peak_src = "measured (MEASURED_PEAKS.json hbm_gbs)"
    else:
        peak, peak_src = 6650.0, "fallback"
    traffic, traffic_src = hist_traffic(n_rows, world)

    # ---- end-to-end legs: the public fit() on HOST buffers -----------------------------------------
    F_s = res["F_s"]
    lists_bytes = CFG["max_depth"] * 3 * F_s * 4

    def e2e_leg(X_src, sharded):
        set_layout(sharded)
        barrier()
        t0 = time.perf_counter()
        b2 = PackBoost(PackBoostConfig(device="cuda", **CFG))
        b2.fit(X_src, y_host, era_host, num_rounds=args.steps)
        p = b2.train_predictions()          # device -> host read of the result
        barrier()
        wall = max_over_ranks(time.perf_counter() - t0)
        digest = model_digest(b2, p)
        set_layout(False)
        # whole job: every rank brings over its own strip of columns, together the matrix once
        h2d = (n_rows * n_feat + world * (n_rows * 4 + (n_eras + 1) * 4)) / args.steps + world * lists_bytes
        d2h = world * (b2._trainer.log_bytes + n_rows * 4 / args.steps)
        del b2
        torch.cuda.empty_cache()
        return {"value": args.steps / wall, "unit": UNIT, "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                "seconds": wall}, digest, p

    e2e = e2e_sharded = e2e_numpy = None
    digests = {}
    train_corr = None
    if not args.no_e2e:
        X_host = torch.empty((n_rows, n_feat), dtype=torch.uint8).pin_memory()
        X_host.copy_(X)
        del X
        torch.cuda.empty_cache()
        e2e, digests["model_digest"], p = e2e_leg(X_host, False)
        e2e["note"] = ("whole PackBoost.fit on a page-locked host tensor: packing + one-time matrix upload amortised "
                       "over the timed rounds, per-round feature lists up and decision log down, final predictions down")
        from packboost_b200.booster import _era_correlation_np
        train_corr = _era_correlation_np(era_host, y_host, p)
        if world > 1:
            e2e_sharded, digests["model_digest_sharded"], _ = e2e_leg(X_host, True)
            e2e_sharded["note"] = "the same with each rank holding only its own feature columns (PACKBOOST_SHARD_CODES=1)"
        # the reference's API takes numpy arrays (packboost/booster.py:375-385): the same fit on a
        # pageable array, staged through page-locked buffers by the library
        try:
            import psutil
            room = psutil.virtual_memory().available > 2.5 * n_rows * n_feat * max(world, 1)
        except Exception:
            room = world == 1
        if world > 1:   # every rank takes the same decision (a rank that skipped the leg would leave the others waiting)
            flag = torch.tensor([1 if room else 0], dtype=torch.int32, device=dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            room = bool(int(flag.item()))
        if room:
            X_np = np.empty((n_rows, n_feat), dtype=np.uint8)
            np.copyto(X_np, X_host.numpy())
            del X_host
            import gc
            gc.collect()
            torch.cuda.empty_cache()   # the page-locked copy is released here, not inside the next timed fit
            e2e_numpy, digests["model_digest_numpy"], _ = e2e_leg(X_np, False)
            e2e_numpy["note"] = "the same fit on a pageable numpy array (the input type of the reference's API)"
            del X_np

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    cpu_baseline = cpu_native = None
    if world == 1 and not args.no_cpu:
        from oracle import native_ref
        cores = os.cpu_count() or 1
        sizes = cpu_baseline_two_sizes(n_rows, n_feat, n_eras, 32, 2, 1, "port")   # ~15 s of CPU work
        cpu_baseline = {"value": sizes[-1]["extrapolated_rounds_per_sec"], "unit": UNIT, "cores": cores, "kind": "port",
                        "sample": f"2 timed rounds (1 warm-up) of the oracle's restatement of the reference torch frontier "
                                  f"on the first 16 and the first 32 of {n_eras} eras ({n_feat} features), rounds/s scaled "
                                  f"by eras (both extrapolations in samples)",
                        "samples": sizes}
        if native_ref.available():
            nsz = cpu_baseline_two_sizes(n_rows, n_feat, n_eras, 32, 2, 1, "native")
            cpu_native = {"value": nsz[-1]["extrapolated_rounds_per_sec"], "unit": UNIT, "cores": cores,
                          "kind": "reference",
                          "sample": "the reference's own compiled C++/OpenMP split finder (oracle/_ref) on the same samples",
                          "samples": nsz}

    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "int64", "data": "synthetic", "config": config,
            "roofline": {"bound": "hbm", "kernel": "hist_lane_kernel (fused flush)", "achieved": achieved, "peak": peak,
                         "unit": "GB/s", "frac": achieved / peak, "traffic": traffic, "traffic_source": traffic_src,
                         "peak_source": peak_src,
                         "bytes": "input bytes only (packed codes of the sampled columns, row state, era offsets): the "
                                  "histogram is never stored (fused flush), so its term is 0; achieved_with_output also "
                                  "counts the (gain, weight) rows the kernel writes instead",
                         "achieved_with_output": achieved_out, "frac_with_output": achieved_out / peak,
                         "timing": "CUDA events around every launch in a second pass of the same number of rounds "
                                   "with the round graph off",
                         "launches": hist_launches, "avg_launch_ms": hist_ms / max(hist_launches, 1),
                         "algorithmic_bytes_per_launch": res["in_bytes"] / max(hist_launches, 1)},
            "cpu_baseline": cpu_baseline, "cpu_baseline_native": cpu_native,
            "e2e": e2e, "e2e_sharded": e2e_sharded, "e2e_numpy": e2e_numpy,
            "value_sharded": res_sharded["value"] if res_sharded else None,
            "gpu_launches": res["launches"], "clocks": res["clocks"], "phases": res["phases"],
            "train_corr_after_e2e": train_corr}
    line.update(digests)
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def source_digest(path):
    """sha256 of a C++/CUDA source without its // comments and blank lines, so that editing a
    comment does not look like a kernel change."""
    import hashlib
    import re
    lines = []
    for line in open(path, encoding="utf-8"):
        code = re.sub(r"//.*$", "", line).strip()
        if code:
            lines.append(code)
    return hashlib.sha256("\n".join(lines).encode()).hexdigest()


def hist_traffic(n_rows, world):
    """DRAM bytes per histogram launch from the committed ncu summary of the kernel that is timed
    (read + written at the captured row count, scaled by rows: the traffic is proportional to rows x
    sampled features).  The summary records the sha256 of the kernel source it was taken from
    (comments and blank lines left out, see source_digest); when the code has changed since, the
    figure is withheld and the reason is given instead."""
    import hashlib
    import re
    path = os.path.join(ROOT, "profiles", "hist_lane_kernel_fused_config3_small.md")
    src = os.path.join(ROOT, "packboost_b200", "csrc", "hist.cu")
    if not os.path.exists(path):
        return None, "no ncu summary of the fused kernel is committed"
    text = open(path).read()
    m_bytes = re.search(r"dram_bytes_per_launch:\s*([0-9.eE+]+)", text)
    m_rows = re.search(r"captured_rows:\s*([0-9]+)", text)
    m_sha = re.search(r"hist_cu_sha256:\s*([0-9a-f]+)", text)
    if not (m_bytes and m_rows and m_sha):
        return None, "the committed ncu summary lacks the traffic fields"
    now = source_digest(src)
    if not now.startswith(m_sha.group(1)):
        return None, "hist.cu has changed since the committed ncu capture: traffic withheld until it is re-captured"
    return float(m_bytes.group(1)) * n_rows / float(m_rows.group(1)) / world, \
        "ncu dram__bytes_read+write of the committed small-case capture of this kernel source, scaled by rows"


if __name__ == "__main__":
    main()
