"""Direct drivers of single kernels of the native library on caller-supplied tensors.

They back the helper methods the reference booster exposes for its own tests
(``PackBoost._batched_histograms_nodes``, ``packboost/booster.py:933-977``) and the
kernel-level parity tests; the training loop does not use them.
"""

from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import backends as B
from .data import pack_feature_major


def _fixed_point(values: torch.Tensor, bits: int) -> tuple[torch.Tensor, float]:
    """``rint(values * scale)`` as int32 with ``scale`` the power of two that keeps every entry
    below ``2**bits`` in magnitude; returns the integers and ``1 / scale``."""
    m = float(values.abs().max().item()) if values.numel() else 0.0
    if not (m > 0.0) or not np.isfinite(m):
        return torch.zeros_like(values, dtype=torch.int32), 1.0
    _, ex = np.frexp(m)
    sh = int(bits - ex)
    q = torch.round(values.to(torch.float64) * (2.0 ** sh)).to(torch.int32)
    return q, 2.0 ** (-sh)


def histograms_nodes(bins_matrix: torch.Tensor, grad_rows: torch.Tensor, hess_rows: torch.Tensor,
                     era_ids: torch.Tensor, node_ids: torch.Tensor, num_nodes: int, num_eras: int,
                     num_bins: int) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Counts (int64) and float32 gradient / hessian sums per ``[feature, node, era, bin]`` of the
    rows given (``bins_matrix`` is ``[rows, features]``), built by the histogram kernel: rows are
    ordered by era, packed feature-major, and the kernel runs once with the gradients and once with
    the hessians as its fixed-point addend.  Sums are exact in fixed point and converted once."""
    dev = torch.device("cuda", torch.cuda.current_device())
    R, F = int(bins_matrix.shape[0]), int(bins_matrix.shape[1])
    if R == 0 or F == 0:
        z = torch.zeros((F, num_nodes, num_eras, num_bins), device=dev)
        return z.to(torch.int64), z.to(torch.float32), z.to(torch.float32)
    cnt, sums = histograms_raw(bins_matrix, [grad_rows, hess_rows], era_ids, node_ids, num_nodes, num_eras, num_bins)
    out = [(q.to(torch.float64) * inv).to(torch.float32).permute(0, 2, 1, 3).contiguous() for q, inv in sums]
    return cnt.to(torch.int64).permute(0, 2, 1, 3).contiguous(), out[0], out[1]


def histograms_raw(bins_matrix: torch.Tensor, addends: list[torch.Tensor], era_ids: torch.Tensor,
                   node_ids: torch.Tensor, num_nodes: int, num_eras: int, num_bins: int):
    """``(cnt int32 [F, E, nodes, bins], [(sum int64 [F, E, nodes, bins], inv_scale), ...])``: one
    histogram pass per per-row addend, each quantised to fixed point with its own power-of-two
    scale (``sum * inv_scale`` is the float sum)."""
    lib = B.lib()
    dev = torch.device("cuda", torch.cuda.current_device())
    R, F = int(bins_matrix.shape[0]), int(bins_matrix.shape[1])
    if num_nodes > 65534:
        raise ValueError("too many nodes")
    era = era_ids.to(dev).to(torch.int64)
    order = torch.sort(era, stable=True).indices
    codes_src = bins_matrix.to(dev).index_select(0, order).to(torch.uint8).contiguous()
    matrix = pack_feature_major(codes_src, None, num_bins)
    counts_e = torch.bincount(era, minlength=num_eras)[:num_eras]
    era_offsets = torch.cat([torch.zeros(1, dtype=torch.int64, device=dev), counts_e.cumsum(0)]).to(torch.int32)
    npad = matrix.rows_padded
    slot = torch.full((npad,), -1, dtype=torch.int16, device=dev)
    slot[:R] = node_ids.to(dev).index_select(0, order).to(torch.int16)
    dummy_f = torch.zeros(R, dtype=torch.float32, device=dev)
    leaf = torch.zeros(npad, dtype=torch.int16, device=dev)
    gq = torch.zeros(npad, dtype=torch.int32, device=dev)
    thr = torch.arange(max(num_bins - 1, 1), dtype=torch.int32, device=dev)
    feat_local = torch.arange(F, dtype=torch.int32, device=dev)
    ctl = torch.zeros(int(lib.pb_ctl_bytes()), dtype=torch.uint8, device=dev)

    st = B.TrainState()
    st.n_rows, st.n_features_total, st.n_features_local, st.n_eras = R, F, F, num_eras
    st.max_bins, st.code_bits, st.pitch = num_bins, matrix.code_bits, matrix.pitch
    st.max_depth, st.pack_size, st.min_samples_leaf = 1, 1, 1
    st.n_thresholds, st.feature_block_size = max(num_bins - 1, 1), 32
    st.lambda_l2, st.learning_rate = 1.0, 1.0
    st.codes, st.era_offsets, st.thr_ids = matrix.codes.data_ptr(), era_offsets.data_ptr(), thr.data_ptr()
    st.feat_local, st.y, st.preds = feat_local.data_ptr(), dummy_f.data_ptr(), dummy_f.data_ptr()
    st.gq, st.slot, st.leaf, st.ctl = gq.data_ptr(), slot.data_ptr(), leaf.data_ptr(), ctl.data_ptr()
    st.workspace, st.workspace_bytes = None, 0
    eo_host = era_offsets.cpu().numpy().astype(np.int32)
    B.check(lib.pb_train_prepare(C.byref(st), eo_host.ctypes.data))

    feats = torch.arange(F, dtype=torch.int32, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    cells = (F, num_eras, num_nodes, num_bins)
    out = []
    cnt = torch.empty(cells, dtype=torch.int32, device=dev)
    for values in addends:
        q, inv = _fixed_point(values.to(dev).to(torch.float32).index_select(0, order), int(st.gq_bits))
        gq[:R] = q
        gsum = torch.empty(cells, dtype=torch.int64, device=dev)
        B.check(lib.pb_hist_build(C.byref(st), feats.data_ptr(), F, num_nodes, num_nodes, cnt.data_ptr(),
                                  gsum.data_ptr(), stream))
        out.append((gsum, inv))
    torch.cuda.current_stream().synchronize()   # (the temporaries above are released after the kernels ran)
    return cnt, out


_SPLIT_DT = np.dtype([("score", "<f4"), ("k", "<i4"), ("threshold", "<i4"), ("has_nan", "<i4"),
                      ("left_count", "<i8"), ("left_gq", "<i8"), ("left_hq", "<i8")])


def best_split_one_node(codes: torch.Tensor, grad: torch.Tensor, hess: torch.Tensor, era_ids: torch.Tensor,
                        features: np.ndarray, num_eras: int, *, max_bins: int, thr_ids: np.ndarray, lambda_l2: float,
                        lambda_dro: float, direction_weight: float, era_alpha: float, direction_form: int,
                        min_samples_leaf: int, feature_block_size: int) -> dict | None:
    """Best split of one node whose rows are given (``codes`` is ``[rows, len(features)]``), with
    arbitrary per-row hessians: histograms by the histogram kernel (gradients and hessians as
    fixed-point addends), per-feature best thresholds by ``pb_score_node_general``, then the
    reference's order over the features (inside a block of ``feature_block_size`` sampled features:
    score, left count, later position; across blocks: score, left count, feature id, threshold;
    ``packboost/booster.py:1912-1981``).  Returns the fields of a ``SplitDecision`` or ``None``."""
    lib = B.lib()
    dev = torch.device("cuda", torch.cuda.current_device())
    R, F = int(codes.shape[0]), int(codes.shape[1])
    if R < 2 * min_samples_leaf or F == 0:
        return None
    node_ids = torch.zeros(R, dtype=torch.int64, device=dev)
    cnt, sums = histograms_raw(codes, [grad, hess], era_ids, node_ids, 1, num_eras, max_bins)
    (gsum, inv_g), (hsum, inv_h) = sums
    total_gq = int(gsum[0].sum().item())
    total_hq = int(hsum[0].sum().item())
    thr_t = torch.from_numpy(np.ascontiguousarray(thr_ids, dtype=np.int32)).to(dev)
    out = torch.zeros(F * _SPLIT_DT.itemsize, dtype=torch.uint8, device=dev)
    B.check(lib.pb_score_node_general(cnt.data_ptr(), gsum.data_ptr(), hsum.data_ptr(), F, num_eras, max_bins,
                                      thr_t.data_ptr(), int(thr_t.numel()), float(inv_g), float(inv_h), float(lambda_l2),
                                      float(lambda_dro), float(direction_weight), float(era_alpha), int(direction_form),
                                      int(min_samples_leaf), R, total_gq, out.data_ptr(),
                                      torch.cuda.current_stream().cuda_stream))
    rec = out.cpu().numpy().view(_SPLIT_DT)
    blk = feature_block_size if 0 < feature_block_size <= F else F
    best = None   # (score, left_count, feature, threshold, position)
    for b0 in range(0, F, blk):
        inblk = None
        if rec["has_nan"][b0:b0 + blk].any():
            continue   # a NaN score voids the block's maximum, as torch.max does
        for p in range(b0, min(F, b0 + blk)):
            r = rec[p]
            if r["k"] < 0:
                continue
            key = (float(r["score"]), int(r["left_count"]), p)
            if inblk is None or key[:2] > inblk[0][:2] or (key[:2] == inblk[0][:2] and p > inblk[0][2]):
                inblk = (key, p)
        if inblk is None:
            continue
        p = inblk[1]
        cand = (float(rec[p]["score"]), int(rec[p]["left_count"]), int(features[p]), int(rec[p]["threshold"]), p)
        if best is None or cand[:4] > best[:4]:
            best = cand
    if best is None:
        return None
    p = best[4]
    f32 = np.float32
    lg = f32(f32(int(rec[p]["left_gq"])) * f32(inv_g))
    lh = f32(f32(int(rec[p]["left_hq"])) * f32(inv_h))
    tg = f32(f32(total_gq) * f32(inv_g))
    th = f32(f32(total_hq) * f32(inv_h))
    return {"feature": best[2], "threshold": best[3], "score": best[0], "left_grad": float(lg), "left_hess": float(lh),
            "right_grad": float(tg) - float(lg), "right_hess": float(th) - float(lh), "left_count": best[1],
            "right_count": R - best[1]}
