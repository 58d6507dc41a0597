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
    lib = B.lib()
    dev = torch.device("cuda", torch.cuda.current_device())
    R, F = int(bins_matrix.shape[0]), int(bins_matrix.shape[1])
    if R == 0 or F == 0:
        z = torch.zeros((F, num_nodes, num_eras, num_bins), device=dev)
        return z.to(torch.int64), z.to(torch.float32), z.to(torch.float32)
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
    for values in (grad_rows, hess_rows):
        q, inv = _fixed_point(values.to(dev).to(torch.float32).index_select(0, order), int(st.gq_bits))
        gq[:R] = q
        gsum = torch.empty(cells, dtype=torch.int64, device=dev)
        B.check(lib.pb_hist_build(C.byref(st), feats.data_ptr(), F, num_nodes, num_nodes, cnt.data_ptr(),
                                  gsum.data_ptr(), stream))
        out.append((gsum.to(torch.float64) * inv).to(torch.float32).permute(0, 2, 1, 3).contiguous())
    counts = cnt.to(torch.int64).permute(0, 2, 1, 3).contiguous()
    return counts, out[0], out[1]
