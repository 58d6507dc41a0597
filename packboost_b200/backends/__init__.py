"""Native backend boundary: ``libpackboost_b200.so`` loaded with ctypes.

The module keeps the seven dispatch names of the reference plugin boundary
(``packboost/backends/__init__.py:10-18``): ``cpu_available``,
``find_best_splits_batched``, ``cuda_available``,
``find_best_splits_batched_cuda``, ``partition_frontier_cuda``,
``predict_bins_cuda`` and ``predict_pack_cuda``.  The two predictors keep
their argument lists and return values.  The two frontier calls are superseded:
the training loop no longer ships row-index lists to the device, it drives the
phase entry points (``lib().pb_round_begin`` ...) on a device-resident
row -> node map, so those names raise a ``RuntimeError`` that says so.

There is no CPU implementation behind this module: without the shared library
or without a CUDA device every compute entry point raises.
"""

from __future__ import annotations

import ctypes as C
import os
from typing import Any

__all__ = [
    "cpu_available",
    "find_best_splits_batched",
    "cuda_available",
    "find_best_splits_batched_cuda",
    "partition_frontier_cuda",
    "predict_bins_cuda",
    "predict_pack_cuda",
    "lib",
    "TrainState",
    "check",
]

# PACKBOOST_DEBUG_LIB=1 loads the build with index checks compiled in (python -m packboost_b200.build --debug-bounds)
_LIB_PATH = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))),
                         "libpackboost_b200_dbg.so" if os.getenv("PACKBOOST_DEBUG_LIB") == "1" else "libpackboost_b200.so")
_LIB: C.CDLL | None = None
_LOAD_ERROR: str | None = None

PB_MAX_DEPTH = 12
SLOT_NONE = 0xFFFF

i64 = C.c_int64
vp = C.c_void_p


class TrainState(C.Structure):
    """Mirror of ``pb_train_state`` (include/packboost_b200.h): every field is 8 bytes."""

    _fields_ = [
        ("n_rows", i64), ("n_features_total", i64), ("n_features_local", i64), ("n_eras", i64),
        ("max_bins", i64), ("code_bits", i64), ("pitch", i64),
        ("max_depth", i64), ("pack_size", i64), ("min_samples_leaf", i64), ("n_thresholds", i64),
        ("feature_block_size", i64),
        ("lambda_l2", C.c_double), ("lambda_dro", C.c_double), ("direction_weight", C.c_double),
        ("era_alpha", C.c_double), ("learning_rate", C.c_double),
        ("codes", vp), ("era_offsets", vp), ("thr_ids", vp), ("feat_local", vp), ("y", vp),
        ("preds", vp), ("gq", vp), ("slot", vp), ("leaf", vp), ("ctl", vp), ("workspace", vp),
        ("workspace_bytes", i64),
        ("max_era_rows", i64), ("hist_rows_per_tile", i64), ("gq_bits", i64), ("count_bits", i64),
        ("lo_bits", i64), ("cut_mass", i64), ("profile", vp), ("direction_form", i64),
    ]


_PROTOS: dict[str, tuple[Any, list[Any]]] = {
    "pb_last_error": (C.c_char_p, []),
    "pb_abi_version": (C.c_int, []),
    "pb_device_count": (C.c_int, []),
    "pb_profile_create": (vp, []),
    "pb_profile_destroy": (None, [vp]),
    "pb_profile_collect": (C.c_int, [vp, vp, vp]),
    "pb_profile_collect_launches": (C.c_int, [vp, vp, vp, i64, vp]),
    "pb_launch_count": (i64, []),
    "pb_debug_bounds_enabled": (C.c_int, []),
    "pb_debug_flags": (C.c_int, [C.POINTER(TrainState), vp]),
    "pb_bin_pack_f32": (C.c_int, [vp, i64, i64, i64, vp, i64, i64, vp, vp, i64, i64, vp]),
    "pb_pack_codes_u8": (C.c_int, [vp, i64, i64, i64, vp, vp, i64, i64, vp]),
    "pb_pack_rows": (C.c_int, [vp, i64, i64, i64, vp, i64, i64, vp, i64, i64, vp]),
    "pb_train_state_bytes": (i64, []),
    "pb_ctl_bytes": (i64, []),
    "pb_workspace_min_bytes": (i64, [C.POINTER(TrainState)]),
    "pb_train_prepare": (C.c_int, [C.POINTER(TrainState), vp]),
    "pb_round_begin": (C.c_int, [C.POINTER(TrainState), i64, vp]),
    "pb_depth_hist_score": (C.c_int, [C.POINTER(TrainState), i64, vp, vp, i64, i64, vp]),
    "pb_static_scratch_bytes": (i64, []),
    "pb_depth_hist_score_static": (C.c_int, [C.POINTER(TrainState), i64, vp, vp, i64, i64, vp, vp]),
    "pb_candidates_buffer": (C.c_int, [C.POINTER(TrainState), i64, i64, C.POINTER(vp), C.POINTER(i64)]),
    "pb_depth_clear_candidates": (C.c_int, [C.POINTER(TrainState), i64, i64, vp]),
    "pb_depth_select": (C.c_int, [C.POINTER(TrainState), i64, vp, i64, vp]),
    "pb_depth_select_cand": (C.c_int, [C.POINTER(TrainState), i64, vp, i64, vp, vp]),
    "pb_depth_partition": (C.c_int, [C.POINTER(TrainState), i64, vp]),
    "pb_depth_goleft_bits": (C.c_int, [C.POINTER(TrainState), i64, vp, vp]),
    "pb_depth_apply_bits": (C.c_int, [C.POINTER(TrainState), i64, vp, vp]),
    "pb_comm_unique_id": (C.c_int, [vp]),
    "pb_comm_init": (C.c_int, [C.POINTER(vp), vp, i64, i64]),
    "pb_comm_allreduce_candidates": (C.c_int, [vp, C.POINTER(TrainState), i64, i64, vp]),
    "pb_comm_allreduce_mask": (C.c_int, [vp, vp, i64, vp]),
    "pb_comm_destroy": (C.c_int, [vp]),
    "pb_round_end": (C.c_int, [C.POINTER(TrainState), vp]),
    "pb_apply_leaf_delta": (C.c_int, [C.POINTER(TrainState), vp]),
    "pb_era_correlation": (C.c_int, [vp, vp, vp, i64, vp, vp]),
    "pb_round_log_buffer": (C.c_int, [C.POINTER(TrainState), C.POINTER(vp), C.POINTER(i64)]),
    "pb_hist_build": (C.c_int, [C.POINTER(TrainState), vp, i64, i64, i64, vp, vp, vp]),
    "pb_score_node_general": (C.c_int, [vp, vp, vp, i64, i64, i64, vp, i64, C.c_float, C.c_float, C.c_float, C.c_float,
                                        C.c_float, C.c_float, i64, i64, i64, i64, vp, vp]),
    "pb_predict_rows": (C.c_int, [vp, i64, i64, i64, vp, vp, vp, vp, vp, vp, vp, vp, i64, C.c_float, vp, vp, vp]),
    "pb_predict_rows_packed": (C.c_int, [vp, i64, i64, i64, vp, vp, vp, i64, i64, C.c_float, vp, vp, vp]),
    "pb_predict_bins_fm": (C.c_int, [vp, i64, i64, vp, vp, vp, vp, vp, vp, i64, vp, vp]),
    "pb_predict_pack_fm": (C.c_int, [vp, i64, i64, vp, vp, vp, vp, vp, vp, vp, i64, C.c_float, vp, vp]),
}

EXPORTED_SYMBOLS = tuple(_PROTOS)


def library_path() -> str:
    return _LIB_PATH


def lib() -> C.CDLL:
    """The loaded shared library; raises if it has not been built."""
    global _LIB, _LOAD_ERROR
    if _LIB is not None:
        return _LIB
    if not os.path.exists(_LIB_PATH):
        _LOAD_ERROR = f"{_LIB_PATH} is missing; build it with `python -m packboost_b200.build`"
        raise RuntimeError("Native backend is not built: " + _LOAD_ERROR)
    handle = C.CDLL(_LIB_PATH)
    for name, (res, args) in _PROTOS.items():
        fn = getattr(handle, name)
        fn.restype = res
        fn.argtypes = args
    if handle.pb_abi_version() != 1 or handle.pb_train_state_bytes() != C.sizeof(TrainState):
        raise RuntimeError("libpackboost_b200.so ABI mismatch; rebuild it with `python -m packboost_b200.build`")
    _LIB = handle
    return handle


def check(rc: int) -> None:
    """Turn a negative status into the exception the reference's callers expect:
    messages of failed CUDA calls start with ``CUDA error`` (the reference's
    booster matches on that text, ``packboost/booster.py:1611-1613``)."""
    if rc == 0:
        return
    msg = lib().pb_last_error().decode("utf-8", "replace")
    if rc == -1:
        raise ValueError(msg)
    raise RuntimeError(msg)


def _stream() -> int:
    import torch
    return torch.cuda.current_stream().cuda_stream


def _ptr(t) -> int:
    return t.data_ptr() if t is not None else 0


# ------------------------------ CPU API ---------------------------------


def cpu_available() -> bool:
    """The reference's optional OpenMP split finder has no counterpart here."""
    return False


def find_best_splits_batched(*args: Any, **kwargs: Any):
    raise RuntimeError("CPU backend is unavailable in this build.")


# ------------------------------ CUDA API --------------------------------


def cuda_available() -> bool:
    """True when the library loads and a compute-capability-10.x device is visible."""
    try:
        return lib().pb_device_count() > 0
    except Exception:
        return False


_SUPERSEDED = (
    "{name} is superseded in the B200 backend: training runs on a device-resident row->node map through "
    "pb_round_begin / pb_depth_hist_score / pb_depth_select / pb_depth_partition (see include/packboost_b200.h)."
)


def find_best_splits_batched_cuda(*args: Any, **kwargs: Any):
    raise RuntimeError(_SUPERSEDED.format(name="find_best_splits_batched_cuda"))


def partition_frontier_cuda(*args: Any, **kwargs: Any):
    raise RuntimeError(_SUPERSEDED.format(name="partition_frontier_cuda"))


def _need_cuda(*tensors) -> None:
    for t in tensors:
        if t.device.type != "cuda":
            raise RuntimeError("CUDA predict needs tensors on a CUDA device")
        if not t.is_contiguous():
            raise ValueError("tensors must be contiguous")


def predict_bins_cuda(bins_fm, feature, threshold, left, right, value, is_leaf):
    """One tree over feature-major ``uint8 [F, N]`` codes -> ``float32 [N]`` leaf values
    (argument list of ``predict_bins_cuda``, ``packboost/backends/cuda/frontier_cuda.cu:853-861``)."""
    import torch
    if bins_fm.dim() != 2:
        raise ValueError("bins must be 2D [F, N]")
    bins_fm = bins_fm.to(torch.uint8)
    feature, threshold, left, right = (t.to(torch.int32).contiguous() for t in (feature, threshold, left, right))
    value = value.to(torch.float32).contiguous()
    is_leaf = is_leaf.to(torch.uint8).contiguous()
    _need_cuda(bins_fm, feature, threshold, left, right, value, is_leaf)
    F, N = bins_fm.shape
    from ..forest import validate_forest
    validate_forest(feature.cpu().numpy(), threshold.cpu().numpy(), left.cpu().numpy(), right.cpu().numpy(),
                    is_leaf.cpu().numpy(), [0, feature.numel()], n_features=F)
    out = torch.empty(N, dtype=torch.float32, device=bins_fm.device)
    check(lib().pb_predict_bins_fm(_ptr(bins_fm), F, N, _ptr(feature), _ptr(threshold), _ptr(left), _ptr(right),
                                   _ptr(value), _ptr(is_leaf), feature.numel(), _ptr(out), _stream()))
    return out


def predict_pack_cuda(bins_fm, feature, threshold, left_abs, right_abs, value, is_leaf, offsets, tree_weight):
    """One pack over feature-major ``uint8 [F, N]`` codes -> ``tree_weight * sum_t leaf_t``
    (argument list of ``predict_pack_cuda``, ``packboost/backends/cuda/frontier_cuda.cu:989-999``)."""
    import torch
    if bins_fm.dim() != 2:
        raise ValueError("bins must be 2D [F, N]")
    bins_fm = bins_fm.to(torch.uint8)
    feature, threshold, left_abs, right_abs, offsets = (
        t.to(torch.int32).contiguous() for t in (feature, threshold, left_abs, right_abs, offsets))
    value = value.to(torch.float32).contiguous()
    is_leaf = is_leaf.to(torch.uint8).contiguous()
    _need_cuda(bins_fm, feature, threshold, left_abs, right_abs, value, is_leaf, offsets)
    F, N = bins_fm.shape
    from ..forest import validate_forest
    validate_forest(feature.cpu().numpy(), threshold.cpu().numpy(), left_abs.cpu().numpy(), right_abs.cpu().numpy(),
                    is_leaf.cpu().numpy(), offsets.cpu().numpy(), n_features=F, absolute_children=True)
    out = torch.empty(N, dtype=torch.float32, device=bins_fm.device)
    check(lib().pb_predict_pack_fm(_ptr(bins_fm), F, N, _ptr(feature), _ptr(threshold), _ptr(left_abs),
                                   _ptr(right_abs), _ptr(value), _ptr(is_leaf), _ptr(offsets), offsets.numel() - 1,
                                   float(tree_weight), _ptr(out), _stream()))
    return out
