"""Binning and bit-packing of features for the B200 backend.

Host-facing names follow the reference's data utilities
(``packboost/data.py``): ``BinningResult``, ``detect_prebinned``,
``quantile_bin``, ``preprocess_features``, ``apply_bins``, ``build_era_index``.
The code assignment (``searchsorted`` against the per-feature edges) and the
packing into 4-bit / 8-bit lanes run on the device; the quantile edges
themselves are order statistics interpolated in float64 by ``np.quantile``,
exactly as the reference computes them, so that bin codes are bit-identical.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Iterable, Sequence

import numpy as np
import torch

from . import backends as B


@dataclass(slots=True)
class BinningResult:
    """Preprocessed training data (``packboost/data.py:12-18``).  ``bins`` is only
    materialised on request; training keeps the packed device matrix instead."""

    bins: np.ndarray | None
    bin_edges: np.ndarray | None
    prebinned: bool


def ensure_numpy(array) -> np.ndarray:
    if isinstance(array, np.ndarray):
        return array
    if isinstance(array, torch.Tensor):
        return array.detach().cpu().numpy()
    return np.asarray(array)


def detect_prebinned(X: np.ndarray, max_bins: int) -> bool:
    """Integer input whose values already are bin ids (``packboost/data.py:32-42``)."""
    if not np.issubdtype(X.dtype, np.integer):
        return False
    if X.size and X.min() < 0:
        return False
    top = int(X.max()) if X.size else 0
    if top >= max_bins:
        return False
    return top <= 127


def quantile_edges(X: np.ndarray, max_bins: int) -> np.ndarray:
    """``[max_bins-1, F]`` float32 edges at the interior quantiles (``packboost/data.py:49-50``)."""
    q = np.linspace(0.0, 1.0, max_bins + 1, dtype=np.float64)[1:-1]
    return np.quantile(X, q, axis=0, method="linear").astype(np.float32)


def edges_from_sorted(sorted_cols: torch.Tensor, max_bins: int) -> np.ndarray:
    """Interior quantile edges of columns that are already sorted ascending (NaN last), with the
    arithmetic of ``np.quantile(..., method="linear")`` step for step: virtual index
    ``(n - 1) * q`` in float64, the two neighbours taken from the float32 column, their float32
    difference, then ``a + d * t`` (``b - d * (1 - t)`` where ``t >= 0.5``) in float64.  A column
    that holds a NaN gets NaN edges.  Only the two gathers touch the big array; the interpolation
    runs on the host on ``2 * (max_bins - 1) * F`` numbers.  ``float64 [max_bins - 1, F]``."""
    n = int(sorted_cols.shape[0])
    q = np.linspace(0.0, 1.0, max_bins + 1, dtype=np.float64)[1:-1]
    virtual = (n - 1) * q
    prev = np.floor(virtual).astype(np.int64)
    nxt = prev + 1
    above = virtual >= n - 1
    prev[above] = n - 1
    nxt[above] = n - 1
    below = virtual < 0
    prev[below] = 0
    nxt[below] = 0
    dev = sorted_cols.device
    a = sorted_cols[torch.from_numpy(prev).to(dev)].cpu().numpy()
    b = sorted_cols[torch.from_numpy(nxt).to(dev)].cpu().numpy()
    has_nan = torch.isnan(sorted_cols[-1]).cpu().numpy()
    t = (virtual - prev).reshape(-1, 1)
    d = np.subtract(b, a)                      # float32, as in numpy's _lerp
    with np.errstate(invalid="ignore"):
        out = np.add(a, d * t)
        np.subtract(b, d * (1 - t), out=out, where=np.broadcast_to(t >= 0.5, out.shape))
    out[:, has_nan] = np.nan
    return out


def quantile_edges_device(X: np.ndarray | torch.Tensor, max_bins: int) -> np.ndarray:
    """``quantile_edges`` with the sort on the GPU (a column sort of 500 000 x 256 floats takes
    seconds on the host and milliseconds on the device); same result bit for bit up to the sign
    of a zero.  ``X``: float32 ``[N, F]``, host array or tensor on either side."""
    dev = _device()
    n, f = X.shape
    cols = max(1, min(f, (256 << 20) // max(4 * n, 1)))   # about 256 MB of floats per sort
    out = np.empty((max_bins - 1, f), dtype=np.float64)
    for c0 in range(0, f, cols):
        c1 = min(f, c0 + cols)
        if isinstance(X, torch.Tensor):
            block = X[:, c0:c1].to(device=dev, dtype=torch.float32)
        else:
            block = torch.from_numpy(np.ascontiguousarray(X[:, c0:c1], dtype=np.float32)).to(dev)
        out[:, c0:c1] = edges_from_sorted(torch.sort(block, dim=0).values, max_bins)
    return out.astype(np.float32)


def code_bits_for(max_bins: int) -> int:
    return 4 if max_bins <= 16 else 8


def _device() -> torch.device:
    if not B.cuda_available():
        raise RuntimeError("packboost_b200 needs its CUDA library and a B200-class device; there is no CPU path")
    return torch.device("cuda", torch.cuda.current_device())


_CHUNK_BYTES = 256 << 20


def _row_chunks(n_rows: int, row_bytes: int, chunk_bytes: int = _CHUNK_BYTES) -> Iterable[tuple[int, int]]:
    step = max(256, (chunk_bytes // max(row_bytes, 1)) // 256 * 256)
    for a in range(0, n_rows, step):
        yield a, min(n_rows, a + step)


class PackedMatrix:
    """Feature-major packed bin codes on the device (layout of ``pb_train_state.codes``)."""

    def __init__(self, n_rows: int, n_features_local: int, code_bits: int, device: torch.device,
                 pitch: int | None = None):
        self.n_rows = int(n_rows)
        self.rows_padded = (self.n_rows + 255) // 256 * 256
        self.code_bits = int(code_bits)
        self.pitch = (self.rows_padded * code_bits // 8 + 127) // 128 * 128
        if pitch is not None:
            if pitch % 128 or pitch < self.pitch:
                raise ValueError("pitch must be a multiple of 128 that covers the padded rows")
            self.pitch = int(pitch)
        self.n_features_local = int(n_features_local)
        self.max_code = 0   # largest pre-binned code seen while packing (when validation was asked for)
        self.codes = torch.zeros((max(self.n_features_local, 1), self.pitch), dtype=torch.uint8, device=device)

    def unpack(self) -> torch.Tensor:
        """``uint8 [F_local, n_rows]`` (tests and the legacy feature-major predictors)."""
        if self.code_bits == 8:
            return self.codes[: self.n_features_local, : self.n_rows].contiguous()
        lo = self.codes & 0xF
        hi = self.codes >> 4
        full = torch.stack([lo, hi], dim=2).reshape(self.codes.shape[0], -1)
        return full[: self.n_features_local, : self.n_rows].contiguous()


_STAGE: dict = {}


def _parallel_copy(dst: np.ndarray, src: np.ndarray) -> None:
    """``dst[...] = src`` for 2-D arrays with the rows dealt over a few threads (numpy releases the
    GIL while it copies): one thread moves ~10 GB/s, the host link takes five times that."""
    import os
    from concurrent.futures import ThreadPoolExecutor
    n = src.shape[0]
    workers = max(1, min(8, (os.cpu_count() or 2) // 2, n // 4096))
    if workers == 1:
        np.copyto(dst, src, casting="unsafe")
        return
    pool = _STAGE.get("pool")
    if pool is None:
        pool = _STAGE["pool"] = ThreadPoolExecutor(max_workers=8)
    step = (n + workers - 1) // workers
    futs = [pool.submit(np.copyto, dst[a:a + step], src[a:a + step], "unsafe") for a in range(0, n, step)]
    for f in futs:
        f.result()


def _staging(nbytes: int) -> list[tuple[torch.Tensor, torch.cuda.Event]]:
    """Two reusable page-locked buffers (and the events that guard their reuse) for bringing
    pageable host arrays to the device chunk by chunk."""
    have = _STAGE.get("bufs")
    if have is None or have[0][0].numel() < nbytes:
        have = [(torch.empty(nbytes, dtype=torch.uint8).pin_memory(), torch.cuda.Event()) for _ in range(2)]
        _STAGE["bufs"] = have
    return have


def pack_feature_major(
    X: np.ndarray | torch.Tensor,
    edges: np.ndarray | None,
    max_bins: int,
    *,
    row_order: np.ndarray | None = None,
    feature_map: np.ndarray | None = None,
    n_features_local: int | None = None,
    validate_codes: bool = False,
    rows: tuple[int, int] | None = None,
    out: "PackedMatrix | None" = None,
    defer_validation: bool = False,
) -> PackedMatrix:
    """Bin (when ``edges`` is given) and pack host or device data into a device ``PackedMatrix``.

    ``row_order`` lists source rows in destination order (era-sorted rows);
    ``feature_map[j]`` is the destination feature row of column ``j`` or -1.
    ``rows=(r0, r1)`` packs only that range of destination rows, into rows ``0 .. r1 - r0`` of
    ``out`` (one rank's share when several GPUs split the upload).  ``out`` packs into an existing
    matrix.  ``validate_codes`` checks on the device that pre-binned input stays below ``max_bins``
    (negative int8 values show up as codes >= 128) and raises ``ValueError`` otherwise; with
    ``defer_validation`` the largest code seen is only recorded in ``PackedMatrix.max_code`` (several
    ranks must agree before any of them raises).

    Host input reaches the device asynchronously: a page-locked tensor is read in place, a pageable
    array goes through two reusable page-locked staging buffers so that the host copy of chunk
    ``i + 1`` overlaps the transfer and the packing of chunk ``i``.
    """
    dev = _device()
    lib = B.lib()
    n_rows, n_feat = X.shape
    bits = code_bits_for(max_bins)
    r0, r1 = (0, n_rows) if rows is None else (int(rows[0]), int(rows[1]))
    n_local = n_feat if n_features_local is None else n_features_local
    pm = out if out is not None else PackedMatrix(r1 - r0, n_local, bits, dev)
    if r1 <= r0:
        return pm
    fmap_t = None
    if feature_map is not None:
        fmap_t = torch.from_numpy(np.ascontiguousarray(feature_map, dtype=np.int32)).to(dev)
    is_f32 = edges is not None
    edges_t = torch.from_numpy(np.ascontiguousarray(edges, dtype=np.float32)).to(dev) if is_f32 else None
    stream = torch.cuda.current_stream().cuda_stream
    is_tensor = isinstance(X, torch.Tensor)
    want = torch.float32 if is_f32 else torch.uint8
    item = 4 if is_f32 else 1
    np_want = np.float32 if is_f32 else np.uint8
    # a tensor that torch can hand to the copy engine as it is: on the device, or page-locked
    direct = is_tensor and (X.is_cuda or X.is_pinned())
    order_t = None
    if row_order is not None and is_tensor:
        order_t = torch.from_numpy(np.ascontiguousarray(row_order, dtype=np.int64)).to(X.device)
    top = torch.zeros((), dtype=torch.uint8, device=dev)
    # (smaller pieces for a pageable source: its two page-locked staging buffers are allocated on first
    # use, at about half a second per GB)
    chunks = [(r0 + a, r0 + b) for a, b in _row_chunks(r1 - r0, n_feat * item, _CHUNK_BYTES if direct else 64 << 20)]
    stage = None
    for i, (a, b) in enumerate(chunks):
        n = b - a
        if direct:
            src = X[a:b] if order_t is None else X.index_select(0, order_t[a:b])
            if src.dtype == torch.int8 and not is_f32:
                src = src.view(torch.uint8)
            chunk = src.to(device=dev, dtype=want, non_blocking=True).contiguous()
        else:
            # pageable source: through a page-locked staging buffer
            if stage is None:
                stage = _staging((chunks[0][1] - chunks[0][0]) * n_feat * item)
            buf, ev = stage[i % 2]
            ev.synchronize()                       # the transfer that last used this buffer is done
            dst = buf[: n * n_feat * item].view(want).view(n, n_feat)
            if is_tensor:
                src = X[a:b] if order_t is None else X.index_select(0, order_t[a:b])
                if src.dtype == torch.int8 and not is_f32:
                    src = src.view(torch.uint8)
                dst.copy_(src)
            else:
                src = X[a:b] if row_order is None else X[row_order[a:b]]
                if src.dtype == np.int8 and not is_f32:
                    src = src.view(np.uint8)
                _parallel_copy(dst.numpy(), src)
            chunk = dst.to(dev, non_blocking=True)
            ev.record()
        if validate_codes and not is_f32:
            top = torch.maximum(top, chunk.max())
        if is_f32:
            B.check(lib.pb_bin_pack_f32(chunk.data_ptr(), n, n_feat, a - r0, edges_t.data_ptr(), edges_t.shape[0],
                                        max_bins, B._ptr(fmap_t), pm.codes.data_ptr(), pm.pitch, bits, stream))
        else:
            B.check(lib.pb_pack_codes_u8(chunk.data_ptr(), n, n_feat, a - r0, B._ptr(fmap_t), pm.codes.data_ptr(),
                                         pm.pitch, bits, stream))
        # no synchronisation per chunk: the copy, the pack kernel and the release of `chunk` are
        # ordered on the current stream
    torch.cuda.current_stream().synchronize()
    pm.max_code = max(pm.max_code, int(top.item())) if validate_codes else pm.max_code
    if validate_codes and not defer_validation and pm.max_code >= min(max_bins, 128):
        raise ValueError("prebinned=True requires X to contain integer bins within [0, max_bins).")
    return pm


def rows_per_rank(n_rows: int, world: int) -> int:
    """Rows each rank packs when the upload is split by rows: equal shares rounded up to 256 rows
    (128 bytes of 4-bit codes), so that every rank's bytes of a feature row are a whole, aligned
    segment of it."""
    per = (n_rows + world - 1) // max(world, 1)
    return (per + 255) // 256 * 256


def pack_feature_major_distributed(X, edges, max_bins, *, row_order, rank: int, world: int, n_features: int,
                                   keep: tuple[int, int] | None, validate_codes: bool = False) -> PackedMatrix:
    """Pack the matrix with ``world`` GPUs sharing the host -> device transfer.

    Rank ``r`` brings over and packs only rows ``[r * R, (r + 1) * R)`` (``R = rows_per_rank``): a
    contiguous piece of the caller's row-major matrix, 1 / world of the bytes, at the full speed of
    its own host link.  The packed pieces are then exchanged between the GPUs (NVLink): with
    ``keep=None`` every rank ends up with the whole feature-major matrix (all-gather), with
    ``keep=(c0, c1)`` with all rows of its own features ``c0 .. c1`` only (all-to-all; every rank
    owns a block of ``ceil(F / world)`` features).  The result is laid out exactly like the matrix a
    single GPU would pack, with ``pitch = world * R * code_bits / 8``."""
    import torch.distributed as dist
    dev = _device()
    n_rows = X.shape[0]
    bits = code_bits_for(max_bins)
    per = rows_per_rank(n_rows, world)
    seg = per * bits // 8                                   # bytes of one feature row per rank (multiple of 128)
    blk = (n_features + world - 1) // world
    f_pad = blk * world
    slab = PackedMatrix(per, f_pad, bits, dev)
    assert slab.pitch == seg
    r0, r1 = min(n_rows, rank * per), min(n_rows, (rank + 1) * per)
    pack_feature_major(X, edges, max_bins, row_order=row_order, validate_codes=validate_codes, rows=(r0, r1), out=slab,
                       defer_validation=True)
    if keep is None:
        full = PackedMatrix(n_rows, f_pad, bits, dev, pitch=world * seg)
        parts = torch.empty((world, f_pad, seg), dtype=torch.uint8, device=dev)
        dist.all_gather_into_tensor(parts, slab.codes)
        full.codes.view(f_pad, world, seg).copy_(parts.permute(1, 0, 2))
        full.n_features_local = n_features
    else:
        full = PackedMatrix(n_rows, blk, bits, dev, pitch=world * seg)
        parts = torch.empty((world, blk, seg), dtype=torch.uint8, device=dev)
        dist.all_to_all_single(parts, slab.codes.view(world, blk, seg))
        full.codes.view(blk, world, seg).copy_(parts.permute(1, 0, 2))
        full.n_features_local = keep[1] - keep[0]
    full.max_code = slab.max_code
    return full


class PackedRows:
    """Row-major packed codes on the device (input layout of ``pb_predict_rows``)."""

    def __init__(self, n_rows: int, n_features: int, code_bits: int, device: torch.device):
        self.n_rows = int(n_rows)
        self.n_features = int(n_features)
        self.code_bits = int(code_bits)
        need = (n_features + 1) // 2 if code_bits == 4 else n_features
        self.pitch_row = (need + 15) // 16 * 16
        self.codes = torch.empty((max(self.n_rows, 1), self.pitch_row), dtype=torch.uint8, device=device)


def pack_row_major(X: np.ndarray | torch.Tensor, edges: np.ndarray | None, max_bins: int) -> PackedRows:
    """Bin (when ``edges`` is given) and pack rows for prediction.  ``X`` may already be a
    device tensor (float32 or uint8)."""
    dev = _device()
    lib = B.lib()
    bits = code_bits_for(max_bins)
    is_f32 = edges is not None
    n_rows, n_feat = X.shape
    pr = PackedRows(n_rows, n_feat, bits, dev)
    edges_t = torch.from_numpy(np.ascontiguousarray(edges, dtype=np.float32)).to(dev) if is_f32 else None
    stream = torch.cuda.current_stream().cuda_stream
    want = torch.float32 if is_f32 else torch.uint8
    for a, b in _row_chunks(n_rows, n_feat * (4 if is_f32 else 1)):
        if isinstance(X, torch.Tensor):
            chunk = X[a:b].to(device=dev, dtype=want).contiguous()
        else:
            chunk = torch.from_numpy(np.ascontiguousarray(X[a:b], dtype=np.float32 if is_f32 else np.uint8)).to(dev)
        out = pr.codes[a:b]
        B.check(lib.pb_pack_rows(chunk.data_ptr(), 1 if is_f32 else 0, b - a, n_feat, B._ptr(edges_t),
                                 edges_t.shape[0] if is_f32 else 0, max_bins, out.data_ptr(), pr.pitch_row, bits,
                                 stream))
        torch.cuda.current_stream().synchronize()
    return pr


# ---- reference-named host helpers ------------------------------------------------------------


def quantile_bin(X: np.ndarray, max_bins: int) -> tuple[np.ndarray, np.ndarray]:
    """Quantile-bin ``X`` column-wise (``packboost/data.py:45-58``): ``(int8 codes [N,F], edges)``."""
    if max_bins > 128:
        raise ValueError("PackBoost currently supports up to 128 bins (int8 storage)")
    Xf = np.ascontiguousarray(X, dtype=np.float32)
    edges = quantile_edges(Xf, max_bins)
    pm = pack_feature_major(Xf, edges, max_bins)
    bins = pm.unpack().t().contiguous().cpu().numpy().astype(np.int8)
    return bins, edges


def preprocess_features(X: np.ndarray, max_bins: int, *, assume_prebinned: bool = False) -> BinningResult:
    """``packboost/data.py:61-93``; the returned ``bins`` are int8 ``[N, F]``."""
    X_np = ensure_numpy(X)
    if assume_prebinned and not detect_prebinned(X_np, max_bins):
        raise ValueError("prebinned=True requires X to contain integer bins within [0, max_bins).")
    if assume_prebinned or detect_prebinned(X_np, max_bins):
        return BinningResult(bins=X_np.astype(np.int8, copy=False), bin_edges=None, prebinned=True)
    bins, edges = quantile_bin(X_np.astype(np.float32, copy=False), max_bins=max_bins)
    return BinningResult(bins=bins, bin_edges=edges, prebinned=False)


def apply_bins(X: np.ndarray, bin_edges: np.ndarray | None, max_bins: int) -> np.ndarray:
    """Bin ``X`` with stored edges (``packboost/data.py:96-111``) -> int8 ``[N, F]``."""
    X_np = ensure_numpy(X)
    if bin_edges is None:
        if not detect_prebinned(X_np, max_bins):
            raise ValueError("Input must already be prebinned when no edges are provided")
        return X_np.astype(np.int8, copy=False)
    Xf = np.ascontiguousarray(X_np, dtype=np.float32)
    pm = pack_feature_major(Xf, bin_edges, max_bins)
    return pm.unpack().t().contiguous().cpu().numpy().astype(np.int8)


def build_era_index(era_ids: Iterable[int] | np.ndarray, num_eras: int | None) -> list[torch.Tensor]:
    """Per-era ascending row-id tensors (``packboost/data.py:114-134``)."""
    era_np = np.asarray(era_ids, dtype=np.int16)
    if era_np.ndim != 1:
        raise ValueError("era_ids must be 1D")
    if num_eras is None:
        num_eras = 1 if era_np.size == 0 else int(era_np.max()) + 1
    order = np.argsort(era_np, kind="stable")
    counts = np.bincount(era_np[era_np >= 0].astype(np.int64), minlength=int(num_eras))[: int(num_eras)]
    offs = np.concatenate([[0], np.cumsum(counts)])
    valid = order[era_np[order] >= 0]
    return [torch.from_numpy(valid[offs[e]:offs[e + 1]].astype(np.int64)) for e in range(int(num_eras))]
