"""Environmental selection operators backed by the CUDA kernels.

Function names, argument order, dtypes and return values follow the reference
(evox/operators/selection/non_dominate.py:172-254, rvea_selection.py:32-99).
"""

from __future__ import annotations

import torch

from .. import _cabi

__all__ = ["non_dominate_rank", "non_dominate_rank_sharded", "crowding_distance", "nd_environmental_selection", "ref_vec_guided",
           "ref_vec_guided_sharded", "raise_on_kernel_errors"]

_workspaces: dict[tuple[str, torch.device], torch.Tensor] = {}
_rvea_vectors: dict[torch.device, tuple | None] = {}  # per device: (reference-vector tensor, its version, workspace address)

# Status words of rank computations that were launched without `check=True`; `raise_on_kernel_errors()`
# reads them later (one host synchronisation), e.g. once per NSGA-II generation.
_pending_status: list[torch.Tensor] = []


def _remember(status: torch.Tensor) -> None:
    _pending_status.append(status)
    if len(_pending_status) > 64:  # nobody is checking: keep only the most recent ones
        del _pending_status[:-64]


def raise_on_kernel_errors() -> None:
    """Check the status word of every non-dominated sort launched since the last call."""
    pending, _pending_status[:] = list(_pending_status), []
    for status in pending:
        _raise_on_status(status)


def _workspace(kind: str, device: torch.device, nbytes: int) -> torch.Tensor:
    """A per-device scratch buffer that only grows; kernels using it are ordered by the stream."""
    key = (kind, device)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(nbytes, dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def _check_objectives(f: torch.Tensor, name: str) -> torch.Tensor:
    if f.ndim != 2:
        raise _cabi.EvoxKernelError(f"{name} must be 2-D (n, m), got shape {tuple(f.shape)}")
    return f.to(torch.float32).contiguous()


def _raise_on_status(status: torch.Tensor) -> None:
    code = int(status[0])
    if code != 0:
        raise _cabi.EvoxKernelError(
            "non-dominated sort did not finish: " + ("a grid-barrier wait timed out" if code == 1 else "no progress")
        )


def non_dominate_rank(x: torch.Tensor, check: bool = False) -> torch.Tensor:
    """Non-domination rank (int32, 0 = non-dominated) of each row of `x` (n, m).

    `check=True` reads the kernel's status word back (one host synchronisation) and raises if the
    bounded device-side waits gave up; the default leaves the call asynchronous."""
    f = _check_objectives(x, "x")
    n, m = f.shape
    rank = torch.empty(n, dtype=torch.int32, device=f.device)
    if n == 0:
        return rank
    nbytes = _cabi.lib.evox_nds_workspace_bytes(n, m)
    ws = _workspace("nds", f.device, nbytes)
    status = torch.zeros(2, dtype=torch.int32, device=f.device)
    _cabi.check(
        _cabi.lib.evox_nd_rank(
            _cabi.ptr(f), n, m, _cabi.ptr(rank), _cabi.ptr(status), _cabi.ptr(ws), ws.numel(), _cabi.stream_ptr(f.device)
        )
    )
    if check:
        _raise_on_status(status)
    else:
        _remember(status)
    return rank


def _shard_geometry(n: int, world: int) -> tuple[int, int]:
    """(rows per shard, columns of the split matrix): equal shards of a multiple of 1,024 rows that cover n."""
    shard_rows = -(-n // (world * 1024)) * 1024
    return shard_rows, shard_rows * world


def non_dominate_rank_sharded(x: torch.Tensor, group=None, check_every: int = 8, _emulate: tuple[int, int] | None = None):
    """`non_dominate_rank` with the dominance matrix split over the ranks of `group`: every rank passes the same
    `x` (n, m) and gets the same ranks back. Rank r builds and keeps only its rows of the bit matrix
    (n^2 / 8 / world bytes) and peels its columns; after every front the ranks allgather their slices of the
    unranked mask (n / 8 bytes in all) — the one exchange per peeling round. The host looks at the mask every
    `check_every` fronts (one synchronisation) to see whether anything is left.

    `_emulate=(rank, world)` runs one shard without a process group and returns its state (tests drive several
    shards on one GPU with it and do the gather themselves)."""
    import torch.distributed as dist

    f = _check_objectives(x, "x")
    n, m = f.shape
    dev = f.device
    if _emulate is not None:
        rank_id, world = _emulate
    elif dist.is_available() and dist.is_initialized():
        rank_id, world = dist.get_rank(group), dist.get_world_size(group)
    else:
        rank_id, world = 0, 1
    if n == 0:
        return torch.empty(0, dtype=torch.int32, device=dev)
    shard_rows, n_cols = _shard_geometry(n, world)
    begin = rank_id * shard_rows
    # a row order every rank derives alike: first objective descending (NaN last), ties in index order; a row's
    # dominators then start at the first row with the same first objective
    key = torch.where(torch.isnan(f[:, 0]), -torch.inf, f[:, 0])
    perm = torch.argsort(key, descending=True, stable=True)
    sorted_key = key[perm]
    first_equal = torch.searchsorted(-sorted_key, -sorted_key, side="left")
    start_word = torch.zeros(shard_rows, dtype=torch.int32, device=dev)
    hi = min(begin + shard_rows, n)
    if hi > begin:
        start_word[: hi - begin] = (first_equal[begin:hi] // 32).to(torch.int32)
    perm32 = perm.to(torch.int32).contiguous()
    nbytes = _cabi.lib.evox_nds_shard_workspace_bytes(n_cols, m, shard_rows)
    ws = _workspace("nds_shard", dev, nbytes)
    mask_slice = torch.empty(shard_rows // 32, dtype=torch.int32, device=dev)
    rank_local = torch.empty(shard_rows, dtype=torch.int32, device=dev)
    s = _cabi.stream_ptr(dev)
    _cabi.check(
        _cabi.lib.evox_nd_rank_shard_begin(
            _cabi.ptr(f), n, m, _cabi.ptr(perm32), n_cols, begin, shard_rows, _cabi.ptr(start_word), _cabi.ptr(mask_slice),
            _cabi.ptr(rank_local), _cabi.ptr(ws), ws.numel(), s,
        )
    )

    def front(mask_full: torch.Tensor, k: int) -> None:
        _cabi.check(
            _cabi.lib.evox_nd_rank_shard_front(n_cols, m, begin, shard_rows, _cabi.ptr(mask_full), k, _cabi.ptr(mask_slice),
                                               _cabi.ptr(rank_local), _cabi.ptr(ws), ws.numel(), _cabi.stream_ptr(dev))
        )

    if _emulate is not None:
        return {"front": front, "mask_slice": mask_slice, "rank_local": rank_local, "perm": perm, "begin": begin,
                "shard_rows": shard_rows, "n_cols": n_cols}
    mask_full = torch.empty(n_cols // 32, dtype=torch.int32, device=dev)

    def gather() -> None:
        if world > 1:
            dist.all_gather_into_tensor(mask_full, mask_slice, group=group)
        else:
            mask_full.copy_(mask_slice)

    gather()
    k = 0
    while True:
        for _ in range(check_every):
            front(mask_full, k)
            gather()
            k += 1
        if k > n or not bool(mask_full.any()):  # a strict partial order ranks somebody in every front
            break
    if world > 1:
        ranks_all = torch.empty(n_cols, dtype=torch.int32, device=dev)
        dist.all_gather_into_tensor(ranks_all, rank_local, group=group)
    else:
        ranks_all = rank_local
    out = torch.empty(n, dtype=torch.int32, device=dev)
    out[perm] = ranks_all[:n]
    if bool((out < 0).any()):
        raise _cabi.EvoxKernelError("sharded non-dominated sort did not finish: no progress")
    return out


def crowding_distance(costs: torch.Tensor, mask: torch.Tensor | None = None) -> torch.Tensor:
    """Crowding distance of the rows selected by `mask` (all rows if None); -inf elsewhere."""
    f = _check_objectives(costs, "costs")
    n, m = f.shape
    if mask is None:
        mask = torch.ones(n, dtype=torch.bool, device=f.device)
    mask_u8 = mask.to(torch.uint8).contiguous()
    out = torch.empty(n, dtype=torch.float32, device=f.device)
    if n == 0:
        return out
    nbytes = _cabi.lib.evox_nds_workspace_bytes(n, m)
    ws = _workspace("nds", f.device, nbytes)
    _cabi.check(
        _cabi.lib.evox_crowding_distance(
            _cabi.ptr(f), _cabi.ptr(mask_u8), n, m, _cabi.ptr(out), _cabi.ptr(ws), ws.numel(), _cabi.stream_ptr(f.device)
        )
    )
    return out


def nd_environmental_selection(x: torch.Tensor, f: torch.Tensor, topk: int, return_index: bool = False, check: bool = False):
    """Keep the best `topk` rows by (non-domination rank, then crowding distance).

    Returns (x, f, rank, crowding_distance) of the selected rows like the reference; with
    `return_index=True` a fifth tensor holds their row numbers."""
    fo = _check_objectives(f, "f")
    xo = x.to(torch.float32).contiguous()
    n, m = fo.shape
    if xo.ndim != 2 or xo.shape[0] != n:
        raise _cabi.EvoxKernelError(f"x must be (n, d) with n = {n}, got {tuple(x.shape)}")
    dx = xo.shape[1]
    dev = fo.device
    out_x = torch.empty(topk, dx, dtype=torch.float32, device=dev)
    out_f = torch.empty(topk, m, dtype=torch.float32, device=dev)
    out_rank = torch.empty(topk, dtype=torch.int32, device=dev)
    out_crowd = torch.empty(topk, dtype=torch.float32, device=dev)
    out_index = torch.empty(topk, dtype=torch.int64, device=dev)
    status = torch.zeros(2, dtype=torch.int32, device=dev)
    nbytes = _cabi.lib.evox_nds_workspace_bytes(n, m)
    ws = _workspace("nds", dev, nbytes)
    _cabi.check(
        _cabi.lib.evox_nd_environmental_selection(
            _cabi.ptr(xo), dx, _cabi.ptr(fo), n, m, topk, _cabi.ptr(out_x), _cabi.ptr(out_f), _cabi.ptr(out_rank),
            _cabi.ptr(out_crowd), _cabi.ptr(out_index), _cabi.ptr(status), _cabi.ptr(ws), ws.numel(), _cabi.stream_ptr(dev),
        )
    )
    if check:
        _raise_on_status(status)
    else:
        _remember(status)
    if return_index:
        return out_x, out_f, out_rank, out_crowd, out_index
    return out_x, out_f, out_rank, out_crowd


def _plain(t: torch.Tensor, device: torch.device | None = None) -> bool:
    """Already what the kernels take: float32, contiguous, on the (given) CUDA device."""
    return t.dtype == torch.float32 and t.is_cuda and t.is_contiguous() and (device is None or t.device == device)


def ref_vec_guided(x: torch.Tensor, f: torch.Tensor, v: torch.Tensor, theta: torch.Tensor | float, return_index: bool = False):
    """RVEA selection: per reference vector the associated individual with the smallest
    angle-penalised distance. Returns (next_x, next_f) with NaN rows for empty vectors, like the
    reference; `return_index=True` adds the chosen row numbers (-1 for empty vectors)."""
    if f.ndim != 2:
        raise _cabi.EvoxKernelError(f"f must be 2-D (n, m), got shape {tuple(f.shape)}")
    fo = f if _plain(f) else f.to(torch.float32).contiguous()
    n, m = fo.shape
    dev = fo.device
    xo = x if _plain(x, dev) else x.to(device=dev, dtype=torch.float32).contiguous()
    vo = v if _plain(v, dev) else v.to(device=dev, dtype=torch.float32).contiguous()
    if xo.ndim != 2 or xo.shape[0] != n:
        raise _cabi.EvoxKernelError(f"x must be (n, d) with n = {n}, got {tuple(x.shape)}")
    if vo.ndim != 2 or vo.shape[1] != m:
        raise _cabi.EvoxKernelError(f"v must be (nv, {m}), got {tuple(v.shape)}")
    nv, dx = vo.shape[0], xo.shape[1]
    if isinstance(theta, torch.Tensor) and theta.ndim == 0 and _plain(theta, dev):
        th = theta
    else:
        th = torch.as_tensor(theta, dtype=torch.float32, device=dev).reshape(())
    next_x = torch.empty(nv, dx, dtype=torch.float32, device=dev)
    next_f = torch.empty(nv, m, dtype=torch.float32, device=dev)
    next_index = torch.empty(nv, dtype=torch.int64, device=dev)
    nbytes = _cabi.lib.evox_rvea_workspace_bytes(n, m, nv)
    ws = _workspace("rvea", dev, nbytes)
    if dev.index != torch.cuda.current_device():
        raise _cabi.EvoxKernelError(f"f lives on {dev} but the current CUDA device is cuda:{torch.cuda.current_device()}")
    # the unit vectors and gamma derived from `v` stay in the workspace: skip them when this call has the
    # vectors of the previous one — the very same tensor object (the record keeps it alive, so its storage
    # cannot have been handed to another tensor), not written to since (version counter), same workspace
    prev = _rvea_vectors.get(dev)
    ready = prev is not None and prev[0] is v and prev[1] == v._version and prev[2] == ws.data_ptr() and vo is v
    _cabi.check(
        _cabi.lib.evox_ref_vec_guided(
            xo.data_ptr(), dx, fo.data_ptr(), n, m, vo.data_ptr(), nv, th.data_ptr(), int(ready), next_x.data_ptr(),
            next_f.data_ptr(), next_index.data_ptr(), ws.data_ptr(), ws.numel(), torch.cuda.current_stream(dev).cuda_stream,
        )
    )
    # `vo` is `v` itself when it already was a contiguous float32 tensor on the device; a converted copy is a
    # new tensor every call and is never reused
    _rvea_vectors[dev] = (v, v._version, ws.data_ptr()) if vo is v else None
    if return_index:
        return next_x, next_f, next_index
    return next_x, next_f


def ref_vec_guided_sharded(x: torch.Tensor, f: torch.Tensor, v: torch.Tensor, theta: torch.Tensor | float, row_offset: int,
                           group=None, return_index: bool = False):
    """`ref_vec_guided` when every rank of `group` holds a contiguous block of rows (x, f local;
    `row_offset` = global number of the first local row). Three small NCCL exchanges: minimum of the
    ideal point (m floats), minimum of the packed per-vector winners (nv int64), sum of the gathered
    rows. Every rank returns the full (nv, d) / (nv, m) result, identical to the single-GPU call."""
    import torch.distributed as dist

    fo = _check_objectives(f, "f")
    n, m = fo.shape
    dev = fo.device
    xo = x.to(torch.float32).contiguous()
    vo = v.to(device=dev, dtype=torch.float32).contiguous()
    nv, dx = vo.shape[0], xo.shape[1]
    th = torch.as_tensor(theta, dtype=torch.float32, device=dev).reshape(())
    ideal = torch.empty(m, dtype=torch.float32, device=dev)
    keys = torch.empty(nv, dtype=torch.int64, device=dev)
    next_x = torch.empty(nv, dx, dtype=torch.float32, device=dev)
    next_f = torch.empty(nv, m, dtype=torch.float32, device=dev)
    next_index = torch.empty(nv, dtype=torch.int64, device=dev)
    ws = _workspace("rvea", dev, _cabi.lib.evox_rvea_workspace_bytes(n, m, nv))
    _rvea_vectors[dev] = None  # phase 2 overwrites the derived vectors the single-GPU call may have left there

    def phase(k):
        _cabi.check(
            _cabi.lib.evox_ref_vec_guided_phase(
                k, _cabi.ptr(xo), dx, _cabi.ptr(fo), n, m, _cabi.ptr(vo), nv, _cabi.ptr(th), row_offset, _cabi.ptr(ideal),
                _cabi.ptr(keys), _cabi.ptr(next_x), _cabi.ptr(next_f), _cabi.ptr(next_index), _cabi.ptr(ws), ws.numel(),
                _cabi.stream_ptr(dev),
            )
        )

    sharded = dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1
    phase(1)
    if sharded:
        dist.all_reduce(ideal, op=dist.ReduceOp.MIN, group=group)
    phase(2)
    if sharded:
        # keys are unsigned; as int64 the "nobody" key (all ones) is -1, so compare in a shifted domain
        shifted = keys ^ torch.iinfo(torch.int64).min
        dist.all_reduce(shifted, op=dist.ReduceOp.MIN, group=group)
        keys.copy_(shifted ^ torch.iinfo(torch.int64).min)
    phase(3)
    if sharded:
        dist.all_reduce(next_x, op=dist.ReduceOp.SUM, group=group)
        dist.all_reduce(next_f, op=dist.ReduceOp.SUM, group=group)
    empty = (next_index < 0)[:, None]
    next_x = torch.where(empty, torch.nan, next_x)
    next_f = torch.where(empty, torch.nan, next_f)
    if return_index:
        return next_x, next_f, next_index
    return next_x, next_f
