"""Multi-GPU sharding of the operator: one process per GPU over ``torch.distributed``.

The reference has no multi-GPU path.  Two facts make sharding collective-free
or nearly so (flash_colreduce/naive.py:19-37): heads are independent, and so
are query rows (the softmax normalises per row), so a rank that owns a subset
of the rows of a head produces a partial N-vector that is combined with ``+``
(sum, mean) or ``max``.

* ``B*H >= world``: heads are partitioned; every rank owns whole heads and no
  data-path collective is needed (results may stay sharded).
* ``B*H < world``: the ranks of a head split its query rows.  With a causal
  mask the work per row grows with the row index, so the rows are cut into
  ``2 * ranks_per_head`` equal chunks and rank g takes chunks g and
  ``2*ranks_per_head - 1 - g`` (zig-zag).  The partial vectors are combined by
  ONE all-reduce of the fp32 (B*H, N) array, after which the mean divisor is
  applied (flash_colreduce/flash.py:377-384).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Tuple

import torch
import torch.distributed as dist

__all__ = ["ShardSpec", "plan_shards", "sharded_colreduce", "NativeComm", "native_plan_shards",
           "sharded_colreduce_native"]


@dataclass
class ShardSpec:
    """What one rank computes: heads [head_lo, head_hi) of the B*H heads, and for
    each of them the query-row ranges in ``row_ranges``."""

    rank: int
    world: int
    head_lo: int
    head_hi: int
    row_ranges: List[Tuple[int, int]] = field(default_factory=list)
    needs_reduce: bool = False  # rows of a head are spread over several ranks

    @property
    def heads(self) -> int:
        return self.head_hi - self.head_lo


def plan_shards(bh: int, m: int, world: int, rank: int, tile: int = 128) -> ShardSpec:
    """Partition ``bh`` heads of ``m`` query rows over ``world`` ranks."""
    if bh <= 0 or m <= 0 or world <= 0 or not (0 <= rank < world):
        raise ValueError("plan_shards: bh, m, world must be positive and 0 <= rank < world")
    if bh >= world:
        base, extra = divmod(bh, world)
        lo = rank * base + min(rank, extra)
        hi = lo + base + (1 if rank < extra else 0)
        return ShardSpec(rank, world, lo, hi, [(0, m)], False)
    per_head = world // bh          # ranks that share one head; leftover ranks stay idle
    head, g = divmod(rank, per_head)
    if head >= bh:
        return ShardSpec(rank, world, 0, 0, [], True)
    if per_head == 1:
        return ShardSpec(rank, world, head, head + 1, [(0, m)], world > bh)
    chunks = 2 * per_head
    step = -(-m // chunks)
    step = -(-step // tile) * tile  # whole 128-row tiles per chunk
    ranges = []
    for c in (g, chunks - 1 - g):
        lo, hi = min(c * step, m), min((c + 1) * step, m)
        if hi > lo:
            ranges.append((lo, hi))
    return ShardSpec(rank, world, head, head + 1, ranges, True)


def _gpu_partial(q, k, reduction, is_causal, scale, causal_offset):
    from .op import colreduce_partial

    return colreduce_partial(q, k, reduction, is_causal, scale, causal_offset)


def _gpu_finalize(acc, m, reduction, is_causal, dtype):
    from .op import finalize_scores

    return finalize_scores(acc, m, reduction, is_causal, dtype)


def sharded_colreduce(
    query: torch.Tensor,
    key: torch.Tensor,
    reduction: str,
    is_causal: bool = False,
    scale: Optional[float] = None,
    *,
    spec: ShardSpec,
    total_heads: int,
    group: Optional[dist.ProcessGroup] = None,
    gather: bool = True,
    partial_fn: Callable = _gpu_partial,
    finalize_fn: Callable = _gpu_finalize,
) -> torch.Tensor:
    """Column reduction of this rank's shard, combined across ranks.

    ``query`` (1, heads_local, M, D) and ``key`` (1, heads_local, N, D) hold the
    heads ``spec`` assigns to this rank, all rows of them.  Returns the
    (total_heads, N) result in ``query.dtype`` when ``gather`` (after one
    all-reduce of the fp32 partials), else this rank's (heads_local, N) block,
    which is final only when ``spec.needs_reduce`` is False.

    ``partial_fn`` / ``finalize_fn`` default to the CUDA kernels; they are
    parameters so that the host logic can be exercised by CPU ranks.
    """
    if reduction not in ("sum", "mean", "max"):
        raise ValueError(f"Invalid reduction: {reduction}. Must be 'sum', 'mean', or 'max'.")
    m, d = query.shape[2], query.shape[3]
    n = key.shape[2]
    if scale is None:
        scale = 1 / math.sqrt(d)
    c = max(n - m, 0)
    base_red = "max" if reduction == "max" else "sum"
    local = torch.zeros((1, spec.heads, n), dtype=torch.float32, device=query.device)
    for lo, hi in spec.row_ranges:
        if is_causal:
            n_vis = min(n, c + hi)  # keys beyond the last row's reach contribute nothing
            part = partial_fn(query[:, :, lo:hi], key[:, :, :n_vis], base_red, True, scale, c + lo)
        else:
            n_vis = n
            part = partial_fn(query[:, :, lo:hi], key, base_red, False, scale, 0)
        if base_red == "max":
            local[..., :n_vis] = torch.maximum(local[..., :n_vis], part)
        else:
            local[..., :n_vis] += part
    if not gather and not spec.needs_reduce:
        return finalize_fn(local, m, reduction, is_causal, query.dtype)[0]
    full = torch.zeros((1, total_heads, n), dtype=torch.float32, device=query.device)
    full[:, spec.head_lo:spec.head_hi] = local
    if spec.world > 1:
        # zeros are neutral for both operators: partial sums add, probabilities are >= 0
        dist.all_reduce(full, op=dist.ReduceOp.MAX if base_red == "max" else dist.ReduceOp.SUM, group=group)
    return finalize_fn(full, m, reduction, is_causal, query.dtype)[0]


# ---------------------------------------------------------------------------
# The same operator through the library's own multi-GPU entry point
# (fcr_colreduce_sharded): shard plan, kernels, the NCCL all-reduce and the
# finalize step are all queued by one C call; torch.distributed only carries
# the 128-byte NCCL id from rank 0 to the other ranks when the communicator is
# made.


class NativeComm:
    """An NCCL communicator owned by the library (``fcr_comm_init``), one rank per process.

    ``NativeComm(group)`` must be called by every rank of ``group`` (default: the
    world) with its GPU current; rank 0's NCCL id travels through a broadcast on
    that group, which may be a ``gloo`` group.
    """

    def __init__(self, group: Optional[dist.ProcessGroup] = None):
        import ctypes as C

        from . import _native as nat

        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        ident = torch.zeros(nat.FCR_NCCL_ID_BYTES, dtype=torch.uint8)
        if self.rank == 0:
            buf = (C.c_ubyte * nat.FCR_NCCL_ID_BYTES)()
            nat.check(nat.lib.fcr_comm_unique_id(buf), "fcr_comm_unique_id")
            ident = torch.tensor(list(buf), dtype=torch.uint8)
        backend = dist.get_backend(group)
        carrier = ident.cuda() if backend == "nccl" else ident
        dist.broadcast(carrier, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        raw = bytes(carrier.cpu().tolist())
        self.handle = C.c_void_p()
        nat.check(nat.lib.fcr_comm_init(raw, self.world, self.rank, C.byref(self.handle)), "fcr_comm_init")

    def close(self) -> None:
        from . import _native as nat

        if self.handle:
            nat.check(nat.lib.fcr_comm_destroy(self.handle), "fcr_comm_destroy")
            self.handle = None


def native_plan_shards(bh: int, m: int, world: int, rank: int) -> ShardSpec:
    """``fcr_plan_shards`` as a :class:`ShardSpec` (the C twin of :func:`plan_shards`)."""
    import ctypes as C

    from . import _native as nat

    sh = nat.Shard()
    rc = nat.lib.fcr_plan_shards(bh, m, world, rank, C.byref(sh))
    if rc != nat.FCR_OK:
        raise ValueError(nat.last_error())
    ranges = [(sh.row_lo[r], sh.row_hi[r]) for r in range(sh.n_ranges)]
    return ShardSpec(sh.rank, sh.world, sh.head_lo, sh.head_hi, ranges, bool(sh.needs_reduce))


def sharded_colreduce_native(
    query: torch.Tensor,
    key: torch.Tensor,
    reduction: str,
    is_causal: bool = False,
    scale: Optional[float] = None,
    *,
    total_heads: int,
    comm: Optional[NativeComm],
    world: int,
    rank: int,
) -> torch.Tensor:
    """Column reduction of this rank's heads combined across ranks by ``fcr_colreduce_sharded``.

    ``query`` (1, heads_local, M, D) / ``key`` (1, heads_local, N, D) hold the heads
    ``fcr_plan_shards(total_heads, M, world, rank)`` assigns to this rank (all their rows; an
    idle rank passes tensors with zero heads).  Returns the full (total_heads, N) result in
    ``query.dtype`` on every rank.  Everything is queued on the current stream.
    """
    import ctypes as C

    from . import _native as nat
    from .op import _DTYPE_CODES, _tma_ready

    if reduction not in ("sum", "mean", "max"):
        raise ValueError(f"Invalid reduction: {reduction}. Must be 'sum', 'mean', or 'max'.")
    m, n = query.shape[2], key.shape[2]
    if scale is None:
        scale = 1 / math.sqrt(query.shape[3])
    sh = nat.Shard()
    nat.check(nat.lib.fcr_plan_shards(total_heads, m, world, rank, C.byref(sh)), "fcr_plan_shards")
    heads = sh.head_hi - sh.head_lo
    if query.shape[1] != heads or key.shape[1] != heads or query.shape[0] != 1:
        raise ValueError(f"this rank's shard has {heads} head(s); got query {tuple(query.shape)}, key {tuple(key.shape)}")
    dev = query.device
    out = torch.empty((total_heads, n), dtype=query.dtype, device=dev)
    acc = torch.empty((total_heads, n), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev).cuda_stream
        if heads > 0:
            q, k = _tma_ready(query), _tma_ready(key)
            prob = nat.make_problem(1, heads, m, n, q.shape[3], q.stride(), k.stride(), _DTYPE_CODES[q.dtype],
                                    nat.REDUCTION_CODES[reduction], is_causal, scale)
            ws = torch.empty(nat.lib.fcr_sharded_workspace_bytes(C.byref(prob), C.byref(sh)), dtype=torch.uint8, device=dev)
            qp, kp = q.data_ptr(), k.data_ptr()
        else:
            prob = nat.make_problem(1, 1, m, n, query.shape[3], (0, 0, query.shape[3], 1), (0, 0, query.shape[3], 1),
                                    _DTYPE_CODES[query.dtype], nat.REDUCTION_CODES[reduction], is_causal, scale)
            ws = torch.empty(256, dtype=torch.uint8, device=dev)
            qp = kp = None
        rc = nat.lib.fcr_colreduce_sharded(C.byref(prob), C.byref(sh), total_heads, qp, kp, acc.data_ptr(), out.data_ptr(),
                                           _DTYPE_CODES[out.dtype], ws.data_ptr(), ws.numel(),
                                           comm.handle if comm is not None else None, stream)
        nat.check(rc, "fcr_colreduce_sharded")
    return out
