"""Leading-axis sharding of very large arrays over the GPUs of one box.

The reference has no multi-GPU code at all; this module is the one addition on top
of its API.  One process per GPU (`torch.distributed`, NCCL over NVLink); the
leading axis (or the only axis of a 1-D array) is cut into `world` contiguous,
nearly equal row ranges and every rank holds its range in its own memory.  Kernels
never read another GPU's memory; what crosses NVLink is a few bytes per output:

  * elementwise sweeps need no communication (an operand whose leading extent is 1
    is replicated);
  * integer sums and Bit counts: per-rank partial -> all_reduce(SUM) on int64, exact
    and order independent;
  * float sums/means: per-rank partial, widened to float64, all_gather, folded in
    rank order by the library's own float64 sum kernel, so the result does not
    depend on NCCL's algorithm choice;
  * min/max and the index reductions: all_gather of the per-rank answers, folded by
    the library's own min/max/arg kernels, whose rules (a NaN loses unless all are
    NaN; ties go to the lowest global index) then hold across ranks exactly as
    they hold across CTAs;
  * an axis-0 reduction of a row-sharded matrix folds per-column partial vectors the
    same way; an axis-1 reduction is local, and flat (max|min)_index answers get the
    shard's element offset added.

The array backend is a namespace `xp` (the `cumo_b200` package on GPUs; the CPU
oracle's look-alike in the gloo tests, so the partition/fold logic is tested where
there is no GPU).
"""
from __future__ import annotations

import numpy as np


def partition(n_rows: int, world: int, rank: int) -> tuple[int, int]:
    """(start, count) of `rank`'s rows: contiguous, sizes differ by at most one, earlier ranks get the extra row."""
    base, extra = divmod(n_rows, world)
    start = rank * base + min(rank, extra)
    return start, base + (1 if rank < extra else 0)


class Comm:
    """The two collectives this path needs, over torch.distributed (or a single process)."""

    def __init__(self, xp, group=None):
        self.xp = xp
        self.group = group
        try:
            import torch.distributed as dist
            self.dist = dist if dist.is_available() and dist.is_initialized() else None
        except ImportError:  # pragma: no cover
            self.dist = None
        self.world = self.dist.get_world_size(group) if self.dist else 1
        self.rank = self.dist.get_rank(group) if self.dist else 0
        self.on_gpu = getattr(xp, "__name__", "") == "cumo_b200"

    # xp array <-> torch tensor without copying where the backend allows it
    def _to_torch(self, arr):
        import torch
        if self.on_gpu:
            return torch.as_tensor(arr, device="cuda")
        return torch.from_numpy(np.ascontiguousarray(arr.a))

    def _from_torch(self, t, like_type):
        if self.on_gpu:
            return like_type.from_torch(t)
        return like_type.cast(t.numpy())

    def all_gather(self, arr):
        """Stack every rank's `arr` (same shape everywhere) along a new leading axis, in rank order."""
        import torch
        src = self._to_torch(arr.dup() if not arr.contiguous() else arr)
        out = torch.empty((self.world,) + tuple(src.shape), dtype=src.dtype, device=src.device)
        if self.dist:
            self.dist.all_gather_into_tensor(out.view(-1), src.reshape(-1).contiguous(), group=self.group)
        else:
            out[0].copy_(src)
        return self._from_torch(out, type(arr))

    def all_reduce_sum(self, arr):
        """Exact integer sum over ranks (Int64 / UInt64 containers)."""
        import torch
        t = self._to_torch(arr.dup() if not arr.contiguous() else arr)
        if t.dtype == torch.uint64:
            t = t.view(torch.int64)
        t = t.clone()
        if self.dist:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM, group=self.group)
        return self._from_torch(t, self.xp.Int64)


class ShardedArray:
    """This rank's rows [row_start, row_start+rows) of a global array of shape (n_rows, *rest)."""

    def __init__(self, comm: Comm, local, global_rows: int, row_start: int):
        self.comm = comm
        self.local = local
        self.global_rows = global_rows
        self.row_start = row_start

    @classmethod
    def scatter_from_numpy(cls, comm: Comm, array_type, host: np.ndarray):
        """Every rank passes the same host array (or a memmap); each uploads only its own rows."""
        start, count = partition(host.shape[0], comm.world, comm.rank)
        return cls(comm, array_type.from_numpy(np.ascontiguousarray(host[start:start + count])), host.shape[0], start)

    @property
    def shape(self):
        return (self.global_rows,) + tuple(self.local.shape[1:])

    def _like(self, local):
        return ShardedArray(self.comm, local, self.global_rows, self.row_start)

    # ---- elementwise: no communication -------------------------------------------------------
    def _other(self, o):
        if isinstance(o, ShardedArray):
            if o.global_rows != self.global_rows or o.row_start != self.row_start:
                raise ValueError("operands are sharded differently")
            return o.local
        return o   # a scalar or a replicated array whose leading extent is 1 / absent

    def __add__(self, o): return self._like(self.local + self._other(o))
    def __sub__(self, o): return self._like(self.local - self._other(o))
    def __mul__(self, o): return self._like(self.local * self._other(o))
    def __truediv__(self, o): return self._like(self.local / self._other(o))
    def __mod__(self, o): return self._like(self.local % self._other(o))
    def __gt__(self, o): return self._like(self.local > self._other(o))
    def __lt__(self, o): return self._like(self.local < self._other(o))
    def map(self, fn): return self._like(fn(self.local))

    # ---- reductions -------------------------------------------------------------------------------
    def _row_elems(self):
        return int(np.prod(self.local.shape[1:], dtype=np.int64)) if self.local.ndim > 1 else 1

    def _is_float(self):
        return type(self.local).__name__.endswith("Float")

    def sum(self, axis=None, nan=False, mean=False):
        """Full sum (axis=None) or axis-0 sum: replicated result on every rank.  Other axes are local."""
        xp, comm = self.comm.xp, self.comm
        if axis not in (None, 0):
            return self._like(self.local.sum(axis=axis, nan=nan))
        part = self.local.sum(axis=axis, nan=nan) if self._is_float() else self.local.sum(axis=axis)
        if not self._is_float():
            return comm.all_reduce_sum(part)
        wide = xp.DFloat.cast(part)                       # float32 partials are widened before they meet
        total = comm.all_gather(wide).sum(axis=0)          # rank-order fold by the float64 sum kernel
        if mean:
            n = self.global_rows * self._row_elems() if axis is None else self.global_rows
            total = total / float(n)
        return type(self.local).cast(total)

    def mean(self, axis=None):
        if axis not in (None, 0):
            return self._like(self.local.mean(axis=axis))
        return self.sum(axis=axis, mean=True)

    def _extreme(self, op, axis, nan):
        if axis not in (None, 0):
            return self._like(getattr(self.local, op)(axis=axis, nan=nan))
        part = getattr(self.local, op)(axis=axis, nan=nan) if self._is_float() else getattr(self.local, op)(axis=axis)
        gathered = self.comm.all_gather(part)
        return getattr(gathered, op)(axis=0, nan=nan) if self._is_float() else getattr(gathered, op)(axis=0)

    def max(self, axis=None, nan=False): return self._extreme("max", axis, nan)
    def min(self, axis=None, nan=False): return self._extreme("min", axis, nan)

    def _arg(self, want_max, axis, nan, flat):
        """argmax/argmin (flat=False: position along the reduced axes) or max_index/min_index
        (flat=True: element offset in the whole global array)."""
        xp, comm = self.comm.xp, self.comm
        name_local = ("max_index" if want_max else "min_index") if flat else ("argmax" if want_max else "argmin")
        kw = {"nan": nan} if self._is_float() else {}
        if axis not in (None, 0):
            idx = getattr(self.local, name_local)(axis=axis, **kw)
            if flat:
                idx = xp.Int64.cast(idx) + self.row_start * self._row_elems()
            return self._like(idx)
        idx, val = self.local.arg_with_value(name_local, axis=axis, **kw)     # one pass: Int64 index and its value
        # local -> global index
        if axis is None or flat:
            idx = idx + self.row_start * self._row_elems()
        else:
            idx = idx + self.row_start
        vals = comm.all_gather(val)                       # [world] or [world, C]
        idxs = comm.all_gather(idx)
        winner = getattr(vals, "argmax" if want_max else "argmin")(axis=0, **kw)   # lowest rank wins ties
        # idxs[winner[c], c]: a selection among `world` candidates per output, done on the host
        w = np.asarray(winner.to_numpy(), dtype=np.int64)
        cand = np.asarray(idxs.to_numpy(), dtype=np.int64)
        picked = np.take_along_axis(cand, w[None, ...], axis=0)[0]
        return xp.Int64.cast(picked)

    def argmax(self, axis=None, nan=False): return self._arg(True, axis, nan, False)
    def argmin(self, axis=None, nan=False): return self._arg(False, axis, nan, False)
    def max_index(self, axis=None, nan=False): return self._arg(True, axis, nan, True)
    def min_index(self, axis=None, nan=False): return self._arg(False, axis, nan, True)

    def count_true(self):
        """Full count of a sharded Bit mask."""
        local = self.local.count_true()
        return self.comm.all_reduce_sum(local)
