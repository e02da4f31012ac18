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
  * float sums/means: per-rank partial, all_gather, added up in float64 in rank
    order by the library's rank-fold kernel and rounded once, so the result does
    not depend on NCCL's algorithm choice;
  * min/max: all_gather of the per-rank answers, folded by the library's own
    min/max kernels;
  * index reductions: every rank writes {global index, value} of its shard in ONE
    pass into one buffer, one all_gather moves it, and the library's rank-fold
    kernel merges the `world` candidates per output with the same total order
    the single-GPU kernels use (a NaN loses unless all are NaN; ties go to the
    lowest global index), so the rules hold across ranks exactly as they hold
    across CTAs.  Nothing is read back to the host on the way;
  * an axis-0 reduction of a row-sharded matrix folds per-column partial vectors the
    same way; an axis-1 reduction is local, and flat (max|min)_index answers get the
    shard's element offset added.

On GPUs the gather of those partials goes through peer memory when every rank could
open every other rank's exchange buffer (`PeerExchange`: one small kernel per rank
stores its partial into all buffers, flags, and waits with a bound; the fold kernel
then reads local memory) and through NCCL's all_gather otherwise; CB200_PEER_EXCHANGE=0
forces NCCL.

The array backend is a namespace `xp` (the `cumo_b200` package on GPUs; the CPU
oracle's look-alike in the gloo tests, so the partition/fold logic is tested where
there is no GPU).
"""
from __future__ import annotations

import os

import numpy as np


def partition(n_rows: int, world: int, rank: int) -> tuple[int, int]:
    """(start, count) of `rank`'s rows: contiguous, sizes differ by at most one, earlier ranks get the extra row."""
    base, extra = divmod(n_rows, world)
    start = rank * base + min(rank, extra)
    return start, base + (1 if rank < extra else 0)


class PeerExchange:
    """Exchange buffers of all ranks, opened in this process (`cb200_peer_buffer_*`, `cb200_peer_exchange_kernel_launch`).

    Built collectively: every rank creates its buffer, the 64-byte handles travel through `all_gather_object`, every
    rank opens the others', and the ranks agree (an all_reduce of a flag) whether all of that worked everywhere; if
    not, `ok` is False on every rank and the caller stays on NCCL."""

    SLOT_BYTES = 256 << 10

    def __init__(self, dist, group, world, rank):
        import ctypes
        import torch
        from . import _lib
        self.lib = _lib.load()
        self.world, self.rank = world, rank
        self.seq = 0
        self.base = ctypes.c_void_p()
        self.opened = []
        self.bases = (ctypes.c_void_p * world)()
        handle = (ctypes.c_ubyte * 64)()
        ok = self.lib.cb200_peer_buffer_create(ctypes.c_size_t(self.SLOT_BYTES), world, ctypes.byref(self.base), handle) == 0
        handles = [None] * world
        dist.all_gather_object(handles, bytes(handle) if ok else None, group=group)
        if ok and all(h is not None for h in handles):
            for p, h in enumerate(handles):
                if p == rank:
                    self.bases[p] = self.base.value
                    continue
                ptr = ctypes.c_void_p()
                buf = (ctypes.c_ubyte * 64).from_buffer_copy(h)
                if self.lib.cb200_peer_buffer_open(buf, ctypes.byref(ptr)) != 0:
                    ok = False
                    break
                self.opened.append(ptr)
                self.bases[p] = ptr.value
        else:
            ok = False
        agreed = torch.tensor([1 if ok else 0], dtype=torch.int32, device="cuda")
        dist.all_reduce(agreed, op=dist.ReduceOp.MIN, group=group)
        self.ok = bool(agreed.item())
        self.status = torch.zeros(1, dtype=torch.int32, device="cuda")
        self.spin_limit = 0                                # 0 = the library's default (about ten seconds)
        dist.barrier(group=group)                          # nobody writes into a buffer that is not there yet

    def gather(self, src):
        """`src`: this rank's contiguous CUDA byte tensor (same size on every rank, <= SLOT_BYTES).  Returns (pointer,
        byte stride) of the `world` partials in this GPU's own memory, valid for kernels queued after this call."""
        import ctypes
        self.seq += 1
        rc = self.lib.cb200_peer_exchange_kernel_launch(ctypes.c_void_p(src.data_ptr()), ctypes.c_size_t(src.numel() * src.element_size()),
                                                        self.bases, self.world, self.rank, ctypes.c_size_t(self.SLOT_BYTES),
                                                        ctypes.c_ulonglong(self.seq), ctypes.c_uint(self.spin_limit),
                                                        ctypes.c_void_p(self.status.data_ptr()))
        if rc != 0:
            raise RuntimeError(f"peer exchange launch failed with CUDA error {rc}")
        return self.base.value + (self.seq & 1) * self.world * self.SLOT_BYTES, self.SLOT_BYTES

    _DTYPES = {"SFloat": 0, "DFloat": 1, "Int32": 2, "Int64": 3}

    def gather_fold(self, src, out, op, divisor=0.0, nan_wins=False):
        """Exchange and rank fold in one kernel: `src` (this rank's partial, an array of the library) against everyone's,
        folded element by element into `out` (same type and size).  op: "sum", "min" or "max"."""
        import ctypes
        self.seq += 1
        rc = self.lib.cb200_peer_exchange_fold_kernel_launch(
            ctypes.c_void_p(src.data_ptr), self._DTYPES[type(src).__name__], {"sum": 0, "min": 1, "max": 2}[op], src.size, float(divisor),
            int(bool(nan_wins)), ctypes.c_void_p(out.data_ptr), self.bases, self.world, self.rank, ctypes.c_size_t(self.SLOT_BYTES),
            ctypes.c_ulonglong(self.seq), ctypes.c_uint(self.spin_limit), ctypes.c_void_p(self.status.data_ptr()))
        if rc != 0:
            raise RuntimeError(f"peer exchange launch failed with CUDA error {rc}")
        return out

    def gather_merge_arg(self, buf, tname, n_out, val_off, want_max, nan_wins, out):
        """Exchange and merge of an index reduction's {index, value} partials in one kernel (`buf`: a CUDA byte tensor)."""
        import ctypes
        self.seq += 1
        rc = self.lib.cb200_peer_exchange_arg_kernel_launch(
            ctypes.c_void_p(buf.data_ptr()), self._DTYPES[tname], n_out, ctypes.c_size_t(val_off), int(want_max), int(bool(nan_wins)),
            ctypes.c_void_p(out.data_ptr), self.bases, self.world, self.rank, ctypes.c_size_t(self.SLOT_BYTES),
            ctypes.c_ulonglong(self.seq), ctypes.c_uint(self.spin_limit), ctypes.c_void_p(self.status.data_ptr()))
        if rc != 0:
            raise RuntimeError(f"peer exchange launch failed with CUDA error {rc}")
        return out

    def check(self):
        """Synchronises and raises if a bounded wait of an exchange ran out since the last check."""
        if int(self.status.item()) != 0:
            self.status.zero_()
            raise RuntimeError("a peer exchange gave up waiting for another rank: its result is not valid")

    def close(self):
        for ptr in self.opened:
            self.lib.cb200_peer_buffer_close(ptr)
        self.opened = []
        if self.base:
            self.lib.cb200_peer_buffer_destroy(self.base)
            self.base = None


class Comm:
    """The two collectives this path needs, over torch.distributed (or a single process)."""

    def __init__(self, xp, group=None, peer_exchange=None):
        """`peer_exchange`: True/False asks for / forbids the gather through peer memory; None leaves it to the
        environment (CB200_PEER_EXCHANGE, default on).  Must be the same on every rank."""
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
        self.peer = None
        if peer_exchange is None:
            peer_exchange = os.environ.get("CB200_PEER_EXCHANGE", "1") != "0"
        if self.on_gpu and self.dist and self.world > 1 and peer_exchange:
            px = PeerExchange(self.dist, group, self.world, self.rank)
            if px.ok:
                self.peer = px
            else:
                px.close()

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

    def all_gather_bytes(self, buf):
        """`buf`: this rank's contiguous torch tensor -> a (world, *buf.shape) tensor of everyone's, rank order."""
        import torch
        out = torch.empty((self.world,) + tuple(buf.shape), dtype=buf.dtype, device=buf.device)
        if self.dist:
            self.dist.all_gather_into_tensor(out.view(-1), buf.view(-1), group=self.group)
        else:
            out[0].copy_(buf)
        return out

    def gather_partials(self, buf):
        """Every rank's `buf` (a contiguous CUDA byte/element tensor, same size everywhere) side by side in local memory:
        (device pointer, byte stride between ranks, keep-alive object).  Peer memory when set up, NCCL otherwise."""
        nbytes = buf.numel() * buf.element_size()
        if self.peer is not None and nbytes <= PeerExchange.SLOT_BYTES:
            ptr, stride = self.peer.gather(buf)
            return ptr, stride, buf
        out = self.all_gather_bytes(buf)
        return out.data_ptr(), nbytes, out

    def check(self):
        """Raises if an exchange through peer memory timed out since the last check (synchronises)."""
        if self.peer is not None:
            self.peer.check()

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
        if host.shape[0] < comm.world:
            # decided from the global shape alone, so every rank raises here, before any collective: a rank with
            # no rows could not take part in the reductions, and the others would wait for it
            raise ValueError(f"{host.shape[0]} rows cannot be sharded over {comm.world} ranks: every rank needs at least one row")
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
        n = float(self.global_rows * self._row_elems() if axis is None else self.global_rows) if mean else 0.0
        if comm.on_gpu:
            # one gather of the partials as they are, one kernel that adds them in float64 in rank order
            import torch
            from . import _lib
            T = type(self.local)
            part = part if part.contiguous() else part.dup()
            out = T(*part.shape)
            if comm.peer is not None and part.size * (4 if T.__name__ == "SFloat" else 8) <= PeerExchange.SLOT_BYTES:
                return comm.peer.gather_fold(part, out, "sum", divisor=n)          # exchange and fold in one kernel
            src = torch.as_tensor(part, device="cuda")
            ptr, stride, _keep = comm.gather_partials(src)
            fold = getattr(_lib.load(), f"cb200_{T.__name__.lower()}_rank_fold_sum_kernel_launch")
            fold(ptr, stride, comm.world, src.numel(), n, out.data_ptr)
            return out
        wide = xp.DFloat.cast(part)                       # float32 partials are widened before they meet
        total = comm.all_gather(wide).sum(axis=0)          # rank-order fold in float64
        if mean:
            total = total / n
        return type(self.local).cast(total)

    def mean(self, axis=None):
        if axis not in (None, 0):
            return self._like(self.local.mean(axis=axis))
        return self.sum(axis=axis, mean=True)

    def _extreme(self, op, axis, nan):
        if axis not in (None, 0):
            return self._like(getattr(self.local, op)(axis=axis, nan=nan))
        part = getattr(self.local, op)(axis=axis, nan=nan) if self._is_float() else getattr(self.local, op)(axis=axis)
        comm = self.comm
        if comm.on_gpu:
            # the partials meet side by side in local memory (peer exchange or NCCL); one rank-fold kernel merges them
            import torch
            from . import _lib
            T = type(part)
            part = part if part.contiguous() else part.dup()
            out = T(*part.shape)
            if comm.peer is not None and part.size * (4 if T.__name__ in ("SFloat", "Int32") else 8) <= PeerExchange.SLOT_BYTES:
                return comm.peer.gather_fold(part, out, op, nan_wins=bool(nan) and self._is_float())
            src = torch.as_tensor(part, device="cuda")
            ptr, stride, _keep = comm.gather_partials(src)
            fold = getattr(_lib.load(), f"cb200_{T.__name__.lower()}_rank_fold_extreme_kernel_launch")
            fold(ptr, stride, comm.world, src.numel(), int(op == "max"), int(bool(nan) and self._is_float()), out.data_ptr)
            return out
        gathered = comm.all_gather(part)
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
        base = self.row_start * self._row_elems() if (axis is None or flat) else self.row_start      # local -> global index
        if comm.on_gpu:
            return self._arg_on_gpu(name_local, want_max, axis, nan, base)
        idx, val = self.local.arg_with_value(name_local, axis=axis, **kw)     # one pass: Int64 index and its value
        idx = idx + base
        vals = comm.all_gather(val)                       # [world] or [world, C]
        idxs = comm.all_gather(idx)
        winner = getattr(vals, "argmax" if want_max else "argmin")(axis=0, **kw)   # lowest rank wins ties
        # idxs[winner[c], c]: a selection among `world` candidates per output, done on the host
        w = np.asarray(winner.to_numpy(), dtype=np.int64)
        cand = np.asarray(idxs.to_numpy(), dtype=np.int64)
        picked = np.take_along_axis(cand, w[None, ...], axis=0)[0]
        return xp.Int64.cast(picked)

    def _arg_on_gpu(self, name_local, want_max, axis, nan, base):
        """{global index, value} of this shard in one pass into one buffer -> one all_gather -> the library's rank fold.
        Everything is queued on the stream; nothing comes back to the host."""
        import torch
        from ctypes import byref, c_void_p
        from . import _lib
        from .narray import _axis_mask, _raise_last

        comm, lib, loc = self.comm, _lib.load(), self.local
        T = type(loc)
        n_out = int(np.prod(loc.shape[1:], dtype=np.int64)) if axis == 0 else 1
        es = 4 if T.__name__ in ("SFloat", "Int32") else 8
        # [n_out int64 indices | n_out values], the value part starting on a 16-byte boundary
        val_off = (n_out * 8 + 15) // 16 * 16
        buf = torch.empty(val_off + (n_out * es + 15) // 16 * 16, dtype=torch.uint8, device="cuda")
        if lib.cb200_na_arg_with_value_into(name_local.encode(), loc._h, _axis_mask(axis, loc.ndim), int(bool(nan)), int(base),
                                            c_void_p(buf.data_ptr()), c_void_p(buf.data_ptr() + val_off), None, None):
            _raise_last()
        out = comm.xp.Int64(*(loc.shape[1:] if axis == 0 else ()))
        if comm.peer is not None and buf.numel() <= PeerExchange.SLOT_BYTES:
            return comm.peer.gather_merge_arg(buf, T.__name__, n_out, val_off, want_max, bool(nan), out)
        ptr, stride, _keep = comm.gather_partials(buf)
        fold = getattr(lib, f"cb200_{T.__name__.lower()}_rank_fold_arg_kernel_launch")
        fold(ptr, ptr + val_off, stride, comm.world, n_out, int(want_max), int(bool(nan)), out.data_ptr, None)
        return out

    def argmax(self, axis=None, nan=False): return self._arg(True, axis, nan, False)
    def argmin(self, axis=None, nan=False): return self._arg(False, axis, nan, False)
    def max_index(self, axis=None, nan=False): return self._arg(True, axis, nan, True)
    def min_index(self, axis=None, nan=False): return self._arg(False, axis, nan, True)

    def count_true(self):
        """Full count of a sharded Bit mask."""
        local = self.local.count_true()
        return self.comm.all_reduce_sum(local)
