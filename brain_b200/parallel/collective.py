"""Collective interface for CPU ranks and the implementations behind it.

``Collective`` = ``world_size`` + ``all_reduce(sum)`` / ``all_gather`` / ``reduce_scatter`` /
``broadcast(root)`` over flat fp32 tensors, reductions in fixed rank order (bit-reproducible)
— crates/model/src/collective.rs:35-54.  Implementations:

* ``HostCollective``    ranks are threads of this process (native barrier + slots);
* ``NetworkCollective`` ranks are processes on a loopback TCP star (native);
* ``TorchCollective``   a ``torch.distributed`` group (gloo on CPU, NCCL on GPUs) — what the
                        GPU engines use for plumbing and as their baseline.

Unlike the reference's trait (which has no error channel), every op raises ``CollectiveError``
naming the peer when a rank never arrives or a connection drops."""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch

from .. import _host

c = ctypes
_host.register({
    "bbh_hc_new": (c.c_void_p, [c.c_int, c.c_double]),
    "bbh_hc_free": (None, [c.c_void_p]),
    "bbh_hc_abort": (None, [c.c_void_p]),
    "bbh_hc_all_reduce": (c.c_int, [c.c_void_p, c.c_int, c.c_void_p, c.c_int64]),
    "bbh_hc_all_gather": (c.c_int, [c.c_void_p, c.c_int, c.c_void_p, c.c_int64, c.c_void_p]),
    "bbh_hc_reduce_scatter": (c.c_int, [c.c_void_p, c.c_int, c.c_void_p, c.c_int64, c.c_void_p]),
    "bbh_hc_broadcast": (c.c_int, [c.c_void_p, c.c_int, c.c_void_p, c.c_int64, c.c_int]),
    "bbh_hc_barrier": (c.c_int, [c.c_void_p]),
    "bbh_nc_listen": (c.c_void_p, [c.c_int, c.c_int, c.POINTER(c.c_int)]),
    "bbh_nc_accept": (c.c_int, [c.c_void_p]),
    "bbh_nc_connect": (c.c_void_p, [c.c_int, c.c_int, c.c_int]),
    "bbh_nc_free": (None, [c.c_void_p]),
    "bbh_nc_failed_peer": (c.c_int, [c.c_void_p]),
    "bbh_nc_all_reduce": (c.c_int, [c.c_void_p, c.c_void_p, c.c_int64]),
    "bbh_nc_broadcast": (c.c_int, [c.c_void_p, c.c_void_p, c.c_int64, c.c_int]),
    "bbh_nc_all_gather": (c.c_int, [c.c_void_p, c.c_void_p, c.c_int64, c.c_void_p]),
})


class CollectiveError(RuntimeError):
    pass


def _flat32(t: torch.Tensor) -> torch.Tensor:
    assert t.dtype == torch.float32 and t.is_contiguous() and not t.is_cuda
    return t.view(-1)


class _HostShared:
    def __init__(self, world: int, timeout_s: float):
        self.h = _host.lib().bbh_hc_new(world, timeout_s)
        self.world = world

    def __del__(self):
        try:
            if getattr(self, "h", None):
                _host.lib().bbh_hc_free(self.h)
                self.h = None
        except Exception:
            pass


class HostCollective:
    """One handle per rank-thread; build them with ``HostCollective.group(world)``."""

    def __init__(self, shared: _HostShared, rank: int):
        self._s, self.rank, self.world_size = shared, rank, shared.world

    @staticmethod
    def group(world: int, timeout_s: float = 60.0) -> List["HostCollective"]:
        s = _HostShared(world, timeout_s)
        return [HostCollective(s, r) for r in range(world)]

    def _check(self, rc: int, op: str):
        if rc == -1:
            raise CollectiveError(f"rank {self.rank}: {op} timed out waiting for a peer thread")
        if rc == -2:
            raise CollectiveError(f"rank {self.rank}: {op} called with mismatched lengths")

    def abort(self):
        """Break the barrier so peers blocked in a collective raise instead of waiting."""
        _host.lib().bbh_hc_abort(self._s.h)

    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        f = _flat32(t)
        self._check(_host.lib().bbh_hc_all_reduce(self._s.h, self.rank, f.data_ptr(), f.numel()), "all_reduce")
        return t

    def all_gather(self, t: torch.Tensor) -> torch.Tensor:
        f = _flat32(t)
        out = torch.empty(self.world_size * f.numel(), dtype=torch.float32)
        self._check(_host.lib().bbh_hc_all_gather(self._s.h, self.rank, f.data_ptr(), f.numel(),
                                                  out.data_ptr()), "all_gather")
        return out

    def reduce_scatter(self, t: torch.Tensor) -> torch.Tensor:
        f = _flat32(t)
        assert f.numel() % self.world_size == 0
        n = f.numel() // self.world_size
        out = torch.empty(n, dtype=torch.float32)
        self._check(_host.lib().bbh_hc_reduce_scatter(self._s.h, self.rank, f.data_ptr(), n,
                                                      out.data_ptr()), "reduce_scatter")
        return out

    def broadcast(self, t: torch.Tensor, root: int = 0) -> torch.Tensor:
        f = _flat32(t)
        self._check(_host.lib().bbh_hc_broadcast(self._s.h, self.rank, f.data_ptr(), f.numel(), root), "broadcast")
        return t

    def barrier(self):
        self._check(_host.lib().bbh_hc_barrier(self._s.h), "barrier")


class NetworkCollective:
    """TCP coordinator-star over 127.0.0.1.  Rank 0: ``NetworkCollective.coordinator(world)`` then
    ``accept()``; workers: ``NetworkCollective.worker(rank, world, port)``."""

    MAX_MSG_ELEMS = 1 << 28

    def __init__(self, h, rank: int, world: int, port: int):
        self._h, self.rank, self.world_size, self.port = h, rank, world, port

    @staticmethod
    def coordinator(world: int, port: int = 0) -> "NetworkCollective":
        p = c.c_int(0)
        h = _host.lib().bbh_nc_listen(world, port, c.byref(p))
        if not h:
            raise CollectiveError("coordinator could not listen on 127.0.0.1")
        return NetworkCollective(h, 0, world, p.value)

    def accept(self) -> "NetworkCollective":
        rc = _host.lib().bbh_nc_accept(self._h)
        if rc != 0:
            raise CollectiveError("coordinator: a worker announced an invalid or duplicate rank"
                                  if rc == -2 else "coordinator: accept failed")
        return self

    @staticmethod
    def worker(rank: int, world: int, port: int) -> "NetworkCollective":
        h = _host.lib().bbh_nc_connect(rank, world, port)
        if not h:
            raise CollectiveError(f"rank {rank}: cannot reach the coordinator on port {port}")
        return NetworkCollective(h, rank, world, port)

    def close(self):
        if getattr(self, "_h", None):
            _host.lib().bbh_nc_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc: int, op: str):
        if rc == -1:
            peer = _host.lib().bbh_nc_failed_peer(self._h)
            raise CollectiveError(f"rank {self.rank}: {op} lost its connection to rank {peer}")
        if rc == -3:
            raise CollectiveError(f"rank {self.rank}: {op} message exceeds {self.MAX_MSG_ELEMS} elements")

    def all_reduce(self, t):
        f = _flat32(t)
        self._check(_host.lib().bbh_nc_all_reduce(self._h, f.data_ptr(), f.numel()), "all_reduce")
        return t

    def broadcast(self, t, root: int = 0):
        f = _flat32(t)
        self._check(_host.lib().bbh_nc_broadcast(self._h, f.data_ptr(), f.numel(), root), "broadcast")
        return t

    def all_gather(self, t):
        f = _flat32(t)
        out = torch.empty(self.world_size * f.numel(), dtype=torch.float32)
        self._check(_host.lib().bbh_nc_all_gather(self._h, f.data_ptr(), f.numel(), out.data_ptr()), "all_gather")
        return out

    def reduce_scatter(self, t):
        f = _flat32(t).clone()
        n = f.numel() // self.world_size
        self.all_reduce(f)
        return f[self.rank * n:(self.rank + 1) * n].clone()


class TorchCollective:
    def __init__(self, group=None):
        import torch.distributed as dist
        self._d, self.group = dist, group
        self.rank = dist.get_rank(group)
        self.world_size = dist.get_world_size(group)

    def all_reduce(self, t):
        self._d.all_reduce(t, group=self.group)
        return t

    def broadcast(self, t, root: int = 0):
        self._d.broadcast(t, self._d.get_global_rank(self.group, root) if self.group else root, group=self.group)
        return t

    def all_gather(self, t):
        parts = [torch.empty_like(t) for _ in range(self.world_size)]
        self._d.all_gather(parts, t.contiguous(), group=self.group)
        return torch.cat([p.reshape(-1) for p in parts])

    def reduce_scatter(self, t):
        f = t.reshape(-1).clone()
        n = f.numel() // self.world_size
        self._d.all_reduce(f, group=self.group)
        return f[self.rank * n:(self.rank + 1) * n].clone()
