"""Worker-to-worker communicator (reference: ``paracel::Comm`` over MPI,
include/utils/comm.hpp:96-721, src/comm.cpp:20-81).

The same primitive set -- send / isend / recv / sendrecv / bcast / bcastring /
alltoall / alltoallring / allreduce(SUM) / treereduce / split / synchronize --
is provided on top of ``torch.distributed`` process groups: ``gloo`` for CPU
ranks and host objects, ``nccl`` for CUDA tensors.  Arbitrary Python values
(lists of triples, dictionaries, strings) are pickled into byte tensors; tensors
and numpy arrays go through the native collectives.  With no process group the
communicator has size 1 and every primitive degenerates to the identity, which
is the reference's "serial use without servers" mode (include/ps.hpp:89-100).
"""
from __future__ import annotations

import os
import pickle
from typing import Any, Callable, List, Optional, Sequence

import numpy as np
import torch
import torch.distributed as dist


class main_env:
    """Process-group lifetime (reference: ``main_env`` = MPI_Init/Finalize,
    comm.hpp:32-44).  Reads RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT."""

    def __init__(self, backend: Optional[str] = None, timeout_s: float = 1800.0):
        self.owned = False
        world = int(os.environ.get("WORLD_SIZE", "1"))
        if world > 1 and not dist.is_initialized():
            import datetime
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29533")
            if backend is None:
                backend = "cpu:gloo,cuda:nccl" if torch.cuda.is_available() else "gloo"
            dist.init_process_group(backend, rank=int(os.environ.get("RANK", "0")),
                                    world_size=world,
                                    timeout=datetime.timedelta(seconds=timeout_s))
            self.owned = True

    def close(self):
        if self.owned and dist.is_initialized():
            dist.destroy_process_group()
            self.owned = False

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()


class vrequest:
    """Handle of one or more pending non-blocking sends (comm.hpp:46-94)."""

    def __init__(self, works=None, keep=None):
        self.works = list(works or [])
        self._keep = keep

    def append(self, w):
        self.works.append(w)

    def wait(self):
        for w in self.works:
            if w is not None:
                w.wait()
        self.works = []


def _to_bytes_tensor(obj: Any) -> torch.Tensor:
    b = pickle.dumps(obj, protocol=pickle.HIGHEST_PROTOCOL)
    return torch.frombuffer(bytearray(b), dtype=torch.uint8)


class Comm:
    def __init__(self, group=None):
        self.group = group
        self._active = dist.is_initialized()
        self._rank = dist.get_rank(group) if self._active else 0
        self._size = dist.get_world_size(group) if self._active else 1
        self._ranks = (dist.get_process_group_ranks(group) if (self._active and group is not None)
                       else list(range(self._size)))

    # ---------------------------------------------------------------- info
    def get_rank(self) -> int:
        return self._rank

    def get_size(self) -> int:
        return self._size

    def _global(self, r: int) -> int:
        return self._ranks[r]

    def synchronize(self) -> None:
        if self._size > 1:
            dist.barrier(group=self.group)

    sync = synchronize

    def split(self, color: int, key: Optional[int] = None) -> "Comm":
        """Sub-communicator of the ranks that pass the same ``color`` (MPI_Comm_split).
        Collective over this communicator."""
        if self._size == 1:
            return Comm(self.group) if self._active else Comm()
        colors = self.allgather(int(color))
        sub = None
        for c in sorted(set(colors)):
            members = [self._global(r) for r in range(self._size) if colors[r] == c]
            g = dist.new_group(ranks=members)
            if c == color:
                sub = g
        return Comm(sub)

    # -------------------------------------------------------- point to point
    def send(self, data: Any, dest: int, tag: int = 2014) -> None:
        self.isend(data, dest, tag).wait()

    def isend(self, data: Any, dest: int, tag: int = 2014) -> vrequest:
        t = _to_bytes_tensor(data)
        n = torch.tensor([t.numel()], dtype=torch.int64)
        d = self._global(dest)
        w1 = dist.isend(n, d, group=self.group, tag=tag)
        w2 = dist.isend(t, d, group=self.group, tag=tag) if t.numel() else None
        return vrequest([w1, w2], keep=(n, t))

    def recv(self, src: int, tag: int = 2014) -> Any:
        s = self._global(src)
        n = torch.zeros(1, dtype=torch.int64)
        dist.recv(n, s, group=self.group, tag=tag)
        t = torch.empty(int(n.item()), dtype=torch.uint8)
        if t.numel():
            dist.recv(t, s, group=self.group, tag=tag)
        return pickle.loads(t.numpy().tobytes())

    def sendrecv(self, data: Any, dest: int, src: int, stag: int = 2014, rtag: int = 2014) -> Any:
        """Send to ``dest`` while receiving from ``src`` (comm.hpp:505-514)."""
        if self._size == 1:
            return data
        req = self.isend(data, dest, stag)
        out = self.recv(src, rtag)
        req.wait()
        return out

    # ------------------------------------------------------------ collectives
    def bcast(self, data: Any, master: int = 0) -> Any:
        if self._size == 1:
            return data
        box = [data if self._rank == master else None]
        dist.broadcast_object_list(box, src=self._global(master), group=self.group)
        return box[0]

    def allgather(self, data: Any) -> List[Any]:
        if self._size == 1:
            return [data]
        out: List[Any] = [None] * self._size
        dist.all_gather_object(out, data, group=self.group)
        return out

    def bcastring(self, data: Any, func: Callable[[Any], None]) -> None:
        """Every rank sees every rank's ``data`` once: own first, then W-1 ring steps where
        step i sends to (rank - i) and receives from (rank + i) (comm.hpp:541-552)."""
        func(data)
        for i in range(1, self._size):
            dest = (self._rank + self._size - i) % self._size
            src = (self._rank + i) % self._size
            func(self.sendrecv(data, dest, src))

    def alltoall(self, data: Sequence[Any]) -> List[Any]:
        """``data[r]`` goes to rank r; returns what every rank sent to this one (variable
        sizes allowed; W-1 pairwise exchanges like comm.hpp:564-610)."""
        if len(data) != self._size:
            raise ValueError("alltoall needs one item per rank")
        out: List[Any] = [None] * self._size
        out[self._rank] = data[self._rank]
        for i in range(1, self._size):
            dest = (self._rank + self._size - i) % self._size
            src = (self._rank + i) % self._size
            out[src] = self.sendrecv(data[dest], dest, src)
        return out

    def alltoallring(self, data: Sequence[Any], func: Callable[[Any], None]) -> None:
        """Like :meth:`alltoall` but hands each received item to ``func`` as it arrives
        (comm.hpp:613-625)."""
        func(data[self._rank])
        for i in range(1, self._size):
            dest = (self._rank + self._size - i) % self._size
            src = (self._rank + i) % self._size
            func(self.sendrecv(data[dest], dest, src))

    def alltoall_tensors(self, send: List[torch.Tensor]) -> List[torch.Tensor]:
        """Variable-size all-to-all of 1-D tensors through the backend's native collective."""
        if self._size == 1:
            return [send[0]]
        dev = send[0].device
        cnt = torch.tensor([t.numel() for t in send], dtype=torch.int64, device=dev)
        rcnt = torch.empty_like(cnt)
        if dev.type == "cuda":
            dist.all_to_all_single(rcnt, cnt, group=self.group)
            out = torch.empty(int(rcnt.sum().item()), dtype=send[0].dtype, device=dev)
            dist.all_to_all_single(out, torch.cat(send), rcnt.tolist(), cnt.tolist(), group=self.group)
            return list(torch.split(out, rcnt.tolist()))
        got = self.alltoall([t.numpy() for t in send])
        return [torch.from_numpy(np.asarray(g)) for g in got]

    def allreduce(self, data: Any) -> Any:
        """Sum over ranks (the reference supports SUM only, comm.hpp:629-658).  Accepts a
        number, a list of numbers, a numpy array or a tensor; returns the same kind."""
        if self._size == 1:
            return data
        if isinstance(data, torch.Tensor):
            t = data.clone()
            dist.all_reduce(t, group=self.group)
            return t
        if isinstance(data, np.ndarray):
            t = torch.from_numpy(np.ascontiguousarray(data).copy())
            dist.all_reduce(t, group=self.group)
            return t.numpy()
        if isinstance(data, bool):
            data = int(data)
        if isinstance(data, int):
            t = torch.tensor([data], dtype=torch.int64)
            dist.all_reduce(t, group=self.group)
            return int(t.item())
        if isinstance(data, float):
            t = torch.tensor([data], dtype=torch.float64)
            dist.all_reduce(t, group=self.group)
            return float(t.item())
        if isinstance(data, (list, tuple)):
            is_int = all(isinstance(x, int) for x in data)
            t = torch.tensor(list(data), dtype=torch.int64 if is_int else torch.float64)
            dist.all_reduce(t, group=self.group)
            return t.tolist()
        raise TypeError(f"allreduce: unsupported type {type(data)}")

    def treereduce(self, data: Any, func: Callable[[Any, Any], Any], rank: int = 0) -> Any:
        """Binary-tree reduction with a user combiner ``func(mine, received)``; the result
        is valid on ``rank`` (comm.hpp:672-711).  Other ranks get their partial value."""
        size, me = self._size, (self._rank - rank) % self._size  # rotate so that the root is 0
        step = 1
        while step < size:
            if me % (2 * step) == 0:
                partner = me + step
                if partner < size:
                    other = self.recv((partner + rank) % size, tag=4028)
                    data = func(data, other)
            elif me % (2 * step) == step:
                self.send(data, ((me - step) + rank) % size, tag=4028)
                break
            step *= 2
        return data
