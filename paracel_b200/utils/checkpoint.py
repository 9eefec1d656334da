"""Checkpoint / resume.

The reference has no training checkpoint: it offers final model dumps, the ``pkl_dat``
blobs (include/ps.hpp:929-941, ``unpkl_dat`` is an empty TODO) and ALS's warm start from a
previous run's dump (alg/recommendation/als/als.hpp:84-98).  Here a checkpoint is a
directory with one file per rank:

* host parameter servers: ``servers.pkl`` = every shard's raw key -> packed-value map, written
  by rank 0 (``save_servers`` / ``load_servers``);
* device tables and any other per-rank state: ``rank<r>.pt`` = a dict of tensors and plain
  values (``save_rank_state`` / ``load_rank_state``);
* ``meta.json``: world size, SSP clocks, round counter, user metadata.

Writes go to a temporary name and are renamed, so a crash never leaves a half-written
checkpoint that looks complete."""
from __future__ import annotations

import json
import os
import pickle
from typing import Any, Dict


def _atomic_write(path: str, data: bytes) -> None:
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(data)
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, path)


def save_servers(pt, ckpt_dir: str) -> None:
    """Dump every server shard (collective: call on all ranks; rank 0 writes)."""
    os.makedirs(ckpt_dir, exist_ok=True)
    pt.paracel_sync()
    if pt.get_worker_id() == 0:
        shards = [c.pullall_raw() for c in pt.ps_obj.kvm]
        _atomic_write(os.path.join(ckpt_dir, "servers.pkl"), pickle.dumps(shards))
    pt.paracel_sync()


def load_servers(pt, ckpt_dir: str, clear: bool = True) -> None:
    """Restore the shards.  Keys are re-placed with the current ring, so the number of
    servers may differ from the run that saved the checkpoint."""
    pt.paracel_sync()
    if pt.get_worker_id() == 0:
        with open(os.path.join(ckpt_dir, "servers.pkl"), "rb") as f:
            shards = pickle.load(f)
        if clear:
            for c in pt.ps_obj.kvm:
                c.clear()
        for shard in shards:
            buckets: Dict[int, Dict[str, bytes]] = {}
            for k, raw in shard.items():
                buckets.setdefault(pt.ps_obj.p_ring.get_server(k), {})[k] = raw
            for idx, kv in buckets.items():
                keys = list(kv.keys())
                pt.ps_obj.kvm[idx]._call("push", "push_multi", keys, [kv[k] for k in keys])
    pt.paracel_sync()


def save_meta(ckpt_dir: str, meta: Dict[str, Any]) -> None:
    os.makedirs(ckpt_dir, exist_ok=True)
    _atomic_write(os.path.join(ckpt_dir, "meta.json"), json.dumps(meta, indent=1).encode())


def load_meta(ckpt_dir: str) -> Dict[str, Any]:
    with open(os.path.join(ckpt_dir, "meta.json")) as f:
        return json.load(f)


def save_rank_state(ckpt_dir: str, rank: int, state: Dict[str, Any]) -> None:
    import io
    import torch
    os.makedirs(ckpt_dir, exist_ok=True)
    buf = io.BytesIO()
    torch.save({k: (v.detach().cpu() if hasattr(v, "detach") else v) for k, v in state.items()}, buf)
    _atomic_write(os.path.join(ckpt_dir, f"rank{rank}.pt"), buf.getvalue())


def load_rank_state(ckpt_dir: str, rank: int) -> Dict[str, Any]:
    import torch
    return torch.load(os.path.join(ckpt_dir, f"rank{rank}.pt"), map_location="cpu", weights_only=False)


def exists(ckpt_dir: str) -> bool:
    return os.path.exists(os.path.join(ckpt_dir, "meta.json"))
