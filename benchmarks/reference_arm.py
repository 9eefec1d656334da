"""Reference arm of bench.py: drive an installed, unmodified build of the reference through
its own executables for the same metric (rating updates/s of one MF-SGD round).

The reference is a CMake C++11 project (no Python packaging); a build installs
``bin/start_server``, ``bin/paracelrun_cpp_proxy`` and ``bin/mf`` plus ``lib/libmf_update.so``
and ``lib/libmf_filter.so``.  When such a tree exists under ``baseline/_ref`` this module plays
the role of the reference's ``prun.py`` local mode (prun.py:144-176, which is Python 2): it
starts the servers, collects their ``host:ports`` lines through the rendezvous proxy, runs
``mpirun -n W bin/mf --server_info ... --cfg_file ...`` on a rating file in the reference's input
format (``user item date rating``, mf.hpp:39-43) and times the run around the worker command.
Nothing of this repository's models or kernels is on that path.

When no build is installed the arm prints one line that names what is missing.
"""
from __future__ import annotations

import json
import os
import shutil
import subprocess
import tempfile
import time
from pathlib import Path
from typing import Dict, List, Optional

ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "baseline" / "_ref"
NEEDED = ("start_server", "paracelrun_cpp_proxy", "mf")
BUILD_DEPS = ("MPI (mpicxx/mpirun)", "ZeroMQ >= 3.2", "msgpack-c", "Boost", "Eigen3", "gflags", "glog")


def find_reference_install() -> Optional[Dict[str, Path]]:
    """Paths of the reference's executables under baseline/_ref, or None."""
    found: Dict[str, Path] = {}
    for name in NEEDED:
        for cand in (REF / "bin" / name, REF / name, REF / "local" / "bin" / name):
            if cand.is_file() and os.access(cand, os.X_OK):
                found[name] = cand
                break
    return found if len(found) == len(NEEDED) else None


def _missing_reason() -> str:
    parts: List[str] = []
    if not REF.exists() or not any(REF.iterdir()):
        parts.append("no reference build under baseline/_ref")
    else:
        have = find_reference_install() or {}
        parts.append("baseline/_ref lacks " + ", ".join(n for n in NEEDED if n not in have))
    parts.append("the reference is a CMake C++11 project without setup.py/pyproject.toml (pip cannot "
                 "install it) and its build needs " + ", ".join(BUILD_DEPS))
    absent = [t for t in ("mpirun", "mpicxx", "cmake") if shutil.which(t) is None]
    if absent:
        parts.append("not on this machine: " + ", ".join(absent))
    for hdr, what in (("/usr/include/zmq.h", "zmq.h"), ("/usr/include/msgpack.hpp", "msgpack.hpp"),
                      ("/usr/include/boost/version.hpp", "boost"), ("/usr/include/eigen3", "eigen3"),
                      ("/usr/include/gflags/gflags.h", "gflags"), ("/usr/include/glog/logging.h", "glog")):
        if not os.path.exists(hdr):
            parts.append("no " + what)
    return "; ".join(parts)


def _write_ratings(path: Path, args) -> int:
    """The bench's synthetic ratings in the reference's text format.  Generated on the CPU with
    the same seeded stream as the GPU arm (torch generators are device specific, so the draws
    differ from the GPU stream; the distribution and the sizes are the same)."""
    import torch
    from paracel_b200.utils.synth import MfRatingStream
    st = MfRatingStream(args.users, args.items, args.nnz, s=args.zipf_s, seed=args.seed, device="cpu",
                        chunk=1 << 22)
    n = 0
    with open(path, "w") as f:
        for u, i, r in st:
            rows = torch.stack([u, i, torch.zeros_like(u), r.long()], 1).tolist()
            f.write("".join("%d %d %d %d\n" % tuple(row) for row in rows))
            n += len(rows)
    return n


def run_reference_arm(args) -> dict:
    inst = find_reference_install()
    if inst is None or shutil.which("mpirun") is None:
        return {"impl": "reference", "unavailable": _missing_reason()}
    nworkers = max(1, int(os.environ.get("PCL_REF_WORKERS", str(os.cpu_count() or 1))))
    nservers = max(1, int(os.environ.get("PCL_REF_SERVERS", str(max(1, nworkers // 5)))))
    work = Path(tempfile.mkdtemp(prefix="pcl_ref_"))
    env = dict(os.environ, LD_LIBRARY_PATH=str(REF / "lib") + os.pathsep + os.environ.get("LD_LIBRARY_PATH", ""))
    servers = proxy = None
    try:
        t0 = time.time()
        nnz = _write_ratings(work / "ratings.txt", args)
        prep_s = time.time() - t0
        rounds = args.steps + args.warmup
        cfg = {"input": str(work / "ratings.txt"), "predict_input": "", "output": str(work / "out") + "/",
               "update_file": str(REF / "lib" / "libmf_update.so"),
               "update_functions": ["cnt_updater", "mf_fac_updater", "mf_bias_updater"],
               "filter_file": str(REF / "lib" / "libmf_filter.so"),
               "filter_functions": ["mf_ubias_filter", "mf_ibias_filter", "mf_W_filter", "mf_H_filter"],
               "k": args.rank, "rounds": rounds, "alpha": args.alpha, "beta": args.beta, "debug": False,
               "ssp_switch": True, "limit_s": args.staleness}
        (work / "cfg.json").write_text(json.dumps(cfg))
        port = 7773
        proxy = subprocess.Popen([str(inst["paracelrun_cpp_proxy"]), "--nsrv", str(nservers), "--init_port",
                                  str(port)], stdout=subprocess.PIPE, env=env, text=True)
        servers = subprocess.Popen(["mpirun", "-n", str(nservers), str(inst["start_server"]), "--start_host",
                                    "127.0.0.1", "--init_port", str(port)], env=env)
        server_info = proxy.stdout.readline().strip()
        t1 = time.time()
        rc = subprocess.run(["mpirun", "-n", str(nworkers), str(inst["mf"]), "--server_info", server_info,
                             "--cfg_file", str(work / "cfg.json")], env=env).returncode
        wall = time.time() - t1
        if rc != 0:
            return {"impl": "reference", "unavailable": f"the reference's mf executable exited with code {rc}"}
        # the executable reports no per-round time; loading and initialisation are inside the wall clock
        value = nnz * rounds / wall
        return {"metric": "rating updates/s (MF-SGD)", "value": value, "unit": "rating updates/s",
                "impl": "reference", "n_gpus": 0, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": wall * 1e3 / rounds, "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "fp64", "data": "synthetic (same generator, CPU stream)",
                "config": {"model": "biased MF, SGD, rank %d fp64 (reference executable mf)" % args.rank,
                           "ratings": nnz, "workers": nworkers, "servers": nservers,
                           "timing": "wall clock around mpirun of the worker executable, all rounds "
                                     "including its own file loading; input generation (%.0f s) excluded" % prep_s},
                "e2e": {"value": value, "unit": "rating updates/s", "h2d_bytes_per_step": 0,
                        "d2h_bytes_per_step": 0},
                "gpu_launches": 0}
    finally:
        for p in (servers, proxy):
            if p is not None and p.poll() is None:
                p.terminate()
        shutil.rmtree(work, ignore_errors=True)
