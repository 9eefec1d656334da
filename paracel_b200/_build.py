"""In-tree build of the native parts of paracel_b200.

Two artefacts are produced under ``paracel_b200/_lib``:

* ``libpcl_kernels.so`` -- every ``csrc/cuda/*.cu`` compiled by nvcc for
  sm_100a only (``-gencode arch=compute_100a,code=sm_100a``) and linked into
  one shared object with a plain C ABI (loaded through ctypes);
* ``_pcl_core*.so`` -- the host runtime (KV store, parameter-server daemon,
  wire protocol client, msgpack codec, hash ring, partitioner, parsers,
  ball tree, default handlers) as a pybind11 module.

The reference builds its native parts with CMake (CMakeLists.txt:1-75,
src/CMakeLists.txt:1-16); this file plays that role.  nvcc cross-compiles, so
the build needs no GPU.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
import sysconfig
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIB = ROOT / "_lib"
OBJ = ROOT / "_lib" / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-pthread", "-Wall",
             "-Wno-unused-function"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _stamp(paths, extra="") -> str:
    h = hashlib.sha1(extra.encode())
    for p in sorted(paths):
        h.update(str(p).encode())
        h.update(Path(p).read_bytes())
    return h.hexdigest()


def _run(cmd, verbose):
    if verbose:
        print(" ".join(map(str, cmd)), flush=True)
    r = subprocess.run(list(map(str, cmd)), capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("build failed: %s\n%s\n%s" % (" ".join(map(str, cmd)), r.stdout, r.stderr))
    if verbose and (r.stdout or r.stderr):
        print(r.stdout, r.stderr, flush=True)
    return r


def kernels_path() -> Path:
    return LIB / "libpcl_kernels.so"


def core_path() -> Path:
    return LIB / ("_pcl_core" + sysconfig.get_config_var("EXT_SUFFIX"))


def build_kernels(force=False, verbose=False, ptxas_v=False) -> Path:
    LIB.mkdir(exist_ok=True)
    OBJ.mkdir(exist_ok=True)
    cu = sorted((CSRC / "cuda").glob("*.cu"))
    hdr = sorted((CSRC / "cuda").glob("*.cuh")) + sorted((CSRC / "cuda").glob("*.h"))
    out = kernels_path()
    hdr_stamp = _stamp(hdr, " ".join(NVCC_FLAGS))
    nvcc = _nvcc()
    jobs = []
    objs = []
    for src in cu:
        obj = OBJ / (src.stem + ".o")
        stamp_file = OBJ / (src.stem + ".stamp")
        st = _stamp([src], hdr_stamp)
        objs.append(obj)
        if not force and obj.exists() and stamp_file.exists() and stamp_file.read_text() == st:
            continue
        cmd = [nvcc, *NVCC_FLAGS, "-I", CSRC / "cuda", "-c", src, "-o", obj]
        if ptxas_v:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        jobs.append((cmd, stamp_file, st))
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            futs = [ex.submit(_run, cmd, verbose or ptxas_v) for cmd, _, _ in jobs]
            for f, (_, stamp_file, st) in zip(futs, jobs):
                r = f.result()
                if ptxas_v:
                    print(r.stderr)
                stamp_file.write_text(st)
    if jobs or not out.exists():
        _run([nvcc, "-shared", "-o", out, *objs, "-lcudart"], verbose)
    return out


def build_core(force=False, verbose=False) -> Path:
    import pybind11

    LIB.mkdir(exist_ok=True)
    srcs = sorted((CSRC / "core").glob("*.cpp"))
    hdrs = sorted((CSRC / "core").glob("*.hpp"))
    out = core_path()
    if not srcs:
        return out
    st = _stamp(srcs + hdrs, " ".join(CXX_FLAGS))
    stamp_file = LIB / "core.stamp"
    if not force and out.exists() and stamp_file.exists() and stamp_file.read_text() == st:
        return out
    inc = ["-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"], "-I", CSRC / "core"]
    OBJ.mkdir(exist_ok=True)
    objs = []
    cmds = []
    for s in srcs:
        o = OBJ / ("core_" + s.stem + ".o")
        objs.append(o)
        cmds.append(["g++", *CXX_FLAGS, *inc, "-c", s, "-o", o])
    with cf.ThreadPoolExecutor(max_workers=8) as ex:
        list(ex.map(lambda c: _run(c, verbose), cmds))
    _run(["g++", "-shared", "-pthread", "-o", out, *objs], verbose)
    stamp_file.write_text(st)
    return out


def build_all(force=False, verbose=False):
    k = build_kernels(force=force, verbose=verbose)
    c = build_core(force=force, verbose=verbose)
    return k, c


if __name__ == "__main__":
    force = "--force" in sys.argv
    if "--ptxas" in sys.argv:
        build_kernels(force=True, ptxas_v=True)
    else:
        print(build_all(force=force, verbose="-v" in sys.argv))
