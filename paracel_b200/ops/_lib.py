"""ctypes access to ``libpcl_kernels.so`` (the hand-written sm_100a kernels).

Every exported launcher has a C ABI, takes raw device pointers plus a CUDA
stream, and returns a ``cudaError_t``.  The table below is the single place
where the argument types are declared; ``call(name, *args)`` converts tensors
to their data pointers, checks the return code, and raises on failure.

If a CUDA device is present but the library has not been built the import of
any op fails loudly: there is no silent PyTorch fallback for these ops.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

import torch

_LIB = None
_LIB_PATH = Path(__file__).resolve().parent.parent / "_lib" / "libpcl_kernels.so"

_T = {
    "p": ctypes.c_void_p,
    "i": ctypes.c_int,
    "q": ctypes.c_longlong,
    "Q": ctypes.c_ulonglong,
    "f": ctypes.c_float,
    "d": ctypes.c_double,
    "z": ctypes.c_size_t,
}

# name -> argument spec (stream is the trailing "p" where present)
SIGS = {
    "pcl_symm_alloc": "zpp",
    "pcl_symm_open": "pp",
    "pcl_symm_close": "p",
    "pcl_symm_free": "p",
    "pcl_device_sync": "",
    "pcl_rows_pull_f32": "ppiiqpppqQpiqp",
    "pcl_rows_push_f32": "ppiiqpppfiiqqpip",
    "pcl_scalars_pull_f32": "ppiqppqpip",
    "pcl_scalars_push_f32": "ppiqpppiiqpip",
    "pcl_rows_pull_i32": "ppiiqppqpip",
    "pcl_rows_push_i32": "ppiiqppiqpip",
    "pcl_mf_sgd_pass": "pppqppppppifffiifipipppp",
    "pcl_mf_sgd_pass_h16": "pppqppppppfffiifippppipip",
    "pcl_mf_sse": "pppqppppifppp",
    "pcl_gemm_tf32": "pppiiiqipppppiiiiipip",
    "pcl_gemm_tf32_2sm": "pppiiiqipppppiiiiipiip",
    "pcl_split3_tf32": "ppqiip",
    "pcl_dense_read": "ppqqiipqQpp",
    "pcl_dense_bupdate": "ppqqiiiffpqQppppp",
    "pcl_publish_flag": "piiqp",
    "pcl_dense_push": "ppqqiifp",
    "pcl_validate_ids": "piqqqqpip",
    "pcl_lr_dense_grad": "pppqiippppip",
    "pcl_lr_sparse_grad": "pppppqiippip",
    "pcl_pagerank_pull": "ppppqfppppiqpip",
    "pcl_pagerank_pull_stream": "ppppqqppfpppppip",
    "pcl_lda_gibbs": "ppppppqifffQip",
    "pcl_lda_loglik": "ppppppqifffpp",
    "pcl_als_solve": "pppppppppppqifip",
    "pcl_kmeans_accumulate": "ppqippp",
    "pcl_topk_rows": "pqiippfippp",
    "pcl_balltree_search": "pppppppiiipppp",
    "pcl_partition_count": "ppqiipp",
    "pcl_partition_scatter": "pppqiipqppppip",
    "pcl_gram": "pqipp",
    "pcl_spmm_csr": "pppqpipp",
    "pcl_spmm_csr_t": "pppqpipp",
    "pcl_chol_factor": "pippdpp",
    "pcl_allreduce_sum_f64": "ppipppiiiqQpp",
    "pcl_ssp_commit": "piiqpp",
    "pcl_ssp_wait": "piqQpip",
}


class KernelLibraryMissing(RuntimeError):
    pass


def lib_path() -> Path:
    return _LIB_PATH


def register(name: str, spec: str) -> None:
    """Declare the signature of one more exported launcher."""
    SIGS[name] = spec
    if _LIB is not None:
        _bind(name, spec)


def _bind(name, spec):
    fn = getattr(_LIB, name)
    fn.argtypes = [_T[c] for c in spec]
    fn.restype = ctypes.c_int
    return fn


def load():
    global _LIB
    if _LIB is not None:
        return _LIB
    if not _LIB_PATH.exists():
        if os.environ.get("PCL_NO_AUTOBUILD", "0") != "1":
            try:
                from .. import _build
                _build.build_kernels()
            except Exception as e:  # pragma: no cover - build environment specific
                raise KernelLibraryMissing(
                    f"{_LIB_PATH} is missing and could not be built: {e}") from e
        if not _LIB_PATH.exists():
            raise KernelLibraryMissing(f"{_LIB_PATH} is missing; run python -m paracel_b200._build")
    _LIB = ctypes.CDLL(str(_LIB_PATH))
    for name, spec in SIGS.items():
        if hasattr(_LIB, name):
            _bind(name, spec)
    _LIB.pcl_error_string.restype = ctypes.c_char_p
    _LIB.pcl_error_string.argtypes = [ctypes.c_int]
    return _LIB


def available() -> bool:
    return torch.cuda.is_available() and _LIB_PATH.exists()


def _conv(a):
    if a is None:
        return None
    if isinstance(a, torch.Tensor):
        return a.data_ptr()
    return a


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


_LAUNCHES = 0


def launches() -> int:
    """Number of kernel-launching calls made through :func:`call` so far."""
    return _LAUNCHES


def call(name: str, *args) -> None:
    global _LAUNCHES
    lib = load()
    fn = getattr(lib, name)
    rc = fn(*[_conv(a) for a in args])
    _LAUNCHES += 1
    if rc != 0:
        msg = lib.pcl_error_string(rc).decode()
        raise RuntimeError(f"{name} failed: CUDA error {rc} ({msg})")


class DeviceWaitTimeout(RuntimeError):
    """A bounded device-side wait (SSP clock, table flag, tile flag) ran out."""

    def __init__(self, what, rank, wait_id, expected, seen):
        super().__init__(f"{what}: rank {rank}: device wait {wait_id} timed out: expected >= "
                         f"{expected}, saw {seen}")
        self.rank, self.wait_id, self.expected, self.seen = rank, wait_id, expected, seen


class BadDeviceId(IndexError):
    """A kernel met an id outside its table; the access was skipped."""

    def __init__(self, what, rank, where, position, bad_id):
        super().__init__(f"{what}: rank {rank}: id {bad_id} at position {position} is outside the "
                         f"table (kernel {where}); the access was skipped")
        self.rank, self.where, self.position, self.bad_id = rank, where, position, bad_id


def new_status(device) -> torch.Tensor:
    """A zeroed status block (``PclStatus``: code, rank, wait id, pad as four 32-bit words, then
    the expected and the seen value as 64-bit words) that kernels report through."""
    return torch.zeros(4, dtype=torch.int64, device=device)


def check_status(status: torch.Tensor, what: str = "device status") -> None:
    """Read a status block back (synchronises its stream), clear it and raise what it holds:
    code 1 -> :class:`DeviceWaitTimeout`, code 2 -> :class:`BadDeviceId`."""
    st = status.cpu()
    word0 = int(st[0].item())
    code = word0 & 0xFFFFFFFF
    if code == 0:
        return
    rank = (word0 >> 32) & 0xFFFFFFFF
    where = int(st[1].item()) & 0xFFFFFFFF
    a, b = int(st[2].item()), int(st[3].item())
    status.zero_()
    if code == 2:
        raise BadDeviceId(what, rank, where, a, b)
    raise DeviceWaitTimeout(what, rank, where, a, b)


def validate_ids(ids: torch.Tensor, lo: int, hi: int, what: str, skip=None) -> None:
    """Range check of an id array on the device (one pass, then one 32-byte read): raises
    :class:`BadDeviceId` if an element is outside ``[lo, hi)`` and not equal to ``skip``."""
    if ids.numel() == 0:
        return
    if ids.dtype not in (torch.int32, torch.int64) or not ids.is_contiguous():
        raise ValueError(f"{what}: ids must be contiguous int32 or int64")
    st = new_status(ids.device)
    call("pcl_validate_ids", ids, int(ids.dtype == torch.int64), ids.numel(), int(lo), int(hi),
         int(lo if skip is None else skip), st, 0, stream_ptr())
    check_status(st, what)


def check_cuda(t: torch.Tensor, dtype, name: str):
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor")
    if t.dtype != dtype:
        raise ValueError(f"{name} must be {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    return t
