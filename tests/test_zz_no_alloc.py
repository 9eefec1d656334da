"""The allocation-free dense-gradient entry point, called through its exported C symbol.

Embedders that may not allocate device memory (a server whose HBM is already owned by one
arena, a plug-in inside another framework's pool, a loop that cannot take cudaMalloc's
device-wide synchronisation) call ``pcl_lr_dense_grad_noalloc``; its scratch is an array
inside the library.  The test checks it against ``pcl_lr_dense_grad`` (caller-provided
scratch) on two calls in a row with different inputs, that a request beyond the built-in
array is refused with a message, and that no device memory is allocated by the calls.
This file sorts last on purpose: a run that stops at the first failure has then already
run every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from paracel_b200.ops import _lib as L
    L.load()
    lib = ctypes.CDLL(str(L.lib_path()))
    fn = lib.pcl_lr_dense_grad_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int,
                   ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
    err = lib.pcl_lr_dense_grad_noalloc_error
    err.restype = ctypes.c_char_p
    return fn, err


def test_no_alloc_entry_point_matches_regular_entry_point_twice():
    from paracel_b200.ops.linear import DenseGrad
    fn, err = _lib()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator(device=dev).manual_seed(123)
    stream = torch.cuda.current_stream().cuda_stream
    for call, (n, d, logistic) in enumerate(((6000, 101, 1), (2500, 257, 0))):
        X = torch.randn(n, d, device=dev, generator=g)
        y = (torch.rand(n, device=dev, generator=g) < 0.4).float()
        theta = 0.2 * torch.randn(d, device=dev, generator=g)
        ref_g = torch.empty(d, device=dev)
        ref_loss = DenseGrad(d, dev)(X, y, theta, ref_g, logistic=bool(logistic)).clone()
        out_g = torch.full((d,), float("nan"), device=dev)
        out_loss = torch.full((1,), float("nan"), device=dev, dtype=torch.float64)
        torch.cuda.synchronize()
        before = torch.cuda.mem_get_info()[0]
        rc = fn(X.data_ptr(), y.data_ptr(), theta.data_ptr(), n, d, logistic, out_g.data_ptr(),
                out_loss.data_ptr(), 0, stream)
        assert rc == 0, err().decode()
        torch.cuda.synchronize()
        after = torch.cuda.mem_get_info()[0]
        assert after >= before - (1 << 20), "the call must not allocate device memory"
        torch.testing.assert_close(out_g, ref_g, rtol=2e-4, atol=2e-3)
        assert abs(float(out_loss.item()) - float(ref_loss.item())) <= 1e-3 * abs(float(ref_loss.item())) + 1e-6


def test_no_alloc_entry_point_rejects_oversized_requests():
    fn, err = _lib()
    dev = torch.device("cuda", 0)
    n, d = 4000, 8000  # 296 blocks x 8000 floats > 1 Mi floats
    X = torch.zeros(n, d, device=dev)
    y = torch.zeros(n, device=dev)
    theta = torch.zeros(d, device=dev)
    out_g = torch.zeros(d, device=dev)
    out_loss = torch.zeros(1, device=dev, dtype=torch.float64)
    rc = fn(X.data_ptr(), y.data_ptr(), theta.data_ptr(), n, d, 1, out_g.data_ptr(),
            out_loss.data_ptr(), 0, torch.cuda.current_stream().cuda_stream)
    assert rc != 0
    assert b"floats of scratch" in err()
    # fewer blocks fit
    rc = fn(X.data_ptr(), y.data_ptr(), theta.data_ptr(), n, d, 1, out_g.data_ptr(),
            out_loss.data_ptr(), 64, torch.cuda.current_stream().cuda_stream)
    assert rc == 0, err().decode()
    torch.cuda.synchronize()
