"""tcgen05 / TMEM tf32 GEMM against a plain PyTorch fp32 reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(A, B):
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        return (A.double() @ B.double().T).float()
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev


@pytest.mark.parametrize("M,N,K", [(128, 128, 32), (256, 128, 64), (300, 200, 100), (1000, 1024, 128),
                                   (4096, 384, 36), (77, 5, 4)])
def test_gemm_nt_tf32_and_3xtf32(M, N, K):
    from paracel_b200.ops.gemm import gemm_nt
    g = torch.Generator(device="cuda").manual_seed(M * 7 + N)
    A = torch.randn(M, K, device="cuda", generator=g)
    B = torch.randn(N, K, device="cuda", generator=g)
    ref = _ref(A, B)
    C = gemm_nt(A, B)
    torch.cuda.synchronize()
    scale = ref.abs().max().item() + 1e-6
    assert (C - ref).abs().max().item() / scale < 5e-3       # tf32: 10-bit mantissa
    C3 = gemm_nt(A, B, precise=True)
    torch.cuda.synchronize()
    assert (C3 - ref).abs().max().item() / scale < 2e-5      # 3xTF32: fp32-level


def test_gemm_argmin_epilogue_matches_cdist():
    from paracel_b200.ops.gemm import argmin_nt
    g = torch.Generator(device="cuda").manual_seed(5)
    X = torch.randn(5000, 64, device="cuda", generator=g)
    Cn = torch.randn(300, 64, device="cuda", generator=g) * 2
    mn, arg = argmin_nt(X, Cn, precise=True)
    torch.cuda.synchronize()
    d = torch.cdist(X.double(), Cn.double()) ** 2
    ref_arg = d.argmin(1)
    ref_min = d.min(1).values - (X.double() ** 2).sum(1)
    same = (arg.long() == ref_arg)
    # ties / near ties may differ: the chosen centre must be (almost) as close as the best one
    chosen = d[torch.arange(X.shape[0]), arg.long()]
    assert same.float().mean() > 0.999
    assert torch.all(chosen <= d.min(1).values + 1e-3)
    torch.testing.assert_close(mn.double(), ref_min, rtol=1e-4, atol=1e-3)


def test_dense_read_gemm_single_rank():
    from paracel_b200.ops.gemm import DenseReadGemm
    g = torch.Generator(device="cuda").manual_seed(9)
    N, K, M = 260, 64, 700
    op = DenseReadGemm(N, K)
    op.shard.copy_(torch.randn(N, K, device="cuda", generator=g))
    A = torch.randn(M, K, device="cuda", generator=g)
    C = op(A)
    op.check()
    ref = _ref(A, op.shard)
    assert (C - ref).abs().max().item() / ref.abs().max().item() < 5e-3
    op.free()
