"""Two-CTA (tcgen05 cta_group::2) tf32 GEMM against a plain PyTorch fp32 reference and
against the one-CTA kernel."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(A, B):
    return (A.double() @ B.double().T).float()


# wide: 0 = 256 x 256 items, 1 = 256 x 512 items (the last item of a row block is half empty when
# the number of column tiles is odd), -1 = the launcher's choice
@pytest.mark.parametrize("wide", [0, 1, -1])
@pytest.mark.parametrize("M,N,K", [(256, 256, 32), (512, 256, 64), (300, 200, 100), (1000, 1024, 128),
                                   (4096, 384, 36), (77, 5, 4), (2048, 2048, 512), (700, 1300, 1024)])
def test_gemm_2sm_matches_reference(M, N, K, wide):
    from paracel_b200.ops.gemm import check_status, gemm_nt
    g = torch.Generator(device="cuda").manual_seed(M * 7 + N)
    A = torch.randn(M, K, device="cuda", generator=g)
    B = torch.randn(N, K, device="cuda", generator=g)
    ref = _ref(A, B)
    C = gemm_nt(A, B, kernel="2sm", wide=wide)
    check_status()
    scale = ref.abs().max().item() + 1e-6
    assert (C - ref).abs().max().item() / scale < 5e-3
    C1 = gemm_nt(A, B, kernel="1sm")
    check_status()
    assert (C - C1).abs().max().item() / scale < 1e-5      # same products, same order of K steps
    C3 = gemm_nt(A, B, precise=True, kernel="2sm", wide=wide)
    check_status()
    assert (C3 - ref).abs().max().item() / scale < 2e-5


@pytest.mark.parametrize("wide", [0, 1])
def test_gemm_2sm_strided_output_and_argmin(wide):
    from paracel_b200.ops.gemm import argmin_nt, check_status, gemm_nt
    g = torch.Generator(device="cuda").manual_seed(11)
    A = torch.randn(700, 64, device="cuda", generator=g)
    B = torch.randn(520, 64, device="cuda", generator=g)
    big = torch.full((700, 1024), -7.0, device="cuda")
    out = big[:, 256:256 + 520]
    gemm_nt(A, B, out=out, kernel="2sm", wide=wide)
    check_status()
    ref = _ref(A, B)
    assert (out - ref).abs().max().item() / ref.abs().max().item() < 5e-3
    assert torch.all(big[:, :256] == -7.0) and torch.all(big[:, 256 + 520:] == -7.0)

    X = torch.randn(5000, 64, device="cuda", generator=g)
    Cn = torch.randn(300, 64, device="cuda", generator=g) * 2
    mn, arg = argmin_nt(X, Cn, precise=True, kernel="2sm", wide=wide)
    check_status()
    d = torch.cdist(X.double(), Cn.double()) ** 2
    chosen = d[torch.arange(X.shape[0]), arg.long()]
    assert (arg.long() == d.argmin(1)).float().mean() > 0.999
    assert torch.all(chosen <= d.min(1).values + 1e-3)
    ref_min = d.min(1).values - (X.double() ** 2).sum(1)
    torch.testing.assert_close(mn.double(), ref_min, rtol=1e-4, atol=1e-3)


@pytest.mark.parametrize("wide", [0, 1])
def test_dense_read_gemm_2sm_single_rank(wide):
    from paracel_b200.ops.gemm import DenseReadGemm
    g = torch.Generator(device="cuda").manual_seed(9)
    N, K, M = 260, 64, 700
    op = DenseReadGemm(N, K, kernel="2sm", wide=wide)
    op.shard.copy_(torch.randn(N, K, device="cuda", generator=g))
    A = torch.randn(M, K, device="cuda", generator=g)
    C = op(A)
    op.check()
    ref = _ref(A, op.shard)
    assert (C - ref).abs().max().item() / ref.abs().max().item() < 5e-3
    op.free()
