"""Four-CTA-cluster variant of the two-CTA tf32 GEMM (B shared between the pairs by TMA multicast)
against a plain PyTorch fp32 reference and against the pair kernel.  The kernel ships in an
optional single-GPU library; where that is not installed the tests are skipped."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _need_single():
    from paracel_b200.ops import _lib
    if _lib.load_single() is None:
        pytest.skip("single-GPU kernel library not installed")


def _ref(A, B):
    return (A.double() @ B.double().T).float()


# shapes: one tile pair, an odd number of 256-row blocks (the second pair of the last cluster row
# multiplies rows beyond M), ragged edges, K that is not a multiple of the 32-deep block, many tiles
@pytest.mark.parametrize("M,N,K", [(512, 256, 32), (256, 256, 64), (768, 512, 64), (300, 200, 100),
                                   (1000, 1024, 128), (4096, 384, 36), (77, 5, 4), (2048, 2048, 512),
                                   (5000, 3000, 256)])
def test_gemm_mc_matches_reference(M, N, K):
    _need_single()
    from paracel_b200.ops.gemm import check_status, gemm_nt
    g = torch.Generator(device="cuda").manual_seed(M * 7 + N)
    A = torch.randn(M, K, device="cuda", generator=g)
    B = torch.randn(N, K, device="cuda", generator=g)
    ref = _ref(A, B)
    C = gemm_nt(A, B, kernel="2sm_mc")
    check_status()
    scale = ref.abs().max().item() + 1e-6
    assert (C - ref).abs().max().item() / scale < 5e-3
    C2 = gemm_nt(A, B, kernel="2sm")
    check_status()
    assert (C - C2).abs().max().item() / scale < 1e-5      # same products, same order of K steps
    C3 = gemm_nt(A, B, precise=True, kernel="2sm_mc")
    check_status()
    assert (C3 - ref).abs().max().item() / scale < 2e-5


def test_gemm_mc_strided_output_and_argmin():
    _need_single()
    from paracel_b200.ops.gemm import argmin_nt, check_status, gemm_nt
    g = torch.Generator(device="cuda").manual_seed(11)
    A = torch.randn(700, 64, device="cuda", generator=g)
    B = torch.randn(520, 64, device="cuda", generator=g)
    big = torch.full((700, 1024), -7.0, device="cuda")
    out = big[:, 256:256 + 520]
    gemm_nt(A, B, out=out, kernel="2sm_mc")
    check_status()
    ref = _ref(A, B)
    assert (out - ref).abs().max().item() / ref.abs().max().item() < 5e-3
    assert torch.all(big[:, :256] == -7.0) and torch.all(big[:, 256 + 520:] == -7.0)

    X = torch.randn(5000, 64, device="cuda", generator=g)
    Cn = torch.randn(300, 64, device="cuda", generator=g) * 2
    mn, arg = argmin_nt(X, Cn, precise=True, kernel="2sm_mc")
    check_status()
    d = torch.cdist(X.double(), Cn.double()) ** 2
    chosen = d[torch.arange(X.shape[0]), arg.long()]
    assert (arg.long() == d.argmin(1)).float().mean() > 0.999
    assert torch.all(chosen <= d.min(1).values + 1e-3)


def test_default_kernel_is_multicast_only_in_single_process():
    _need_single()
    from paracel_b200.ops import gemm
    assert gemm._entry("auto") == "pcl_gemm_tf32_2sm_mc"
    op = gemm.DenseReadGemm(260, 64)
    assert op.entry == "pcl_gemm_tf32_2sm"        # shards can be peers' memory
    op.free()
