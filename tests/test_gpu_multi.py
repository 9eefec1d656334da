"""Multi-GPU tests (2 ranks, one process per GPU, NCCL for plumbing and plain
peer loads/stores in the kernels).  NVLS is switched off for these runs."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


needs2 = pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")


def _job(n):
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    from paracel_b200.launch.local import LocalJob
    return LocalJob(n, 0, backend="cpu:gloo,cuda:nccl")


@needs2
def test_symmetric_buffers_and_row_tables_across_ranks():
    from paracel_b200.testing.gpu_workers import symm_and_rows
    res = _job(2).run(symm_and_rows, timeout_s=300)
    for r in res:
        assert r["peer_vals"] == [1.0, 2.0]
        assert r["pull_ok"] and r["push_ok"] and r["int_ok"]


@needs2
def test_device_ssp_clock_bound_and_timeout():
    from paracel_b200.testing.gpu_workers import ssp_clock
    res = _job(2).run(ssp_clock, timeout_s=300)
    assert res[0]["max_ahead"] <= 2
    assert res[0]["timeout"] not in (None, "none")
    assert res[0]["alive"] == 4.0


@needs2
def test_mf_two_ranks_converges_like_one_rank():
    from paracel_b200.testing.gpu_workers import mf_train
    args = (3000, 800, 200_000, 32, 5, 2)
    two = _job(2).run(mf_train, args, timeout_s=300)
    one = _job(1).run(mf_train, args, timeout_s=300)
    assert two[0]["nnz_local"] + two[1]["nnz_local"] == 200_000
    assert abs(two[0]["rmse1"] - two[1]["rmse1"]) < 1e-6  # all-reduced metric
    assert two[0]["rmse1"] < two[0]["rmse0"]
    assert abs(two[0]["rmse1"] - one[0]["rmse1"]) < 0.05 * one[0]["rmse1"]


@needs2
@pytest.mark.parametrize("kernel", ["1sm", "2sm"])
def test_fused_allgather_gemm_two_ranks(kernel):
    from paracel_b200.testing.gpu_workers import fused_gather_gemm
    res = _job(2).run(fused_gather_gemm, (1000, 64, 900, kernel), timeout_s=300)
    for r in res:
        assert r["err0"] < 5e-3 and r["err1"] < 5e-3, r
        assert r["argmin_ok"]


@needs2
def test_dense_table_reduce_scatter_handler_two_ranks():
    from paracel_b200.testing.gpu_workers import dense_table_two_ranks
    assert all(_job(2).run(dense_table_two_ranks, timeout_s=300))


@needs2
def test_sparse_l1lr_and_pagerank_two_ranks():
    from paracel_b200.testing.gpu_workers import l1lr_and_pagerank_two_ranks
    for ok_lr, ok_pr in _job(2).run(l1lr_and_pagerank_two_ranks, timeout_s=300):
        assert ok_lr and ok_pr


@needs2
def test_kmeans_allreduce_lda_two_ranks():
    from paracel_b200.testing.gpu_workers import kmeans_allreduce_lda_two_ranks
    for r in _job(2).run(kmeans_allreduce_lda_two_ranks, timeout_s=300):
        assert r["allreduce"] and r["kmeans"], r
        assert r["lda_counts"][0] == r["lda_counts"][2] == r["lda_counts"][1], r
        assert r["lda_ll_up"] and r["lda_consistent"], r


@needs2
@pytest.mark.parametrize("pattern", ["fmap", "fsmap"])
def test_device_loader_exchange_two_ranks(pattern):
    from paracel_b200.testing.gpu_workers import device_exchange_ranks
    res = _job(2).run(device_exchange_ranks, (pattern,), timeout_s=300)
    assert sum(r["n"] for r in res) == 100_000
    for r in res:
        assert r["triples"] and r["maps"] and r["idx"], r
