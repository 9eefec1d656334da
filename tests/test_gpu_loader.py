"""Device loader exchange (placement + scatter kernels, id compaction, CSR) against plain tensor code."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_partition_kernels_with_four_virtual_destinations():
    """One GPU plays all four destinations: the pointer table names four local receive buffers."""
    from paracel_b200.ops import _lib
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(3)
    n, npx, npy = 200_003, 2, 2
    a = torch.randint(0, 5000, (n,), device=dev, generator=g)
    b = torch.randint(0, 7000, (n,), device=dev, generator=g)
    w = torch.rand(n, device=dev, generator=g)
    world = npx * npy
    counts = torch.zeros(world, dtype=torch.int64, device=dev)
    _lib.call("pcl_partition_count", a, b, n, npx, npy, counts, _lib.stream_ptr())
    owner = (a % npx) * npy + (b % npy)
    ref_counts = torch.bincount(owner, minlength=world)
    assert torch.equal(counts, ref_counts)
    cap = int(ref_counts.max().item())
    cap += cap % 2
    bufs = [torch.zeros(2 * cap + cap // 2, dtype=torch.int64, device=dev) for _ in range(world)]
    table = torch.tensor([t.data_ptr() for t in bufs], dtype=torch.int64, device=dev)
    base = torch.zeros(world, dtype=torch.int64, device=dev)
    cursor = torch.zeros(world, dtype=torch.int64, device=dev)
    status = torch.zeros(4, dtype=torch.int64, device=dev)
    _lib.call("pcl_partition_scatter", a, b, w, n, npx, npy, table, cap, base, counts, cursor, status, 0,
              _lib.stream_ptr())
    torch.cuda.synchronize()
    assert int(status[0].item()) == 0
    assert torch.equal(cursor, ref_counts)
    for d in range(world):
        m = int(ref_counts[d].item())
        ra, rb = bufs[d][:m], bufs[d][cap:cap + m]
        rw = bufs[d][2 * cap:].view(torch.float32)[:m]
        sel = owner == d
        got = torch.stack([ra.double(), rb.double(), rw.double()], 1)
        ref = torch.stack([a[sel].double(), b[sel].double(), w[sel].double()], 1)
        # same multiset of triples
        kg = got[:, 0] * 1e6 + got[:, 1] + got[:, 2]
        kr = ref[:, 0] * 1e6 + ref[:, 1] + ref[:, 2]
        assert torch.allclose(torch.sort(kg).values, torch.sort(kr).values)


def test_scatter_refuses_to_overrun_a_short_quota():
    from paracel_b200.ops import _lib
    dev = torch.device("cuda")
    n = 1000
    a = torch.zeros(n, dtype=torch.int64, device=dev)
    b = torch.zeros(n, dtype=torch.int64, device=dev)
    w = torch.ones(n, device=dev)
    cap = 1000
    buf = torch.full((2 * cap + cap // 2,), -1, dtype=torch.int64, device=dev)
    table = torch.tensor([buf.data_ptr()], dtype=torch.int64, device=dev)
    base = torch.zeros(1, dtype=torch.int64, device=dev)
    quota = torch.tensor([10], dtype=torch.int64, device=dev)      # counted 10, but 1000 arrive
    cursor = torch.zeros(1, dtype=torch.int64, device=dev)
    status = torch.zeros(4, dtype=torch.int64, device=dev)
    _lib.call("pcl_partition_scatter", a, b, w, n, 1, 1, table, cap, base, quota, cursor, status, 0,
              _lib.stream_ptr())
    torch.cuda.synchronize()
    assert int(status[0].item()) & 0xFFFFFFFF == 2
    assert int((buf[:cap] == 0).sum().item()) == 10 and bool((buf[10:cap] == -1).all())


def test_device_exchange_single_rank_csr():
    from paracel_b200.load.device_exchange import DeviceExchange
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(5)
    a = torch.randint(0, 300, (5000,), device=dev, generator=g) * 7 + 3
    b = torch.randint(0, 200, (5000,), device=dev, generator=g) * 5 + 1
    w = torch.rand(5000, device=dev, generator=g)
    ex = DeviceExchange("fmap")
    rowptr, col, val, rm, cm = ex.load(a, b, w)
    assert torch.equal(rm, torch.unique(a)) and torch.equal(cm, torch.unique(b))
    dense = torch.zeros(rm.numel(), cm.numel(), dtype=torch.float64, device=dev)
    dense.index_put_((torch.searchsorted(rm, a), torch.searchsorted(cm, b)), w.double(), accumulate=True)
    rows = torch.repeat_interleave(torch.arange(rm.numel(), device=dev), rowptr[1:] - rowptr[:-1])
    back = torch.zeros_like(dense)
    back.index_put_((rows, col.long()), val.double(), accumulate=True)
    assert torch.allclose(dense, back)
    # columns ascend inside every row
    same_row = rows[1:] == rows[:-1]
    assert bool((col[1:][same_row] >= col[:-1][same_row]).all())


def test_paralg_device_matrix_load_matches_host_loader(tmp_path):
    """Same file through the host loader (scipy CSR) and the device loader: same maps, same matrix."""
    import numpy as np
    from paracel_b200.load.parser import gen_parser, parser_a
    from paracel_b200.paralg import paralg
    from paracel_b200.parallel.comm import Comm
    rng = np.random.default_rng(8)
    rows = rng.integers(0, 200, 3000) * 3 + 1
    cols = rng.integers(0, 150, 3000) * 2
    vals = rng.random(3000).round(4)
    seen = {}
    for r, c, v in zip(rows, cols, vals):
        seen[(int(r), int(c))] = float(v)          # unique (row, col) pairs
    p = tmp_path / "m.txt"
    p.write_text("".join(f"{r},{c},{v}\n" for (r, c), v in seen.items()))
    pa = paralg(Comm())
    host_m, host_rm, host_cm = pa.paracel_load_as_matrix(str(p), gen_parser(parser_a, ","), "fsmap")
    rowptr, col, val, rm, cm = pa.paracel_load_as_matrix_device(str(p), gen_parser(parser_a, ","), "fsmap")
    assert rm.cpu().tolist() == [host_rm[i] for i in range(len(host_rm))]
    assert cm.cpu().tolist() == [host_cm[i] for i in range(len(host_cm))]
    dense = np.zeros(host_m.shape)
    rp = rowptr.cpu().numpy()
    ri = np.repeat(np.arange(len(rp) - 1), np.diff(rp))
    dense[ri, col.cpu().numpy()] = val.cpu().numpy()
    assert np.allclose(dense, host_m.toarray(), atol=1e-6)
