"""World-size-2 `gloo` test of the row-sharded SpMM plumbing on CPU: nnz-balanced shard bounds, CSR slicing, the
all-gather of the dense blocks (plain and feature-chunked) and reassembly.  The local product is a stand-in (the
oracle's vectorised SpMM) because the product has no CPU path; what is under test is everything around it."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import PACKAGE_DIR, ROOT


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _make_graph():
    gen = torch.Generator().manual_seed(31)
    rows, cols, feat = 400, 64, 12
    degree = torch.randint(0, 6, (rows,), generator=gen)
    degree[3] = 900  # a hub row: equal-row sharding would put almost all edges on rank 0
    rowptr = torch.zeros(rows + 1, dtype=torch.int64)
    rowptr[1:] = degree.cumsum(0)
    col = torch.randint(0, cols, (int(rowptr[-1]),), generator=gen)
    value = torch.rand(col.numel(), generator=gen)
    x = torch.randn(cols, feat, generator=gen)
    return rowptr, col, value, x


def _worker(rank, world, port, chunks, result_dir):
    import sys

    for path in (ROOT, PACKAGE_DIR):
        if path not in sys.path:
            sys.path.insert(0, path)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from ops_gnn.distributed import RowShardedSpmm, balanced_row_bounds, shard_csr
    from oracle.spmm import csr_spmm_sum_vectorised

    rowptr, col, value, x = _make_graph()
    bounds = balanced_row_bounds(rowptr, world)
    ptr, c, v = shard_csr(rowptr, col, value, bounds[rank], bounds[rank + 1])
    block = x.size(0) // world
    op = RowShardedSpmm(ptr, c, v, block, x.size(1), x.dtype, torch.device("cpu"),
                        local_spmm=csr_spmm_sum_vectorised, feature_chunks=chunks)
    mine = op.split_block(x[rank * block:(rank + 1) * block])
    out = torch.cat(op(mine), dim=1)
    torch.save({"bounds": bounds, "out": out, "edges": c.numel()}, os.path.join(result_dir, f"rank{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def _halo_worker(rank, world, port, result_dir):
    import sys

    for path in (ROOT, PACKAGE_DIR):
        if path not in sys.path:
            sys.path.insert(0, path)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from ops_gnn.distributed import HaloShardedSpmm, balanced_row_bounds, shard_csr
    from oracle.spmm import csr_spmm_sum_vectorised

    rowptr, col, value, _ = _make_graph()
    gen = torch.Generator().manual_seed(5)
    x = torch.randn(rowptr.numel() - 1, 12, generator=gen)      # square: X is owned by the same row ranges as A
    col = col * 6 % x.size(0)                                    # columns over all of X, most rows never referenced
    bounds = balanced_row_bounds(rowptr, world, row_cost=1.0)
    ptr, c, v = shard_csr(rowptr, col, value, bounds[rank], bounds[rank + 1])
    op = HaloShardedSpmm(ptr, c, v, bounds, x.size(1), x.dtype, torch.device("cpu"),
                         local_spmm=csr_spmm_sum_vectorised, gather_rows=lambda block, index: block[index])
    out = op(x[bounds[rank]:bounds[rank + 1]])
    again = op(op.own_block)                                     # producing the block in place skips the copy
    assert torch.equal(out, again)
    from ops_gnn.distributed import HaloShardedSddmm
    from oracle import sddmm_oracle

    other = torch.randn(x.size(0), 12, generator=torch.Generator().manual_seed(6))
    edge_op = HaloShardedSddmm(ptr, c, bounds, x.size(1), x.dtype, torch.device("cpu"),
                               local_sddmm=lambda p_, c_, lhs, rhs: sddmm_oracle(p_, c_, lhs, rhs, "dot", "u", "v"),
                               gather_rows=lambda block, index: block[index])
    dots = edge_op(other[bounds[rank]:bounds[rank + 1]], x[bounds[rank]:bounds[rank + 1]])
    torch.save({"out": out, "exchange": op.exchange_rows(), "rows": x.size(0), "col": col, "dots": dots},
               os.path.join(result_dir, f"halo{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def _staged_worker(rank, world, port, fractions, result_dir):
    import sys

    for path in (ROOT, PACKAGE_DIR):
        if path not in sys.path:
            sys.path.insert(0, path)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from ops_gnn.distributed import StagedHaloSpmm, balanced_row_bounds, shard_csr, staged_row_bounds
    from oracle.spmm import csr_spmm_sum_vectorised

    rowptr, col, value, _ = _make_graph()
    x = torch.randn(rowptr.numel() - 1, 12, generator=torch.Generator().manual_seed(5))
    col = col * 6 % x.size(0)
    bounds = balanced_row_bounds(rowptr, world, row_cost=1.0)
    ptr, c, v = shard_csr(rowptr, col, value, bounds[rank], bounds[rank + 1])
    op = StagedHaloSpmm(ptr, c, v, bounds, x.size(1), x.dtype, torch.device("cpu"), stage_fractions=fractions,
                        row_cost=1.0,
                        spmm_into=lambda p_, c_, v_, mat, out: out.copy_(csr_spmm_sum_vectorised(p_, c_, v_, mat)),
                        gather_rows=lambda block, index, outs, ctas: torch.cat(list(outs)).copy_(block[index])
                        if len(outs) > 1 else outs[0].copy_(block[index]))
    out = op(x[bounds[rank]:bounds[rank + 1]])
    assert torch.equal(out, op(op.own_block))                    # producing the block in place skips the copy
    stage_bounds = staged_row_bounds(ptr, fractions, row_cost=1.0)
    assert stage_bounds == op.stage_rows and stage_bounds[0] == 0 and stage_bounds[-1] == ptr.numel() - 1
    assert all(a <= b for a, b in zip(stage_bounds, stage_bounds[1:]))
    # every remote row is fetched once, by the first stage that references it
    remote = torch.unique(c[(c < bounds[rank]) | (c >= bounds[rank + 1])])
    assert op.exchange_rows()[1] == remote.numel() == sum(op.halo_counts)
    torch.save({"out": out, "exchange": op.exchange_rows(), "col": col, "stages": op.halo_counts},
               os.path.join(result_dir, f"staged{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def _check_staged(world, fractions, tmp_path):
    mp.spawn(_staged_worker, args=(world, _free_port(), fractions, str(tmp_path)), nprocs=world, join=True)
    parts = [torch.load(tmp_path / f"staged{r}.pt") for r in range(world)]
    rowptr, _, value, _ = _make_graph()
    x = torch.randn(rowptr.numel() - 1, 12, generator=torch.Generator().manual_seed(5))
    from oracle.spmm import csr_spmm_sum_vectorised

    want = csr_spmm_sum_vectorised(rowptr, parts[0]["col"], value, x)
    got = torch.cat([p["out"] for p in parts], dim=0)
    assert torch.allclose(got, want, rtol=1e-5, atol=1e-5)
    assert sum(p["exchange"][0] for p in parts) == sum(p["exchange"][1] for p in parts) > 0
    return parts


def test_staged_halo_spmm_gloo(tmp_path):
    """Exchange and product overlap stage by stage: three stages on two ranks, an empty stage, and three ranks."""
    parts = _check_staged(2, (0.2, 0.3, 0.5), tmp_path)
    assert all(len(p["stages"]) == 3 for p in parts)
    _check_staged(2, (0.5, 0.0, 0.5), tmp_path)
    _check_staged(3, (1.0,), tmp_path)


def test_halo_sharded_spmm_gloo(tmp_path):
    world = 2
    mp.spawn(_halo_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    parts = [torch.load(tmp_path / f"halo{r}.pt") for r in range(world)]
    rowptr, _, value, _ = _make_graph()
    col = parts[0]["col"]
    x = torch.randn(rowptr.numel() - 1, 12, generator=torch.Generator().manual_seed(5))
    from oracle.spmm import csr_spmm_sum_vectorised

    want = csr_spmm_sum_vectorised(rowptr, col, value, x)
    got = torch.cat([p["out"] for p in parts], dim=0)
    assert torch.allclose(got, want, rtol=1e-5, atol=1e-5)
    sent = sum(p["exchange"][0] for p in parts)
    received = sum(p["exchange"][1] for p in parts)
    assert sent == received and 0 < received < x.size(0)        # fewer rows move than an all-gather would move
    from oracle import sddmm_oracle

    other = torch.randn(x.size(0), 12, generator=torch.Generator().manual_seed(6))
    want_dots = sddmm_oracle(rowptr, col, other, x, "dot", "u", "v")
    assert torch.allclose(torch.cat([p["dots"] for p in parts]), want_dots, rtol=1e-5, atol=1e-5)


def _run(chunks, tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), chunks, str(tmp_path)), nprocs=world, join=True)
    parts = [torch.load(tmp_path / f"rank{r}.pt") for r in range(world)]
    rowptr, col, value, x = _make_graph()
    from oracle.spmm import csr_spmm_sum_vectorised

    want = csr_spmm_sum_vectorised(rowptr, col, value, x)
    got = torch.cat([p["out"] for p in parts], dim=0)
    assert torch.allclose(got, want, rtol=1e-5, atol=1e-5)
    assert parts[0]["bounds"] == parts[1]["bounds"]
    edges = [p["edges"] for p in parts]
    assert sum(edges) == col.numel()
    assert max(edges) <= 0.5 * col.numel() + 900  # balanced up to one row's worth of edges


def test_row_sharded_spmm_gloo(tmp_path):
    _run(1, tmp_path)


def test_row_sharded_spmm_gloo_feature_chunks(tmp_path):
    _run(3, tmp_path)


def test_balanced_bounds_properties():
    import sys

    sys.path.insert(0, PACKAGE_DIR)
    from ops_gnn.distributed import balanced_row_bounds

    rowptr = torch.tensor([0, 0, 0, 10, 10, 11, 30, 30, 31])
    for parts in (1, 2, 3, 8):
        bounds = balanced_row_bounds(rowptr, parts)
        assert bounds[0] == 0 and bounds[-1] == 8 and len(bounds) == parts + 1
        assert all(a <= b for a, b in zip(bounds, bounds[1:]))
    empty = balanced_row_bounds(torch.zeros(5, dtype=torch.int64), 2)
    assert empty[0] == 0 and empty[-1] == 4
    # with a cost per row, a graph without edges is split by rows, and short-row shards get fewer edges
    assert balanced_row_bounds(torch.zeros(5, dtype=torch.int64), 2, row_cost=1.0) == [0, 2, 4]
    degree = torch.cat([torch.full((10,), 100), torch.ones(1000, dtype=torch.int64)])
    skewed = torch.zeros(degree.numel() + 1, dtype=torch.int64)
    skewed[1:] = degree.cumsum(0)
    by_edges = balanced_row_bounds(skewed, 2)
    by_work = balanced_row_bounds(skewed, 2, row_cost=1.0)
    assert by_edges == [0, 10, 1010]
    assert by_work[1] > by_edges[1]
    work = [int(skewed[b] - skewed[a]) + (b - a) for a, b in zip(by_work, by_work[1:])]
    assert abs(work[0] - work[1]) <= 101


def test_host_leg_bounds_pick_the_lightest_busiest_rank():
    """The host-buffer leg of the bench balances its shards on the bytes a rank moves over PCIe: the automatic choice is
    never worse than a fixed row cost, is a valid partition, and is a pure function of the graph."""
    import importlib.util
    import sys

    sys.path.insert(0, PACKAGE_DIR)
    from ops_gnn.distributed import balanced_row_bounds

    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(os.path.dirname(PACKAGE_DIR), "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    generator = torch.Generator().manual_seed(5)
    degree = (torch.rand(50000, generator=generator) ** -0.8).long().clamp(max=4000).sort(descending=True).values
    rowptr = torch.cat([torch.zeros(1, dtype=torch.int64), degree.cumsum(0)])
    for world in (2, 4, 8):
        bounds, choice = bench.host_leg_bounds(rowptr, world, 1024, -1.0, balanced_row_bounds)
        again, _ = bench.host_leg_bounds(rowptr, world, 1024, -1.0, balanced_row_bounds)
        assert bounds == again and bounds[0] == 0 and bounds[-1] == 50000 and len(bounds) == world + 1
        assert all(a <= b for a, b in zip(bounds, bounds[1:]))
        for fixed in (1.0, 51.0, 1e7):
            _, other = bench.host_leg_bounds(rowptr, world, 1024, fixed, balanced_row_bounds)
            assert choice["busiest_rank_bytes"] <= other["busiest_rank_bytes"]
