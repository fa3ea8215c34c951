"""Two-GPU check of the row-sharded SpMM (needs two CUDA devices; skipped otherwise): every exchange form — all-gather,
needed-rows all-to-all, needed rows pulled from the peer's symmetric memory — must reproduce the one-GPU product."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

from conftest import PACKAGE_DIR, ROOT, requires_gpu

pytestmark = requires_gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _graph():
    gen = torch.Generator().manual_seed(41)
    nodes, feat = 20000, 256
    degree = torch.randint(0, 24, (nodes,), generator=gen)
    degree[3], degree[4] = 30000, 0
    rowptr = torch.zeros(nodes + 1, dtype=torch.int64)
    rowptr[1:] = degree.cumsum(0)
    col = torch.randint(0, nodes, (int(rowptr[-1]),), generator=gen)
    col[::3] = col[::3] % 500                                   # hot columns, as in a power-law graph
    value = torch.rand(col.numel(), generator=gen)
    x = torch.randn(nodes, feat, generator=gen)
    return rowptr, col, value, x


def _worker(rank, world, port, result_dir):
    import sys

    for path in (ROOT, PACKAGE_DIR):
        if path not in sys.path:
            sys.path.insert(0, path)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    from ops_gnn.distributed import HaloShardedSpmm, RowShardedSpmm, balanced_row_bounds, shard_csr

    rowptr, col, value, x = (t.to(device) for t in _graph())
    nodes = x.size(0)
    bounds = balanced_row_bounds(rowptr, world, row_cost=4.0)
    ptr, c, v = shard_csr(rowptr, col, value, bounds[rank], bounds[rank + 1])
    results = {}
    gathered = RowShardedSpmm(ptr, c, v, nodes // world, x.size(1), x.dtype, device)
    results["allgather"] = gathered([x[rank * (nodes // world):(rank + 1) * (nodes // world)].contiguous()])[0].cpu()
    mine = x[bounds[rank]:bounds[rank + 1]].contiguous()
    for transport in ("alltoall", "pull"):
        op = HaloShardedSpmm(ptr, c, v, bounds, x.size(1), x.dtype, device, transport=transport)
        first = op(mine)
        second = op(op.own_block)
        assert torch.equal(first, second), transport
        results[transport] = first.cpu()
        results[transport + "_exchange"] = op.exchange_rows()
    from ops_gnn.distributed import StagedHaloSpmm

    for transport in ("alltoall", "push", "copy"):
        op = StagedHaloSpmm(ptr, c, v, bounds, x.size(1), x.dtype, device, stage_fractions=(0.3, 0.3, 0.4),
                            transport=transport)
        first = op(mine)
        second = op(op.own_block)
        assert torch.equal(first, second), "staged " + transport
        results["staged_" + transport] = first.cpu()
        results["staged_" + transport + "_exchange"] = op.exchange_rows()
    from ops_gnn.distributed import HaloShardedSddmm

    left = torch.randn(nodes, 64, generator=torch.Generator().manual_seed(43)).to(device)
    right = torch.randn(nodes, 64, generator=torch.Generator().manual_seed(44)).to(device)
    for transport in ("alltoall", "pull"):
        edge_op = HaloShardedSddmm(ptr, c, bounds, 64, left.dtype, device, transport=transport)
        results["dots_" + transport] = edge_op(left[bounds[rank]:bounds[rank + 1]].contiguous(),
                                               right[bounds[rank]:bounds[rank + 1]].contiguous()).cpu()
    from ops_gnn.distributed import ShardedGatLayer

    heads, width = 4, 64
    feats = torch.randn(nodes, heads, width, generator=torch.Generator().manual_seed(45)).to(device)
    el = torch.randn(nodes, heads, generator=torch.Generator().manual_seed(46)).to(device)
    er = torch.randn(nodes, heads, generator=torch.Generator().manual_seed(47)).to(device)
    own = slice(bounds[rank], bounds[rank + 1])
    layer = ShardedGatLayer(ptr, c, bounds, heads, width, feats.dtype, device, transport="pull")
    results["gat"] = layer(feats[own].contiguous(), el[own].contiguous(), er[own].contiguous()).cpu()
    fused_layer = ShardedGatLayer(ptr, c, bounds, heads, width, feats.dtype, device, transport="alltoall", fused=True)
    results["gat_fused"] = fused_layer(feats[own].contiguous(), el[own].contiguous(), er[own].contiguous()).cpu()
    torch.cuda.synchronize()
    torch.save(results, os.path.join(result_dir, f"rank{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_sharded_spmm_two_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    parts = [torch.load(tmp_path / f"rank{r}.pt") for r in range(world)]
    import sys

    sys.path.insert(0, PACKAGE_DIR)
    from ops_gnn.torch_sparse_spmm import csr_spmm

    rowptr, col, value, x = (t.to("cuda:0") for t in _graph())
    want = csr_spmm(rowptr, col, value, x, "sum").cpu()
    assert parts[0]["staged_alltoall_exchange"] == parts[0]["alltoall_exchange"]   # every remote row moves once
    for form in ("allgather", "alltoall", "pull", "staged_alltoall", "staged_push", "staged_copy"):
        got = torch.cat([p[form] for p in parts], dim=0)
        assert got.shape == want.shape
        # shard boundaries do not move edges between rows and the kernel's order inside a row depends only on the
        # row's own edges, but rows may straddle different block boundaries: compare within the fp32 sum tolerance
        scale = want.abs().max().item()
        assert float((got - want).abs().max()) <= 1e-5 * max(scale, 1.0), form
    import ops_gnn

    left = torch.randn(x.size(0), 64, generator=torch.Generator().manual_seed(43)).to("cuda:0")
    right = torch.randn(x.size(0), 64, generator=torch.Generator().manual_seed(44)).to("cuda:0")
    want_dots = ops_gnn.sddmm_csr(rowptr, col, left, right, "dot", "u", "v").cpu()
    for transport in ("alltoall", "pull"):
        got_dots = torch.cat([p["dots_" + transport] for p in parts])
        assert torch.equal(got_dots, want_dots), "sharded SDDMM, " + transport  # a dot product has one summation order
    heads, width = 4, 64
    feats = torch.randn(x.size(0), heads, width, generator=torch.Generator().manual_seed(45)).to("cuda:0")
    el = torch.randn(x.size(0), heads, generator=torch.Generator().manual_seed(46)).to("cuda:0")
    er = torch.randn(x.size(0), heads, generator=torch.Generator().manual_seed(47)).to("cuda:0")
    edge_rows = ops_gnn.ptr2ind(rowptr, col.numel())
    scores = torch.nn.functional.leaky_relu(ops_gnn.sddmm_csr(rowptr, col, el, er, "add", "u", "v"), 0.2)
    alpha = ops_gnn.scatter_softmax(scores, edge_rows, 0, x.size(0))
    want_gat = ops_gnn.bspmm(rowptr, col, feats, "mul", "sum", rhs=alpha.unsqueeze(-1)).cpu()
    got_gat = torch.cat([p["gat"] for p in parts]).view(-1, heads, width)
    assert float((got_gat - want_gat).abs().max()) <= 1e-5 * max(float(want_gat.abs().max()), 1.0), "sharded GAT layer"
    got_fused = torch.cat([p["gat_fused"] for p in parts]).view(-1, heads, width)
    assert float((got_fused - want_gat).abs().max()) <= 1e-5 * max(float(want_gat.abs().max()), 1.0), "sharded fused GAT layer"
    sent = sum(p["alltoall_exchange"][0] for p in parts)
    received = sum(p["alltoall_exchange"][1] for p in parts)
    assert sent == received and 0 < received < x.size(0)


def _single_rank_worker(rank, world, port, result_dir):
    import sys

    for path in (ROOT, PACKAGE_DIR):
        if path not in sys.path:
            sys.path.insert(0, path)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    dist.init_process_group("nccl", rank=0, world_size=1, device_id=device)
    from ops_gnn.distributed import StagedHaloSpmm
    from ops_gnn.torch_sparse_spmm import csr_spmm

    rowptr, col, value, x = (t.to(device) for t in _graph())
    op = StagedHaloSpmm(rowptr, col, value, [0, x.size(0)], x.size(1), x.dtype, device, stage_fractions=(0.2, 0.3, 0.5))
    staged = op(x)
    want = csr_spmm(rowptr, col, value, x, "sum")
    torch.cuda.synchronize()
    # stage boundaries fall on row boundaries, so every row sees its own edges in the one-GPU order; rows that are cut
    # by other thread-block boundaries than in the one-GPU launch differ in the last bits only
    worst = float((staged - want).abs().max())
    torch.save({"worst": worst, "scale": float(want.abs().max()), "stages": op.stage_rows}, os.path.join(result_dir, "single.pt"))
    dist.destroy_process_group()


def test_staged_spmm_one_gpu(tmp_path):
    """The staged product (three stages, side stream, `csr_spmm_into` writing row ranges of one output) on a single
    rank: no exchange, so it must reproduce the one-launch product; runs on every box, the two-GPU test needs two."""
    mp.spawn(_single_rank_worker, args=(1, _free_port(), str(tmp_path)), nprocs=1, join=True)
    result = torch.load(tmp_path / "single.pt")
    assert len(result["stages"]) == 4 and result["stages"][0] == 0
    assert result["worst"] <= 1e-5 * max(result["scale"], 1.0)
