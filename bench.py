#!/usr/bin/env python
"""Headline benchmark: CSR SpMM-sum on an R-MAT graph (BASELINE config 4), nnz*feat/s and fraction of HBM peak.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--scale S] [--feat F] [--dtype fp32|bf16]

One "step" is one SpMM over the whole graph: out = A @ X with A an R-MAT(0.57/0.19/0.19/0.05) graph of 2**scale
nodes and 16 * 2**scale drawn edges (deduplicated), fp32 edge weights U[0,1), X ~ N(0,1) with `feat` columns.  The
default (scale 24, feat 256, fp32: 16.7M nodes, 256M drawn edges) is the configuration the metric is quoted on.
All inputs are seeded synthetic tensors generated on the GPU; no dataset is read.

The line printed by rank 0 carries
  value         whole-job nnz*feat/s with inputs resident in HBM (CUDA events, K steps, max over ranks),
  e2e           the same metric through the public API `ops_gnn.torch_sparse_spmm.csr_spmm` with HOST buffers: the
                pinned-host -> device copies of rowptr/col/value/X and the device -> host copy of the result are inside
                the timed region (N > 1: every rank moves its own CSR slice, block of X and output rows through
                `ops_gnn.distributed.RowShardedSpmm`),
  roofline      algorithmic bytes of one step / measured step time against the measured HBM copy bandwidth (N > 1: per
                rank, the local product alone),
  parity_check  rows of the timed product copied to the host and compared with the float64 CPU oracle of the same rows
                (N > 1: every rank checks rows of its own shard against the oracle fed with the TRUE rows of X, so a
                wrong exchange shows; the verdicts are reduced over the ranks),
  cpu_baseline  the CPU oracle (vectorised restatement of the reference's golden) on a bounded row sample, all host
                threads (N = 1 only),
  ops           the other half of the metric after the timed SpMM: at N = 1 `sddmm_csr` dot on BASELINE config 3 (nnz/s,
                roofline) and the GAT layer of config 5 by the functions of bench_ops.py; at N > 1 the sharded SDDMM and
                the sharded fused GAT layer,
  clocks        SM clock and throttle reasons sampled by nvidia-smi during the timed region.
  step_ms       min / median / max of the K single steps (rank 0), beside ms_per_step = timed region / K.

N > 1 (torchrun, one rank per GPU; strong scaling: the graph is fixed): output rows are split into contiguous ranges
of equal work (edges + 6 per row) and X is owned by the same row ranges.  Each step moves only the rows of X a shard
references.  `--exchange staged` cuts every shard into consecutive row stages whose exchanges (packs on one stream,
NCCL all-to-alls of a high-priority group on another) run while the products of earlier stages compute;
`--exchange staged_push` is the same pipeline with the gather kernel storing the rows straight into the peers'
symmetric-memory buffers; `--exchange staged_copy` moves the packed rows with copy-engine transfers;
`--exchange halo` / `pull` are the unstaged forms (whole exchange, then the product); `--exchange allgather`
all-gathers all of X.  The default picks what measured fastest at each N: staged_push at 2, staged up to 4, halo beyond.
`sharding.phases_ms` gives, for one extra step after the timed region, the time from the step's start to the end of
every phase (max over ranks); the `x_resident` record times the local SpMM alone.  The host-buffer leg at N > 1 uses
the all-gather form with shard bounds balanced on the bytes every rank moves over PCIe (`--e2e-row-cost`).
`--impl reference` times the reference's CPU algorithm (the oracle port) on the host cores for the same metric.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "ops-gnn_b200"))
sys.path.insert(0, ROOT)

RMAT = (0.57, 0.19, 0.19, 0.05)
# dram__bytes_read.sum + dram__bytes_write.sum of one ReduceKernel launch, from a 1-pass ncu capture of this workload at
# full size (a profiler figure, copied here; not measured by this script; the capture's summary is kept under profiles/)
NCU_DRAM_TRAFFIC = {"rmat_s24_ef16_f256_fp32_spmm_sum": 203.84e9, "rmat_s24_ef16_f256_bf16_spmm_sum": 87.44e9}
SEED = 20261125 + 4


# ---- synthetic workload -------------------------------------------------------------------------------------------------
def rmat_csr(scale, edges_drawn, device, seed=SEED, index_dtype=torch.int64):
    """Deduplicated, row-sorted R-MAT graph as (rowptr, col); 2**scale nodes, no vertex permutation."""
    a, b, c, _ = RMAT
    gen = torch.Generator(device=device).manual_seed(seed)
    chunk = min(edges_drawn, 1 << 26)
    keys = []
    for start in range(0, edges_drawn, chunk):
        count = min(chunk, edges_drawn - start)
        row = torch.zeros(count, dtype=torch.int64, device=device)
        col = torch.zeros(count, dtype=torch.int64, device=device)
        for _ in range(scale):
            u = torch.rand(count, device=device, generator=gen)
            row_bit = u >= a + b
            col_bit = ((u >= a) & (u < a + b)) | (u >= a + b + c)
            row = (row << 1) | row_bit
            col = (col << 1) | col_bit
        keys.append((row << scale) | col)
        del row, col, u, row_bit, col_bit
    keys = torch.cat(keys) if len(keys) > 1 else keys[0]
    keys = torch.unique_consecutive(torch.sort(keys).values)
    rows = keys >> scale
    col = (keys & ((1 << scale) - 1)).to(index_dtype)
    del keys
    nodes = 1 << scale
    counts = torch.bincount(rows, minlength=nodes)
    del rows
    rowptr = torch.zeros(nodes + 1, dtype=torch.int64, device=device)
    torch.cumsum(counts, 0, out=rowptr[1:])
    return rowptr.to(index_dtype), col


def algorithmic_bytes(rows, nnz, feat, elem, index_bytes=8):
    """nnz*(col + weight + one dense row) + rows*(pointer + one output row): no cache credit for the gathers."""
    return nnz * (index_bytes + elem + feat * elem) + rows * (index_bytes + feat * elem)


# ---- clocks ---------------------------------------------------------------------------------------------------------------
class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        self.proc.wait()
        self.file.flush()
        self.file.seek(0)
        clocks, maxima, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.file.read().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                clocks.append(float(parts[1]))
                maxima.append(float(parts[2]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[5:9]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.file.name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": max(maxima) if maxima else None,
                "reasons": sorted(reasons), "samples": len(clocks)}


# ---- CPU arm and parity sample ---------------------------------------------------------------------------------------------
def row_sample(rowptr, col, value, x_rows_of, target_edges, base=0):
    """A contiguous row range around the median edge of (rowptr, col) holding about `target_edges` edges, as a graph of
    its own on the host: pointers rebased, columns relabelled to the distinct rows they reference, and those rows of X
    (`x_rows_of(ids)` gathers them on the device).  Returns a dict of host tensors plus the row range."""
    nnz = int(rowptr[-1]) - int(rowptr[0])
    start = int(rowptr[0])
    probe = torch.tensor([start + nnz // 2, start + min(nnz // 2 + target_edges, nnz)], device=rowptr.device, dtype=rowptr.dtype)
    first = max(int(torch.searchsorted(rowptr, probe[:1], right=True)) - 1, 0)
    last = min(max(int(torch.searchsorted(rowptr, probe[1:], right=False)), first + 1), rowptr.numel() - 1)
    lo, hi = int(rowptr[first]) - start, int(rowptr[last]) - start
    distinct, local = torch.unique(col[lo:hi], return_inverse=True)
    return {"ptr": (rowptr[first:last + 1] - rowptr[first]).cpu(), "col": local.cpu(), "value": value[lo:hi].float().cpu(),
            "x": x_rows_of(distinct).float().cpu(), "first": first + base, "last": last + base, "rows": (first, last),
            "edges": hi - lo}


def parity_of(sample, gpu_rows, tolerance):
    """Largest |gpu - oracle| over the sample's rows, relative to the magnitude each row summed (float64 oracle)."""
    from oracle.spmm import csr_spmm_sum_vectorised

    torch.set_num_threads(os.cpu_count() or 1)
    want = csr_spmm_sum_vectorised(sample["ptr"], sample["col"], sample["value"].double(), sample["x"].double())
    size = csr_spmm_sum_vectorised(sample["ptr"], sample["col"], sample["value"].double().abs(), sample["x"].double().abs())
    error = float(((gpu_rows.double().cpu() - want).abs() / size.clamp(min=1.0)).max()) if want.numel() else 0.0
    return {"rows": [sample["first"], sample["last"]], "edges": sample["edges"], "max_rel_err": error,
            "tolerance": tolerance, "ok": bool(error <= tolerance),
            "oracle": "oracle.spmm.csr_spmm_sum_vectorised in float64; error relative to max(1, sum |w x|) of the row"}


def time_cpu(sample, repeats):
    from oracle.spmm import csr_spmm_sum_vectorised

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    args = (sample["ptr"], sample["col"], sample["value"], sample["x"])
    csr_spmm_sum_vectorised(*args)  # warm the allocator and the thread pool
    times = []
    for _ in range(repeats):
        start = time.perf_counter()
        csr_spmm_sum_vectorised(*args)
        times.append(time.perf_counter() - start)
    return min(times), threads


# ---- main -----------------------------------------------------------------------------------------------------------------
def parse():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=10)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="ours", choices=("ours", "reference"))
    parser.add_argument("--scale", type=int, default=24, help="log2(nodes); 24 is the quoted configuration")
    parser.add_argument("--edge-factor", type=int, default=16)
    parser.add_argument("--feat", type=int, default=256)
    parser.add_argument("--dtype", default="fp32", choices=("fp32", "bf16"))
    parser.add_argument("--exchange", default="auto",
                        choices=("auto", "staged", "staged_push", "staged_copy", "allgather", "halo", "pull"),
                        help="N > 1: staged = row stages whose pack + NCCL all-to-all overlap with the products of "
                             "earlier stages; staged_push = the same with the gather kernel storing into the peers' "
                             "symmetric memory; staged_copy = packed rows moved by copy-engine transfers into the peers' "
                             "symmetric memory; halo / pull = the unstaged forms; allgather = all of X every step; "
                             "auto = staged_push between two GPUs, staged up to four, halo beyond (what measured fastest)")
    parser.add_argument("--stages", default="0.1,0.2,0.3,0.4",
                        help="staged exchanges: shares of a shard's work per stage, in row order")
    parser.add_argument("--copy-streams", type=int, default=4,
                        help="N > 1, --exchange staged_copy: streams the per-peer copies of a stage are spread over")
    parser.add_argument("--nccl-priority", type=int, default=1,
                        help="N > 1, --exchange staged: 1 = the all-to-alls run in a NCCL group with a high-priority stream")
    parser.add_argument("--exchange-ctas", type=int, default=148,
                        help="staged exchanges: thread blocks of the pack / push kernel that runs beside the products")
    parser.add_argument("--row-cost", type=float, default=6.0, help="N > 1: cost of one output row in edges (shard balance)")
    parser.add_argument("--e2e-row-cost", type=float, default=-1.0,
                        help="N > 1: the same for the host-buffer leg; negative = pick, among a few candidates, the one whose "
                             "busiest rank moves the fewest bytes over PCIe")
    parser.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    parser.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg (profiling runs)")
    parser.add_argument("--no-ops", action="store_true", help="skip the SDDMM / GAT legs, single-GPU and sharded (profiling runs)")
    return parser.parse_args()


def workload_name(args):
    return f"rmat_s{args.scale}_ef{args.edge_factor}_f{args.feat}_{args.dtype}_spmm_sum"


SAMPLE_EDGES = 1 << 22          # CPU sample of the N = 1 run (timed as the CPU baseline and used as the parity check)
SHARD_SAMPLE_EDGES = 1 << 20    # parity sample of every rank at N > 1


def main():
    args = parse()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference" and rank != 0:
        return 0
    if not torch.cuda.is_available():
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "no CUDA device to generate the seeded workload"}))
            return 0
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    distributed = world > 1 and args.impl == "ours"
    args.host_binding = bind_near_gpu(local) if distributed else None
    if distributed:
        # plain peer loads / stores and NCCL rings only: no NVLS, no multicast binding of symmetric memory
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=device)
    dtype = torch.float32 if args.dtype == "fp32" else torch.bfloat16
    elem = 4 if dtype == torch.float32 else 2
    tolerance = 1e-5 if dtype == torch.float32 else 1e-2
    nodes = 1 << args.scale

    # ---- inputs (seeded; identical on every rank) ------------------------------------------------------------------
    rowptr, col = rmat_csr(args.scale, args.edge_factor * nodes, device)
    nnz = col.numel()
    gen = torch.Generator(device=device).manual_seed(SEED + 1)
    value = torch.rand(nnz, device=device, generator=gen).to(dtype)
    x = torch.randn(nodes, args.feat, device=device, generator=gen, dtype=torch.float32).to(dtype)
    # the same keys in both arms: the driver compares the two `config` objects
    config = {"workload": workload_name(args), "nodes": nodes, "nnz": nnz, "feat": args.feat,
              "index_dtype": "int64", "l2": "inputs_larger_than_l2", "seed": SEED}

    if args.impl == "reference":
        return reference_arm(args, rowptr, col, value, x, config)

    import ops_gnn
    from ops_gnn.torch_sparse_spmm import csr_spmm

    forward = ops_gnn._pybind.torch_sparse_spmm.forward
    out_code = 0 if dtype == torch.float32 else 2
    sharding = {"parallelism": "single_gpu"}

    # ---- shard (work-balanced contiguous row ranges) -------------------------------------------------------------------
    sharded = None
    if distributed:
        from ops_gnn.distributed import (HaloShardedSpmm, RowShardedSpmm, StagedHaloSpmm, balanced_row_bounds, shard_csr)

        # a row end costs the kernel about four edges on this graph (measured per rank: 0.13 ns per edge, 0.6 ns per row)
        bounds = balanced_row_bounds(rowptr, world, row_cost=args.row_cost)
        my_ptr, my_col, my_val = shard_csr(rowptr, col, value, bounds[rank], bounds[rank + 1])
        sharding = {"shard_rows": [bounds[k + 1] - bounds[k] for k in range(world)], "row_cost": args.row_cost}
        # parity sample of this rank, taken while all of X is still here: rows of the shard around its median edge with
        # the TRUE rows of X they reference (global column ids), so the check below does not depend on the exchange
        sample = row_sample(my_ptr, my_col, my_val, lambda ids: x[ids], SHARD_SAMPLE_EDGES, base=bounds[rank])
        host_shard = None
        if not args.no_e2e:
            # The host-buffer leg is bound by PCIe, not by the kernel: it gets its own shard bounds (balanced on the bytes
            # every rank moves, see host_leg_bounds) and equal blocks of X.
            e2e_bounds, e2e_choice = host_leg_bounds(rowptr, world, args.feat * elem, args.e2e_row_cost, balanced_row_bounds)
            sharding["e2e_shards"] = e2e_choice
            block = nodes // world
            pieces = shard_csr(rowptr, col, value, e2e_bounds[rank], e2e_bounds[rank + 1])
            host_shard = [torch.empty(t.shape, dtype=t.dtype, pin_memory=True).copy_(t)
                          for t in (*pieces, x[rank * block:(rank + 1) * block])]
            del pieces
        if args.exchange == "auto":
            # measured on this graph, ms per step: 2 GPUs 22.5 (staged_push) / 22.2 - 23.7 (staged_copy) / 24.4 (staged) /
            # 25.5 (halo); 4 GPUs 18.7 / - / 17.6 / 18.8; 8 GPUs, three boxes: halo 12.4 - 15.1, staged 12.3 - 12.5 on the
            # box where halo took 12.4, staged_copy 13.8 where halo took 15.1, staged_push 18.6 where halo took 13.7
            args.exchange = "staged_push" if world == 2 else ("staged" if world <= 4 else "halo")
        if args.exchange in ("halo", "pull", "staged", "staged_push", "staged_copy"):
            # X is owned by the same row ranges as the output (a layer's output rows are the next layer's input)
            x_block = x[bounds[rank]:bounds[rank + 1]].clone()
            del rowptr, col, value, x
            torch.cuda.empty_cache()
            fractions = [float(f) for f in args.stages.split(",")]

            exchange_group = None
            if args.exchange in ("staged", "staged_copy") and args.nccl_priority:
                from ops_gnn.distributed import high_priority_group

                try:
                    exchange_group = high_priority_group()
                    sharding["nccl_stream"] = "high priority"
                except (RuntimeError, AttributeError, TypeError) as exc:  # the option is missing in this torch build
                    sharding["nccl_stream"] = f"default priority ({type(exc).__name__})"

            def build(kind):
                if kind in ("staged", "staged_push", "staged_copy"):
                    return StagedHaloSpmm(my_ptr, my_col, my_val, bounds, args.feat, dtype, device,
                                          group=exchange_group if kind == "staged" else None,
                                          barrier_group=exchange_group if kind == "staged_copy" else None,
                                          stage_fractions=fractions, row_cost=args.row_cost,
                                          transport={"staged": "alltoall", "staged_push": "push", "staged_copy": "copy"}[kind],
                                          exchange_ctas=args.exchange_ctas, copy_streams=args.copy_streams)
                return HaloShardedSpmm(my_ptr, my_col, my_val, bounds, args.feat, dtype, device,
                                       transport="pull" if kind == "pull" else "alltoall")

            fallback = {"staged_push": "staged", "staged_copy": "staged", "pull": "halo"}
            try:
                sharded, failure = build(args.exchange), None
            except (RuntimeError, ImportError, AttributeError) as exc:  # symmetric memory unavailable on this box
                sharded, failure = None, f"{type(exc).__name__}: {exc}"[:200]
            agreed = torch.tensor([0 if failure else 1], device=device)
            dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
            if int(agreed.item()) == 0:  # every rank falls back together
                if args.exchange not in fallback:
                    raise RuntimeError(f"sharded SpMM set-up failed: {failure}")
                sharded = None
                torch.cuda.empty_cache()
                args.exchange = fallback[args.exchange]
                sharded = build(args.exchange)
                sharding["exchange_fallback"] = failure or "symmetric memory set-up failed on another rank"
            x_block = sharded.own_block.copy_(x_block)        # produce the block where the exchange reads it
            sent, received = sharded.exchange_rows()
            sharding["parallelism"] = f"row_shard{world}_{args.exchange}_x"
            sharding["halo_rows_rank0"] = {"sent": sent, "received": received}
            if args.exchange.startswith("staged"):
                sharding["stage_fractions"] = fractions
                sharding["exchange_ctas"] = args.exchange_ctas
                sharding["stage_halo_rows_rank0"] = sharded.halo_counts
            local_ptr, local_col, local_x = my_ptr, sharded.col, sharded.compact
        else:
            block = nodes // world
            x_block = x[rank * block:(rank + 1) * block].clone()
            del rowptr, col, value, x
            torch.cuda.empty_cache()
            sharded = RowShardedSpmm(my_ptr, my_col, my_val, block, args.feat, dtype, device)
            local_ptr, local_col, local_x = my_ptr, my_col, sharded.gathered[0]  # filled by every step's all-gather
            sharding["parallelism"] = f"row_shard{world}_allgather_x"
    else:
        my_ptr, my_col, my_val = rowptr, col, value
        x_block = None
        sample = None if args.no_cpu else row_sample(rowptr, col, value, lambda ids: x[ids], SAMPLE_EDGES)

    def step():
        if distributed:
            return sharded([x_block])[0] if args.exchange == "allgather" else sharded(x_block)
        return forward(my_ptr, my_col, my_val, x, 0, out_code)[0]

    def barrier():
        torch.cuda.synchronize()
        if distributed:
            dist.barrier()
        torch.cuda.synchronize()

    out = None
    for _ in range(max(args.warmup, 3)):
        out = step()
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    marks = []
    for _ in range(args.steps):
        out = step()
        marks.append(torch.cuda.Event(enable_timing=True))
        marks[-1].record()             # one more event per step: shows how the K steps spread around their mean
    stop.record()
    barrier()
    clocks = sampler.stop() if sampler else None
    elapsed = torch.tensor([start.elapsed_time(stop)], device=device)
    if distributed:
        dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
    ms_per_step = float(elapsed.item()) / args.steps
    each = sorted(a.elapsed_time(b) for a, b in zip([start] + marks[:-1], marks))
    step_spread = {"min": round(each[0], 3), "median": round(statistics.median(each), 3), "max": round(each[-1], 3),
                   "note": "single steps on rank 0's stream; ms_per_step is the whole region / steps, max over ranks"}
    ops_gnn.check_device_status()      # a device-side wait that ran out would have left rows unwritten: fail loudly

    # ---- parity: rows of the timed product against the float64 CPU oracle -------------------------------------------------
    parity = None
    if sample is not None:
        first, last = sample["rows"]
        parity = parity_of(sample, out[first:last], tolerance)
        if distributed:
            verdict = torch.tensor([1.0 if parity["ok"] else 0.0, -parity["max_rel_err"]], device=device, dtype=torch.float64)
            dist.all_reduce(verdict, op=dist.ReduceOp.MIN)
            edges = torch.tensor([parity["edges"]], device=device)
            dist.all_reduce(edges)
            parity = {"ok": bool(verdict[0].item() == 1.0), "max_rel_err": -float(verdict[1].item()), "tolerance": tolerance,
                      "ranks_checked": world, "edges": int(edges.item()), "rows_rank0": parity["rows"],
                      "oracle": parity["oracle"] + "; every rank checks rows of its own shard against the oracle fed "
                                "with the true rows of X (taken before X was sharded)"}

    # ---- N > 1: the local product alone, per-phase times of one more step, per-rank roofline ---------------------------
    resident_ms = None
    if distributed:
        barrier()
        start.record()
        for _ in range(args.steps):
            forward(local_ptr, local_col, my_val, local_x, 0, out_code)
        stop.record()
        barrier()
        local_ms = torch.tensor([start.elapsed_time(stop) / args.steps], device=device)
        every_ms = torch.empty(world, device=device)
        dist.all_gather_into_tensor(every_ms, local_ms)
        resident_ms = float(every_ms.max().item())
        resident_per_rank = [round(v, 3) for v in every_ms.tolist()]
        shard_bytes = torch.tensor([float(algorithmic_bytes(my_ptr.numel() - 1, my_col.numel(), args.feat, elem))],
                                   device=device, dtype=torch.float64)
        every_bytes = torch.empty(world, device=device, dtype=torch.float64)
        dist.all_gather_into_tensor(every_bytes, shard_bytes)
        if isinstance(sharded, StagedHaloSpmm):
            sharded.timing = True
            barrier()
            step()
            barrier()
            names = list(sharded.phase_ms().keys())
            mine = torch.tensor(list(sharded.phase_ms().values()), device=device)
            sharded.timing = False
            dist.all_reduce(mine, op=dist.ReduceOp.MAX)
            sharding["phases_ms"] = {n: round(float(v), 3) for n, v in zip(names, mine.tolist())}
            sharding["phases_note"] = ("one step after the timed region: ms from the step's start to the END of each phase, "
                                       "max over ranks; pack/exchange run on the side stream, product on the main stream")

    launches_per_step = 2
    if distributed and args.exchange.startswith("staged"):
        launches_per_step = len(sharded.stage_ptr) * 3   # per stage: one gather (pack or push), ReduceKernel, FixupKernel
    elif distributed and args.exchange == "halo":
        launches_per_step = 4
    elif distributed and args.exchange == "pull":
        launches_per_step = 2 * world
    result = {
        "metric": "spmm_sum_nnz_feat_per_s", "value": nnz * args.feat / (ms_per_step * 1e-3), "unit": "nnz*feat/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32" if elem == 4 else "bf16",
        "data": "synthetic", "config": config, "sharding": sharding, "clocks": clocks, "parity_check": parity,
        # ReduceKernel + FixupKernel per product and per pack gather on every rank (plans are cached after warm-up);
        # NCCL's own kernels are not counted
        "gpu_launches": args.steps * world * launches_per_step, "step_ms": step_spread,
    }

    peaks = {}
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as handle:
            peaks = json.load(handle)
    except OSError:
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))
    shape = "4,2" if elem == 4 else "8,1"
    kernel = f"opsgnn::ReduceKernel<{args.dtype},{args.dtype},int64,int64,{shape},sum,lean,bulk>"
    if resident_ms is not None:
        result["x_resident"] = {"ms_per_step": resident_ms, "value": nnz * args.feat / (resident_ms * 1e-3),
                                "per_rank_ms": resident_per_rank,
                                "note": "local SpMM only, X already in place (no exchange in the step)"}
        per_rank = [b / (ms * 1e-3) / 1e9 for b, ms in zip(every_bytes.tolist(), every_ms.tolist())]
        result["roofline"] = {
            "bound": "hbm", "achieved": min(per_rank), "peak": peak, "unit": "GB/s", "frac": min(per_rank) / peak,
            "traffic": None, "peak_source": "measured" if peaks else "fallback",
            "per_rank_achieved": [round(v, 1) for v in per_rank], "per_rank_frac": [round(v / peak, 3) for v in per_rank],
            "kernel": kernel + " of every rank's local product, timed alone (x_resident); achieved = the slowest rank's "
                      "algorithmic bytes / its time",
        }
    elif rank == 0:
        total = algorithmic_bytes(nodes, nnz, args.feat, elem)
        achieved = total / (ms_per_step * 1e-3) / 1e9
        result["roofline"] = {
            "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
            "traffic": NCU_DRAM_TRAFFIC.get(config["workload"]),
            "peak_source": "measured" if peaks else "fallback", "algorithmic_bytes_per_launch": total,
            "kernel": kernel + " (+ FixupKernel, 0.8 % of the step, inside the same timed region)",
        }

    # ---- N > 1: the other sharded operators north_star names (SDDMM, GAT layer) ---------------------------------------------
    out = None
    if distributed and not args.no_ops:
        del sharded, local_x, x_block, local_ptr, local_col, my_ptr, my_col, my_val
        sharded = local_x = x_block = None
        torch.cuda.empty_cache()
        result["ops"] = sharded_operators(dist, device, world, rank, max(3, min(args.steps, 10)))

    # ---- end to end through the public API with host buffers -----------------------------------------------------------
    torch.cuda.empty_cache()
    if not args.no_e2e:
        if distributed:
            sharded = local_x = x_block = None
            torch.cuda.empty_cache()
            result["e2e"] = end_to_end_sharded(args, host_shard, nnz, dist, device, world)
        else:
            result["e2e"] = end_to_end(args, csr_spmm, rowptr, col, value, x, nnz)[0]

    if rank == 0 and not distributed and not args.no_cpu:
        seconds, threads = time_cpu(sample, repeats=3)
        result["cpu_baseline"] = {
            "value": sample["edges"] * args.feat / seconds, "unit": "nnz*feat/s", "cores": threads, "kind": "port",
            "sample": f"rows [{sample['first']}, {sample['last']}) of the same graph ({sample['edges']} edges, columns "
                      f"relabelled to the {sample['x'].size(0)} rows of X they reference), best of 3 runs of "
                      f"oracle.spmm.csr_spmm_sum_vectorised ({seconds:.3f} s each)",
        }

    # ---- the other half of the metric: SDDMM nnz/s (config 3) and the GAT layer (config 5) -------------------------------
    if rank == 0 and not distributed and not args.no_ops:
        del rowptr, col, value, x, my_ptr, my_col, my_val
        torch.cuda.empty_cache()
        result["ops"] = other_operators(device, skip_cpu=args.no_cpu)
    if rank == 0:
        print(json.dumps(result))
    if distributed:
        dist.destroy_process_group()
    return 0


def sharded_operators(dist, device, world, rank, steps):
    """N > 1: `sddmm_csr` dot (BASELINE config 3) and the fused GAT layer (config 5) row-sharded over the ranks with the
    needed-rows exchange (`HaloShardedSddmm`, `ShardedGatLayer(fused=True)`): ms per step (CUDA events, max over ranks)
    and, for SDDMM, a check of every rank's first edges against a float64 product formed from the unsharded operands."""
    import ops_gnn
    from ops_gnn.distributed import HaloShardedSddmm, ShardedGatLayer, balanced_row_bounds, shard_csr

    def timed(step):
        for _ in range(3):
            step()
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for _ in range(steps):
            result = step()
        end.record()
        torch.cuda.synchronize()
        ms = torch.tensor([begin.elapsed_time(end) / steps], device=device)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item()), result

    record = {}
    scale = 21
    nodes = 1 << scale
    # ---- config 3: out[e] = <A[row e], B[col e]> -------------------------------------------------------------------------
    indptr, indices = rmat_csr(scale, 32 * nodes, device, seed=20261125 + 3)
    nnz = indices.numel()
    gen = torch.Generator(device=device).manual_seed(20261125 + 3)
    a = torch.randn(nodes, 64, device=device, generator=gen)
    b = torch.randn(nodes, 64, device=device, generator=gen)
    bounds = balanced_row_bounds(indptr, world, row_cost=1.0)
    ptr, col, _ = shard_csr(indptr, indices, None, bounds[rank], bounds[rank + 1])
    own = slice(bounds[rank], bounds[rank + 1])
    probe = min(col.numel(), 1 << 18)
    local_rows = ops_gnn.ptr2ind(ptr, col.numel())[:probe]
    want = (a[own][local_rows].double() * b[col[:probe]].double()).sum(-1)
    size = (a[own][local_rows].double().abs() * b[col[:probe]].double().abs()).sum(-1).clamp(min=1.0)
    op = HaloShardedSddmm(ptr, col, bounds, 64, a.dtype, device)
    a_block, b_block = a[own].contiguous(), op.own_block.copy_(b[own])
    del a, b, indptr, indices
    ms, dots = timed(lambda: op(a_block, b_block))
    error = torch.tensor([float(((dots[:probe].double() - want).abs() / size).max()) if probe else 0.0], device=device)
    dist.all_reduce(error, op=dist.ReduceOp.MAX)
    record["sddmm_sharded"] = {"ms_per_step": ms, "nnz_per_s": nnz / (ms * 1e-3), "nnz": nnz,
                               "parity_check": {"max_rel_err": float(error.item()), "tolerance": 1e-5,
                                                "ok": bool(error.item() <= 1e-5), "edges_per_rank": probe}}
    del op, a_block, b_block, dots, want, size
    torch.cuda.empty_cache()
    # ---- config 5: the GAT layer -------------------------------------------------------------------------------------------
    heads, width = 8, 64
    indptr, indices = rmat_csr(scale, 16 * nodes, device, seed=20261125 + 5)
    rows = ops_gnn.ptr2ind(indptr, indices.numel())
    loops = torch.arange(nodes, device=device)
    keys = torch.unique(torch.cat([(rows << scale) | indices, (loops << scale) | loops]))
    rows, indices = keys >> scale, keys & (nodes - 1)
    indptr = ops_gnn.ind2ptr(rows, nodes)
    del keys, loops, rows
    gen = torch.Generator(device=device).manual_seed(20261125 + 5)
    x = torch.randn(nodes, heads, width, device=device, generator=gen)
    left = torch.randn(nodes, heads, device=device, generator=gen)
    right = torch.randn(nodes, heads, device=device, generator=gen)
    bounds = balanced_row_bounds(indptr, world, row_cost=4.0)
    ptr, col, _ = shard_csr(indptr, indices, None, bounds[rank], bounds[rank + 1])
    own = slice(bounds[rank], bounds[rank + 1])
    layer = ShardedGatLayer(ptr, col, bounds, heads, width, x.dtype, device, fused=True)
    blocks = (x[own].contiguous(), left[own].contiguous(), right[own].contiguous())
    nnz = indices.numel()
    del x, left, right, indptr, indices
    ms, _ = timed(lambda: layer(*blocks))
    record["gat_layer_sharded"] = {"ms_per_step": ms, "nnz": nnz, "form": "needed-rows exchange of x and right, then gat_aggregate"}
    return record


def other_operators(device, skip_cpu):
    """`sddmm_csr` dot on BASELINE config 3 and the GAT layer of config 5 at full size, by the functions of bench_ops.py
    (5 warm + 20 timed launches each, one CUDA-event pair per launch, median)."""
    import types

    import bench_ops

    report = bench_ops.Report(types.SimpleNamespace(warm=5, timed=20, no_cpu=skip_cpu), echo=False)
    bench_ops.config3(report, device, 21)
    torch.cuda.empty_cache()
    bench_ops.config5(report, device, 21)
    torch.cuda.empty_cache()
    lines = {line["op"]: line for line in report.lines}
    dot = lines["sddmm_csr_dot_u_v"]
    summary = {
        "sddmm_nnz_per_s": dot["metric"]["value"], "sddmm_ms": dot["ms_median"],
        "sddmm_roofline": {"bound": "hbm", "achieved": dot["achieved_gbs"], "peak": dot["peak_gbs"], "unit": "GB/s",
                           "frac": dot["frac"], "traffic": dot.get("traffic"),
                           "algorithmic_bytes_per_launch": dot["algorithmic_bytes"],
                           "note": "B (0.5 GB) stays in L2, so the algorithmic rate exceeds the DRAM rate"},
        "sddmm_cpu_baseline": dot.get("cpu_baseline"),
        "gat_layer_ms": {op: lines[op]["ms_median"] for op in lines if op.startswith("gat_")},
        "lines": report.lines,
    }
    return summary


def bind_near_gpu(local):
    """Best effort: restrict this process to the CPUs of the NUMA node the GPU hangs off, so pinned host buffers
    (first touch) land in the memory closest to its PCIe root.  Returns what was done, for the record."""
    try:
        props = torch.cuda.get_device_properties(local)
        address = f"{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{address}/numa_node") as handle:
            node = int(handle.read().strip())
        if node < 0:
            return {"numa_node": None, "note": "the platform reports no NUMA node for the GPU"}
        with open(f"/sys/devices/system/node/node{node}/cpulist") as handle:
            text = handle.read().strip()
        cpus = set()
        for part in text.split(","):
            low, _, high = part.partition("-")
            cpus.update(range(int(low), int(high or low) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if not allowed:
            return {"numa_node": node, "note": "none of the node's CPUs is available to this process"}
        os.sched_setaffinity(0, allowed)
        return {"numa_node": node, "cpus": len(allowed)}
    except (OSError, ValueError, AttributeError) as exc:
        return {"numa_node": None, "note": f"not bound: {type(exc).__name__}"}


def copy_rates(pinned, staging, out_host, out_like, sync):
    """GB/s of this rank's host -> device and device -> host copies: each direction alone, then both at once (what
    the pipelined step does).  `sync()` lines the ranks up before each probe, so the rates are those of all ranks
    copying at the same time."""
    up_bytes = sum(t.numel() * t.element_size() for t in pinned)
    down_bytes = out_host.numel() * out_host.element_size()
    side = torch.cuda.Stream()
    rates = {}

    def timed(upload, download):
        sync()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        main = torch.cuda.current_stream()
        begin.record(main)
        side.wait_event(begin)
        if upload:
            for dev, host in zip(staging, pinned):
                dev.copy_(host, non_blocking=True)
        if download:
            with torch.cuda.stream(side):
                out_host.copy_(out_like, non_blocking=True)
        main.wait_stream(side)
        end.record(main)
        torch.cuda.synchronize()
        return begin.elapsed_time(end) * 1e-3

    rates["h2d_alone_gbs"] = up_bytes / timed(True, False) / 1e9
    rates["d2h_alone_gbs"] = down_bytes / timed(False, True) / 1e9
    both = timed(True, True)
    rates["both_directions_gbs"] = (up_bytes + down_bytes) / both / 1e9
    rates["both_directions_ms"] = both * 1e3
    return rates


def host_leg_bounds(rowptr, world, row_bytes, row_cost, balanced_row_bounds):
    """Shard bounds of the host-buffer leg.  That leg is bound by the host side of PCIe: measured with four ranks copying
    at once, a rank's uploads and downloads together ran at the rate of one direction alone (26 - 32 GB/s), so a rank's
    step takes about (bytes up + bytes down) / that rate - up = its CSR slice + an equal block of X, down = its output
    rows.  With a negative `row_cost` several shard balances are tried and the one whose busiest rank moves the fewest
    bytes is taken (a pure function of the graph, so every rank picks the same)."""
    rows = rowptr.numel() - 1

    def busiest(bounds):
        worst = 0
        for k in range(world):
            mine, edges = bounds[k + 1] - bounds[k], int(rowptr[bounds[k + 1]]) - int(rowptr[bounds[k]])
            up = edges * 12 + (mine + 1) * 8 + (rows // world) * row_bytes  # col + weight per edge, pointers, block of X
            down = mine * row_bytes
            worst = max(worst, up + down)
        return worst

    if row_cost >= 0:
        bounds = balanced_row_bounds(rowptr, world, row_cost=row_cost)
        return bounds, {"row_cost": row_cost, "busiest_rank_bytes": busiest(bounds)}
    best = None
    for candidate in (1.0, 4.0, 12.0, 25.0, 51.0, 100.0, 400.0, 1e7):
        bounds = balanced_row_bounds(rowptr, world, row_cost=candidate)
        cost = busiest(bounds)
        if best is None or cost < best[0]:
            best = (cost, candidate, bounds)
    return best[2], {"row_cost": best[1], "busiest_rank_bytes": best[0],
                     "rule": "smallest maximum over ranks of upload + download bytes"}


def host_available_bytes():
    try:
        with open("/proc/meminfo") as handle:
            info = dict(line.split(":") for line in handle.read().splitlines())
        return int(info["MemAvailable"].split()[0]) * 1024
    except (OSError, KeyError, ValueError):
        return None


def run_pipelined(pinned, like, product, out_host, steps, sync):
    """Milliseconds per step of: upload `pinned` into device staging, `product(staging)`, download into `out_host`.

    The three legs run on three streams with two sets of staging buffers, so the upload of step k+1 overlaps the
    product and the download of step k (PCIe is full duplex).  Every step uploads all inputs and downloads the whole
    output; the timed region (CUDA events on the product stream, which joins the copy streams before the stop event)
    covers all of it.  `sync()` brackets the timed region (device synchronise, plus a barrier when there are ranks).
    """
    slots = 2
    staging = [[torch.empty_like(t) for t in like] for _ in range(slots)]
    main = torch.cuda.current_stream()
    upload, download = torch.cuda.Stream(), torch.cuda.Stream()
    consumed = [None] * slots   # the product that read staging[s] has finished
    drained = [None] * slots    # the download that read outputs[s] has finished
    outputs = [None] * slots

    def step(k):
        s = k % slots
        with torch.cuda.stream(upload):
            if consumed[s] is not None:
                upload.wait_event(consumed[s])
            for dev, host in zip(staging[s], pinned):
                dev.copy_(host, non_blocking=True)
            ready = torch.cuda.Event()
            ready.record(upload)
        main.wait_event(ready)
        if drained[s] is not None:
            main.wait_event(drained[s])  # the allocator may hand the old output's memory to the next product
        outputs[s] = None
        out = product(staging[s])
        consumed[s] = torch.cuda.Event()
        consumed[s].record(main)
        with torch.cuda.stream(download):
            download.wait_event(consumed[s])
            out_host.copy_(out, non_blocking=True)
            drained[s] = torch.cuda.Event()
            drained[s].record(download)
        outputs[s] = out

    for k in range(slots):
        step(k)
    main.wait_stream(download)
    sync()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record(main)
    for k in range(steps):
        step(k)
    main.wait_stream(download)
    main.wait_stream(upload)
    stop.record(main)
    sync()
    return start.elapsed_time(stop) / steps


def end_to_end(args, csr_spmm, rowptr, col, value, x, nnz):
    """K steps of: pinned host -> device copies of every input, csr_spmm, device -> host copy of the result.

    The three legs run on three streams with two sets of device staging buffers, so the upload of step k+1 overlaps
    the product and the download of step k (PCIe is full duplex); every step still uploads all of its inputs and
    downloads all of its output, and the timed region covers all of it.  Returns (record, pinned host inputs).
    """
    inputs = (rowptr, col, value, x)
    in_bytes = sum(t.numel() * t.element_size() for t in inputs)
    rows = rowptr.numel() - 1
    out_bytes = rows * args.feat * x.element_size()
    available = host_available_bytes()
    if available is not None and available < 2 * (in_bytes + out_bytes):
        return {"value": None, "unit": "nnz*feat/s", "h2d_bytes_per_step": in_bytes, "d2h_bytes_per_step": out_bytes,
                "note": f"skipped: host has {available >> 30} GiB available, pinned staging needs "
                        f"{(in_bytes + out_bytes) >> 30} GiB"}, None
    pinned = [torch.empty(t.shape, dtype=t.dtype, pin_memory=True) for t in inputs]
    for host, dev in zip(pinned, inputs):
        host.copy_(dev)
    out_host = torch.empty((rows, args.feat), dtype=x.dtype, pin_memory=True)
    steps = max(3, min(args.steps, 5))
    ms = run_pipelined(pinned, inputs, lambda dev: csr_spmm(dev[0], dev[1], dev[2], dev[3], "sum"), out_host, steps,
                       torch.cuda.synchronize)
    checksum = float(out_host[:: max(1, out_host.size(0) // 1024)].double().sum())
    torch.cuda.empty_cache()
    return {"value": nnz * args.feat / (ms * 1e-3), "unit": "nnz*feat/s", "ms_per_step": ms, "steps": steps,
            "h2d_bytes_per_step": in_bytes, "d2h_bytes_per_step": out_bytes, "api": "ops_gnn.torch_sparse_spmm.csr_spmm",
            "overlap": "upload of step k+1 runs beside product and download of step k (2 staging sets, 3 streams)",
            "result_checksum": checksum}, pinned


def end_to_end_sharded(args, pinned, nnz, dist, device, world):
    """N > 1: every rank uploads its CSR slice and its block of X, runs the sharded step (all-gather of X + local
    SpMM through `ops_gnn.distributed.RowShardedSpmm`) and downloads its output rows.  `pinned` holds the rank's
    (rowptr, col, value, block of X) in pinned host memory."""
    from ops_gnn.distributed import RowShardedSpmm

    like = [torch.empty(t.shape, dtype=t.dtype, device=device) for t in pinned]
    rows = pinned[0].numel() - 1
    block_rows, dtype = pinned[3].size(0), pinned[3].dtype
    out_host = torch.empty((rows, args.feat), dtype=dtype, pin_memory=True)
    sharded = RowShardedSpmm(None, None, None, block_rows, args.feat, dtype, device)

    def product(dev):
        sharded.rowptr, sharded.col, sharded.value = dev[0], dev[1], dev[2]
        return sharded([dev[3]])[0]

    def barrier():
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()

    steps = max(3, min(args.steps, 5))
    # what bounds the leg: this rank's copy rates with every rank copying at once, and the device part of a step alone
    rates = copy_rates(pinned, like, out_host, torch.empty((rows, args.feat), dtype=dtype, device=device), barrier)
    for dev, host in zip(like, pinned):
        dev.copy_(host)
    barrier()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    product(like)
    begin.record()
    product(like)
    end.record()
    barrier()
    rates["device_part_ms"] = begin.elapsed_time(end)
    gathered_rates = [None] * world
    dist.all_gather_object(gathered_rates, {k: round(v, 2) for k, v in rates.items()})
    local_ms = run_pipelined(pinned, like, product, out_host, steps, barrier)
    del like
    elapsed = torch.tensor([local_ms * steps], device=device)
    in_bytes = torch.tensor([sum(t.numel() * t.element_size() for t in pinned)], device=device)
    out_bytes = torch.tensor([rows * args.feat * out_host.element_size()], device=device)
    dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
    dist.all_reduce(in_bytes)
    dist.all_reduce(out_bytes)
    ms = float(elapsed.item()) / steps
    return {"value": nnz * args.feat / (ms * 1e-3), "unit": "nnz*feat/s", "ms_per_step": ms, "steps": steps,
            "h2d_bytes_per_step": int(in_bytes.item()), "d2h_bytes_per_step": int(out_bytes.item()),
            "api": "ops_gnn.distributed.RowShardedSpmm", "rows_rank0": rows,
            "overlap": "upload of step k+1 runs beside product and download of step k (2 staging sets, 3 streams)",
            "note": "bytes are summed over ranks; time is the max over ranks",
            "per_rank": gathered_rates,
            "per_rank_note": "GB/s of each rank's pinned-host copies with all ranks copying at once (each direction alone, "
                             "then both), and the device part of one step (validate + plan + all-gather + product); a "
                             "step cannot be shorter than both_directions_ms of the slowest rank",
            "host_binding": args.host_binding}


def reference_arm(args, rowptr, col, value, x, config):
    """The reference's CPU algorithm (oracle port of its vectorised golden) on the host cores, same metric."""
    sample = row_sample(rowptr, col, value, lambda ids: x[ids], SAMPLE_EDGES)
    del rowptr, col, value, x
    torch.cuda.empty_cache()
    from oracle.spmm import csr_spmm_sum_vectorised

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    operands = (sample["ptr"], sample["col"], sample["value"], sample["x"])
    for _ in range(max(args.warmup, 1)):
        csr_spmm_sum_vectorised(*operands)
    begin = time.perf_counter()
    for _ in range(args.steps):
        csr_spmm_sum_vectorised(*operands)
    seconds = (time.perf_counter() - begin) / args.steps
    rate = sample["edges"] * args.feat / seconds
    text = (f"each step = rows [{sample['first']}, {sample['last']}) of the graph ({sample['edges']} edges, columns "
            f"relabelled to the {sample['x'].size(0)} rows of X they reference) through oracle.spmm.csr_spmm_sum_vectorised")
    print(json.dumps({
        "impl": "reference", "metric": "spmm_sum_nnz_feat_per_s", "value": rate, "unit": "nnz*feat/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": max(args.warmup, 1), "ms_per_step": seconds * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config,
        "cpu_baseline": {"value": rate, "unit": "nnz*feat/s", "cores": threads, "kind": "port", "sample": text},
        "e2e": {"value": rate, "unit": "nnz*feat/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))
    return 0


if __name__ == "__main__":
    sys.exit(main())
