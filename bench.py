#!/usr/bin/env python
"""Headline benchmark: CSR SpMM-sum on an R-MAT graph (BASELINE config 4), nnz*feat/s and fraction of HBM peak.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--scale S] [--feat F] [--dtype fp32|bf16]

One "step" is one SpMM over the whole graph: out = A @ X with A an R-MAT(0.57/0.19/0.19/0.05) graph of 2**scale
nodes and 16 * 2**scale drawn edges (deduplicated), fp32 edge weights U[0,1), X ~ N(0,1) with `feat` columns.  The
default (scale 24, feat 256, fp32: 16.7M nodes, 256M drawn edges) is the configuration the metric is quoted on.
All inputs are seeded synthetic tensors generated on the GPU; no dataset is read.

The line printed by rank 0 carries
  value       whole-job nnz*feat/s with inputs resident in HBM (CUDA events, K steps, max over ranks),
  e2e         the same metric through the public API `ops_gnn.torch_sparse_spmm.csr_spmm` with HOST buffers: the
              pinned-host -> device copies of rowptr/col/value/X and the device -> host copy of the result are inside
              the timed region (N > 1: every rank moves its own CSR slice, block of X and output rows through
              `ops_gnn.distributed.RowShardedSpmm`),
  roofline    algorithmic bytes of one step / measured step time against the measured HBM copy bandwidth,
  cpu_baseline  the CPU oracle (vectorised restatement of the reference's golden) on a bounded row sample, all host
              threads,
  clocks      SM clock and throttle reasons sampled by nvidia-smi during the timed region.

N > 1 (torchrun, one rank per GPU; strong scaling: the graph is fixed): output rows are split into contiguous ranges
of equal work (edges + 6 per row).  X is owned by the same row ranges and each step moves only the rows of X a shard
references into a compact buffer before the local SpMM: `--exchange pull` runs the gather kernel once per peer with
the peer's block (symmetric memory) as its source; `--exchange halo` packs the rows and sends them with one NCCL
all-to-all (also the fallback when symmetric memory cannot be set up).  The default `auto` takes pull between two
GPUs and halo beyond.  `--exchange allgather`: every rank owns an equal row block of X and each step all-gathers all
of X.  The
`x_resident` record times the local SpMM alone.  The host-buffer leg at N > 1 uses the all-gather form with its own
shard bounds (`--e2e-row-cost`).
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


# ---- CPU arm ----------------------------------------------------------------------------------------------------------------
def cpu_sample(rowptr, col, value, x, target_edges):
    """Contiguous row range around the median edge holding about `target_edges` edges (host tensors)."""
    nnz = int(rowptr[-1])
    middle = nnz // 2
    first = int(torch.searchsorted(rowptr, torch.tensor(middle), right=True)) - 1
    last = int(torch.searchsorted(rowptr, torch.tensor(min(middle + target_edges, nnz)), right=False))
    last = max(last, first + 1)
    lo, hi = int(rowptr[first]), int(rowptr[last])
    return (rowptr[first:last + 1] - lo).clone(), col[lo:hi].clone(), value[lo:hi].clone(), first, last


def time_cpu(rowptr, col, value, x, repeats):
    from oracle.spmm import csr_spmm_sum_vectorised

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    csr_spmm_sum_vectorised(rowptr, col, value, x)  # warm the allocator and the thread pool
    times = []
    for _ in range(repeats):
        start = time.perf_counter()
        csr_spmm_sum_vectorised(rowptr, col, value, x)
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
    parser.add_argument("--exchange", default="auto", choices=("auto", "allgather", "halo", "pull"),
                        help="N > 1: all-gather of X; an all-to-all of only the rows each shard references (halo); or "
                             "the same rows pulled from the peers' symmetric memory by the gather kernel (pull); "
                             "auto = pull between two GPUs (where it has been measured), halo beyond")
    parser.add_argument("--row-cost", type=float, default=6.0, help="N > 1: cost of one output row in edges (shard balance)")
    parser.add_argument("--e2e-row-cost", type=float, default=1.0,
                        help="N > 1: the same for the host-buffer leg (measured at 4 GPUs: 272 ms per step with 1, 310 with 50)")
    parser.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    parser.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg (profiling runs)")
    return parser.parse_args()


def workload_name(args):
    return f"rmat_s{args.scale}_ef{args.edge_factor}_f{args.feat}_{args.dtype}_spmm_sum"


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
    if distributed:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=device)
    dtype = torch.float32 if args.dtype == "fp32" else torch.bfloat16
    elem = 4 if dtype == torch.float32 else 2
    nodes = 1 << args.scale

    # ---- inputs (seeded; identical on every rank) ------------------------------------------------------------------
    rowptr, col = rmat_csr(args.scale, args.edge_factor * nodes, device)
    nnz = col.numel()
    gen = torch.Generator(device=device).manual_seed(SEED + 1)
    value = torch.rand(nnz, device=device, generator=gen).to(dtype)
    x = torch.randn(nodes, args.feat, device=device, generator=gen, dtype=torch.float32).to(dtype)
    config = {"workload": workload_name(args), "nodes": nodes, "nnz": nnz, "feat": args.feat,
              "index_dtype": "int64", "l2": "inputs_larger_than_l2", "seed": SEED}

    if args.impl == "reference":
        return reference_arm(args, rowptr, col, value, x, config)

    import ops_gnn
    from ops_gnn.torch_sparse_spmm import csr_spmm

    forward = ops_gnn._pybind.torch_sparse_spmm.forward
    out_code = 0 if dtype == torch.float32 else 2

    # ---- shard (nnz-balanced contiguous row ranges) ---------------------------------------------------------------------
    sharded = None
    if distributed:
        from ops_gnn.distributed import HaloShardedSpmm, RowShardedSpmm, balanced_row_bounds, shard_csr

        # a row end costs the kernel about four edges on this graph (measured per rank: 0.13 ns per edge, 0.6 ns per row)
        bounds = balanced_row_bounds(rowptr, world, row_cost=args.row_cost)
        my_ptr, my_col, my_val = shard_csr(rowptr, col, value, bounds[rank], bounds[rank + 1])
        config["shard_rows"] = bounds[rank + 1] - bounds[rank]
        host_shard = None
        if not args.no_e2e:
            # The host-buffer leg is bound by PCIe, not by the kernel: it gets its own shard bounds (balanced on edges +
            # e2e_row_cost per row; weighing a row like the 50 edges its bytes amount to measured slower) and equal
            # blocks of X.
            e2e_bounds = balanced_row_bounds(rowptr, world, row_cost=args.e2e_row_cost)
            block = nodes // world
            pieces = shard_csr(rowptr, col, value, e2e_bounds[rank], e2e_bounds[rank + 1])
            host_shard = [torch.empty(t.shape, dtype=t.dtype, pin_memory=True).copy_(t)
                          for t in (*pieces, x[rank * block:(rank + 1) * block])]
            del pieces
        if args.exchange == "auto":
            args.exchange = "pull" if world == 2 else "halo"
        if args.exchange in ("halo", "pull"):
            # X is owned by the same row ranges as the output (a layer's output rows are the next layer's input)
            x_block = x[bounds[rank]:bounds[rank + 1]].clone()
            del rowptr, col, value, x
            torch.cuda.empty_cache()
            transport = "pull" if args.exchange == "pull" else "alltoall"
            try:
                sharded = HaloShardedSpmm(my_ptr, my_col, my_val, bounds, args.feat, dtype, device, transport=transport)
                failure = None
            except (RuntimeError, ImportError, AttributeError) as exc:  # symmetric memory unavailable on this box
                sharded, failure = None, f"{type(exc).__name__}: {exc}"[:200]
            agreed = torch.tensor([0 if failure else 1], device=device)
            dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
            if int(agreed.item()) == 0:  # every rank falls back together
                if transport == "alltoall":
                    raise RuntimeError(f"sharded SpMM set-up failed: {failure}")
                sharded = None
                torch.cuda.empty_cache()
                sharded = HaloShardedSpmm(my_ptr, my_col, my_val, bounds, args.feat, dtype, device, transport="alltoall")
                args.exchange = "halo"
                config["exchange_fallback"] = failure or "symmetric memory set-up failed on another rank"
            my_col = sharded.col
            x = sharded.compact
            sent, received = sharded.exchange_rows()
            config["parallelism"] = (f"row_shard{world}_halo_pull_x" if args.exchange == "pull"
                                     else f"row_shard{world}_halo_alltoall_x")
            config["halo_rows_rank0"] = {"sent": sent, "received": received}
        else:
            block = nodes // world
            x_block = x[rank * block:(rank + 1) * block].clone()
            del rowptr, col, value, x
            torch.cuda.empty_cache()
            sharded = RowShardedSpmm(my_ptr, my_col, my_val, block, args.feat, dtype, device)
            x = sharded.gathered[0]  # filled by the all-gather of every step, never by the generator
            config["parallelism"] = f"row_shard{world}_allgather_x"
    else:
        my_ptr, my_col, my_val = rowptr, col, value
        x_block = None
        config["parallelism"] = "single_gpu"

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
    for _ in range(args.steps):
        out = step()
    stop.record()
    barrier()
    clocks = sampler.stop() if sampler else None
    elapsed = torch.tensor([start.elapsed_time(stop)], device=device)
    if distributed:
        dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
    ms_per_step = float(elapsed.item()) / args.steps

    # kernel-only scaling figure for N > 1: the same local SpMM with X already replicated
    resident_ms = None
    if distributed:
        barrier()
        start.record()
        for _ in range(args.steps):
            forward(my_ptr, my_col, my_val, x, 0, out_code)
        stop.record()
        barrier()
        local_ms = torch.tensor([start.elapsed_time(stop) / args.steps], device=device)
        every_ms = torch.empty(world, device=device)
        dist.all_gather_into_tensor(every_ms, local_ms)
        resident_ms = float(every_ms.max().item())
        resident_per_rank = [round(v, 3) for v in every_ms.tolist()]

    result = {
        "metric": "spmm_sum_nnz_feat_per_s", "value": nnz * args.feat / (ms_per_step * 1e-3), "unit": "nnz*feat/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32" if elem == 4 else "bf16",
        "data": "synthetic", "config": config, "clocks": clocks,
        # ReduceKernel + FixupKernel per step on every rank (the plan is cached after warm-up); NCCL's kernels not counted
        # (the halo step adds the pack gather, again ReduceKernel + FixupKernel; the pull step one gather per peer)
        "gpu_launches": args.steps * world * (2 if not distributed or args.exchange == "allgather"
                                              else 4 if args.exchange == "halo" else 2 * world),
    }
    if resident_ms is not None:
        result["x_resident"] = {"ms_per_step": resident_ms, "value": nnz * args.feat / (resident_ms * 1e-3),
                                "per_rank_ms": resident_per_rank,
                                "note": "local SpMM only, X already replicated (no all-gather in the step)"}

    if rank == 0:
        peaks = {}
        try:
            with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as handle:
                peaks = json.load(handle)
        except OSError:
            pass
        peak = float(peaks.get("hbm_gbs", 6650.0))
        if not distributed:
            total = algorithmic_bytes(nodes, nnz, args.feat, elem)
            achieved = total / (ms_per_step * 1e-3) / 1e9
            shape = "4,2" if elem == 4 else "8,1"
            result["roofline"] = {
                "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": NCU_DRAM_TRAFFIC.get(config["workload"]),
                "peak_source": "measured" if peaks else "fallback", "algorithmic_bytes_per_launch": total,
                "kernel": f"opsgnn::ReduceKernel<{args.dtype},{args.dtype},int64,int64,{shape},sum,lean,bulk> "
                          "(+ FixupKernel, 0.8 % of the step, inside the same timed region)",
            }

    # ---- end to end through the public API with host buffers -----------------------------------------------------------
    host_inputs = None
    out = None
    torch.cuda.empty_cache()
    if not args.no_e2e:
        if distributed:
            result["e2e"] = end_to_end_sharded(args, host_shard, nnz, dist, device, world)
        else:
            result["e2e"], host_inputs = end_to_end(args, csr_spmm, rowptr, col, value, x, nnz)

    if rank == 0 and not distributed and not args.no_cpu:
        if host_inputs is None:
            host_inputs = [t.cpu() for t in (rowptr, col, value, x)]
        del rowptr, col, value, x
        *host, x_host = host_inputs
        sample_ptr, sample_col, sample_val, first, last = cpu_sample(*host, x_host, 1 << 22)
        seconds, threads = time_cpu(sample_ptr, sample_col, sample_val.float(), x_host.float(), repeats=3)
        result["cpu_baseline"] = {
            "value": sample_col.numel() * args.feat / seconds, "unit": "nnz*feat/s", "cores": threads, "kind": "port",
            "sample": f"rows [{first}, {last}) of the same graph: {sample_col.numel()} edges, best of 3 runs of "
                      f"oracle.spmm.csr_spmm_sum_vectorised ({seconds:.3f} s each)",
        }
    if rank == 0:
        print(json.dumps(result))
    if distributed:
        dist.destroy_process_group()
    return 0


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
            "api": "ops_gnn.distributed.RowShardedSpmm", "shard_row_cost": args.e2e_row_cost, "rows_rank0": rows,
            "overlap": "upload of step k+1 runs beside product and download of step k (2 staging sets, 3 streams)",
            "note": "bytes are summed over ranks; time is the max over ranks"}


def reference_arm(args, rowptr, col, value, x, config):
    """The reference's CPU algorithm (oracle port of its vectorised golden) on the host cores, same metric."""
    host = [t.cpu() for t in (rowptr, col, value)]
    x_host = x.float().cpu()
    del rowptr, col, value, x
    sample_ptr, sample_col, sample_val, first, last = cpu_sample(*host, x_host, 1 << 22)
    sample_val = sample_val.float()
    from oracle.spmm import csr_spmm_sum_vectorised

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    for _ in range(max(args.warmup, 1)):
        csr_spmm_sum_vectorised(sample_ptr, sample_col, sample_val, x_host)
    begin = time.perf_counter()
    for _ in range(args.steps):
        csr_spmm_sum_vectorised(sample_ptr, sample_col, sample_val, x_host)
    seconds = (time.perf_counter() - begin) / args.steps
    rate = sample_col.numel() * args.feat / seconds
    sample = (f"each step = rows [{first}, {last}) of the graph ({sample_col.numel()} edges) through "
              f"oracle.spmm.csr_spmm_sum_vectorised")
    print(json.dumps({
        "impl": "reference", "metric": "spmm_sum_nnz_feat_per_s", "value": rate, "unit": "nnz*feat/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": max(args.warmup, 1), "ms_per_step": seconds * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config,
        "cpu_baseline": {"value": rate, "unit": "nnz*feat/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": rate, "unit": "nnz*feat/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))
    return 0


if __name__ == "__main__":
    sys.exit(main())
