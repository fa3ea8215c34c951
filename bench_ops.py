#!/usr/bin/env python
"""Per-operator measurements for the rest of the message-passing path: BASELINE configs 2, 3 and 5 on one B200.

    python bench_ops.py [--config 2|3|5|all] [--warm 20] [--timed 50] [--no-cpu] [--scale S]

`bench.py` measures the headline (config 4, SpMM-sum).  This script times every other operator family of the path
through the public `ops_gnn` API with inputs resident in HBM and prints ONE JSON line per operator:

    {"op": ..., "config": ..., "ms_median": ..., "ms_p90": ..., "algorithmic_bytes": B, "achieved_gbs": B / median,
     "peak_gbs": measured copy bandwidth, "frac": ..., "metric": {...}, "cpu_baseline": {...}}

Every launch is bracketed by its own pair of CUDA events on the current stream (`--warm` untimed calls first); the
working sets are larger than L2 (config 2: 512 MiB of src; config 3: 16 GB of gathers), so no flush is needed.  The
algorithmic bytes are written beside every call below (every gathered row counted as a DRAM read).  The CPU
baseline is the oracle of the same operator on a bounded sample with all host threads.  All inputs are seeded
synthetic tensors (seed = 20261125 + config number).
"""
import argparse
import json
import os
import statistics
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "ops-gnn_b200"))
sys.path.insert(0, ROOT)

from bench import rmat_csr  # noqa: E402  (the seeded R-MAT generator of the headline benchmark)

BASE_SEED = 20261125


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as handle:
            return float(json.load(handle)["hbm_gbs"]), "measured"
    except (OSError, KeyError, ValueError):
        return 6650.0, "fallback"


def time_launches(fn, warm, timed):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    pairs = []
    for _ in range(timed):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        stop.record()
        pairs.append((start, stop))
    torch.cuda.synchronize()
    times = sorted(a.elapsed_time(b) for a, b in pairs)
    return statistics.median(times), times[min(len(times) - 1, int(0.9 * len(times)))]


def time_cpu(fn, repeats=3):
    torch.set_num_threads(os.cpu_count() or 1)
    fn()
    best = None
    for _ in range(repeats):
        begin = time.perf_counter()
        fn()
        elapsed = time.perf_counter() - begin
        best = elapsed if best is None else min(best, elapsed)
    return best


# dram__bytes_read.sum + dram__bytes_write.sum of one launch from an ncu capture of the same call (profiler figures copied
# here, not measured by this script; the captures are summarised under profiles/)
NCU_DRAM_TRAFFIC = {"sddmm_csr_dot_u_v": 3.2e9}


class Report:
    """Times one public call and prints (echo) or collects (lines) its JSON record."""

    def __init__(self, args, echo=True):
        self.args = args
        self.echo = echo
        self.lines = []
        self.peak, self.peak_source = measured_peak()

    def emit(self, op, config, fn, nbytes, metric=None, cpu=None):
        median, p90 = time_launches(fn, self.args.warm, self.args.timed)
        line = {"op": op, "config": config, "ms_median": median, "ms_p90": p90, "algorithmic_bytes": nbytes,
                "achieved_gbs": nbytes / (median * 1e-3) / 1e9, "peak_gbs": self.peak, "peak_source": self.peak_source,
                "launches_timed": self.args.timed}
        line["frac"] = line["achieved_gbs"] / self.peak
        if op in NCU_DRAM_TRAFFIC:
            line["traffic"] = NCU_DRAM_TRAFFIC[op]
        if metric:
            name, units = metric
            line["metric"] = {"name": name, "value": units / (median * 1e-3)}
        if cpu is not None and not self.args.no_cpu:
            seconds, units, what = cpu()
            line["cpu_baseline"] = {"value": units / seconds, "unit": (metric[0] if metric else "units/s"),
                                    "cores": os.cpu_count() or 1, "kind": "port", "sample": what}
        self.lines.append(line)
        if self.echo:
            print(json.dumps(line), flush=True)


# ---- config 2: segment / scatter reductions and grouped softmax ------------------------------------------------------------
def config2(report, device):
    import ops_gnn
    from oracle import grouped_softmax_oracle, segment_coo_oracle, segment_csr_oracle, segment_logsumexp_oracle

    n, k = 1 << 20, 128
    gen = torch.Generator().manual_seed(BASE_SEED + 2)
    lengths = torch.empty(n // 4).geometric_(1.0 / 8, generator=gen).long()   # trials until success: >= 1, mean 8
    ends = lengths.cumsum(0)
    count = int(torch.searchsorted(ends, torch.tensor(n), right=False)) + 1
    lengths = lengths[:count].clone()
    lengths[-1] -= int(ends[count - 1]) - n
    indptr_host = torch.zeros(count + 1, dtype=torch.int64)
    indptr_host[1:] = lengths.cumsum(0)
    index_host = torch.repeat_interleave(torch.arange(count), lengths)
    src_host = torch.randn(n, k, generator=gen)
    shuffle = torch.randperm(n, generator=gen)
    indptr, index, src = indptr_host.to(device), index_host.to(device), src_host.to(device)
    index_shuffled = index[shuffle.to(device)].contiguous()
    s = count
    name = f"config2_n{n}_k{k}_segments{s}_fp32"
    row = k * 4
    sample_rows = 1 << 17                       # CPU sample: the first 131,072 rows of src and their segments
    sample_segments = int(index_host[sample_rows - 1]) + 1
    ptr_sample = indptr_host[:sample_segments + 1].clone()
    ptr_sample[-1] = sample_rows
    src_sample, index_sample = src_host[:sample_rows], index_host[:sample_rows]
    what = f"first {sample_rows} rows ({sample_segments} segments), best of 3"

    def cpu_of(fn):
        return lambda: (time_cpu(fn), sample_rows * k, what)

    for reduce in ("sum", "mean", "max", "min"):
        arg = s * k * 8 if reduce in ("max", "min") else 0
        call = {"sum": ops_gnn.segment_sum_csr, "mean": ops_gnn.segment_mean_csr, "max": ops_gnn.segment_max_csr,
                "min": ops_gnn.segment_min_csr}[reduce]
        report.emit(f"segment_csr_{reduce}", name, lambda c=call: c(src, indptr),
                    n * row + (s + 1) * 8 + s * row + arg, ("elements/s", n * k),
                    cpu_of(lambda r=reduce: segment_csr_oracle(src_sample, ptr_sample, r)))
    for reduce in ("sum", "max"):
        arg = s * k * 8 if reduce == "max" else 0
        call = ops_gnn.segment_sum_coo if reduce == "sum" else ops_gnn.segment_max_coo
        report.emit(f"segment_coo_{reduce}", name, lambda c=call: c(src, index, None, s),
                    n * row + n * 8 + s * row + arg, ("elements/s", n * k),
                    cpu_of(lambda r=reduce: segment_coo_oracle(src_sample, index_sample, None, sample_segments, r)))
    report.emit("segment_logsumexp", name, lambda: ops_gnn.segment_logsumexp(src, indptr),
                n * row + (s + 1) * 8 + s * row, ("elements/s", n * k),
                cpu_of(lambda: segment_logsumexp_oracle(src_sample, ptr_sample)))
    report.emit("scatter_logsumexp_sorted", name, lambda: ops_gnn.scatter_logsumexp(src, index, 0, s),
                n * row + n * 8 + s * row, ("elements/s", n * k))
    for label, idx in (("sorted", index), ("shuffled", index_shuffled)):
        report.emit(f"scatter_softmax_{label}", name, lambda i=idx: ops_gnn.scatter_softmax(src, i, 0, s),
                    2 * n * row + n * 8, ("elements/s", n * k),
                    cpu_of(lambda: grouped_softmax_oracle(src_sample, index_sample, 0, sample_segments)))
        report.emit(f"scatter_log_softmax_{label}", name, lambda i=idx: ops_gnn.scatter_log_softmax(src, i, 0, s),
                    2 * n * row + n * 8, ("elements/s", n * k))
    for reduce in ("sum", "max"):
        arg = s * k * 8 if reduce == "max" else 0
        call = ops_gnn.scatter_sum if reduce == "sum" else ops_gnn.scatter_max
        report.emit(f"scatter_{reduce}_shuffled", name, lambda c=call: c(src, index_shuffled, 0, None, s),
                    n * row + n * 8 + s * row + arg, ("elements/s", n * k))
    report.emit("ind2ptr", name, lambda: ops_gnn.ind2ptr(index, s), 8 * (n + s + 1), ("indices/s", n))
    report.emit("ptr2ind", name, lambda: ops_gnn.ptr2ind(indptr, n), 8 * (n + s + 1), ("indices/s", n))


# ---- config 3: SDDMM on an R-MAT graph --------------------------------------------------------------------------------------
def config3(report, device, scale):
    import ops_gnn
    from oracle import sddmm_oracle

    nodes, feat = 1 << scale, 64
    indptr, indices = rmat_csr(scale, 32 * nodes, device, seed=BASE_SEED + 3, index_dtype=torch.int32)
    nnz = indices.numel()
    gen = torch.Generator(device=device).manual_seed(BASE_SEED + 3)
    a = torch.randn(nodes, feat, device=device, generator=gen)
    b = torch.randn(nodes, feat, device=device, generator=gen)
    name = f"config3_rmat_s{scale}_nnz{nnz}_f{feat}_fp32_int32"
    out = torch.empty(nnz, device=device)
    first = nodes // 2
    last = int(torch.searchsorted(indptr, indptr[first] + (1 << 22)).item())
    lo, hi = int(indptr[first]), int(indptr[last])
    ptr_s = (indptr[first:last + 1] - lo).cpu()
    idx_s, a_s, b_host = indices[lo:hi].cpu(), a[first:last].cpu(), b.cpu()
    what = f"rows [{first}, {last}) of the same graph: {hi - lo} edges, best of 3"
    report.emit("sddmm_csr_dot_u_v", name, lambda: ops_gnn.sddmm_csr(indptr, indices, a, b, "dot", "u", "v", out=out),
                nnz * (4 + feat * 4 + 4) + nodes * (4 + feat * 4), ("nnz/s", nnz),
                lambda: (time_cpu(lambda: sddmm_oracle(ptr_s, idx_s, a_s, b_host, "dot", "u", "v")), hi - lo, what))
    out2 = torch.empty(nnz, feat, device=device)
    report.emit("sddmm_csr_mul_u_v", name, lambda: ops_gnn.sddmm_csr(indptr, indices, a, b, "mul", "u", "v", out=out2),
                nnz * (4 + feat * 4 + feat * 4) + nodes * (4 + feat * 4), ("nnz/s", nnz))
    del out2
    x16 = a.half()
    report.emit("spmm_max_copy_lhs_fp16", name, lambda: ops_gnn.spmm(indptr, indices, x16, reduce="max"),
                nnz * (4 + feat * 2) + nodes * (4 + feat * 2), ("nnz*feat/s", nnz * feat))


# ---- config 5: a GAT-style attention layer --------------------------------------------------------------------------------
def config5(report, device, scale):
    import ops_gnn

    nodes, heads, width = 1 << scale, 8, 64
    indptr, indices = rmat_csr(scale, 16 * nodes, device, seed=BASE_SEED + 5, index_dtype=torch.int64)
    # add the self loops the configuration names (edges stay sorted by row; duplicates of existing loops are merged)
    rows = ops_gnn.ptr2ind(indptr, indices.numel())
    loops = torch.arange(nodes, device=device)
    keys = torch.unique(torch.cat([(rows << scale) | indices, (loops << scale) | loops]))
    rows, indices = keys >> scale, keys & (nodes - 1)
    indptr = ops_gnn.ind2ptr(rows, nodes)
    nnz = indices.numel()
    del keys, loops
    gen = torch.Generator(device=device).manual_seed(BASE_SEED + 5)
    x = torch.randn(nodes, heads, width, device=device, generator=gen)
    att_l = torch.randn(heads, width, device=device, generator=gen) / width ** 0.5
    att_r = torch.randn(heads, width, device=device, generator=gen) / width ** 0.5
    left = (x * att_l).sum(-1)      # [N, H] per-node halves of the logit (dense torch work, not on the sparse path)
    right = (x * att_r).sum(-1)
    name = f"config5_rmat_s{scale}_nnz{nnz}_h{heads}_d{width}_fp32"
    state = {}

    def logits():
        state["e"] = ops_gnn.sddmm_csr(indptr, indices, left, right, "add", "u", "v")

    def activation():
        state["a"] = torch.nn.functional.leaky_relu(state["e"], 0.2)

    def softmax():
        state["alpha"] = ops_gnn.scatter_softmax(state["a"], rows, 0, nodes)

    def aggregate():
        state["out"] = ops_gnn.bspmm(indptr, indices, x, "mul", "sum", rhs=state["alpha"].unsqueeze(-1))

    def layer():
        logits()
        activation()
        softmax()
        aggregate()

    row = heads * width * 4
    report.emit("gat_sddmm_add_logits", name, logits, nnz * (8 + 2 * heads * 4) + nodes * (8 + heads * 4),
                ("nnz/s", nnz))
    activation()
    report.emit("gat_scatter_softmax", name, softmax, 2 * nnz * heads * 4 + nnz * 8, ("nnz/s", nnz))
    report.emit("gat_bspmm_mul_sum", name, aggregate, nnz * (8 + heads * 4 + row) + nodes * (8 + row),
                ("nnz*feat/s", nnz * heads * width))
    total = (nnz * (8 + 2 * heads * 4) + nodes * (8 + heads * 4) + 2 * nnz * heads * 4 + 2 * nnz * heads * 4 + nnz * 8
             + nnz * (8 + heads * 4 + row) + nodes * (8 + row))
    report.emit("gat_layer_composed", name, layer, total, ("nnz/s", nnz))
    # the fused form: log-sum-exp of the logits from the edge list and the [N, H] halves, then the aggregation with the
    # weights formed in the gather ring; no [E, H] tensor is written or read
    fused_bytes = (nnz * (8 + 8 + heads * 4) + nodes * heads * 8) + (nnz * (8 + heads * 4 + row) + nodes * (8 + 2 * heads * 4 + row))
    report.emit("gat_layer_fused", name, lambda: ops_gnn.gat_aggregate(indptr, indices, x, left, right, 0.2, edge_rows=rows),
                fused_bytes, ("nnz/s", nnz))


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--config", default="all", choices=("2", "3", "5", "all"))
    parser.add_argument("--warm", type=int, default=20)
    parser.add_argument("--timed", type=int, default=50)
    parser.add_argument("--scale", type=int, default=21, help="log2(nodes) of the R-MAT graphs of configs 3 and 5")
    parser.add_argument("--no-cpu", action="store_true")
    args = parser.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("bench_ops.py needs a CUDA device: the product has no CPU path")
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    report = Report(args)
    if args.config in ("2", "all"):
        config2(report, device)
        torch.cuda.empty_cache()
    if args.config in ("3", "all"):
        config3(report, device, args.scale)
        torch.cuda.empty_cache()
    if args.config in ("5", "all"):
        config5(report, device, args.scale)
    return 0


if __name__ == "__main__":
    sys.exit(main())
