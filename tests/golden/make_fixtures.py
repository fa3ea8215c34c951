"""Generate the golden fixtures of this directory by RUNNING THE REFERENCE'S OWN golden functions.

Run it where the reference checkout exists: ``python tests/golden/make_fixtures.py /path/to/ops-gnn``.  For every
operator on the sparse message-passing path it loads the reference's ``golden.py``
(or ``python/ops_gnn/scatter.py`` for the ordered scatter reference) with ``runpy``, feeds it small seeded inputs that
cover the edge cases the reference tests name (empty rows and segments, hub rows, NaN / +-inf, ties, batched pointers,
caller-provided outputs, every dtype) and stores inputs and outputs in ``<op>.pt``.  The committed ``.pt`` files are what
``tests/test_oracle_golden.py`` (CPU) and the ``-m gpu`` parity tests compare against; nothing at test time reads the
reference checkout.
"""
import os
import runpy
import sys

import torch

if len(sys.argv) != 2:
    raise SystemExit("usage: python tests/golden/make_fixtures.py /path/to/ops-gnn")
REFERENCE = sys.argv[1]
HERE = os.path.dirname(os.path.abspath(__file__))


def load(relative):
    return runpy.run_path(os.path.join(REFERENCE, relative))


def save(name, cases):
    path = os.path.join(HERE, name + ".pt")
    torch.save(cases, path)
    print(f"{name}: {len(cases)} cases, {os.path.getsize(path) / 1024:.1f} KiB")


def random_csr(gen, rows, cols, max_degree, hub=None, dtype=torch.int64):
    degree = torch.randint(0, max_degree + 1, (rows,), generator=gen)
    degree[rows // 3] = 0
    if hub is not None:
        degree[1] = hub
    ptr = torch.zeros(rows + 1, dtype=torch.int64)
    ptr[1:] = degree.cumsum(0)
    col = torch.randint(0, cols, (int(ptr[-1]),), generator=gen)
    return ptr.to(dtype), col.to(dtype)


def fixtures_torch_sparse_spmm():
    g = load("test/torch_sparse_spmm/arch35/golden.py")
    golden, sample, combos = g["golden"], g["sample"], g["COMBOS"]
    cases = []
    for dtype, outdtype in combos:
        for batch, wide in ((False, False), (True, False), (False, True), (True, True)):
            ptr, col, v, mat = sample(dtype, batch=batch, feature_values=wide)
            for reduce in ("sum", "mean", "min", "max"):
                for weighted in (True, False):
                    value = v if weighted else None
                    out, arg = golden(ptr, col, value, mat, reduce, outdtype=outdtype)
                    cases.append(dict(ptr=ptr, col=col, value=value, mat=mat, reduce=reduce, outdtype=outdtype,
                                      out=out, arg=arg))
    gen = torch.Generator().manual_seed(1234)
    for k in (1, 7, 64, 132):
        ptr, col = random_csr(gen, 40, 30, 9, hub=600)
        mat = torch.randn(30, k, generator=gen)
        value = torch.rand(col.numel(), generator=gen) * 2 - 1
        if k == 64:  # special values: NaN products are ignored, infinities compare normally, exact ties
            mat[3, :8] = float("nan")
            mat[5, 8:16] = float("inf")
            mat[7, 16:24] = -float("inf")
            mat[9] = mat[11]
            value[:] = 1.0
        for reduce in ("sum", "mean", "min", "max"):
            out, arg = golden(ptr, col, value, mat, reduce, outdtype=torch.float32)
            cases.append(dict(ptr=ptr, col=col, value=value, mat=mat, reduce=reduce, outdtype=torch.float32, out=out,
                              arg=arg))
    save("torch_sparse_spmm", cases)


def fixtures_spmm_copy():
    unified = load("test/unified_spmm/arch22/golden.py")["unified_spmm_reference"]
    spmm_sum = load("test/spmm_sum/arch22/golden.py")["spmm_sum_reference"]
    spmm_max = load("test/spmm_max/arch22/golden.py")["spmm_max_reference"]
    gen = torch.Generator().manual_seed(77)
    cases = []
    for index_dtype in (torch.int32, torch.int64):
        ptr, col = random_csr(gen, 33, 21, 6, hub=300, dtype=index_dtype)
        for n in (1, 15, 16, 17, 33, 127):
            for dtype in (torch.float32, torch.float16):
                x = torch.randn(21, n, generator=gen).to(dtype)
                if n == 17:
                    x[2, 0], x[4, 1], x[6, 2] = float("nan"), float("inf"), -float("inf")
                for reduce in ("sum", "max", "min", "mean"):
                    out = unified(ptr, col, x, reduce, "copy_lhs")
                    cases.append(dict(kind="unified", indptr=ptr, indices=col, x=x, op="copy_lhs", reduce=reduce, out=out))
            edge = torch.randn(col.numel(), n, generator=gen)
            for reduce in ("sum", "max", "min"):
                out = unified(ptr, col, edge, reduce, "copy_rhs")
                cases.append(dict(kind="unified", indptr=ptr, indices=col, x=edge, op="copy_rhs", reduce=reduce, out=out))
        x3 = torch.randn(21, 3, 10, generator=gen).half()
        cases.append(dict(kind="spmm_sum", indptr=ptr, indices=col, x=x3, reduce="sum", out=spmm_sum(ptr, col, x3, fp32=True)))
        cases.append(dict(kind="spmm_max", indptr=ptr, indices=col, x=x3, reduce="max", out=spmm_max(ptr, col, x3)))
        rhs = torch.randn(col.numel(), 3, 1, generator=gen)
        x3f = x3.float()
        for op in ("add", "sub", "mul", "div"):
            for reduce in ("sum", "mean", "max", "min"):
                out = unified(ptr, col, x3f, reduce, op, rhs)
                cases.append(dict(kind="binary", indptr=ptr, indices=col, x=x3f, rhs=rhs, op=op, reduce=reduce, out=out))
    save("spmm_copy", cases)


def fixtures_sddmm():
    ref = load("test/sddmm_csr/arch22/golden.py")["sddmm_reference"]
    gen = torch.Generator().manual_seed(5)
    cases = []
    for index_dtype in (torch.int32, torch.int64):
        ptr, col = random_csr(gen, 25, 25, 5, hub=70, dtype=index_dtype)
        e = col.numel()
        for feat in (1, 3, 16, 65):
            for dtype in (torch.float32, torch.float16):
                node_a = torch.randn(25, feat, generator=gen).to(dtype)
                node_b = torch.randn(25, feat, generator=gen).to(dtype)
                edge = torch.randn(e, feat, generator=gen).to(dtype)
                for op in ("dot", "add", "sub", "mul", "div", "copy_lhs", "copy_rhs"):
                    for lt, rt in ((0, 2), (2, 0), (0, 1), (1, 2), (1, 1)):
                        lhs = edge if lt == 1 else node_a
                        rhs = edge if rt == 1 else node_b
                        out = ref(ptr, col, lhs, rhs, op, lt, rt)
                        cases.append(dict(indptr=ptr, indices=col, lhs=lhs, rhs=rhs, op=op, lhs_target=lt,
                                          rhs_target=rt, out=out))
        vec_a, vec_b = torch.randn(25, generator=gen), torch.randn(25, generator=gen)
        for op in ("dot", "mul", "copy_lhs"):
            cases.append(dict(indptr=ptr, indices=col, lhs=vec_a, rhs=vec_b, op=op, lhs_target=0, rhs_target=2,
                              out=ref(ptr, col, vec_a, vec_b, op, 0, 2)))
    cases = cases[::3]  # keep the file small; a stride of 3 over 7 ops x 5 target pairs still hits every combination
    save("sddmm_csr", cases)


def _values(gen, shape, dtype):
    if dtype.is_floating_point:
        return torch.randn(shape, generator=gen).to(dtype)
    if dtype == torch.uint8:
        return torch.randint(0, 200, shape, generator=gen).to(dtype)
    return torch.randint(-100, 100, shape, generator=gen).to(dtype)


def fixtures_segment_csr():
    g = load("test/segment_csr/arch35/golden.py")
    values, args = g["segment_csr_cpu"], g["segment_argminmax_cpu"]
    gen = torch.Generator().manual_seed(9)
    cases = []
    dtypes = (torch.float32, torch.float16, torch.bfloat16, torch.int8, torch.uint8, torch.int32, torch.int64)
    lengths = torch.tensor([3, 0, 1, 40, 0, 0, 2, 300, 5])
    ptr = torch.zeros(lengths.numel() + 1, dtype=torch.int64)
    ptr[1:] = lengths.cumsum(0)
    total = int(ptr[-1])
    for dtype in dtypes:
        for k in (1, 5, 32):
            src = _values(gen, (total + 4, k), dtype)  # four trailing rows belong to no segment
            for reduce in ("sum", "mean", "min", "max"):
                out = values(src, ptr, reduce)
                arg = args(src, ptr, reduce) if reduce in ("min", "max") else None
                cases.append(dict(src=src, indptr=ptr, reduce=reduce, out=out, arg=arg))
    # pointers that start after row 0, batched / broadcast pointers, exact ties
    src = torch.randn(2, 12, 3, generator=gen)
    shared = torch.tensor([[2, 5, 5, 12]])
    per_batch = torch.tensor([[0, 4, 4, 9], [1, 1, 7, 12]])
    tied = torch.tensor([[1.0, 2.0], [3.0, 2.0], [3.0, 0.0], [0.5, 2.0]])
    for s, p in ((src, shared), (src, per_batch), (tied, torch.tensor([0, 4]))):
        for reduce in ("sum", "mean", "min", "max"):
            out = values(s, p, reduce)
            arg = args(s, p, reduce) if reduce in ("min", "max") else None
            cases.append(dict(src=s, indptr=p, reduce=reduce, out=out, arg=arg))
    save("segment_csr", cases)


def fixtures_segment_coo():
    g = load("test/segment_coo/arch35/golden.py")
    ref, options = g["segment_coo_reference"], g["ReferenceOptions"]
    gen = torch.Generator().manual_seed(10)
    cases = []
    index = torch.tensor([0, 0, 0, 2, 3, 3, 3, 3, 3, 3, 3, 3, 3, 3, 3, 6, 6])
    for dtype in (torch.float32, torch.float16, torch.bfloat16, torch.int8, torch.uint8, torch.int32, torch.int64):
        for k in (1, 6):
            src = _values(gen, (index.numel(), k), dtype)
            for reduce in ("sum", "mean", "min", "max"):
                for dim_size in (None, 9):
                    got = ref(src, index, None, dim_size, options(reduce, reduce in ("min", "max")))
                    out, arg = got if isinstance(got, tuple) else (got, None)
                    cases.append(dict(src=src, index=index, out_in=None, dim_size=dim_size, reduce=reduce, out=out, arg=arg))
    src = torch.randn(index.numel(), 4, generator=gen)
    src[3:15, 0] = 1.5  # ties inside a long segment
    seed = torch.randn(8, 4, generator=gen)
    for reduce in ("sum", "mean", "min", "max"):
        got = ref(src, index, seed.clone(), None, options(reduce, reduce in ("min", "max")))
        out, arg = got if isinstance(got, tuple) else (got, None)
        cases.append(dict(src=src, index=index, out_in=seed, dim_size=None, reduce=reduce, out=out, arg=arg))
    batched_src = torch.randn(2, 6, 3, generator=gen)
    batched_index = torch.tensor([[0, 0, 1, 1, 1, 3], [1, 2, 2, 2, 2, 2]])
    for idx in (batched_index, batched_index[:1]):
        for reduce in ("sum", "mean", "min", "max"):
            got = ref(batched_src, idx, None, 4, options(reduce, reduce in ("min", "max")))
            out, arg = got if isinstance(got, tuple) else (got, None)
            cases.append(dict(src=batched_src, index=idx, out_in=None, dim_size=4, reduce=reduce, out=out, arg=arg))
    special = torch.tensor([[1.0], [float("nan")], [2.0], [-float("inf")], [float("inf")]])
    for reduce in ("min", "max"):
        out, arg = ref(special, torch.tensor([0, 0, 0, 1, 2]), None, 3, options(reduce, True))
        cases.append(dict(src=special, index=torch.tensor([0, 0, 0, 1, 2]), out_in=None, dim_size=3, reduce=reduce,
                          out=out, arg=arg))
    save("segment_coo", cases)


def fixtures_scatter():
    element_loop = load("test/scatter/arch35/golden.py")["scatter_cpu"]
    module = load("python/ops_gnn/scatter.py")
    ordered, request = module["_reference_forward"], module["_ScatterRequest"]
    gen = torch.Generator().manual_seed(11)
    cases = []
    for dtype in (torch.float32, torch.float16, torch.bfloat16, torch.int8, torch.uint8, torch.int16, torch.int32,
                  torch.int64, torch.float64):
        for shape, dim in (((40,), 0), ((30, 5), 0), ((4, 25), 1), ((2, 12, 3), 1)):
            src = _values(gen, shape, dtype)
            if not dtype.is_floating_point:
                src = src.clamp(-3, 3) if dtype != torch.uint8 else src.clamp(0, 3)
            index = torch.randint(0, 7, shape, generator=gen)
            for reduce in ("sum", "mul", "mean", "min", "max"):
                got = element_loop(src, index, dim=dim, dim_size=9, reduce=reduce)
                out, arg = got if isinstance(got, tuple) else (got, None)
                cases.append(dict(src=src, index=index, dim=dim, dim_size=9, reduce=reduce, out_in=None, out=out, arg=arg,
                                  source="scatter_cpu"))
    src = torch.randn(50, 4, generator=gen)
    src[10:20, 1] = 0.25  # ties: the later position wins
    index = torch.randint(0, 6, (50, 4), generator=gen)
    seed = torch.randn(6, 4, generator=gen)
    for reduce in ("sum", "mul", "mean", "min", "max"):
        shape = (6, 4)
        out, arg = ordered(src, index, request(0, seed.clone(), None, reduce), shape)
        cases.append(dict(src=src, index=index, dim=0, dim_size=None, reduce=reduce, out_in=seed, out=out, arg=arg,
                          source="_reference_forward"))
        out, arg = ordered(src, index, request(0, None, 6, reduce), shape)
        cases.append(dict(src=src, index=index, dim=0, dim_size=6, reduce=reduce, out_in=None, out=out, arg=arg,
                          source="_reference_forward"))
    save("scatter", cases)


def fixtures_grouped():
    g = load("test/common/grouped_softmax_golden.py")
    shared = load("test/common/grouped_softmax_cases.py")
    grouped, lse = g["grouped_reference"], g["grouped_logsumexp_reference"]
    gen = torch.Generator().manual_seed(shared["SEED"])
    cases = []
    for index, shape, dim, dim_size in shared["CASES"]:
        for dtype in shared["DTYPES"]:
            src = (torch.randn(shape, generator=gen) * 3).to(dtype)
            cases.append(dict(src=src, index=torch.tensor(index), dim=dim, dim_size=dim_size,
                              softmax=grouped(src, index, dim, dim_size, torch.softmax),
                              log_softmax=grouped(src, index, dim, dim_size, torch.log_softmax),
                              logsumexp=lse(src, index, dim, dim_size)))
    index = torch.randint(0, 11, (400,), generator=gen)  # unsorted
    src = torch.randn(400, 9, generator=gen) * 4
    src[5, 0], src[9, 1], src[17, 2] = float("inf"), -float("inf"), float("nan")
    src[index == 3, 3] = -float("inf")
    cases.append(dict(src=src, index=index, dim=0, dim_size=12,
                      softmax=grouped(src, index, 0, 12, torch.softmax),
                      log_softmax=grouped(src, index, 0, 12, torch.log_softmax),
                      logsumexp=lse(src, index, 0, 12)))
    save("grouped_softmax", cases)


def fixtures_segment_logsumexp():
    ref = load("test/segment_logsumexp/golden.py")["reference"]
    gen = torch.Generator().manual_seed(12)
    cases = []
    for dtype in (torch.float32, torch.float16, torch.bfloat16):
        for ptr in ([0, 3, 3, 4, 200, 200, 230], [2, 5, 230], [0, 230]):
            for feat in ((), (7,), (2, 16)):
                src = (torch.randn((230,) + feat, generator=gen) * 5).to(dtype)
                if feat == (7,):
                    src[0, 0], src[1, 1], src[3, 2] = float("inf"), float("nan"), -float("inf")
                cases.append(dict(src=src, indptr=torch.tensor(ptr), out=ref(src, ptr)))
    save("segment_logsumexp", cases)


def fixtures_convert():
    g = load("test/sparse/arch35/golden.py")
    ind2ptr, ptr2ind, make = g["ind2ptr_cpu"], g["ptr2ind_cpu"], g["make_sorted_row_indices"]
    cases = []
    for edges, rows, seed in ((0, 5, 0), (1, 1, 1), (50, 8, 2), (500, 1000, 3), (3000, 17, 4)):
        ind = make(edges, rows, seed)
        ptr = ind2ptr(ind, rows)
        cases.append(dict(ind=ind, rows=rows, ptr=ptr, back=ptr2ind(ptr, edges)))
    save("convert", cases)


def fixtures_gather():
    g = load("test/gather_csr/arch35/golden.py")
    by_ptr, by_index = g["gather_csr_cpu"], g["gather_csr_coo_cpu"]
    cases = []
    # the golden file's own known-answer table, every dtype it lists
    for src_data, index_data, ptr_data, expected in g["CASES"]:
        for dtype in g["DTYPES"]:
            src, ptr = torch.tensor(src_data, dtype=dtype), torch.tensor(ptr_data, dtype=torch.int64)
            out = by_ptr(src, ptr)
            assert torch.equal(out, torch.tensor(expected, dtype=dtype)) and torch.equal(by_index(src, ptr), out)
            cases.append(dict(src=src, indptr=ptr, index=torch.tensor(index_data, dtype=torch.int64), out=out, source="table"))
    # seeded cases: empty segments, an uncovered prefix, broadcast and per-batch pointers, wide and odd feature widths
    gen = torch.Generator().manual_seed(91)
    for shape, ptr_rank, prefix in (((40,), 1, 0), ((40, 7), 1, 3), ((3, 13, 16), 2, 0), ((3, 13, 5), 2, 2),
                                    ((2, 3, 7, 9), 3, 0), ((9, 132), 1, 0), ((1, 9, 2, 3), 2, 1)):
        for dtype in (torch.float32, torch.float16, torch.bfloat16, torch.float64, torch.int8, torch.uint8, torch.int16,
                      torch.int32, torch.int64):
            dim = ptr_rank - 1
            segments = shape[dim]
            lead = [1 if (ptr_rank == 1 or k % 2) else shape[k] for k in range(dim)] if ptr_rank > 1 else []
            count = 1
            for extent in lead:
                count *= extent
            rows = 37
            cuts = torch.sort(torch.randint(prefix, rows + 1, (count, segments - 1), generator=gen), dim=1).values
            ptr = torch.cat([torch.full((count, 1), prefix), cuts, torch.full((count, 1), rows)], dim=1).to(torch.int64)
            ptr = ptr.reshape(lead + [segments + 1]) if lead else ptr.reshape(segments + 1)
            src = (torch.randn(shape, generator=gen) * 9).to(dtype)
            out = by_ptr(src, ptr)
            case = dict(src=src, indptr=ptr, out=out, source="seeded")
            if prefix == 0:
                full = ptr.expand([shape[k] for k in range(dim)] + [segments + 1]).reshape(-1, segments + 1)
                index = torch.stack([torch.arange(segments).repeat_interleave(row[1:] - row[:-1]) for row in full])
                case["index"] = index.reshape([shape[k] for k in range(dim)] + [rows])
                assert torch.equal(by_index(src, ptr), out)
            cases.append(case)
    save("gather", cases)


if __name__ == "__main__":
    torch.set_num_threads(4)
    fixtures_torch_sparse_spmm()
    fixtures_spmm_copy()
    fixtures_sddmm()
    fixtures_segment_csr()
    fixtures_segment_coo()
    fixtures_scatter()
    fixtures_grouped()
    fixtures_segment_logsumexp()
    fixtures_convert()
    fixtures_gather()
