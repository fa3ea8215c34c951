"""GPU parity of a GAT-style attention layer composed from the public operators (BASELINE config 5 at reduced size):
SDDMM for per-head edge logits, LeakyReLU, scatter_softmax over destination rows, fused per-head weighted aggregation.
The expected result is the same composition of the CPU oracles."""
import pytest
import torch

import oracle
from conftest import assert_close, requires_gpu

pytestmark = requires_gpu


def _rmat(scale, edges, gen):
    a, b, c = 0.57, 0.19, 0.19
    row = torch.zeros(edges, dtype=torch.int64)
    col = torch.zeros(edges, dtype=torch.int64)
    for _ in range(scale):
        u = torch.rand(edges, generator=gen)
        row = (row << 1) | (u >= a + b)
        col = (col << 1) | (((u >= a) & (u < a + b)) | (u >= a + b + c))
    loops = torch.arange(1 << scale)
    keys = torch.unique(torch.cat([(row << scale) | col, (loops << scale) | loops]))
    return keys >> scale, keys & ((1 << scale) - 1)


def test_attention_layer_matches_oracle_composition(cuda_device):
    import ops_gnn

    gen = torch.Generator().manual_seed(20261125 + 5)
    scale, heads, width = 12, 8, 64
    nodes = 1 << scale
    rows, cols = _rmat(scale, 16 * nodes, gen)
    x = torch.randn(nodes, heads, width, generator=gen)
    att_l = torch.randn(heads, width, generator=gen) / width ** 0.5
    att_r = torch.randn(heads, width, generator=gen) / width ** 0.5
    left, right = (x * att_l).sum(-1), (x * att_r).sum(-1)

    d_rows, d_cols, d_x = rows.to(cuda_device), cols.to(cuda_device), x.to(cuda_device)
    indptr = ops_gnn.ind2ptr(d_rows, nodes)
    assert torch.equal(ops_gnn.ptr2ind(indptr, rows.numel()).cpu(), rows)
    logits = ops_gnn.sddmm_csr(indptr, d_cols, left.to(cuda_device), right.to(cuda_device), "add", "u", "v")
    alpha = ops_gnn.scatter_softmax(torch.nn.functional.leaky_relu(logits, 0.2), d_rows, 0, nodes)
    out = ops_gnn.bspmm(indptr, d_cols, d_x, "mul", "sum", rhs=alpha.unsqueeze(-1))

    ptr = oracle.ind2ptr_oracle(rows, nodes)
    want_logits = oracle.sddmm_oracle(ptr, cols, left, right, "add", "u", "v")
    assert_close(logits, want_logits, what="edge logits")
    want_alpha = oracle.grouped_softmax_oracle(torch.nn.functional.leaky_relu(want_logits, 0.2), rows, 0, nodes)
    assert_close(alpha, want_alpha, what="attention weights")
    sums = torch.zeros(nodes, heads, dtype=torch.float64).index_add_(0, rows, alpha.cpu().double())
    assert float((sums - 1).abs().max()) <= 1e-5, "every destination's weights sum to one (self loops: no empty row)"
    want = torch.zeros(nodes, heads, width, dtype=torch.float64).index_add_(
        0, rows, x.double()[cols] * want_alpha.double().unsqueeze(-1))
    magnitude = torch.zeros(nodes, heads, width, dtype=torch.float64).index_add_(
        0, rows, (x.double()[cols] * want_alpha.double().unsqueeze(-1)).abs()).clamp(min=1.0)
    error = ((out.cpu().double() - want).abs() / magnitude).max().item()
    assert error <= 2e-5, f"aggregated features: conditioned error {error:.3g}"
    # the fused form of the same layer: no [E, H] tensor in memory, weights formed inside the aggregation kernel
    fused, lse = ops_gnn.gat_aggregate(indptr, d_cols, d_x, left.to(cuda_device), right.to(cuda_device), 0.2, return_lse=True)
    assert torch.equal(fused, ops_gnn.gat_aggregate(indptr, d_cols, d_x, left.to(cuda_device), right.to(cuda_device), 0.2,
                                                    edge_rows=d_rows)), "bitwise reproducible"
    want_lse = oracle.grouped_logsumexp_oracle(torch.nn.functional.leaky_relu(want_logits, 0.2), rows, 0, nodes)
    assert_close(lse, want_lse.float(), what="log-sum-exp of the logits")
    error = ((fused.cpu().double() - want).abs() / magnitude).max().item()
    assert error <= 1e-5, f"fused layer: conditioned error {error:.3g}"


@pytest.mark.parametrize("heads,width,index_dtype", [(8, 64, torch.int64), (4, 64, torch.int32), (16, 32, torch.int64), (8, 32, torch.int32)])
def test_fused_attention_shapes_and_hub_rows(cuda_device, heads, width, index_dtype):
    """Rows that span thread blocks and 32-edge chunks, rows without edges, both index widths, every head count the fused
    kernel takes; and the shapes it refuses."""
    import ops_gnn

    gen = torch.Generator().manual_seed(8)
    nodes = 3000
    degree = torch.randint(0, 30, (nodes,), generator=gen)
    degree[7], degree[8], degree[9], degree[2000] = 9000, 0, 0, 2500
    ptr = torch.zeros(nodes + 1, dtype=torch.int64)
    ptr[1:] = degree.cumsum(0)
    col = torch.randint(0, nodes, (int(ptr[-1]),), generator=gen)
    rows = torch.repeat_interleave(torch.arange(nodes), degree)
    x = torch.randn(nodes, heads, width, generator=gen)
    left, right = torch.randn(nodes, heads, generator=gen) * 2, torch.randn(nodes, heads, generator=gen) * 2
    right[col[5], 0] = 60.0                                           # one dominant logit: the others must underflow cleanly
    args = (ptr.to(index_dtype).to(cuda_device), col.to(index_dtype).to(cuda_device), x.to(cuda_device), left.to(cuda_device),
            right.to(cuda_device))
    fused, lse = ops_gnn.gat_aggregate(*args, 0.2, return_lse=True)
    logits = torch.nn.functional.leaky_relu(left.double()[rows] + right.double()[col], 0.2)
    alpha = oracle.grouped_softmax_oracle(logits, rows, 0, nodes)
    terms = x.double()[col] * alpha.unsqueeze(-1)
    want = torch.zeros(nodes, heads, width, dtype=torch.float64).index_add_(0, rows, terms)
    magnitude = torch.zeros_like(want).index_add_(0, rows, terms.abs()).clamp(min=1.0)
    error = ((fused.cpu().double() - want).abs() / magnitude).max().item()
    assert error <= 1e-5, f"fused layer {heads}x{width}: conditioned error {error:.3g}"
    assert_close(lse, oracle.grouped_logsumexp_oracle(logits, rows, 0, nodes).float(), what="lse")
    assert bool((fused[8] == 0).all()) and bool(torch.isinf(lse[8]).all()), "a row without edges gives 0 and lse = -inf"
    composed = ops_gnn.bspmm(args[0], args[1], args[2], "mul", "sum",
                             rhs=ops_gnn.scatter_softmax(torch.nn.functional.leaky_relu(
                                 ops_gnn.sddmm_csr(args[0], args[1], args[3], args[4], "add", "u", "v"), 0.2),
                                 rows.to(cuda_device), 0, nodes).unsqueeze(-1))
    assert float((fused - composed).abs().max()) <= 2e-5 * max(float(composed.abs().max()), 1.0), "fused vs composed on the GPU"


def test_fused_attention_refuses_other_shapes(cuda_device):
    import ops_gnn

    ptr = torch.tensor([0, 1, 2], device=cuda_device)
    col = torch.tensor([1, 0], device=cuda_device)
    for heads, width in ((3, 64), (8, 20), (24, 32)):
        with pytest.raises(RuntimeError, match="unsupported shape"):
            ops_gnn.gat_aggregate(ptr, col, torch.randn(2, heads, width, device=cuda_device),
                                  torch.randn(2, heads, device=cuda_device), torch.randn(2, heads, device=cuda_device))
    with pytest.raises(RuntimeError, match="float32"):
        ops_gnn.gat_aggregate(ptr, col, torch.randn(2, 8, 64, device=cuda_device).half(), torch.randn(2, 8, device=cuda_device),
                              torch.randn(2, 8, device=cuda_device))
