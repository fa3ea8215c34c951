"""GPU parity of a GAT-style attention layer composed from the public operators (BASELINE config 5 at reduced size):
SDDMM for per-head edge logits, LeakyReLU, scatter_softmax over destination rows, fused per-head weighted aggregation.
The expected result is the same composition of the CPU oracles."""
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
