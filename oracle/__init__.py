"""CPU oracle of the ops-gnn sparse message-passing path.  TEST INFRASTRUCTURE ONLY.

Each function restates, in vectorised torch-on-CPU, the algorithm of one of the reference's `golden.py` files (the
reference ships those goldens as per-row / per-segment / per-element Python loops that cannot finish at benchmark
sizes).  Only `tests/`, `__graft_entry__.smoke()` and the `cpu_baseline` / `--impl reference` legs of `bench.py` may
import this package; the product (`ops-gnn_b200/`) never does and has no CPU path.

Parity is pinned: `tests/golden/make_fixtures.py` ran the reference's own golden functions in a container that had
the reference checked out and stored their inputs and outputs under `tests/golden/`; `tests/test_oracle_golden.py`
checks every oracle function against those fixtures and against the known-answer vectors found in the reference's
test files.
"""
from .convert import ind2ptr_oracle, ptr2ind_oracle
from .gather import gather_coo_oracle, gather_csr_oracle
from .grouped import grouped_logsumexp_oracle, grouped_softmax_oracle
from .scatter import scatter_oracle
from .sddmm import sddmm_oracle
from .segment import segment_coo_oracle, segment_csr_oracle, segment_logsumexp_oracle
from .spmm import csr_spmm_oracle, spmm_copy_oracle

__all__ = [
    "csr_spmm_oracle", "spmm_copy_oracle", "sddmm_oracle", "segment_csr_oracle", "segment_coo_oracle",
    "segment_logsumexp_oracle", "scatter_oracle", "grouped_softmax_oracle", "grouped_logsumexp_oracle",
    "ind2ptr_oracle", "ptr2ind_oracle", "gather_csr_oracle", "gather_coo_oracle",
]
