"""DGL-style ``segment_reduce`` (python/ops_gnn/segment_reduce.py:30-66 of ops-gnn): a thin wrapper that promotes
int32 offsets to the int64 pointers ``segment_csr`` takes."""
from typing import Optional

import torch

from .segment_csr import segment_csr


def segment_reduce(src: torch.Tensor, offsets: torch.Tensor, out: Optional[torch.Tensor] = None,
                   reduce: str = "sum") -> torch.Tensor:
    """``out[i] = reduce(src[offsets[i]:offsets[i + 1]])``; values only for every reduction."""
    if offsets.dtype != torch.int64:
        offsets = offsets.to(torch.int64)
    return segment_csr(src, offsets, out, reduce)
