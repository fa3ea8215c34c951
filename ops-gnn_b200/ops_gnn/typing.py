"""Tensor aliases used in the public signatures."""
from typing import Optional

import torch

Tensor = torch.Tensor
OptTensor = Optional[torch.Tensor]

__all__ = ["Tensor", "OptTensor"]
