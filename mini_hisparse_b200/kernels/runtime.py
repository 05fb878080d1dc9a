"""The runtime for a compute dtype: which kernels a model's parts call for their matrix products."""
from __future__ import annotations

import torch

from ..parts.base import Runtime


def make_runtime(device, dtype: torch.dtype) -> Runtime:
    return Runtime(device, dtype)
