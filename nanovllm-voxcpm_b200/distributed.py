"""Tensor-parallel rank / world-size getters (``nanovllm_voxcpm/utils/distributed.py``).

One process per GPU; the TP group is the default ``torch.distributed`` group.
"""

from __future__ import annotations

import torch.distributed as dist


def get_tp_world_size() -> int:
    return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1


def get_tp_rank() -> int:
    return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
