"""B200-native batched multi-LoRA linear path (drop-in for nanovllm_voxcpm's
``lora.py`` / ``lora_ops`` / ``layers/lora.py`` operator interface).

Compute happens only in ``lib/libb200lora.so`` (hand-written sm_100a CUDA behind a C
ABI, see ``include/b200_lora.h``); importing the package needs no GPU, calling an
operator without the library or a CUDA device raises.
"""

from .lora import (  # noqa: F401
    B200LoRABackend,
    LoRAAvailability,
    LoRABackend,
    LoRAMetadata,
    assert_available,
    get_availability,
    get_backend,
    install_into_reference,
    is_available,
    set_backend_for_testing,
)
from .lora_ops import LoRAKernelMeta, lora_expand, lora_shrink  # noqa: F401

__all__ = [
    "B200LoRABackend", "LoRAAvailability", "LoRABackend", "LoRAMetadata", "LoRAKernelMeta", "lora_shrink",
    "lora_expand", "get_backend", "set_backend_for_testing", "get_availability", "is_available",
    "assert_available", "install_into_reference",
]
