"""Prefill entry point with built-in scratch (`lora_b200_add_prefill_noalloc`).

Some users of this library may not allocate device memory where they call it: code that is
being captured into (or replayed from) a CUDA graph, plug-ins that only receive the input and
output buffers of their host framework, serving loops that must never reach cudaMalloc because
it stalls the whole device.  For them the prefill kernels can run on a fixed 8 MiB array that
ships inside the library.  This file checks, through the C ABI, that the entry point gives the
same result as the regular one (which takes caller-provided scratch), on two calls in a row
(the second call finds the first call's intermediate still in the shared array), that an
oversized batch is refused with a clear message, and that no device memory is allocated.

The file name sorts last on purpose: a failure here stops a `-x` run only after every other
test has run.
"""

import pytest
import torch

from helpers import assert_lora_close
from nanovllm_voxcpm_b200 import _native as N
from nanovllm_voxcpm_b200 import lora as LORA
from nanovllm_voxcpm_b200 import workloads as W
from oracle import lora_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _noalloc_add(d: W.Projection, y: torch.Tensor, scaling: float = 1.0) -> int:
    return N.lib().lora_b200_add_prefill_noalloc(
        y.data_ptr(), y.stride(0), d.x.data_ptr(), d.x.stride(0), d.x.size(0), d.x.size(1), len(d.a_slabs),
        N.ptr_array(d.a_slabs), N.ptr_array(d.b_slabs), N.int_array(d.out_sizes), N.int_array(d.col_offsets),
        d.a_slabs[0].size(0), d.a_slabs[0].size(1), None, d.token_to_slot.data_ptr(), scaling,
        torch.cuda.current_stream().cuda_stream,
    )


def _regular_add(d: W.Projection, y: torch.Tensor, scaling: float = 1.0) -> None:
    meta = LORA.LoRAMetadata(d.token_to_slot, None, None, None, None, False, 0)
    LORA.launch_add(y, d.x, d.a_slabs, d.b_slabs, d.out_sizes, d.col_offsets, meta, scaling, impl=N.IMPL_SGMV)


def test_noalloc_matches_regular_entry_point_twice_in_a_row():
    cases = [
        W.prefill_projection("qkv", seed=5, lengths=[300, 90, 211]),   # first call
        W.prefill_projection("o", seed=6, lengths=[64, 500, 129, 7]),  # second call: other shapes, stale scratch
    ]
    cases[1].token_to_slot[70:90] = -1
    for i, p in enumerate(cases):
        d = p.to_device(DEV)
        y_regular, y_noalloc = d.y.clone(), d.y.clone()
        _regular_add(d, y_regular)
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        rc = _noalloc_add(d, y_noalloc)
        torch.cuda.synchronize()
        assert rc == 0, N.lib().lora_b200_last_error().decode()
        assert torch.cuda.memory_allocated() == before, "the no-allocation entry point must not allocate"
        # same kernels, same inputs: the tolerance of the path is far wider than needed
        assert_lora_close(y_noalloc, y_regular.float(), what=f"call {i}: noalloc vs regular")
        assert torch.equal(y_noalloc, y_regular)
        ref = O.add_lora(p.y, p.x, p.a_slabs, p.b_slabs, p.token_to_slot, 1.0, p.col_offsets)
        assert_lora_close(y_noalloc, ref, what=f"call {i}: noalloc vs oracle")
        none = p.token_to_slot < 0
        assert torch.equal(y_noalloc.cpu()[none], p.y[none])
    assert N.device_status() == 0


def test_noalloc_rejects_batches_beyond_the_builtin_scratch():
    cap = N.lib().lora_b200_static_scratch_bytes()
    assert cap == 8 << 20
    T = 40000  # 2 slices x 40000 tokens x rank 64 x 2 bytes = 10.2 MB > 8 MiB
    assert N.workspace_bytes(T, 2, 64) > cap
    x = torch.zeros(T, 64, dtype=torch.bfloat16, device=DEV)
    y = torch.zeros(T, 128, dtype=torch.bfloat16, device=DEV)
    a = [torch.zeros(1, 64, 64, dtype=torch.bfloat16, device=DEV) for _ in range(2)]
    b = [torch.zeros(1, 64, 64, dtype=torch.bfloat16, device=DEV) for _ in range(2)]
    d = W.Projection(x, y, a, b, [64, 64], [0, 64], torch.tensor([64]), torch.zeros(T, dtype=torch.int32, device=DEV))
    rc = _noalloc_add(d, y)
    assert rc == N.E_WORKSPACE
    msg = N.lib().lora_b200_last_error().decode()
    assert "built-in scratch" in msg and str(cap) in msg
    torch.cuda.synchronize()
    assert not y.any()  # nothing was launched
