"""The bounds-checked build of the library (``lib/libb200lora_debug.so``, compiled with
``-DB200_LORA_DEBUG_BOUNDS``): every index that comes from caller-provided metadata is checked on the
device before use. On valid inputs it must stay silent and compute the same results; on corrupt
metadata it must raise bit 8 of the device status word and skip the access - no trap, no fault. The
product build ignores the same corrupt entries silently (they are treated as "no adapter").

The checked library is loaded in a child process (``B200_LORA_LIB`` selects the file at import time).
"""

import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r'''
import os, sys
import torch
sys.path.insert(0, os.environ["B200_TEST_ROOT"]); sys.path.insert(0, os.path.join(os.environ["B200_TEST_ROOT"], "tests"))
from helpers import assert_lora_close
from nanovllm_voxcpm_b200 import _native as N, batch_plan as BP, lora as LORA, workloads as W
from oracle import lora_oracle as O

DEV = "cuda"
expect_reports = os.environ["B200_EXPECT_REPORTS"] == "1"

def meta_of(slots):
    ctx = BP.build_lora_context_from_batch_plan(BP.build_lora_batch_plan_from_token_to_slot({}, slots.tolist()), device=DEV)
    return LORA.LoRAMetadata(ctx.token_to_slot, ctx.token_indices_sorted_by_slot, ctx.active_slot_ids,
                             ctx.num_tokens_per_slot, ctx.slot_start_offsets, False, ctx.num_active_loras)

def run(p, impl, meta=None):
    d = p.to_device(DEV)
    y = d.y.clone()
    LORA.launch_add(y, d.x, d.a_slabs, d.b_slabs, d.out_sizes, d.col_offsets, meta or meta_of(p.token_to_slot), 1.0, impl=impl)
    torch.cuda.synchronize()
    return y.cpu()

# ---- valid inputs: every kernel family, small exhaustive shapes; silent and correct
cases = [(W.decode_projection("qkv", seed=1, T=96, S=8), N.IMPL_BGMV), (W.decode_projection("down", seed=2, T=70, S=4), N.IMPL_BGMV),
         (W.make_projection(3, 200, 1024, [1024, 128, 128], 2, 32, p_none=0.2), N.IMPL_BGMV),          # several passes per bucket
         (W.make_projection(9, 70, 2048, [2048, 256, 256], 6, 64, ranks=[8, 16, 64, 8, 16, 64]), N.IMPL_BGMV),
         (W.make_projection(4, 8, 1000, [64], 2, 16), N.IMPL_GENERIC),
         (W.prefill_projection("o", seed=3, lengths=[200, 77, 133, 128, 64]), N.IMPL_SGMV)]
for p, impl in cases:
    out = run(p, impl)
    assert_lora_close(out, O.add_lora(p.y, p.x, p.a_slabs, p.b_slabs, p.token_to_slot, 1.0, p.col_offsets), what=f"impl {impl}")
assert N.device_status() == 0, "the checked build reported a violation on valid inputs"

# ---- corrupt metadata: reported (checked build) or ignored (product build); never a fault
p = W.decode_projection("o", seed=5, T=64, S=8)
good = meta_of(p.token_to_slot)
want = O.add_lora(p.y, p.x, p.a_slabs, p.b_slabs, p.token_to_slot, 1.0, p.col_offsets)

def with_(meta, **kw):
    f = dict(token_to_slot=meta.token_to_slot, token_indices_sorted_by_slot=meta.token_indices_sorted_by_slot,
             active_slot_ids=meta.active_slot_ids, num_tokens_per_slot=meta.num_tokens_per_slot,
             slot_start_offsets=meta.slot_start_offsets, no_lora_flag=False, num_active_loras=meta.num_active_loras)
    f.update(kw)
    return LORA.LoRAMetadata(**f)

# (a) a sorted row index beyond the batch
bad_rows = good.token_indices_sorted_by_slot.clone(); bad_rows[3] = 10_000
# (b) a bucket whose row range leaves the batch
bad_off = good.slot_start_offsets.clone(); bad_off[1] = 64 - 1
bad_cnt = good.num_tokens_per_slot.clone(); bad_cnt[1] = 40
# (c) a slot id beyond the slabs
bad_ids = good.active_slot_ids.clone(); bad_ids[0] = 99
for name, meta in (("row index", with_(good, token_indices_sorted_by_slot=bad_rows)),
                   ("bucket range", with_(good, slot_start_offsets=bad_off, num_tokens_per_slot=bad_cnt)),
                   ("slot id", with_(good, active_slot_ids=bad_ids))):
    out = run(p, N.IMPL_BGMV, meta)
    status = N.device_status(reset=True)
    assert bool(status & 8) == expect_reports, f"{name}: status {status}"
    assert torch.isfinite(out.float()).all()
# (d) slot ids outside [-1, S) in the slot map of the per-token and the tensor-core kernels
q = W.prefill_projection("o", seed=3, lengths=[300, 300])
q.token_to_slot[5] = 77
q.token_to_slot[400] = -9
raw_map = q.token_to_slot.to(DEV)
for impl in (N.IMPL_GENERIC, N.IMPL_SGMV):
    # bucket arrays from a sane copy of the map; the kernels under test read the raw map itself
    out = run(q, impl, with_(meta_of(q.token_to_slot.clamp(min=-1, max=15)), token_to_slot=raw_map))
    status = N.device_status(reset=True)
    assert bool(status & 8) == expect_reports, f"slot map, impl {impl}: status {status}"
# an ordinary launch afterwards
assert_lora_close(run(p, N.IMPL_BGMV), want, what="after the corrupt cases")
assert N.device_status() == 0
print("CHILD-OK")
'''


def _run_child(lib: str | None, expect_reports: bool):
    env = dict(os.environ, B200_TEST_ROOT=ROOT, B200_EXPECT_REPORTS="1" if expect_reports else "0")
    env.pop("B200_LORA_LIB", None)
    if lib is not None:
        env["B200_LORA_LIB"] = lib
    proc = subprocess.run([sys.executable, "-c", CHILD], env=env, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0 and "CHILD-OK" in proc.stdout, proc.stdout[-2000:] + proc.stderr[-4000:]


def test_bounds_checked_build_is_silent_on_valid_inputs_and_reports_corrupt_metadata():
    from nanovllm_voxcpm_b200.build import DEBUG_LIB_PATH, build_library

    if not os.path.exists(DEBUG_LIB_PATH):
        build_library(debug_bounds=True)  # nvcc is part of the image; the file normally travels prebuilt
    assert torch.cuda.is_available()
    _run_child(DEBUG_LIB_PATH, expect_reports=True)


def test_product_build_ignores_the_same_corrupt_metadata_without_a_fault():
    _run_child(None, expect_reports=False)
