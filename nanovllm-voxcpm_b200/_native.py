"""ctypes binding of the C-ABI library (``lib/libb200lora.so``).

The library is the only compute path of this package: there is no Python or
CPU fallback. Importing this module without the built library raises; calling a
launch function without a CUDA device raises.  The C declarations live in
``include/b200_lora.h``.
"""

from __future__ import annotations

import contextlib
import ctypes
import os
from ctypes import POINTER, c_char_p, c_float, c_int32, c_int64, c_size_t, c_void_p

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
#: B200_LORA_LIB points at another build of the same ABI (e.g. an instrumented one)
LIB_PATH = os.environ.get("B200_LORA_LIB") or os.path.join(_HERE, "lib", "libb200lora.so")

ABI_VERSION = 1

DT_BF16, DT_F16, DT_F32 = 0, 1, 2
IMPL_AUTO, IMPL_GENERIC, IMPL_BGMV, IMPL_SGMV = 0, 1, 2, 3
MAX_SLICES = 4

E_INVAL, E_UNSUPPORTED, E_CUDA, E_WORKSPACE = -1, -2, -3, -4

_DTYPES = {torch.bfloat16: DT_BF16, torch.float16: DT_F16, torch.float32: DT_F32}

#: every symbol declared in include/b200_lora.h, with (restype, argtypes)
_SIGNATURES = {
    "lora_b200_version": (c_int32, []),
    "lora_b200_last_error": (c_char_p, []),
    "lora_b200_add": (
        c_int32,
        [c_void_p, c_int64, c_void_p, c_int64, c_int32, c_int32, c_int32, POINTER(c_void_p), POINTER(c_void_p),
         POINTER(c_int32), POINTER(c_int32), c_int32, c_int32, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
         c_void_p, c_void_p, c_int32, c_float, c_int32, c_int32, c_void_p, c_size_t, c_void_p],
    ),
    "lora_b200_delta": (
        c_int32,
        [c_void_p, c_int64, c_void_p, c_int64, c_int32, c_int32, c_int32, POINTER(c_void_p), POINTER(c_void_p),
         POINTER(c_int32), POINTER(c_int32), c_int32, c_int32, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
         c_void_p, c_void_p, c_int32, c_float, c_int32, c_int32, c_void_p, c_size_t, c_void_p],
    ),
    "lora_b200_shrink": (
        c_int32,
        [c_void_p, c_int32, c_void_p, c_int64, c_int32, c_int32, c_int32, POINTER(c_void_p), c_int32, c_int32,
         c_void_p, c_float, c_int32, c_void_p],
    ),
    "lora_b200_expand": (
        c_int32,
        [c_void_p, c_int64, c_void_p, c_int32, c_int32, c_int32, POINTER(c_void_p), POINTER(c_int32),
         POINTER(c_int32), c_int32, c_int32, c_void_p, c_int32, c_int32, c_void_p],
    ),
    "lora_b200_workspace_bytes": (c_size_t, [c_int32, c_int32, c_int32]),
    "lora_b200_linear_lora": (
        c_int32,
        [c_void_p, c_int64, c_void_p, c_int64, c_int32, c_int32, c_void_p, c_int64, c_int32, c_void_p, c_int32,
         POINTER(c_void_p), POINTER(c_void_p), POINTER(c_int32), POINTER(c_int32), c_int32, c_int32, c_void_p,
         c_void_p, c_float, c_void_p, c_size_t, c_void_p],
    ),
    "lora_b200_add_prefill_noalloc": (
        c_int32,
        [c_void_p, c_int64, c_void_p, c_int64, c_int32, c_int32, c_int32, POINTER(c_void_p), POINTER(c_void_p),
         POINTER(c_int32), POINTER(c_int32), c_int32, c_int32, c_void_p, c_void_p, c_float, c_void_p],
    ),
    "lora_b200_static_scratch_bytes": (c_size_t, []),
    "lora_b200_build_metadata": (
        c_int32, [c_void_p, c_int32, c_int32, c_int32, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    ),
    "lora_b200_load_slot": (c_int32, [c_void_p, c_int32, c_int64, c_void_p]),
    "lora_b200_glue_add_rmsnorm": (
        c_int32, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int32, c_int32,
                  c_float, c_int32, c_int32, c_void_p],
    ),
    "lora_b200_glue_rope_kv_store": (
        c_int32, [c_void_p, c_int64, c_int32, c_int32, c_int32, c_int32, c_void_p, c_void_p, c_void_p, c_int32, c_int32,
                  c_int32, c_void_p, c_void_p, c_void_p, c_int32, c_void_p],
    ),
    "lora_b200_glue_silu_mul": (c_int32, [c_void_p, c_int64, c_void_p, c_int64, c_int32, c_int32, c_int32, c_void_p]),
    "lora_b200_tp_allreduce": (
        c_int32, [c_void_p, c_void_p, c_int32, POINTER(c_void_p), c_int32, c_int32, c_int32, c_void_p],
    ),
    "lora_b200_tp_exchange_bytes": (c_size_t, [c_int32, c_int32]),
    "lora_b200_shrink_allreduce_expand": (
        c_int32,
        [c_void_p, c_int64, c_void_p, c_int64, c_int32, c_int32, c_int32, POINTER(c_void_p), POINTER(c_void_p),
         POINTER(c_int32), POINTER(c_int32), c_int32, c_int32, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
         c_void_p, c_void_p, c_int32, c_float, c_int32, c_void_p, POINTER(c_void_p), c_int32, c_int32, c_int32, c_void_p],
    ),
    "lora_b200_set_option": (c_int32, [c_int32, c_int32]),
    "lora_b200_device_status": (c_int32, [POINTER(c_int32), c_int32]),
}

OPT_CLUSTER, OPT_PDL, OPT_RING_KB, OPT_KSPLIT, OPT_PEER_POLL_LIMIT = 1, 2, 3, 6, 7
META_GRAPH, META_KERNEL, META_EAGER = 0, 1, 2


class NativeLibraryError(RuntimeError):
    pass


def _load() -> ctypes.CDLL:
    if not os.path.exists(LIB_PATH):
        raise NativeLibraryError(
            f"{LIB_PATH} is missing: build it with `python -m nanovllm_voxcpm_b200.build` "
            "(nvcc, sm_100a). This package has no fallback path."
        )
    lib = ctypes.CDLL(LIB_PATH)
    for name, (restype, argtypes) in _SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the build is stale
        fn.restype = restype
        fn.argtypes = argtypes
    got = lib.lora_b200_version()
    if got != ABI_VERSION:
        raise NativeLibraryError(f"{LIB_PATH} has ABI version {got}, this package needs {ABI_VERSION}: rebuild it")
    return lib


_LIB: ctypes.CDLL | None = None


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        _LIB = _load()
    return _LIB


def exported_symbols() -> list[str]:
    return list(_SIGNATURES)


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise ValueError(f"unsupported LoRA dtype {dtype}; expected bfloat16, float16 or float32") from None


def check(rc: int) -> None:
    """Map a C status to the exceptions the reference raises before launch."""
    if rc == 0:
        return
    msg = lib().lora_b200_last_error().decode("utf-8", "replace")
    if rc == E_INVAL:
        raise ValueError(msg)
    raise RuntimeError(msg)


def require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError(
                "nanovllm_voxcpm_b200 runs on CUDA tensors only (sm_100a kernels, no CPU fallback); "
                f"got a tensor on {t.device}"
            )


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


_PTR_ARRAYS: dict[tuple, ctypes.Array] = {}
_INT_ARRAYS: dict[tuple, ctypes.Array] = {}


def ptr_array(tensors) -> ctypes.Array:
    """Host array of device pointers; arrays are kept per pointer tuple (a layer passes the same slabs every call)."""
    key = tuple(t.data_ptr() if t is not None else 0 for t in tensors)
    arr = _PTR_ARRAYS.get(key)
    if arr is None:
        if len(_PTR_ARRAYS) > 4096:
            _PTR_ARRAYS.clear()
        arr = (c_void_p * len(key))(*[v or None for v in key])
        _PTR_ARRAYS[key] = arr
    return arr


def int_array(values) -> ctypes.Array:
    key = tuple(int(v) for v in values)
    arr = _INT_ARRAYS.get(key)
    if arr is None:
        if len(_INT_ARRAYS) > 4096:
            _INT_ARRAYS.clear()
        arr = (c_int32 * len(key))(*key)
        _INT_ARRAYS[key] = arr
    return arr


_RAW_STREAM = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_NULL_CONTEXT = contextlib.nullcontext()


def current_stream(device: torch.device) -> int:
    """Raw ``cudaStream_t`` of torch's current stream on ``device`` (a few hundred nanoseconds)."""
    if _RAW_STREAM is not None:
        return _RAW_STREAM(device.index if device.index is not None else torch.cuda.current_device())
    return torch.cuda.current_stream(device).cuda_stream


def on_device(device: torch.device):
    """Context manager that makes ``device`` current; nothing happens when it already is (the usual case: the
    full ``torch.cuda.device`` guard costs several microseconds per launch)."""
    if device.index is None or device.index == torch.cuda.current_device():
        return _NULL_CONTEXT
    return torch.cuda.device(device)


def set_option(key: int, value: int) -> None:
    check(lib().lora_b200_set_option(key, value))


def device_status(reset: bool = False) -> int:
    """Status word of the current CUDA device (0 = healthy); synchronises."""
    out = c_int32(0)
    check(lib().lora_b200_device_status(ctypes.byref(out), 1 if reset else 0))
    return out.value


def build_metadata(token_to_slot, S: int, convention: int, sorted_idx, slot_ids, counts, offsets, info=None) -> None:
    """``lora_b200_build_metadata`` on the current stream: index arrays of the step from the device-resident
    slot map, without host loops or copies (arrays as documented in include/b200_lora.h)."""
    require_cuda(token_to_slot, sorted_idx, slot_ids, counts, offsets, info)
    for name, t in (("token_to_slot", token_to_slot), ("sorted_idx", sorted_idx), ("slot_ids", slot_ids),
                    ("counts", counts), ("offsets", offsets), ("info", info)):
        if t is not None and (t.dtype != torch.int32 or not t.is_contiguous()):
            raise ValueError(f"{name} must be a contiguous int32 tensor")
    T = token_to_slot.numel()
    if sorted_idx.numel() < T or counts.numel() < S + 1 or offsets.numel() < S + 2 or \
            (slot_ids is not None and slot_ids.numel() < S + 1) or (info is not None and info.numel() < 3):
        raise ValueError("metadata arrays are too small for T rows and S slots")
    with on_device(token_to_slot.device):
        check(lib().lora_b200_build_metadata(ptr(token_to_slot), T, S, convention, ptr(sorted_idx), ptr(slot_ids),
                                             ptr(counts), ptr(offsets), ptr(info), current_stream(token_to_slot.device)))


_WORKSPACE_BYTES: dict[tuple[int, int, int], int] = {}


def workspace_bytes(T: int, n_slices: int, r_max: int) -> int:
    key = (T, n_slices, r_max)
    got = _WORKSPACE_BYTES.get(key)
    if got is None:
        if len(_WORKSPACE_BYTES) > 4096:
            _WORKSPACE_BYTES.clear()
        got = _WORKSPACE_BYTES[key] = int(lib().lora_b200_workspace_bytes(T, n_slices, r_max))
    return got
