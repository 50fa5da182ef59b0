"""Loads the sm_100a kernel library and exposes its C entry points.

There is no other implementation behind these functions: if the library cannot be built or
loaded, or the device is not a compute-capability-10 GPU, the import of an op fails with the
reason.  Nothing here falls back to the CPU or to a library's model code.
"""

from __future__ import annotations

import ctypes
import threading
from ctypes import c_char_p, c_float, c_int, c_longlong, c_ulonglong, c_void_p

import torch

from ..csrc import build

GK_F32, GK_BF16 = 0, 1
INTERFACE_VERSION = 1


class KernelError(RuntimeError):
    """A kernel entry point refused its arguments or a launch failed."""


_lock = threading.Lock()
_lib: ctypes.CDLL | None = None

P, I, L, F, U = c_void_p, c_int, c_longlong, c_float, c_ulonglong

_SIGNATURES: dict[str, list] = {
    "gk_embed_rows": [P, I, P, P, I, I, P],
    "gk_add_rmsnorm": [P, P, I, P, I, P, I, P, I, I, F, P],
    "gk_swiglu": [P, P, I, I, I, I, P],
    "gk_decode_layers_plan": [I, I, I, I, I, I, I, I, P],
    "gk_decode_layers": [P, I, I, I, I, I, I, I, P, P, P, P, P, L, P, P, P, P, I, I, P, P, I, I, I, F, P, P, P],
    "gk_qk_norm_rope_write": [P, I, P, P, I, P, P, I, P, P, P, P, P, P, P, I, I, I, I, I, I, F, I, I, P],
    "gk_gemm_f32": [P, I, P, P, I, I, I, I, L, L, L, P],
    "gk_attention_exact": [P, P, P, P, I, P, P, P, P, I, I, I, I, I, I, F, I, P],
    "gk_attention_decode_bf16": [P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, F, I, I, P],
    "gk_gemm_bf16_tc": [P, I, L, P, I, L, I, P, I, L, L, I, I, I, I, I, P, P],
    "gk_gemm_bf16_tc_qkv": [P, I, P, I, I, I, I, P, P, I, I, F, P, P, I, I, P, P, P, P, I, I, P, P, P, P, P],
    "gk_gemv_bf16": [P, I, I, L, P, I, L, P, I, I, P],
    "gk_gemv_bf16_stream": [P, I, I, L, P, I, L, P, I, I, P, L, P, I, F, P, L, P],
    "gk_set_pdl": [I],
    "gk_attention_decode_resident_clusters": [I, I],
    "gk_set_gemm_pairs": [I],
    "gk_set_attention_prefill_keys": [I],
    "gk_set_attention_prefill_one_tile": [I],
    "gk_attention_decode_fused_bf16": [P, P, P, I, I, F, P, P, I, I, I, P, P, P, P, P, P, P, P, I, I, I, I, I, I, F, I, I, P],
    "gk_attention_decode_flat_bf16": [P, P, P, P, I, I, F, P, P, I, I, I, P, P, P, P, P, P, P, P, I, I, I, I, I, I, F, I, I, P],
    "gk_attention_decode_flat_resident_blocks": [I],
    "gk_attention_decode_bf16_no_alloc": [P, P, P, P, P, P, P, I, I, I, I, I, I, F, I, I, P],
    "gk_attention_prefill_bf16": [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, F, I, P],
    "gk_attention_prefill_tc_bf16": [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, L, F, I, P, P],
    "gk_attention_prefill_tc_tokens_bf16": [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, L, F, I, P, P, L],
    "gk_set_attention_prefill_stay": [I],
    "gk_argmax": [P, L, I, I, P, I, P, P],
    "gk_sample": [P, L, I, I, F, I, U, P, P, I, P, I, P, P],
}


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return GK_F32
    if dtype == torch.bfloat16:
        return GK_BF16
    raise KernelError(f"kernels take float32 or bfloat16, not {dtype}")


def library() -> ctypes.CDLL:
    """The loaded library; built on first use."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = build.library_path(build=True)
        lib = ctypes.CDLL(str(path))
        lib.gk_last_error.restype = c_char_p
        lib.gk_last_error.argtypes = []
        lib.gk_interface_version.restype = c_int
        if lib.gk_interface_version() != INTERFACE_VERSION:
            raise KernelError(f"{path} has interface {lib.gk_interface_version()}, expected {INTERFACE_VERSION}; rebuild it")
        for name, argtypes in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = c_int
        lib.gk_device_capability.restype = c_int
        _lib = lib
        return lib


_checked_devices: set[int] = set()


def require_device(device: torch.device) -> None:
    """Fails loudly unless ``device`` is a CUDA device of compute capability 10.x."""
    if device.type != "cuda":
        raise KernelError(f"this library runs on a B200 (sm_100a) only; got device {device}")
    index = device.index if device.index is not None else torch.cuda.current_device()
    if index in _checked_devices:
        return
    major, minor = torch.cuda.get_device_capability(index)
    if major != 10:
        raise KernelError(f"kernels are built for sm_100a; device {index} has compute capability {major}.{minor}")
    library()
    _checked_devices.add(index)


def ptr(tensor: torch.Tensor | None) -> int | None:
    return None if tensor is None else tensor.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream_ptr() -> int:
    """The current CUDA stream of the current device as a raw handle.  Asked for at every launch (a graph
    capture switches streams), so through the one C call that does nothing else where torch has it: building
    a ``torch.cuda.Stream`` object costs more than launching the kernel."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


launch_count = 0  # entries into the kernel library since import (each is one or more kernel launches)


_entries: dict[str, object] = {}  # name -> the library's function, looked up once


def call(name: str, *args) -> None:
    global launch_count
    launch_count += 1
    entry = _entries.get(name)
    if entry is None:
        entry = _entries[name] = getattr(library(), name)
    if entry(*args) != 0:
        raise KernelError(f"{name}: {library().gk_last_error().decode(errors='replace')}")
