"""ctypes binding of libaiter_b200.so, marshalled the way the reference's FFI does it
(aiter/jit/core.py:1306-1620): tensors as pointers to the aiter_tensor_t POD
(aiter/utility/aiter_types.py:66-86), None as NULL, the current CUDA stream appended last,
int status + thread-local error string turned into RuntimeError.

There is no fallback: if the library is missing or does not load, importing an op fails loudly."""

from __future__ import annotations

import ctypes
import os

import torch

from .dtypes import AITER_DTYPE

_HERE = os.path.dirname(os.path.abspath(__file__))
# AITER_B200_LIB points at a library built elsewhere (same C-ABI); default: the in-tree build
LIB_PATH = os.environ.get("AITER_B200_LIB") or os.path.join(_HERE, "libaiter_b200.so")


class aiter_tensor_t(ctypes.Structure):
    _fields_ = [
        ("ptr", ctypes.c_void_p),
        ("numel_", ctypes.c_size_t),
        ("ndim", ctypes.c_int),
        ("shape", ctypes.c_int64 * 8),
        ("strides", ctypes.c_int64 * 8),
        ("dtype_", ctypes.c_int),
        ("device_id", ctypes.c_int),
    ]


assert ctypes.sizeof(aiter_tensor_t) == 160

_T = ctypes.POINTER(aiter_tensor_t)
_SIGNATURES = {
    "aiter_ctypes_abi_version": (ctypes.c_int, []),
    "aiter_get_last_error": (ctypes.c_char_p, []),
    "aiter_clear_last_error": (None, []),
    "b200_moe_sorting_get_workspace_size": (ctypes.c_int64, [ctypes.c_int] * 4),
    "b200_moe_sorting_fwd": (ctypes.c_int, [_T] * 7 + [ctypes.c_int, ctypes.c_int, _T, _T, _T,
                                                ctypes.c_int, _T, _T, _T, ctypes.c_void_p]),
    "b200_moe_sorting_fwd_noalloc": (ctypes.c_int, [_T] * 7 + [ctypes.c_int, ctypes.c_int, _T, _T, _T,
                                                        ctypes.c_void_p]),
    "b200_moe_quant_1x128": (ctypes.c_int, [_T] * 4 + [ctypes.c_int, ctypes.c_int, ctypes.c_void_p]),
    "b200_moe_quant_per_token": (ctypes.c_int, [_T] * 4 + [ctypes.c_int, ctypes.c_void_p]),
    "b200_moe_stage1": (ctypes.c_int, [_T] * 10 + [ctypes.c_int, _T, ctypes.c_int, ctypes.c_void_p]),
    "b200_moe_stage2": (ctypes.c_int, [_T] * 10 + [ctypes.c_int] * 5 + [ctypes.c_void_p]),
    "b200_biased_grouped_topk": (ctypes.c_int, [_T] * 4 + [ctypes.c_int] * 3 + [ctypes.c_float, ctypes.c_void_p]),
    "b200_topk_softmax": (ctypes.c_int, [_T] * 4 + [ctypes.c_int, ctypes.c_void_p]),
    "b200_moe_finalize": (ctypes.c_int, [_T] * 2 + [ctypes.c_void_p]),
    "b200_moe_quant_per_tensor": (ctypes.c_int, [_T] * 6 + [ctypes.c_void_p]),
    "b200_ep_dispatch": (ctypes.c_int, [_T] * 5 + [ctypes.c_int] * 3 + [_T, ctypes.c_void_p]),
    "b200_ep_quant_dispatch": (ctypes.c_int, [_T] * 4 + [ctypes.c_int] * 3 + [_T, ctypes.c_void_p]),
    "b200_ep_push_partials": (ctypes.c_int, [_T] * 3 + [ctypes.c_int] * 3 + [_T] + [ctypes.c_int] * 3 + [ctypes.c_void_p]),
    "b200_ep_combine": (ctypes.c_int, [_T] * 4 + [ctypes.c_int] * 3 + [_T, ctypes.c_void_p]),
    "b200_ep_ipc_export": (ctypes.c_int, [_T, ctypes.c_void_p, ctypes.POINTER(ctypes.c_int64)]),
    "b200_ep_ipc_open": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(ctypes.c_int64)]),
    "b200_ep_ipc_close": (ctypes.c_int, [ctypes.c_int64, ctypes.c_int]),
    "b200_moe_debug_config": (ctypes.c_int, [ctypes.c_int64, ctypes.c_int]),
}

_lib = None

# Kernel launches behind one call of an entry point (the sort takes three kernels above 16384 routes, one below;
# the per-tensor quantiser two). ``launch_count`` adds them up for callers that report how many kernels they ran.
_KERNELS_PER_CALL = {"b200_moe_quant_per_tensor": 2}
launch_count = 0


def lib():
    """Loads the shared library once; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m aiter_b200.build` "
                "(there is no CPU or PyTorch fallback for these ops)")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError if the symbol is not exported
            fn.restype = res
            fn.argtypes = args
        if handle.aiter_ctypes_abi_version() != 4:
            raise RuntimeError("libaiter_b200.so: unexpected C-ABI version")
        _lib = handle
    return _lib


def exported_symbols():
    return sorted(_SIGNATURES)


def to_aiter(t: torch.Tensor | None):
    """torch.Tensor -> aiter_tensor_t (None -> NULL). The struct only borrows the storage."""
    if t is None:
        return None
    if t.dtype not in AITER_DTYPE:
        raise TypeError(f"unsupported dtype for the C-ABI: {t.dtype}")
    if t.dim() > 8:
        raise ValueError("tensors of more than 8 dimensions are not supported")
    s = aiter_tensor_t()
    s.ptr = t.data_ptr()
    s.numel_ = t.numel()
    s.ndim = t.dim()
    for i in range(t.dim()):
        s.shape[i] = t.shape[i]
        s.strides[i] = t.stride(i)
    s.dtype_ = AITER_DTYPE[t.dtype]
    s.device_id = t.device.index if t.is_cuda else -1
    return s


def call_plain(name: str, *args):
    """Calls an int-status entry point that takes plain integers and no stream."""
    handle = lib()
    status = getattr(handle, name)(*args)
    if status != 0:
        msg = handle.aiter_get_last_error()
        raise RuntimeError(f"{name} failed: {msg.decode() if msg else 'unknown error'}")


def call(name: str, *args, device: torch.device | None = None):
    """Calls an int-status entry point; tensors are marshalled, the stream of ``device`` (or of
    the first CUDA tensor) is appended."""
    handle = lib()
    fn = getattr(handle, name)
    keep = []
    cargs = []
    for a in args:
        if isinstance(a, torch.Tensor):
            if device is None and a.is_cuda:
                device = a.device
            s = to_aiter(a)
            keep.append(s)
            cargs.append(ctypes.byref(s))
        elif a is None:
            cargs.append(None)
        else:
            cargs.append(a)
    if device is None:
        raise RuntimeError(f"{name}: no CUDA tensor among the arguments")
    stream = torch.cuda.current_stream(device).cuda_stream
    global launch_count
    if name == "b200_moe_sorting_fwd":
        launch_count += 3 if args[0].numel() > 16384 else 1
    else:
        launch_count += _KERNELS_PER_CALL.get(name, 1)
    status = fn(*cargs, ctypes.c_void_p(stream))
    if status != 0:
        msg = handle.aiter_get_last_error()
        raise RuntimeError(f"{name} failed: {msg.decode() if msg else 'unknown error'}")
