"""ctypes binding of ``libevox_b200.so`` (the C ABI declared in ``include/evox_b200.h``).

There is no CPU fallback: if the library has not been built, importing this module raises.
Tensors are passed as raw device pointers; `ptr()` checks device, dtype and contiguity first.
"""

from __future__ import annotations

import ctypes
import re
from ctypes import c_char_p, c_float, c_int32, c_int64, c_size_t, c_uint64, c_void_p
from pathlib import Path

import torch

from . import _build

_TYPE_MAP = {
    "int": c_int32,
    "int32_t": c_int32,
    "int64_t": c_int64,
    "uint64_t": c_uint64,
    "uint32_t": ctypes.c_uint32,
    "size_t": c_size_t,
    "float": c_float,
    "double": ctypes.c_double,
    "const char*": c_char_p,
}


def _parse_header(path: Path) -> dict[str, tuple[object, list[object]]]:
    """Read every prototype of the header and turn it into (restype, argtypes)."""
    text = re.sub(r"/\*.*?\*/", " ", path.read_text(), flags=re.S)
    text = "\n".join(line for line in text.splitlines() if not line.lstrip().startswith("#"))
    protos = {}
    for m in re.finditer(r"([A-Za-z_][\w\s\*]*?)\b(evox_\w+)\s*\(([^)]*)\)\s*;", text):
        ret, name, args = m.group(1).strip(), m.group(2), m.group(3).strip()
        ret = ret.replace('extern "C"', "").strip()
        restype = _TYPE_MAP.get(ret.replace(" *", "*"), None)
        if restype is None:
            raise RuntimeError(f"unsupported return type {ret!r} of {name}")
        argtypes = []
        if args and args != "void":
            for a in args.split(","):
                a = " ".join(a.split())
                if "*" in a:
                    argtypes.append(c_void_p)
                else:
                    base = a.rsplit(" ", 1)[0].replace("const ", "").strip()
                    argtypes.append(_TYPE_MAP[base])
        protos[name] = (restype, argtypes)
    return protos


HEADER = _build.INCLUDE / "evox_b200.h"
PROTOTYPES = _parse_header(HEADER)


def _load() -> ctypes.CDLL:
    path = _build.LIB_PATH
    if not _build.is_current():
        try:
            _build.build()  # fresh checkout or edited sources: compile once (needs nvcc)
        except Exception as exc:
            raise ImportError(
                f"{path} is missing and could not be built ({exc}). The evox_b200 CUDA kernels are "
                "required; there is no CPU fallback."
            ) from exc
    lib = ctypes.CDLL(str(path))
    for name, (restype, argtypes) in PROTOTYPES.items():
        fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
        fn.restype = restype
        fn.argtypes = argtypes
    return lib


lib = _load()


class EvoxKernelError(RuntimeError):
    """A C-ABI call returned a non-zero code."""


def check(rc: int) -> None:
    if rc != 0:
        msg = lib.evox_last_error()
        raise EvoxKernelError(f"evox_b200 error {rc}: {msg.decode() if msg else '?'}")


def ptr(t: torch.Tensor | None, dtype: torch.dtype | None = None, name: str = "tensor") -> int | None:
    """Device pointer of a contiguous CUDA tensor (None passes through as NULL)."""
    if t is None:
        return None
    if not t.is_cuda:
        raise EvoxKernelError(f"{name} must live on a CUDA device (evox_b200 has no CPU path), got {t.device}")
    if dtype is not None and t.dtype != dtype:
        raise EvoxKernelError(f"{name} must have dtype {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise EvoxKernelError(f"{name} must be contiguous")
    if t.device.index != torch.cuda.current_device():
        # the library launches on the calling thread's current device
        raise EvoxKernelError(
            f"{name} lives on {t.device} but the current CUDA device is cuda:{torch.cuda.current_device()}: "
            f"make the call under `torch.cuda.device({t.device.index})` (or torch.cuda.set_device)"
        )
    return t.data_ptr()


def stream_ptr(device: torch.device | None = None) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def host_floats(values) -> ctypes.Array:
    arr = (c_float * len(values))(*values)
    return arr
