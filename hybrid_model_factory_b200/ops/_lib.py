"""ctypes binding of the in-tree native libraries.

``kernels()`` returns the CUDA kernel library (``_C/libhmf_b200_kernels.so``) and
``runtime()`` the host-only C++ runtime (``_C/libhmf_b200_runtime.so``).  Both are built by
``hybrid_model_factory_b200.build``.  On a machine with a GPU a missing kernel library is an
error (ops never fall back silently to PyTorch there); on a CPU-only machine the pure
PyTorch reference implementations in ``ops/reference.py`` are used instead.
"""
from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path

import torch

_PKG = Path(__file__).resolve().parent.parent
_KERNELS_PATH = _PKG / "_C" / "libhmf_b200_kernels.so"
_RUNTIME_PATH = _PKG / "_C" / "libhmf_b200_runtime.so"

_kernels = None
_runtime = None
_launch_count = 0


class NativeLibraryMissing(RuntimeError):
    pass


class KernelError(RuntimeError):
    pass


_available = None
_force_reference = os.environ.get("HMF_FORCE_REFERENCE", "0") == "1"     # read once: this is on every op's path


def kernels_available() -> bool:
    global _available
    if not _available:           # a positive answer is final; a negative one is re-checked (the library may get built)
        _available = _KERNELS_PATH.exists()
    return _available


def use_cuda_kernels(*tensors: torch.Tensor) -> bool:
    """True when the op must run on the hand-written CUDA path (all tensors on a GPU).

    ``HMF_FORCE_REFERENCE=1`` routes every op to the PyTorch reference (debugging aid);
    without it a CUDA tensor always takes the native path and a missing library raises.
    """
    if not tensors:
        return False
    for t in tensors:
        if t is not None and not t.is_cuda:
            return False
    if _force_reference:
        return False
    if not _available and not kernels_available():
        raise NativeLibraryMissing(
            f"{_KERNELS_PATH} is missing: run `python -m hybrid_model_factory_b200.build` "
            "before using CUDA tensors")
    return True


def kernels() -> ctypes.CDLL:
    global _kernels
    if _kernels is None:
        if not _KERNELS_PATH.exists():
            raise NativeLibraryMissing(
                f"{_KERNELS_PATH} is missing: run `python -m hybrid_model_factory_b200.build`")
        lib = ctypes.CDLL(str(_KERNELS_PATH))
        lib.hmf_last_error.restype = ctypes.c_char_p
        _kernels = lib
    return _kernels


def runtime() -> ctypes.CDLL:
    global _runtime
    if _runtime is None:
        if not _RUNTIME_PATH.exists():
            raise NativeLibraryMissing(
                f"{_RUNTIME_PATH} is missing: run `python -m hybrid_model_factory_b200.build`")
        _runtime = ctypes.CDLL(str(_RUNTIME_PATH))
    return _runtime


_thread_state = threading.local()


def bind_thread(device=None) -> None:
    """Makes ``device`` current for the native library on the calling thread (once per thread and
    device).  Autograd worker threads start without a current CUDA context."""
    idx = torch.cuda.current_device() if device is None or device.index is None else device.index
    if getattr(_thread_state, "device", None) != idx:
        rc = kernels().hmf_set_device(ctypes.c_int(idx))
        if rc != 0:
            raise KernelError(kernels().hmf_last_error().decode(errors="replace"))
        _thread_state.device = idx


def stream_ptr(device=None) -> ctypes.c_void_p:
    idx = -1 if device is None or device.index is None else device.index
    if idx < 0 or getattr(_thread_state, "device", None) != idx:
        bind_thread(device)
        idx = _thread_state.device
    return ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(idx))


def ptr(t: torch.Tensor | None) -> ctypes.c_void_p:
    """Device address of ``t`` for a kernel argument.  The kernels read and write 8- and 16-bit data 16 bytes at a
    time, so such a tensor of 16 bytes or more must start on a 16-byte boundary; a view that does not (a column slice
    of a one-row matrix counts as contiguous and keeps its odd offset) is refused here, on the host, instead of
    faulting on the device.  Index, label and fp32 side inputs are read element by element and only need their natural
    alignment, which every view has."""
    if t is None:
        return ctypes.c_void_p(0)
    p = t.data_ptr()
    if (p & 15) and t.is_cuda and t.element_size() <= 2 and t.numel() * t.element_size() >= 16:
        raise ValueError(f"tensor of shape {tuple(t.shape)} ({t.dtype}) starts at {p:#x}, not on a 16-byte boundary: "
                         "clone the view before handing it to a kernel")
    return ctypes.c_void_p(p)


def aligned(t: torch.Tensor) -> torch.Tensor:
    """``t`` made contiguous, and copied when its first element is not on a 16-byte boundary."""
    t = t.contiguous()
    return t.clone() if (t.data_ptr() & 15) else t


def check(rc: int, what: str) -> None:
    """Raises ``KernelError`` with the library's message when a launcher rejected a call."""
    global _launch_count
    if rc != 0:
        msg = kernels().hmf_last_error().decode(errors="replace")
        raise KernelError(f"{what} failed (code {rc}): {msg}")
    _launch_count += 1


def launch_count() -> int:
    """Number of native kernel launches issued through this binding so far."""
    return _launch_count


def add_launches(n: int) -> None:
    global _launch_count
    _launch_count += n


def read_status(reset: bool = True) -> tuple[int, int, int, int]:
    """Returns the device status block (code, block, detail, count); code 0 means no kernel
    wait ran out since the last reset."""
    out = (ctypes.c_uint * 4)()
    rc = kernels().hmf_read_status(out, ctypes.c_int(1 if reset else 0), stream_ptr())
    if rc != 0:
        raise KernelError(kernels().hmf_last_error().decode(errors="replace"))
    return tuple(int(x) for x in out)


def assert_status_ok() -> None:
    code, block, detail, count = read_status(reset=True)
    if code != 0:
        raise KernelError(
            f"a device-side wait ran out: code={code} block={block} detail={detail:#x} count={count}")
