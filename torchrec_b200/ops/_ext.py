"""Loader for the in-tree native libraries.

Two shared objects are built in-tree (see ``torchrec_b200/csrc/build.py``):

* ``_C_cuda.so``  -- the sm_100a CUDA kernels, registered as ``torch.ops.trb200.*``.
* ``_C_cpu.so``   -- CPU C++ runtime pieces (dynamic-embedding library, batching
  queue, CPU sparse kernels), registered as ``torch.ops.trb200_cpu.*`` and
  ``torch.classes.trb200.*``.

The reference reaches its kernels through ``torch.ops.fbgemm.*`` from an external
wheel (``torchrec/sparse/jagged_tensor.py:32-48``); here the kernels live in the
repository and are loaded from a fixed path so a GPU box sees exactly what was built.

On a machine with a CUDA device, an op that has a CUDA kernel refuses to run without
the CUDA library (``require_cuda_ext``) rather than silently taking a slow path.
"""
from __future__ import annotations

import os
import threading
from typing import Optional

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_PKG = os.path.dirname(_HERE)
CUDA_LIB_PATH = os.path.join(_PKG, "_C_cuda.so")
CPU_LIB_PATH = os.path.join(_PKG, "_C_cpu.so")

_lock = threading.Lock()
_cuda_loaded: Optional[bool] = None
_cpu_loaded: Optional[bool] = None
_cuda_err: Optional[str] = None
_cpu_err: Optional[str] = None


def _try_load(path: str) -> Optional[str]:
    if not os.path.exists(path):
        return f"{path} not built (run `python -c 'import __graft_entry__ as g; g.build()'`)"
    try:
        torch.ops.load_library(path)
        return None
    except Exception as e:  # pragma: no cover - depends on the machine
        return f"{type(e).__name__}: {e}"


def has_cuda_ext() -> bool:
    """True when the CUDA kernel library is loaded (it loads on CPU-only machines too)."""
    global _cuda_loaded, _cuda_err
    if _cuda_loaded is None:
        with _lock:
            if _cuda_loaded is None:
                if os.environ.get("TRB200_DISABLE_CUDA_EXT", "0") == "1":
                    _cuda_err = "disabled by TRB200_DISABLE_CUDA_EXT=1"
                else:
                    _cuda_err = _try_load(CUDA_LIB_PATH)
                _cuda_loaded = _cuda_err is None
    return bool(_cuda_loaded)


def has_cpu_ext() -> bool:
    global _cpu_loaded, _cpu_err
    if _cpu_loaded is None:
        with _lock:
            if _cpu_loaded is None:
                _cpu_err = _try_load(CPU_LIB_PATH)
                _cpu_loaded = _cpu_err is None
    return bool(_cpu_loaded)


def require_cuda_ext(op: str) -> None:
    """Raise if a CUDA tensor reached ``op`` but the kernel library is not loaded."""
    if not has_cuda_ext():
        raise RuntimeError(
            f"torchrec_b200: op '{op}' was called on a CUDA tensor but the sm_100a kernel "
            f"library is not available: {_cuda_err}"
        )


def use_cuda_kernel(t: torch.Tensor, op: str) -> bool:
    """Dispatch rule shared by every op wrapper.

    CUDA tensor -> the hand-written kernel (mandatory; raises when the library is absent).
    CPU tensor  -> the composite torch implementation, which doubles as the numerical oracle.
    """
    if t.is_cuda:
        require_cuda_ext(op)
        return True
    return False


def cuda_ops():
    require_cuda_ext("torch.ops.trb200")
    return torch.ops.trb200


def cpu_ops():
    if not has_cpu_ext():
        raise RuntimeError(f"torchrec_b200: CPU native library unavailable: {_cpu_err}")
    return torch.ops.trb200_cpu


def cpu_error() -> Optional[str]:
    """Why the native CPU library did not load (None when it did or was not tried yet)."""
    return _cpu_err


def cuda_error() -> Optional[str]:
    return _cuda_err
