"""Loading the native library and IO plugins."""
from __future__ import annotations

import torch

from torchrec_b200.ops import _ext


def ensure_native() -> None:
    if not _ext.has_cpu_ext():
        raise RuntimeError("the native CPU library (_C_cpu.so) is not built: " + str(_ext.cpu_error()))


def register_io(plugin_path: str) -> None:
    """Load a storage plugin (a shared library exporting ``trb_tde_io_provider``).  The ``memory://`` store is built in."""
    ensure_native()
    torch.ops.trb_tde.register_io(plugin_path)
