"""Opaque stand-in ops and the encapsulate / decapsulate walk (``torchrec/ir/utils.py:55-183``, ``mark_dynamic_kjt`` ``:194``).

While a model is exported, an embedding module must not be traced into its kernels: its forward is replaced by one custom op that
only produces tensors of the right shape, and the module's configuration travels in a byte buffer.  After export the walk in
``decapsulate_ir_modules`` puts real modules back (possibly quantized or sharded ones built from the same metadata).
"""
from __future__ import annotations

import logging
from typing import Dict, List, Optional, Tuple, Type, Union

import torch
from torch import nn
from torch.export import Dim, ShapesCollection

from torchrec_b200.ir.types import SerializerInterface
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor

logger: logging.Logger = logging.getLogger(__name__)


def qualname(m: Union[nn.Module, type]) -> str:
    t = m if isinstance(m, type) else type(m)
    return f"{t.__module__}.{t.__qualname__}"


def get_device(tensors: List[Optional[torch.Tensor]]) -> Optional[torch.device]:
    for t in tensors:
        if t is not None:
            return t.device
    return None


@torch.library.custom_op("trb200_ir::emb_lookup", mutates_args={})
def ir_emb_lookup(tensors: List[Optional[torch.Tensor]], batch_size: int, dims: List[int]) -> List[torch.Tensor]:
    dev = get_device(tensors)
    return [torch.empty(batch_size, d, device=dev) for d in dims]


@ir_emb_lookup.register_fake
def ir_emb_lookup_fake(tensors: List[Optional[torch.Tensor]], batch_size: int, dims: List[int]) -> List[torch.Tensor]:
    dev = get_device(tensors)
    return [torch.empty(batch_size, d, device=dev) for d in dims]


@torch.library.custom_op("trb200_ir::kt_regroup", mutates_args={})
def ir_kt_regroup(tensors: List[Optional[torch.Tensor]], batch_size: int, dims: List[int], dtype: torch.dtype = torch.float32) -> List[torch.Tensor]:
    dev = get_device(tensors)
    return [torch.empty(batch_size, d, device=dev, dtype=dtype) for d in dims]


@ir_kt_regroup.register_fake
def ir_kt_regroup_fake(tensors: List[Optional[torch.Tensor]], batch_size: int, dims: List[int], dtype: torch.dtype = torch.float32) -> List[torch.Tensor]:
    dev = get_device(tensors)
    return [torch.empty(batch_size, d, device=dev, dtype=dtype) for d in dims]


@torch.library.custom_op("trb200_ir::dynamic_batch_emb_lookup", mutates_args={})
def ir_dynamic_batch_emb_lookup(tensors: List[Optional[torch.Tensor]], batch_size: int, dims: List[int]) -> List[torch.Tensor]:
    dev = get_device(tensors)
    return [torch.empty(batch_size, d, device=dev) for d in dims]


@ir_dynamic_batch_emb_lookup.register_fake
def ir_dynamic_batch_emb_lookup_fake(tensors: List[Optional[torch.Tensor]], batch_size: int, dims: List[int]) -> List[torch.Tensor]:
    dev = get_device(tensors)
    b = torch.library.get_ctx().new_dynamic_size()  # the batch of a variable-batch KJT is not an input dimension
    return [torch.empty(b, d, device=dev) for d in dims]


# the eager bodies under the names the reference gives them (``torchrec/ir/utils.py:54-114``)
ir_emb_lookup_impl = ir_emb_lookup
ir_kt_regroup_impl = ir_kt_regroup
ir_dynamic_batch_emb_lookup_impl = ir_dynamic_batch_emb_lookup


def move_to_copy_nodes_to_device(unflattened_module: nn.Module, device: torch.device) -> nn.Module:
    """Point every ``_to_copy`` node of an unflattened exported module at ``device``: an exported graph carries the devices of the
    machine it was traced on as literals, and a module traced on the host must copy to the serving GPU instead."""
    for node in unflattened_module.graph.nodes:
        if "_to_copy" in node.name:
            node.kwargs = {k: (device if isinstance(v, torch.device) else v) for k, v in node.kwargs.items()}
    return unflattened_module


def _default_serializer() -> Type[SerializerInterface]:
    from torchrec_b200.ir.serializer import JsonSerializer

    return JsonSerializer


def encapsulate_ir_modules(module: nn.Module, serializer: Optional[Type[SerializerInterface]] = None, fqn: str = "") -> Tuple[nn.Module, List[str]]:
    """Serialise every supported submodule in place.  Returns the module and the FQNs to pass as ``preserve_module_call_signature``."""
    serializer = serializer or _default_serializer()
    preserve: List[str] = []
    if qualname(module) in serializer.module_to_serializer_cls:
        children = serializer.encapsulate_module(module)
        preserve.append(fqn)
    else:
        children = [name for name, _ in module.named_children()]
    for child in children:
        _, fqns = encapsulate_ir_modules(module.get_submodule(child), serializer, f"{fqn}.{child}" if fqn else child)
        preserve.extend(fqns)
    return module, preserve


def decapsulate_ir_modules(module: nn.Module, serializer: Optional[Type[SerializerInterface]] = None, device: Optional[torch.device] = None,
                           finalize_interpreter_modules: bool = False) -> nn.Module:
    """Children first, then the module itself when it carries an ``ir_metadata`` buffer."""
    serializer = serializer or _default_serializer()
    for name, child in list(module.named_children()):
        setattr(module, name, decapsulate_ir_modules(child, serializer, device))
    if "ir_metadata" in dict(module.named_buffers(recurse=False)):
        module = serializer.decapsulate_module(module, device)
    if finalize_interpreter_modules:
        from torch.export.unflatten import InterpreterModule

        for m in module.modules():
            if isinstance(m, InterpreterModule):
                m.finalize()
    return module


def _get_dim(name: str, min: Optional[int] = None, max: Optional[int] = None) -> Dim:
    return Dim(name, min=min, max=max)


def mark_dynamic_kjt(kjt: KeyedJaggedTensor, shapes_collection: Optional[ShapesCollection] = None, variable_length: bool = False,
                     vlen: Optional[Dim] = None, llen: Optional[Dim] = None) -> ShapesCollection:
    """Declare the dynamic dimensions of a KJT for export: ``values`` (and ``weights``) share one length, ``lengths`` / ``offsets``
    get theirs when the batch may vary too."""
    sc = shapes_collection if shapes_collection is not None else ShapesCollection()
    n = len(_DIM_COUNTER)
    _DIM_COUNTER.append(n)
    vlen = vlen if vlen is not None else _get_dim(f"vlen{n}")
    has = lambda t: t is not None and t.dim() > 0
    if has(kjt._values):
        sc[kjt._values] = (vlen,)
    if has(kjt._weights):
        sc[kjt._weights] = (vlen,)
    if variable_length:
        llen = llen if llen is not None else _get_dim(f"llen{n}", min=2)
        if has(kjt._lengths):
            sc[kjt._lengths] = (llen,)
        if has(kjt._offsets):
            sc[kjt._offsets] = (llen + 1,)
    return sc


_DIM_COUNTER: List[int] = []
