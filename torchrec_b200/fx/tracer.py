"""fx tracer that treats the embedding modules (sharded or not) as leaves and accepts the sparse types as constants
(``torchrec/fx/tracer.py:27,144``)."""
from __future__ import annotations

import typing
from typing import Any, Callable, Dict, List, Optional, Union

import torch
from torch.fx._compatibility import compatibility
from torch.fx.graph import Graph
from torch.fx.node import Argument

from torchrec_b200.distributed.types import NoWait, ShardedModule

_is_fx_tracing_flag = False


def is_fx_tracing() -> bool:
    return _is_fx_tracing_flag


@compatibility(is_backward_compatible=False)
class Tracer(torch.fx.Tracer):
    """``leaf_modules``: qualified class names kept opaque besides sharded modules."""

    # keep shape arithmetic on proxies out of the graph where possible
    proxy_buffer_attributes = False

    def __init__(self, leaf_modules: Optional[List[str]] = None) -> None:
        super().__init__()
        self._leaf_modules: List[str] = leaf_modules if leaf_modules is not None else []

    def is_leaf_module(self, m: torch.nn.Module, module_qualified_name: str) -> bool:
        if type(m).__name__ in self._leaf_modules or isinstance(m, ShardedModule):
            return True
        return super().is_leaf_module(m, module_qualified_name)

    @compatibility(is_backward_compatible=True)
    def trace(self, root: Union[torch.nn.Module, Callable[..., Any]], concrete_args: Optional[Dict[str, Any]] = None) -> Graph:
        global _is_fx_tracing_flag
        old = _is_fx_tracing_flag
        _is_fx_tracing_flag = True
        try:
            return super().trace(root, concrete_args)
        finally:
            _is_fx_tracing_flag = old

    def create_arg(self, a: Any) -> Argument:
        """``NoWait`` wrappers and sparse-type instances become call nodes that rebuild them at run time."""
        if isinstance(a, NoWait):
            return self.create_node("call_function", target=NoWait, args=self.create_arg((a._obj,)), kwargs={}, type_expr=NoWait)
        from torchrec_b200.sparse.jagged_tensor import JaggedTensor, KeyedJaggedTensor

        if isinstance(a, JaggedTensor):
            return self.create_node("call_function", target=JaggedTensor, args=self.create_arg((a.values(), a.weights_or_none(), a.lengths_or_none(), a.offsets_or_none())), kwargs={})
        if isinstance(a, KeyedJaggedTensor):
            return self.create_node("call_function", target=KeyedJaggedTensor,
                                    args=self.create_arg((a.keys(), a.values(), a.weights_or_none(), a.lengths_or_none(), a.offsets_or_none())), kwargs={})
        return super().create_arg(a)

    def path_of_module(self, mod: torch.nn.Module) -> str:
        """Modules created inside a leaf's forward are not registered in the root: give them a placeholder path instead of failing."""
        try:
            return super().path_of_module(mod)
        except NameError:
            return ""


def symbolic_trace(root: Union[torch.nn.Module, Callable], concrete_args: Optional[Dict[str, Any]] = None, leaf_modules: Optional[List[str]] = None) -> torch.fx.GraphModule:
    tracer = Tracer(leaf_modules)
    graph = tracer.trace(root, concrete_args)
    return torch.fx.GraphModule(root, graph)
