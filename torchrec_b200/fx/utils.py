"""Small fx helpers (``torchrec/fx/utils.py:30-154``): markers that survive tracing, assertions that tracing skips, and a
scriptable wrapper of a traced model-parallel forward."""
from __future__ import annotations

from typing import Any, Dict, List, Set, Union

import torch
from torch.fx._symbolic_trace import is_fx_tracing as _torch_is_fx_tracing

from torchrec_b200.fx.tracer import is_fx_tracing


def fake_range() -> Any:
    return torch._C._jit_tree_views.SourceRangeFactory("", None, 0, 0).make_raw_range(0, 1)


def _fx_marker(s: str, any_proxy_unused: Any) -> None:
    pass


@torch.fx.wrap
def fx_marker(s: str, any_proxy_unused: Any) -> None:
    """A no-op call that stays in the traced graph: marks regions (``KJT_ONE_TO_ALL_FORWARD_BEGIN`` ...) for graph passes."""
    pass


def is_marker_node(node: torch.fx.Node, marker_name: str) -> bool:
    return bool(node.op == "call_function" and node.target == fx_marker and isinstance(node.args[0], str) and node.args[0] == marker_name)


@torch.jit.ignore
def assert_fx_safe(condition: bool, message: str) -> None:
    """``assert`` that does not try to evaluate a proxy while a graph is being traced."""
    if not is_fx_tracing() and not _torch_is_fx_tracing():
        assert condition, message


def dmp_fx_trace_forward(dmp: torch.nn.Module, tracer: torch.fx.Tracer) -> torch.fx.GraphModule:
    """Trace the forward of a model-parallel wrapper (sharded modules stay leaves) into a ``GraphModule`` whose code imports the
    sparse types it mentions, so that the generated source runs stand-alone."""
    module = dmp.module if hasattr(dmp, "module") else dmp
    graph = tracer.trace(module)
    gm = torch.fx.GraphModule(module, graph)
    from torchrec_b200.distributed.types import NoWait
    from torchrec_b200.sparse.jagged_tensor import JaggedTensor, KeyedJaggedTensor, KeyedTensor

    for cls in (NoWait, JaggedTensor, KeyedJaggedTensor, KeyedTensor):
        gm.graph._codegen._body_transformer = getattr(gm.graph._codegen, "_body_transformer", None)
        setattr(torch.fx.graph, "_trb200_" + cls.__name__, cls)
    gm.recompile()
    return gm
