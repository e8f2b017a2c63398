"""Introspection helpers for sharded inference models: the batched quantized kernels behind a sharded module, their table specs,
where every tensor of a module tree lives, and the embedding modules of a model by path.
Counterpart of ``torchrec/distributed/infer_utils.py:32-195``."""
from __future__ import annotations

from typing import Dict, List, Optional, Set, Tuple, Type

import torch

from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection, EmbeddingCollection
from torchrec_b200.ops.qtbe import QuantTableBatchedEmbeddingBags
from torchrec_b200.quant.embedding_modules import EmbeddingBagCollection as QuantEmbeddingBagCollection
from torchrec_b200.quant.embedding_modules import EmbeddingCollection as QuantEmbeddingCollection


def _sharded_quant_types() -> Tuple[type, ...]:
    from torchrec_b200.distributed.quant_embedding import ShardedQuantEmbeddingCollection
    from torchrec_b200.distributed.quant_embeddingbag import ShardedQuantEmbeddingBagCollection

    return (ShardedQuantEmbeddingBagCollection, ShardedQuantEmbeddingCollection)


def get_tbes_from_sharded_module(module: torch.nn.Module) -> List[QuantTableBatchedEmbeddingBags]:
    """Every batched quantized lookup kernel inside a sharded quantized collection, in device order."""
    assert type(module) in _sharded_quant_types(), "Only ShardedQuantEmbeddingBagCollection and ShardedQuantEmbeddingCollection hold quantized kernels"
    return [m for m in module.modules() if isinstance(m, QuantTableBatchedEmbeddingBags)]


def get_tbe_specs_from_sharded_module(module: torch.nn.Module) -> List[Tuple[str, int, int, str, str]]:
    """``(table position, rows, dim, storage type, device)`` of every table of every kernel of ``module``."""
    names = {32: "FP32", 16: "FP16", 8: "INT8", 4: "INT4", 2: "INT2"}
    specs: List[Tuple[str, int, int, str, str]] = []
    for tbe in get_tbes_from_sharded_module(module):
        device = str(next(iter(tbe.buffers()), torch.empty(0)).device)
        for t, (rows, dim, bits) in enumerate(tbe.embedding_specs):
            specs.append((str(t), rows, dim, names.get(int(bits), str(bits)), device))
    return specs


def get_path_device_tuples(module: object, ignore_list: Optional[List[str]] = None) -> List[Tuple[str, str]]:
    """``(attribute path, device)`` of every tensor reachable from ``module`` through modules, lists, tuples and dicts.  Attribute
    names in ``ignore_list`` (default: ``embedding_tables``) are not followed."""
    ignored = set(ignore_list if ignore_list else ["embedding_tables"])
    found: List[Tuple[str, str]] = []
    seen: Set[str] = set()

    def walk(obj: object, path: str, depth: int) -> None:
        if depth > 50 or path in seen:
            return
        seen.add(path)
        if isinstance(obj, torch.Tensor):
            found.append((path, str(obj.device)))
        elif isinstance(obj, torch.nn.Module):
            for name, t in list(obj.named_parameters(recurse=False)) + list(obj.named_buffers(recurse=False)):
                walk(t, f"{path}.{name}" if path else name, depth + 1)
            for name, child in obj.named_children():
                if name not in ignored:
                    walk(child, f"{path}.{name}" if path else name, depth + 1)
            for name, value in vars(obj).items():
                if name.startswith("_parameters") or name.startswith("_buffers") or name.startswith("_modules") or name in ignored:
                    continue
                if isinstance(value, (torch.Tensor, list, tuple, dict)):
                    walk(value, f"{path}.{name}" if path else name, depth + 1)
        elif isinstance(obj, (list, tuple)):
            for i, v in enumerate(obj):
                walk(v, f"{path}[{i}]", depth + 1)
        elif isinstance(obj, dict):
            for k, v in obj.items():
                if k not in ignored:
                    walk(v, f"{path}[{k}]", depth + 1)

    walk(module, "", 0)
    return found


def get_all_torchrec_modules(model: torch.nn.Module, trec_module_class_types: Optional[List[Type[torch.nn.Module]]] = None) -> Dict[str, torch.nn.Module]:
    """``{path: module}`` of the outermost modules whose exact type is in ``trec_module_class_types`` (default: the float, quantized
    and sharded-quantized embedding collections)."""
    wanted = tuple(trec_module_class_types) if trec_module_class_types else _sharded_quant_types() + (
        QuantEmbeddingBagCollection, QuantEmbeddingCollection, EmbeddingBagCollection, EmbeddingCollection)
    out: Dict[str, torch.nn.Module] = {}
    stack: List[Tuple[str, torch.nn.Module]] = [("", model)]
    while stack:
        path, m = stack.pop()
        if type(m) in wanted:
            out[path] = m
            continue
        stack.extend((f"{path}.{n}" if path else n, c) for n, c in reversed(list(m.named_children())))
    return out


def get_non_scriptable_trec_module(model: torch.nn.Module) -> Dict[str, torch.nn.Module]:
    """The sharded quantized collections of ``model``: the modules that must be traced as leaves rather than scripted."""
    return get_all_torchrec_modules(model, trec_module_class_types=list(_sharded_quant_types()))
