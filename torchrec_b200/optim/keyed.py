"""Optimizers whose state dict is keyed by parameter name.

Keys are fully qualified names, so the state survives re-sharding and can be written by a
distributed checkpoint.  ``load_state_dict`` is strict and copies *in place* into existing
``ShardedTensor`` / ``DTensor`` / plain tensor states.  Counterpart of
``torchrec/optim/keyed.py:35-515``.

Layout of this implementation: the recursive walks over nested state (``_export_leaf`` / ``_import_leaf``)
are free functions driven by small per-type handlers, and the param-group bookkeeping lives in
``_GroupIndex``; the classes only wire them to the ``torch.optim.Optimizer`` surface.
"""
from __future__ import annotations

import copy
import json
from typing import Any, Callable, Collection, Dict, Iterable, List, Mapping, Optional, Set, Tuple, Union

import torch
from torch import optim
from torch.distributed._shard.sharded_tensor import ShardedTensor

try:
    from torch.distributed.tensor import DTensor
except Exception:  # pragma: no cover
    DTensor = None  # type: ignore

OptimizerFactory = Callable[[List[Union[torch.Tensor, ShardedTensor]]], optim.Optimizer]
_SAVE_GROUPS = "_save_param_groups"


# ---- nested state: export ------------------------------------------------------------------------------------------
def _export_leaf(value: Any) -> Any:
    """Checkpoint form of one state entry: dicts recurse, stateful objects give their own state dict."""
    if isinstance(value, dict):
        return {name: _export_leaf(child) for name, child in value.items()}
    exporter = getattr(value, "state_dict", None)
    return exporter() if callable(exporter) else value


# ---- nested state: in-place import ---------------------------------------------------------------------------------
def _shard_count_error(have: int, got: int, path: List[Any]) -> ValueError:
    return ValueError(f"Different number of shards {have} vs {got} for the path of {json.dumps(path)}")


def _copy_sharded_tensor(dst: ShardedTensor, src: Any, path: List[Any]) -> None:
    assert isinstance(src, ShardedTensor)
    mine, theirs = dst.local_shards(), src.local_shards()
    if len(mine) != len(theirs):
        raise _shard_count_error(len(mine), len(theirs), path)
    for a, b in zip(mine, theirs):
        if a.tensor.shape != b.tensor.shape:
            a.tensor.resize_(b.tensor.shape)
        a.tensor.detach().copy_(b.tensor)


def _copy_dtensor(dst: Any, src: Any, path: List[Any]) -> None:
    from torchrec_b200.distributed.shards_wrapper import LocalShardsWrapper

    assert isinstance(src, DTensor)
    local = dst.to_local()
    if not isinstance(local, LocalShardsWrapper):
        dst.detach().copy_(src)
        return
    mine, theirs = local.local_shards(), src.to_local().local_shards()
    if len(mine) != len(theirs):
        raise _shard_count_error(len(mine), len(theirs), path)
    for a, b in zip(mine, theirs):
        a.detach().copy_(b)


def _import_leaf(holder: Dict[str, Any], name: str, incoming: Any, path: List[Any]) -> None:
    """Write ``incoming`` into ``holder[name]`` without replacing tensors (their memory may belong to a kernel)."""
    here = holder[name]
    if isinstance(here, dict):
        for child in here:
            _import_leaf(here, child, incoming[child], path + [child])
    elif callable(getattr(here, "load_state_dict", None)):
        here.load_state_dict(incoming)
    elif isinstance(here, ShardedTensor):
        _copy_sharded_tensor(here, incoming, path)
    elif DTensor is not None and isinstance(here, DTensor):
        _copy_dtensor(here, incoming, path)
    elif isinstance(here, torch.Tensor):
        here.detach().copy_(incoming)
    else:
        holder[name] = copy.deepcopy(incoming)


class _GroupIndex:
    """Param groups addressed by the sorted names of their parameters."""

    def __init__(self, names_of: Callable[[Mapping[str, Any]], List[str]], groups: Iterable[Mapping[str, Any]]) -> None:
        self.by_key: Dict[str, Mapping[str, Any]] = {"/".join(names_of(g)): g for g in groups}

    @staticmethod
    def options(group: Mapping[str, Any]) -> Dict[str, Any]:
        return {k: v for k, v in group.items() if k != "params"}


class KeyedOptimizer(optim.Optimizer):
    """Takes ``{name: param}`` and exposes ``state_dict`` by name.

    ``param_groups`` are not saved unless ``save_param_groups(True)``: ranks hold different
    parameters, and groups are normally re-created at start-up anyway.
    """

    def __init__(self, params: Mapping[str, Union[torch.Tensor, ShardedTensor]], state: Mapping[Any, Any], param_groups: Collection[Mapping[str, Any]]) -> None:
        # torch.optim.Optimizer.__init__ is deliberately not called: state and groups are adopted, not built
        self._optimizer_step_pre_hooks: Dict[int, Callable] = {}
        self._optimizer_step_post_hooks: Dict[int, Callable] = {}
        self.params = params
        self.state: Mapping[Any, Any] = state
        self.param_groups: Collection[Mapping[str, Any]] = param_groups
        self.defaults: Dict[str, Any] = {_SAVE_GROUPS: False}
        known = set(params.values())
        strangers = [k for k in state if k not in known]
        if strangers:
            raise ValueError(f"All state keys must be params. The following keys are not: {strangers}.")

    # kept as static methods because subclasses and tests reach them through the class
    @staticmethod
    def _extract_state_dict_content(input_dict: Dict[str, Any]) -> Dict[str, Any]:
        return _export_leaf(input_dict)

    @staticmethod
    def _update_param_state_dict_object(current: Dict[str, Any], to_load: Dict[str, Any], parent_keys: List[Any]) -> None:
        for name in current:
            _import_leaf(current, name, to_load[name], parent_keys + [name])

    def _names(self) -> Dict[Any, str]:
        return {p: n for n, p in self.params.items()}

    def state_dict(self) -> Dict[str, Any]:
        name_of = self._names()
        out: Dict[str, Any] = {"state": {name_of[p]: _export_leaf(s) for p, s in self.state.items()}}
        if self.defaults[_SAVE_GROUPS]:
            out["param_groups"] = [
                {"params": sorted(name_of[p] for p in g["params"]), **copy.deepcopy(_GroupIndex.options(g))} for g in self.param_groups
            ]
        return out

    def post_load_state_dict(self) -> None:
        pass

    def _load_groups(self, saved_groups: List[Mapping[str, Any]]) -> None:
        if len(self.param_groups) != len(saved_groups):
            raise ValueError(f"Different param_groups count: {len(self.param_groups)} vs {len(saved_groups)}")
        name_of = self._names()
        mine = _GroupIndex(lambda g: sorted(name_of[p] for p in g["params"]), self.param_groups)
        theirs = _GroupIndex(lambda g: sorted(g["params"]), saved_groups)
        for key, group in mine.by_key.items():
            saved = theirs.by_key.get(key)
            if saved is None:
                raise ValueError(f"Group {key} not found")
            if len(group) != len(saved):
                raise ValueError(f"Different param_group size: {len(group)} vs {len(saved)}")
            missing = [k for k in group if k not in saved]
            if missing:
                raise ValueError(f"Group key {missing[0]} not found for group {key}")
            for option in _GroupIndex.options(group):
                group[option] = copy.deepcopy(saved[option])  # type: ignore[index]

    def load_state_dict(self, state_dict: Mapping[str, Any]) -> None:
        """Strict, in-place load: keys and shard layouts must match the current state."""
        incoming = state_dict["state"]
        if len(self.state) != len(incoming):
            raise ValueError(f"Different parameter count: {len(self.state)} vs {len(incoming)}")
        for name, param in self.params.items():
            if param not in self.state:
                continue
            slot = self.state[param]
            if name not in incoming:
                raise ValueError(f"Parameter {name} not found")
            if len(slot) != len(incoming[name]):
                raise ValueError(f"Different state size: {len(slot)} vs {len(incoming[name])}")
            self._update_param_state_dict_object(slot, incoming[name], [name])
        if self.defaults[_SAVE_GROUPS]:
            self._load_groups(state_dict["param_groups"])
        self.post_load_state_dict()

    def add_param_group(self, param_group: Any) -> None:
        raise NotImplementedError()

    def init_state(self, sparse_grad_parameter_names: Optional[Set[str]] = None) -> None:
        """Run one step on zero gradients so that all state exists (needed before loading a checkpoint)."""
        sparse = sparse_grad_parameter_names or set()
        for name, p in self.params.items():
            if not p.requires_grad:
                continue
            zero = torch.zeros_like(p)
            p.grad = zero.to_sparse() if name in sparse else zero
        self.step(closure=None)

    def save_param_groups(self, save: bool) -> None:
        self.defaults[_SAVE_GROUPS] = save

    def __getstate__(self) -> Dict[str, object]:
        return self.__dict__


class CombinedOptimizer(KeyedOptimizer):
    """Several keyed optimizers behind one interface; keys may be prefixed per optimizer."""

    def __init__(self, optims: List[Union[KeyedOptimizer, Tuple[str, KeyedOptimizer]]]) -> None:
        self._optims: List[Tuple[str, KeyedOptimizer]] = [o if isinstance(o, tuple) else ("", o) for o in optims]
        flag = self._optims[0][1].defaults[_SAVE_GROUPS] if self._optims else False
        self.defaults: Dict[str, Any] = {_SAVE_GROUPS: flag}
        seen: Set[str] = set()
        for prefix, opt in self._optims:
            assert opt.defaults[_SAVE_GROUPS] == flag
            for name in opt.params:
                full = self.prepend_opt_key(name, prefix)
                if full in seen:
                    raise ValueError(f"Duplicate param key {full}")
                seen.add(full)
        self._optimizer_step_pre_hooks: Dict[int, Callable] = {}
        self._optimizer_step_post_hooks: Dict[int, Callable] = {}
        self._patch_step_function()

    def _patch_step_function(self) -> None:
        pass

    def _each(self) -> Iterable[KeyedOptimizer]:
        return (opt for _, opt in self._optims)

    def __repr__(self) -> str:
        return "\n".join(f"{prefix}: {opt!r}" for prefix, opt in self._optims)

    def zero_grad(self, set_to_none: bool = False) -> None:
        for opt in self._each():
            opt.zero_grad(set_to_none=set_to_none)

    def step(self, closure: Any = None) -> None:
        for opt in self._each():
            opt.step(closure=closure)

    @property
    def optimizers(self) -> List[Tuple[str, KeyedOptimizer]]:
        return self._optims

    @staticmethod
    def prepend_opt_key(name: str, opt_key: str) -> str:
        return ".".join(part for part in (opt_key, name) if part)

    @property
    def param_groups(self) -> Collection[Mapping[str, Any]]:
        groups: List[Mapping[str, Any]] = []
        for opt in self._each():
            groups.extend(opt.param_groups)
        return groups

    @property
    def params(self) -> Mapping[str, Union[torch.Tensor, ShardedTensor]]:
        return {self.prepend_opt_key(name, prefix): p for prefix, opt in self._optims for name, p in opt.params.items()}

    @property
    def state(self) -> Mapping[torch.Tensor, Any]:
        merged: Dict[torch.Tensor, Any] = {}
        for opt in self._each():
            merged.update(opt.state)
        return merged

    def post_load_state_dict(self) -> None:
        for opt in self._each():
            opt.post_load_state_dict()

    def save_param_groups(self, save: bool) -> None:
        self.defaults[_SAVE_GROUPS] = save
        for opt in self._each():
            opt.save_param_groups(save)

    def _forward_optional(self, method: str, *args: Any) -> None:
        for opt in self._each():
            fn = getattr(opt, method, None)
            if fn is not None:
                fn(*args)

    def set_optimizer_step(self, step: int) -> None:
        self._forward_optional("set_optimizer_step", step)

    def update_hyper_parameters(self, params_dict: Dict[str, Any]) -> None:
        self._forward_optional("update_hyper_parameters", params_dict)


class KeyedOptimizerWrapper(KeyedOptimizer):
    """Build a torch optimizer from ``{name: param}`` with ``optim_factory`` and key its state by name."""

    def __init__(self, params: Mapping[str, Union[torch.Tensor, ShardedTensor]], optim_factory: OptimizerFactory) -> None:
        inner = optim_factory([p for p in params.values()])
        self._optimizer: optim.Optimizer = inner
        super().__init__(params, inner.state, inner.param_groups)

    def zero_grad(self, set_to_none: bool = False) -> None:
        self._optimizer.zero_grad(set_to_none=set_to_none)

    def step(self, closure: Any = None) -> None:
        self._optimizer.step(closure=closure)


class OptimizerWrapper(KeyedOptimizer):
    """Base for optimizers that decorate another keyed optimizer (clipping, warm-up, ...)."""

    def __init__(self, optimizer: KeyedOptimizer) -> None:
        self._optimizer = optimizer
        self._adopt()
        self.defaults: Dict[str, Any] = {_SAVE_GROUPS: False}

    def _adopt(self) -> None:
        inner = self._optimizer
        self.params: Mapping[str, Union[torch.Tensor, ShardedTensor]] = inner.params
        self.state: Mapping[Any, Any] = inner.state
        self.param_groups: Collection[Mapping[str, Any]] = inner.param_groups

    def __repr__(self) -> str:
        return repr(self._optimizer)

    def zero_grad(self, set_to_none: bool = False) -> None:
        self._optimizer.zero_grad(set_to_none=set_to_none)

    def step(self, closure: Any = None) -> None:
        self._optimizer.step(closure=closure)

    def add_param_group(self, param_group: Any) -> None:
        raise NotImplementedError()

    def state_dict(self) -> Dict[str, Any]:
        return self._optimizer.state_dict()

    def post_load_state_dict(self) -> None:
        self._optimizer.post_load_state_dict()

    def load_state_dict(self, state_dict: Mapping[str, Any]) -> None:
        self._optimizer.load_state_dict(state_dict)
        self._adopt()  # a wrapped optimizer may have rebuilt its containers while loading
        self.post_load_state_dict()

    def save_param_groups(self, save: bool) -> None:
        self._optimizer.save_param_groups(save)
