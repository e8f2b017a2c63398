"""Data loader that rewrites global ids into cache rows ahead of the training step.

``wrap(url, dataloader, module, configs_dict)`` builds the id-transformer group of ``module`` and returns a loader whose background
thread pulls batches, transforms the KJTs that feed dynamic embedding modules (global id -> row of the HBM-resident table, fetching
rows from the parameter store on a miss) and queues the result; ``__next__`` waits for the fetches of that batch before handing it
out.  ``save(module)`` writes every cached row back to the store.
Counterpart of ``contrib/dynamic_embedding/src/torchrec_dynamic_embedding/dataloader.py:25-240``."""
from __future__ import annotations

import queue
import threading
from typing import Any, Dict, Iterable, List, Optional, Tuple

import torch
from torch import nn

from torchrec_b200.contrib.dynamic_embedding.id_transformer_group import IDTransformerGroup
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor

_POLL_S = 0.5
_END = object()


def _transform_loop(dataloader: Iterable, transform_fn, out_queue: "queue.Queue", done: threading.Event) -> None:
    torch.set_num_threads(1)  # thread-local: keep pinned-memory copies from taking every core
    try:
        for data in dataloader:
            if done.is_set():
                return
            item = transform_fn(data)
            while not done.is_set():
                try:
                    out_queue.put(item, timeout=_POLL_S)
                    break
                except queue.Full:
                    continue
    except BaseException as e:  # surfaced by the consumer
        item = e
        while not done.is_set():
            try:
                out_queue.put(item, timeout=_POLL_S)
                break
            except queue.Full:
                continue
        return
    while not done.is_set():
        try:
            out_queue.put(_END, timeout=_POLL_S)
            return
        except queue.Full:
            continue


class DataLoaderIter:
    def __init__(self, dataloader: Iterable, transform_fn, num_prefetch: int = 0) -> None:
        self._queue: "queue.Queue" = queue.Queue(maxsize=max(num_prefetch, 1))
        self._done = threading.Event()
        self._thread = threading.Thread(target=_transform_loop, args=(dataloader, transform_fn, self._queue, self._done), daemon=True)
        self._thread.start()

    def __iter__(self) -> "DataLoaderIter":
        return self

    def __next__(self) -> Any:
        if self._done.is_set():
            raise StopIteration
        item = self._queue.get()
        if item is _END:
            self._done.set()
            raise StopIteration
        if isinstance(item, BaseException):
            self._done.set()
            raise RuntimeError("id transform thread failed") from item
        data, handles = item
        for h in handles:
            h.wait()
        return data

    def close(self) -> None:
        self._done.set()

    def __del__(self) -> None:
        self._done.set()


class DataLoader:
    """Iterating yields the wrapped loader's batches with the KJTs at ``data_info`` positions rewritten.  A batch may be a single KJT
    (``data_info`` omitted, one path), or a tuple / list indexed by ``data_info``'s keys."""

    def __init__(self, id_transformer_group: IDTransformerGroup, dataloader: Iterable, *, data_info: Optional[Dict[int, str]] = None,
                 paths: Optional[List[str]] = None, num_prefetch: int = 0) -> None:
        self._group = id_transformer_group
        self._dataloader = dataloader
        self._num_prefetch = num_prefetch
        if data_info is not None:
            self._data_info = dict(data_info)
        else:
            assert paths is not None and len(paths) == 1, "data_info is required when more than one module is wrapped"
            self._data_info = {None: paths[0]}  # type: ignore[dict-item]

    def _transform(self, data: Any) -> Tuple[Any, List]:
        if None in self._data_info:  # the batch is the KJT itself
            out, handles = self._group.transform({self._data_info[None]: data})  # type: ignore[index]
            return out[self._data_info[None]], handles  # type: ignore[index]
        picked = {path: data[i] for i, path in self._data_info.items()}
        out, handles = self._group.transform(picked)
        data = list(data)
        for i, path in self._data_info.items():
            data[i] = out[path]
        return tuple(data), handles

    def __iter__(self) -> DataLoaderIter:
        return DataLoaderIter(self._dataloader, self._transform, self._num_prefetch)

    def __len__(self) -> int:
        return len(self._dataloader)  # type: ignore[arg-type]


def wrap(url: str, dataloader: Iterable, module: nn.Module, configs_dict: Dict[str, list], *, data_info: Optional[Dict[int, str]] = None,
         eviction_config: Optional[dict] = None, transform_config: Optional[dict] = None, ps_config: Optional[dict] = None, parallel: bool = True,
         num_prefetch: int = 0) -> Tuple[DataLoader, nn.Module]:
    """``url`` names the parameter store (``memory://...``, ``redis://host:port/?prefix=...``); ``configs_dict`` maps the path of each
    dynamic embedding module inside ``module`` to its table configs; ``data_info`` maps positions in a batch to those paths."""
    group = IDTransformerGroup(url, module, configs_dict, eviction_config=eviction_config, transform_config=transform_config, ps_config=ps_config)
    module._id_transformer_group = group  # type: ignore[assignment]
    return DataLoader(group, dataloader, data_info=data_info, paths=list(configs_dict.keys()), num_prefetch=num_prefetch), module


def save(module: nn.Module) -> None:
    """Write the dynamic-embedding rows cached in ``module`` back to the parameter store."""
    group = getattr(module, "_id_transformer_group", None)
    if not isinstance(group, IDTransformerGroup):
        raise ValueError("module has no id-transformer group: was it returned by wrap()?")
    group.save()
