"""Batch container shared by datasets, models and pipelines (cf. ``torchrec/datasets/utils.py:28``)."""
from __future__ import annotations

from dataclasses import dataclass

import torch

from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor
from torchrec_b200.streamable import Pipelineable


@dataclass
class Batch(Pipelineable):
    dense_features: torch.Tensor
    sparse_features: KeyedJaggedTensor
    labels: torch.Tensor

    def to(self, device: torch.device, non_blocking: bool = False) -> "Batch":
        return Batch(
            dense_features=self.dense_features.to(device=device, non_blocking=non_blocking),
            sparse_features=self.sparse_features.to(device=device, non_blocking=non_blocking),
            labels=self.labels.to(device=device, non_blocking=non_blocking),
        )

    def record_stream(self, stream: torch.Stream) -> None:
        if self.dense_features.is_cuda:
            self.dense_features.record_stream(stream)
            self.labels.record_stream(stream)
        self.sparse_features.record_stream(stream)

    def pin_memory(self) -> "Batch":
        return Batch(
            dense_features=self.dense_features.pin_memory(),
            sparse_features=self.sparse_features.pin_memory(),
            labels=self.labels.pin_memory(),
        )


# ---- small stream stages for file-backed datasets (cf. ``torchrec/datasets/utils.py:58-340``) ------------------------------
# Every stage is an ``IterDataPipe``: re-iterable, composable, and aware of ``DataLoader`` workers where that matters.
import csv as _csv
import math as _math
import random as _random
from typing import Any, Callable, Iterable, Iterator, List, Sequence, Tuple, TypeVar

from torch.utils.data import IterDataPipe, get_worker_info

PATH_MANAGER_KEY = "torchrec_b200"
T = TypeVar("T")


def safe_cast(val: T, dest_type: Callable[[T], T], default: T) -> T:
    """``dest_type(val)``, or ``default`` when the value does not parse (empty fields of a TSV, say)."""
    try:
        return dest_type(val)
    except ValueError:
        return default


class _Keep(IterDataPipe):
    """Passes on the samples whose (index, sample) the predicate accepts."""

    def __init__(self, datapipe: Iterable, accept: Callable[[int], bool]) -> None:
        super().__init__()
        self.datapipe, self.accept = datapipe, accept

    def __iter__(self) -> Iterator[Any]:
        return (sample for i, sample in enumerate(self.datapipe) if self.accept(i))


def _default_key_fn(idx: int) -> int:
    return idx


def train_filter(key_fn: Callable[[int], int], train_perc: float, decimal_places: int, idx: int) -> bool:
    """Deterministic membership: the last ``decimal_places`` digits of the sample's key decide, so the split has the asked proportion."""
    scale = 10 ** decimal_places
    return key_fn(idx) % scale < round(train_perc * scale)


def val_filter(key_fn: Callable[[int], int], train_perc: float, decimal_places: int, idx: int) -> bool:
    return not train_filter(key_fn, train_perc, decimal_places, idx)


def idx_split_train_val(datapipe: Iterable, train_perc: float, decimal_places: int = 2,
                        key_fn: Callable[[int], int] = _default_key_fn) -> Tuple[IterDataPipe, IterDataPipe]:
    """Disjoint train / validation views of ``datapipe`` chosen by sample index (repeatable across epochs and processes)."""
    if not 0.0 < train_perc < 1.0:
        raise ValueError("train_perc must be in range (0.0, 1.0)")
    return (_Keep(datapipe, lambda i: train_filter(key_fn, train_perc, decimal_places, i)),
            _Keep(datapipe, lambda i: val_filter(key_fn, train_perc, decimal_places, i)))


class _RandomKeep(IterDataPipe):
    """Keeps a sample when the draw of a seeded generator falls on the wanted side of ``train_perc``; both views of a split replay the
    same draws, so they are disjoint and together complete."""

    def __init__(self, datapipe: Iterable, train_perc: float, seed: int, want_train: bool) -> None:
        super().__init__()
        self.datapipe, self.train_perc, self.seed, self.want_train = datapipe, train_perc, seed, want_train

    def __iter__(self) -> Iterator[Any]:
        draws = _random.Random(self.seed)
        for sample in self.datapipe:
            if (draws.random() < self.train_perc) == self.want_train:
                yield sample


def rand_split_train_val(datapipe: Iterable, train_perc: float, random_seed: int = 0) -> Tuple[IterDataPipe, IterDataPipe]:
    """Disjoint train / validation views by uniform sampling (the proportion is met in expectation)."""
    if not 0.0 < train_perc < 1.0:
        raise ValueError("train_perc must be in range (0.0, 1.0)")
    return _RandomKeep(datapipe, train_perc, random_seed, True), _RandomKeep(datapipe, train_perc, random_seed, False)


class Limit(IterDataPipe):
    """The first ``limit`` samples."""

    def __init__(self, datapipe: Iterable, limit: int) -> None:
        super().__init__()
        self.datapipe, self.limit = datapipe, limit

    def __iter__(self) -> Iterator[Any]:
        for i, sample in enumerate(self.datapipe):
            if i >= self.limit:
                return
            yield sample


class LoadFiles(IterDataPipe):
    """``(path, open file)`` for every path of ``datapipe``; the file is closed when the consumer asks for the next one."""

    def __init__(self, datapipe: Iterable[str], mode: str = "b", length: int = -1, path_manager_key: str = PATH_MANAGER_KEY, **open_kw: Any) -> None:
        super().__init__()
        if mode not in ("b", "t", "rb", "rt", "r"):
            raise ValueError(f"Invalid mode {mode}")
        self.datapipe, self.mode, self.length, self.open_kw = datapipe, ("r" + mode if "r" not in mode else mode), length, open_kw

    def __iter__(self) -> Iterator[Tuple[str, Any]]:
        for path in self.datapipe:
            with open(path, self.mode, **self.open_kw) as handle:
                yield path, handle

    def __len__(self) -> int:
        if self.length == -1:
            raise NotImplementedError
        return self.length


class ReadLinesFromCSV(IterDataPipe):
    """Rows of the ``(path, open text file)`` pairs of ``datapipe`` as lists of fields."""

    def __init__(self, datapipe: Iterable[Tuple[str, Any]], skip_first_line: bool = False, **csv_kw: Any) -> None:
        super().__init__()
        self.datapipe, self.skip_first_line, self.csv_kw = datapipe, skip_first_line, csv_kw

    def __iter__(self) -> Iterator[List[str]]:
        for _, handle in self.datapipe:
            rows = _csv.reader(handle, **self.csv_kw)
            if self.skip_first_line:
                next(rows, None)
            yield from rows


def _default_dp_selector(datapipes: Sequence[IterDataPipe]) -> Sequence[IterDataPipe]:
    """The slice of ``datapipes`` that this ``DataLoader`` worker reads: contiguous, sizes differing by at most one."""
    info = get_worker_info()
    if info is None:
        return datapipes
    if info.num_workers > len(datapipes):
        raise ValueError(f"Number of workers {info.num_workers} exceeds number of datapipes ({len(datapipes)})!")
    bounds = [0]
    for left in range(info.num_workers, 0, -1):
        bounds.append(bounds[-1] + _math.ceil((len(datapipes) - bounds[-1]) / left))
    return datapipes[bounds[info.id]: bounds[info.id + 1]]


class ParallelReadConcat(IterDataPipe):
    """Concatenation of several datapipes; under a ``DataLoader`` with workers each worker reads its own subset, so the files are read
    in parallel and every sample is produced once."""

    def __init__(self, *datapipes: IterDataPipe, dp_selector: Callable[[Sequence[IterDataPipe]], Sequence[IterDataPipe]] = _default_dp_selector) -> None:
        super().__init__()
        self.datapipes, self.dp_selector = datapipes, dp_selector

    def __iter__(self) -> Iterator[Any]:
        for dp in self.dp_selector(self.datapipes):
            yield from dp
