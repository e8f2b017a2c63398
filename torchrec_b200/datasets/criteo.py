"""Criteo click-logs readers: TSV rows (label, 13 integer features, 26 hashed categorical features) and the pre-processed
``.npy`` triplets (dense / sparse / labels) used for DLRM training (``torchrec/datasets/criteo.py:59-1014``).

The in-memory iterator yields ``Batch``es ready for ``DistributedModelParallel``: dense features are already
``log(x + 3)``-transformed by the pre-processing, sparse ids are taken modulo the table sizes, every feature has exactly
one id per sample (lengths are all 1), and every rank reads a disjoint contiguous slice of every file.
"""
from __future__ import annotations

import os
from typing import Any, Callable, Dict, Iterable, Iterator, List, Optional, Tuple, Union

import numpy as np
import torch
from torch.utils.data import IterableDataset

from torchrec_b200.datasets.utils import Batch
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor

FREQUENCY_THRESHOLD = 3
INT_FEATURE_COUNT = 13
CAT_FEATURE_COUNT = 26
DAYS = 24
DEFAULT_LABEL_NAME = "label"
DEFAULT_INT_NAMES: List[str] = [f"int_{idx}" for idx in range(INT_FEATURE_COUNT)]
DEFAULT_CAT_NAMES: List[str] = [f"cat_{idx}" for idx in range(CAT_FEATURE_COUNT)]
DEFAULT_COLUMN_NAMES: List[str] = [DEFAULT_LABEL_NAME, *DEFAULT_INT_NAMES, *DEFAULT_CAT_NAMES]
TOTAL_TRAINING_SAMPLES = 4195197692  # days 0-22 of the 1 TB dataset
COLUMN_TYPE_CASTERS: List[Callable[[Union[int, str]], Union[int, str]]] = [
    lambda val: int(val) if val else 0, *(lambda val: int(val) if val else 0 for _ in range(INT_FEATURE_COUNT)),
    *(lambda val: val if val else "" for _ in range(CAT_FEATURE_COUNT)),
]


def _default_row_mapper(example: List[str]) -> Dict[str, Union[int, str]]:
    return {DEFAULT_COLUMN_NAMES[idx]: COLUMN_TYPE_CASTERS[idx](val) for idx, val in enumerate(example)}


class CriteoIterDataPipe(IterableDataset):
    """Rows of the raw TSV files as dicts ``{column: value}`` (categoricals stay hex strings)."""

    def __init__(self, paths: Iterable[str], *, row_mapper: Optional[Callable[[List[str]], Any]] = _default_row_mapper, **open_kw: Any) -> None:
        self.paths = list(paths)
        self.row_mapper = row_mapper
        self.open_kw = open_kw

    def __iter__(self) -> Iterator[Any]:
        worker = torch.utils.data.get_worker_info()
        paths = self.paths if worker is None else self.paths[worker.id:: worker.num_workers]
        for path in paths:
            with open(path, "r", **self.open_kw) as f:
                for line in f:
                    row = line.rstrip("\n").split("\t")
                    yield self.row_mapper(row) if self.row_mapper else row


def criteo_terabyte(paths: Iterable[str], *, row_mapper=_default_row_mapper, **open_kw: Any) -> IterableDataset:
    return CriteoIterDataPipe(paths, row_mapper=row_mapper, **open_kw)


def criteo_kaggle(path: str, *, row_mapper=_default_row_mapper, **open_kw: Any) -> IterableDataset:
    return CriteoIterDataPipe((path,), row_mapper=row_mapper, **open_kw)


class BinaryCriteoUtils:
    """TSV -> ``.npy`` conversion and slicing helpers for the pre-processed dataset."""

    @staticmethod
    def tsv_to_npys(in_file: str, out_dense_file: str, out_sparse_file: str, out_labels_file: str, dataset_name: str = "criteo_1tb") -> None:
        dense, sparse, labels = [], [], []
        with open(in_file, "r") as f:
            for line in f:
                row = line.rstrip("\n").split("\t")
                labels.append(int(row[0]) if row[0] else 0)
                dense.append([int(v) if v else 0 for v in row[1: 1 + INT_FEATURE_COUNT]])
                sparse.append([int(v, 16) if v else 0 for v in row[1 + INT_FEATURE_COUNT: 1 + INT_FEATURE_COUNT + CAT_FEATURE_COUNT]])
        np.save(out_dense_file, np.array(dense, dtype=np.float32))
        np.save(out_sparse_file, np.array(sparse, dtype=np.int32))
        np.save(out_labels_file, np.array(labels, dtype=np.int32).reshape(-1, 1))

    @staticmethod
    def get_shape_from_npy(path: str) -> Tuple[int, ...]:
        return tuple(np.load(path, mmap_mode="r").shape)

    @staticmethod
    def get_file_row_ranges_and_remainder(lengths: List[int], rank: int, world_size: int, start_row: int = 0, last_row: Optional[int] = None
                                          ) -> Tuple[Dict[int, Tuple[int, int]], int]:
        """Rows ``[start, end]`` (inclusive) of every file that belong to ``rank`` when the concatenation of all files is cut
        into ``world_size`` contiguous parts; the remainder is spread one row each over the first ranks."""
        total = sum(lengths) if last_row is None else last_row - start_row + 1
        per, rem = divmod(total, world_size)
        lo = start_row + rank * per + min(rank, rem)
        hi = lo + per + (1 if rank < rem else 0) - 1
        out: Dict[int, Tuple[int, int]] = {}
        base = 0
        for i, n in enumerate(lengths):
            a, b = max(lo, base), min(hi, base + n - 1)
            if a <= b:
                out[i] = (a - base, b - base)
            base += n
        return out, rem

    @staticmethod
    def load_npy_range(fname: str, start_row: int, num_rows: int, path_manager_key: str = "", mmap_mode: bool = False) -> np.ndarray:
        data = np.load(fname, mmap_mode="r")
        if start_row + num_rows > data.shape[0]:
            raise ValueError(f"cannot read rows {start_row}..{start_row + num_rows} of {fname} with {data.shape[0]} rows")
        part = data[start_row: start_row + num_rows]
        return part if mmap_mode else np.array(part)

    @staticmethod
    def sparse_to_contiguous(in_files: List[str], output_dir: str, frequency_threshold: int = FREQUENCY_THRESHOLD, columns: int = CAT_FEATURE_COUNT) -> None:
        """Map raw categorical ids to contiguous ids per column; ids rarer than the threshold share id 1."""
        counts: List[Dict[int, int]] = [dict() for _ in range(columns)]
        for f in in_files:
            arr = np.load(f)
            for c in range(columns):
                vals, cnt = np.unique(arr[:, c], return_counts=True)
                for v, n in zip(vals.tolist(), cnt.tolist()):
                    counts[c][v] = counts[c].get(v, 0) + n
        maps = []
        for c in range(columns):
            m = {}
            nxt = 2
            for v, n in sorted(counts[c].items()):
                if n >= frequency_threshold:
                    m[v] = nxt
                    nxt += 1
            maps.append(m)
        os.makedirs(output_dir, exist_ok=True)
        for f in in_files:
            arr = np.load(f)
            out = np.ones_like(arr)
            for c in range(columns):
                out[:, c] = np.array([maps[c].get(v, 1) for v in arr[:, c].tolist()], dtype=arr.dtype)
            np.save(os.path.join(output_dir, os.path.basename(f).replace(".npy", "_contig_freq.npy")), out)

    @staticmethod
    def shuffle(input_dir_labels_and_dense: str, input_dir_sparse: str, output_dir_shuffled: str, rows_per_day: Dict[int, int], seed: int = 0, days: int = 1) -> None:
        rng = np.random.default_rng(seed)
        os.makedirs(output_dir_shuffled, exist_ok=True)
        for d in range(days):
            perm = None
            for kind, src in (("dense", input_dir_labels_and_dense), ("labels", input_dir_labels_and_dense), ("sparse", input_dir_sparse)):
                arr = np.load(os.path.join(src, f"day_{d}_{kind}.npy"))
                if perm is None:
                    perm = rng.permutation(arr.shape[0])
                np.save(os.path.join(output_dir_shuffled, f"day_{d}_{kind}.npy"), arr[perm])


class InMemoryBinaryCriteoIterDataPipe(IterableDataset):
    """Batches from the pre-processed ``.npy`` files, all of this rank's rows held in (optionally memory-mapped) host memory."""

    def __init__(self, stage: str, dense_paths: List[str], sparse_paths: List[str], labels_paths: List[str], batch_size: int, rank: int, world_size: int,
                 drop_last: Optional[bool] = False, shuffle_batches: bool = False, shuffle_training_set: bool = False, shuffle_training_set_random_seed: int = 0,
                 mmap_mode: bool = False, hashes: Optional[List[int]] = None, path_manager_key: str = "") -> None:
        self.stage = stage
        self.batch_size = batch_size
        self.rank, self.world_size = rank, world_size
        self.drop_last = drop_last
        self.shuffle_batches = shuffle_batches
        self.hashes = np.array(hashes).reshape(1, -1) if hashes is not None else None
        self.keys = DEFAULT_CAT_NAMES
        lengths = [BinaryCriteoUtils.get_shape_from_npy(p)[0] for p in dense_paths]
        ranges, _ = BinaryCriteoUtils.get_file_row_ranges_and_remainder(lengths, rank, world_size)
        dense, sparse, labels = [], [], []
        for idx, (lo, hi) in sorted(ranges.items()):
            n = hi - lo + 1
            dense.append(BinaryCriteoUtils.load_npy_range(dense_paths[idx], lo, n, mmap_mode=mmap_mode))
            sparse.append(BinaryCriteoUtils.load_npy_range(sparse_paths[idx], lo, n, mmap_mode=mmap_mode))
            labels.append(BinaryCriteoUtils.load_npy_range(labels_paths[idx], lo, n, mmap_mode=mmap_mode))
        self.dense = np.concatenate(dense) if dense else np.zeros((0, INT_FEATURE_COUNT), np.float32)
        self.sparse = np.concatenate(sparse) if sparse else np.zeros((0, CAT_FEATURE_COUNT), np.int32)
        self.labels = np.concatenate(labels) if labels else np.zeros((0, 1), np.int32)
        if shuffle_training_set and stage == "train":
            perm = np.random.default_rng(shuffle_training_set_random_seed).permutation(self.dense.shape[0])
            self.dense, self.sparse, self.labels = self.dense[perm], self.sparse[perm], self.labels[perm]
        if self.hashes is not None:
            self.sparse = self.sparse % self.hashes
        self.num_rows = self.dense.shape[0]
        self.num_full_batches = self.num_rows // batch_size
        self.last_batch_size = self.num_rows - self.num_full_batches * batch_size
        self._lengths = torch.ones(batch_size * CAT_FEATURE_COUNT, dtype=torch.int32)

    def _np_arrays_to_batch(self, dense: np.ndarray, sparse: np.ndarray, labels: np.ndarray) -> Batch:
        b = dense.shape[0]
        lengths = self._lengths if b == self.batch_size else torch.ones(b * CAT_FEATURE_COUNT, dtype=torch.int32)
        return Batch(
            dense_features=torch.from_numpy(np.ascontiguousarray(dense)),
            sparse_features=KeyedJaggedTensor(keys=self.keys, values=torch.from_numpy(np.ascontiguousarray(sparse.T).reshape(-1)), lengths=lengths, stride=b),
            labels=torch.from_numpy(np.ascontiguousarray(labels).reshape(-1)),
        )

    def __iter__(self) -> Iterator[Batch]:
        n = self.num_full_batches + (1 if self.last_batch_size and not self.drop_last else 0)
        order = np.random.permutation(n) if self.shuffle_batches else np.arange(n)
        for i in order:
            lo = int(i) * self.batch_size
            hi = min(lo + self.batch_size, self.num_rows)
            yield self._np_arrays_to_batch(self.dense[lo:hi], self.sparse[lo:hi], self.labels[lo:hi])

    def __len__(self) -> int:
        return self.num_full_batches + (1 if self.last_batch_size and not self.drop_last else 0)
