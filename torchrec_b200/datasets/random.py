"""Synthetic recommendation data (cf. ``torchrec/datasets/random.py:78-221``).

``RandomRecDataset`` yields ``Batch(dense_features, sparse_features: KJT, labels)`` forever (or for
``num_batches``).  Ids are uniform by default; ``zipf_s`` draws them from a bounded Zipf law whose ranks
are spread over the table by a multiplicative hash, so that hot ids do not cluster in one row block.
"""
from __future__ import annotations

import math
from typing import Iterator, List, Optional, Sequence, Union

import torch
from torch.utils.data.dataset import IterableDataset

from torchrec_b200.datasets.utils import Batch
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


def zipf_ids(n: int, rows: int, s: float, generator: Optional[torch.Generator] = None, device: Optional[torch.device] = None,
             scramble: bool = True, dtype: torch.dtype = torch.int64) -> torch.Tensor:
    """``n`` ids in ``[0, rows)`` with ``P(rank k) ~ k^-s`` (inverse-CDF of the continuous power law, floored).

    With ``scramble`` rank ``k`` maps to id ``(k * A) % rows`` for an ``A`` coprime to ``rows``: a bijection, so
    the frequency profile is unchanged but popular ids are spread over the whole table.
    """
    if rows <= 1:
        return torch.zeros(n, dtype=dtype, device=device)
    u = torch.rand(n, generator=generator, device=device, dtype=torch.float64)
    if abs(s - 1.0) < 1e-9:
        ranks = torch.exp(u * math.log(rows + 1.0))
    else:
        a = 1.0 - s
        ranks = ((float(rows + 1) ** a - 1.0) * u + 1.0) ** (1.0 / a)
    ids = (ranks.floor().to(torch.int64) - 1).clamp_(0, rows - 1)
    if scramble:
        A = _coprime_multiplier(rows)
        ids = (ids * A) % rows
    return ids.to(dtype)


def _coprime_multiplier(rows: int) -> int:
    a = int(rows * 0.6180339887) | 1
    while math.gcd(a, rows) != 1:
        a += 2
    return a


class _RandomRecBatch:
    def __init__(self, keys: List[str], batch_size: int, hash_sizes: List[int], ids_per_features: List[int], num_dense: int,
                 manual_seed: Optional[int] = None, num_generated_batches: int = 10, num_batches: Optional[int] = None,
                 min_ids_per_features: Optional[List[int]] = None, zipf_s: Optional[float] = None, idx_dtype: torch.dtype = torch.int64,
                 label_positive_rate: float = 0.5, dense_log_transform: bool = False) -> None:
        self.keys = keys
        self.keys_length = len(keys)
        self.batch_size = batch_size
        self.hash_sizes = hash_sizes
        self.ids_per_features = ids_per_features
        self.min_ids_per_features = min_ids_per_features if min_ids_per_features else [0] * len(keys)
        self.num_dense = num_dense
        self.num_batches = num_batches
        self.num_generated_batches = num_generated_batches
        self.zipf_s = zipf_s
        self.idx_dtype = idx_dtype
        self.label_positive_rate = label_positive_rate
        self.dense_log_transform = dense_log_transform
        self.batch_index = 0
        self.generator: Optional[torch.Generator] = None
        if manual_seed is not None:
            self.generator = torch.Generator()
            self.generator.manual_seed(manual_seed)
        self._generated_batches: List[Batch] = [self._generate_batch() for _ in range(num_generated_batches)]
        self._batches_idx = 0

    def __iter__(self) -> "_RandomRecBatch":
        self.batch_index = 0
        return self

    def __next__(self) -> Batch:
        if self.batch_index == self.num_batches:
            raise StopIteration
        if self.num_generated_batches >= 0:
            batch = self._generated_batches[self._batches_idx % len(self._generated_batches)]
            self._batches_idx += 1
        else:
            batch = self._generate_batch()
        self.batch_index += 1
        return batch

    def _generate_batch(self) -> Batch:
        values, lengths = [], []
        for key_idx, _ in enumerate(self.keys):
            hash_size = self.hash_sizes[key_idx]
            min_num_ids = self.min_ids_per_features[key_idx]
            max_num_ids = self.ids_per_features[key_idx]
            if min_num_ids == max_num_ids:
                length = torch.full((self.batch_size,), min_num_ids, dtype=torch.int32)
            else:
                length = torch.randint(min_num_ids, max_num_ids + 1, (self.batch_size,), dtype=torch.int32, generator=self.generator)
            n = int(length.sum())
            if self.zipf_s is not None:
                value = zipf_ids(n, hash_size, self.zipf_s, generator=self.generator, dtype=self.idx_dtype)
            else:
                value = torch.randint(0, hash_size, (n,), generator=self.generator).to(self.idx_dtype)
            lengths.append(length)
            values.append(value)
        sparse_features = KeyedJaggedTensor.from_lengths_sync(keys=self.keys, values=torch.cat(values), lengths=torch.cat(lengths))
        dense_features = torch.randn(self.batch_size, self.num_dense, generator=self.generator)
        if self.dense_log_transform:
            dense_features = torch.log1p(100.0 * dense_features.abs())
        labels = (torch.rand(self.batch_size, generator=self.generator) < self.label_positive_rate).float()
        return Batch(dense_features=dense_features, sparse_features=sparse_features, labels=labels)


class RandomRecDataset(IterableDataset[Batch]):
    """Random dataset of ``Batch`` objects.

    Args:
        keys: feature names.  batch_size: samples per batch.
        hash_size / hash_sizes: id range of all / each feature.
        ids_per_feature / ids_per_features: max ids per sample; ``min_ids_per_feature(s)``: min (default 0).
        num_dense: number of dense features.  manual_seed: seed.  num_batches: length (None = endless).
        num_generated_batches: size of the pre-generated pool that is cycled (-1 = always generate).
        zipf_s: draw ids from a Zipf law with this exponent instead of uniformly.
    """

    def __init__(self, keys: List[str], batch_size: int, hash_size: Optional[int] = None, hash_sizes: Optional[List[int]] = None,
                 ids_per_feature: Optional[int] = None, ids_per_features: Optional[List[int]] = None, num_dense: int = 50,
                 manual_seed: Optional[int] = None, num_batches: Optional[int] = None, num_generated_batches: int = 10,
                 min_ids_per_feature: Optional[int] = None, min_ids_per_features: Optional[List[int]] = None,
                 zipf_s: Optional[float] = None, idx_dtype: torch.dtype = torch.int64, label_positive_rate: float = 0.5,
                 dense_log_transform: bool = False) -> None:
        super().__init__()
        if hash_sizes is None:
            hash_sizes = [hash_size if hash_size else 100] * len(keys)
        assert hash_sizes is not None and len(hash_sizes) == len(keys), "length of hash_sizes must be equal to the number of keys"
        if ids_per_features is None:
            ids_per_features = [ids_per_feature if ids_per_feature is not None else 2] * len(keys)
        assert len(ids_per_features) == len(keys), "length of ids_per_features must be equal to the number of keys"
        if min_ids_per_features is None:
            if min_ids_per_feature is None and ids_per_feature is None and ids_per_features is not None:
                min_ids_per_feature = 0
            min_ids_per_features = [min_ids_per_feature if min_ids_per_feature is not None else 0] * len(keys)
        self.batch_generator = _RandomRecBatch(
            keys=keys, batch_size=batch_size, hash_sizes=hash_sizes, ids_per_features=ids_per_features, num_dense=num_dense,
            manual_seed=manual_seed, num_batches=num_batches, num_generated_batches=num_generated_batches,
            min_ids_per_features=min_ids_per_features, zipf_s=zipf_s, idx_dtype=idx_dtype, label_positive_rate=label_positive_rate,
            dense_log_transform=dense_log_transform,
        )
        self.num_batches = num_batches

    def __iter__(self) -> Iterator[Batch]:
        return iter(self.batch_generator)

    def __len__(self) -> int:
        assert self.num_batches is not None
        return self.num_batches
