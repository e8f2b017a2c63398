"""Helpers of ``ebc_benchmarks.py``: a random KJT dataset over a table set and epoch timers for an embedding collection trained
with a separate optimizer or with the optimizer fused into the backward (``benchmarks/ebc_benchmarks_utils.py:22-125`` of the reference)."""
from __future__ import annotations

import time
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

from torchrec_b200.datasets.random import RandomRecDataset
from torchrec_b200.modules.embedding_configs import EmbeddingBagConfig


def get_random_dataset(batch_size: int, num_batches: int, num_dense_features: int, embedding_bag_configs: List[EmbeddingBagConfig],
                       pooling_factors: Optional[Dict[str, int]] = None) -> RandomRecDataset:
    """One feature per table feature name, 64 ids per bag unless ``pooling_factors`` says otherwise."""
    pooling_factors = pooling_factors or {}
    keys = [f for t in embedding_bag_configs for f in t.feature_names]
    return RandomRecDataset(keys=keys, batch_size=batch_size, hash_sizes=[t.num_embeddings for t in embedding_bag_configs for _ in t.feature_names],
                            ids_per_features=[pooling_factors.get(k, 64) for k in keys], num_dense=num_dense_features, num_batches=num_batches)


def _sync(device: torch.device) -> None:
    if device.type == "cuda":
        torch.cuda.synchronize(device)


def train_one_epoch(model: torch.nn.Module, optimizer: Optional[torch.optim.Optimizer], dataset, device: torch.device) -> float:
    """Seconds for one pass: forward, ``sum().backward()``, and ``optimizer.step()`` when an optimizer is given (a fused module updates
    inside its backward)."""
    _sync(device)
    t0 = time.perf_counter()
    for batch in dataset:
        pooled = model(batch.sparse_features.to(device))
        if optimizer is not None:
            optimizer.zero_grad()
        pooled.values().sum().backward()
        if optimizer is not None:
            optimizer.step()
    _sync(device)
    return time.perf_counter() - t0


def train(model: torch.nn.Module, optimizer: Optional[torch.optim.Optimizer], dataset, device: torch.device, epochs: int = 100) -> Tuple[float, float]:
    times = [train_one_epoch(model, optimizer, dataset, device) for _ in range(epochs)]
    return float(np.mean(times)), float(np.std(times))
