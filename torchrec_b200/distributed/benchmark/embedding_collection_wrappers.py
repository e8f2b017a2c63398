"""Wrappers and drivers for module-level embedding benchmarks: ``EBCWrapper`` / ``ECWrapper`` turn a collection's structured output
into plain tensors (so a benchmark can reduce it and call backward), ``get_tables`` makes configs from ``(rows, dim)`` pairs, and
``benchmark_ebc_module`` times one module in a chosen form: as is, quantized, or quantized and placed over the local devices.
Counterpart of ``torchrec/distributed/benchmark/embedding_collection_wrappers.py:72-647``."""
from __future__ import annotations

import dataclasses
import enum
from typing import Dict, List, Optional, Tuple, Union

import torch
from torch import nn

from torchrec_b200.distributed.benchmark.benchmark_base import BenchmarkResult, benchmark_func
from torchrec_b200.modules.embedding_configs import DataType, EmbeddingBagConfig, EmbeddingConfig
from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection, EmbeddingCollection
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


class ModuleForm(enum.Enum):
    FLOAT = "float"  # the module as constructed (training-capable)
    QUANT = "quant"  # row-wise quantized, one device
    QUANT_SHARDED = "quant_sharded"  # quantized and placed table-wise over the local devices


class EBCWrapper(nn.Module):
    """``KJT -> [B, sum(D)]``."""

    def __init__(self, module: nn.Module) -> None:
        super().__init__()
        self._module = module

    def forward(self, input: KeyedJaggedTensor) -> torch.Tensor:
        return self._module(input).values()


class ECWrapper(nn.Module):
    """``KJT -> [values of every feature]`` (one ``[n_f, D]`` tensor per feature)."""

    def __init__(self, module: nn.Module) -> None:
        super().__init__()
        self._module = module

    def forward(self, input: KeyedJaggedTensor) -> List[torch.Tensor]:
        return [jt.values() for jt in self._module(input).values()]


def get_tables(table_sizes: List[Tuple[int, int]], is_pooled: bool = True, data_type: DataType = DataType.INT8) -> Union[List[EmbeddingBagConfig], List[EmbeddingConfig]]:
    cls = EmbeddingBagConfig if is_pooled else EmbeddingConfig
    return [cls(num_embeddings=rows, embedding_dim=dim, name=f"table_{i}", feature_names=[f"feature_{i}"], data_type=data_type) for i, (rows, dim) in enumerate(table_sizes)]


def make_inputs(tables, batch_size: int, pooling: int, num_inputs: int, device: torch.device, seed: int = 0) -> List[KeyedJaggedTensor]:
    gen = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(num_inputs):
        lengths = torch.randint(0, 2 * pooling + 1, (len(tables) * batch_size,), generator=gen)
        per_table = lengths.view(len(tables), batch_size).sum(1).tolist()
        values = torch.cat([torch.randint(0, t.num_embeddings, (n,), generator=gen) for t, n in zip(tables, per_table)])
        out.append(KeyedJaggedTensor(keys=[f for t in tables for f in t.feature_names], values=values, lengths=lengths).to(device))
    return out


def transform_module(module: nn.Module, form: ModuleForm, device: torch.device, world_size: int = 1) -> nn.Module:
    if form == ModuleForm.FLOAT:
        return module.to(device)
    from torchrec_b200.inference.modules import quantize_embeddings, shard_quant_model

    holder = nn.Sequential(module)
    quantize_embeddings(holder, dtype=torch.qint8, inplace=True)
    if form == ModuleForm.QUANT_SHARDED:
        holder, _ = shard_quant_model(holder, world_size=world_size, compute_device=device.type)
        return holder[0]
    return holder[0].to(device)


def benchmark_ebc_module(tables, form: ModuleForm = ModuleForm.FLOAT, batch_size: int = 2048, pooling: int = 10, num_iters: int = 10, warmup_iters: int = 3,
                         device: Optional[torch.device] = None, world_size: int = 1, train: bool = False, profile_dir: str = "") -> BenchmarkResult:
    """Time the forward (and backward + plain SGD step when ``train``) of a collection built from ``tables`` in the given form."""
    device = device if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")
    pooled = isinstance(tables[0], EmbeddingBagConfig)
    # the collection is always built in fp32; quantized forms are derived from it
    float_tables = [dataclasses.replace(t, data_type=DataType.FP32) for t in tables]
    base = EmbeddingBagCollection(tables=float_tables) if pooled else EmbeddingCollection(tables=float_tables)
    module = transform_module(base, form, device, world_size)
    wrapped = EBCWrapper(module) if pooled else ECWrapper(module)
    inputs = make_inputs(tables, batch_size, pooling, 4, device)
    state = {"i": 0}
    params = [p for p in wrapped.parameters() if p.requires_grad] if train else []

    def step() -> None:
        kjt = inputs[state["i"] % len(inputs)]
        state["i"] += 1
        if not train:
            with torch.no_grad():
                wrapped(kjt)
            return
        out = wrapped(kjt)
        (out.sum() if isinstance(out, torch.Tensor) else sum(o.sum() for o in out)).backward()
        with torch.no_grad():
            for p in params:
                if p.grad is not None:
                    p.add_(p.grad, alpha=-0.01)
                    p.grad = None

    return benchmark_func(f"{'ebc' if pooled else 'ec'}-{form.value}{'-train' if train else ''}", step, num_iters=num_iters, warmup_iters=warmup_iters,
                          device=device, rank=0, profile_dir=profile_dir)
