"""Lookups of one rank: the TBE groups of a sharding, fed from one KJT.

``GroupedPooledEmbeddingsLookup`` (pooled, output ``[B, sum(D)]``) and ``GroupedEmbeddingsLookup``
(unpooled, output ``[sum(L), D]``) split the incoming KJT by TBE group, run each group's kernel and
concatenate.  Counterpart of ``torchrec/distributed/embedding_lookup.py:178-711``.
"""
from __future__ import annotations

from typing import Any, Dict, Iterator, List, Optional, Tuple, Union

import torch
import torch.distributed as dist
from torch import nn
from torch.autograd.function import FunctionCtx
from torch.nn.parallel import DistributedDataParallel

from torchrec_b200.distributed.batched_embedding_kernel import (
    BaseEmbedding,
    BatchedDenseEmbedding,
    BatchedDenseEmbeddingBag,
    BatchedFusedEmbedding,
    BatchedFusedEmbeddingBag,
)
from torchrec_b200.distributed.embedding_types import (
    BaseEmbeddingLookup,
    BaseGroupedFeatureProcessor,
    EmbeddingComputeKernel,
    GroupedEmbeddingConfig,
)
from torchrec_b200.distributed.types import ShardedTensor, ShardingType
from torchrec_b200.optim.fused import FusedOptimizerModule
from torchrec_b200.optim.keyed import CombinedOptimizer, KeyedOptimizer
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


def _copy_checkpoint_entry(dst: Any, src: Any) -> None:
    """One state-dict entry into the live table memory; sharded entries are matched shard by shard on (offsets, sizes)."""
    if isinstance(dst, ShardedTensor):
        assert isinstance(src, ShardedTensor), "a sharded table loads from a sharded checkpoint entry"
        ours, theirs = dst.local_shards(), src.local_shards()
        assert len(ours) == len(theirs), f"{len(theirs)} checkpoint shards for {len(ours)} local shards"
        for mine, other in zip(ours, theirs):
            assert (mine.metadata.shard_offsets, mine.metadata.shard_sizes) == (other.metadata.shard_offsets, other.metadata.shard_sizes)
            mine.tensor.detach().copy_(other.tensor)
        return
    if isinstance(src, ShardedTensor):
        src = src.local_shards()[0].tensor
    assert isinstance(src, torch.Tensor) and isinstance(dst, torch.Tensor)
    dst.detach().copy_(src)


def _load_state_dict(emb_modules: "nn.ModuleList", state_dict: Dict[str, Any]) -> Tuple[List[str], List[str]]:
    """Copy checkpoint shards into the local table views.  Returns (keys the kernels hold that the checkpoint lacks, keys
    of the checkpoint that no kernel holds)."""
    missing: List[str] = []
    leftover = dict.fromkeys(state_dict.keys())
    for kernel in emb_modules:
        for key, live in kernel.state_dict().items():
            if key not in state_dict:
                missing.append(key)
                continue
            _copy_checkpoint_entry(live, state_dict[key])
            leftover.pop(key, None)
    return missing, list(leftover)


_FUSED_KERNELS = (EmbeddingComputeKernel.FUSED, EmbeddingComputeKernel.FUSED_UVM, EmbeddingComputeKernel.FUSED_UVM_CACHING)


def _kernel_class(compute_kernel: EmbeddingComputeKernel, dense_cls: type, fused_cls: type) -> type:
    """The UVM kinds run as HBM-resident fused kernels: 180 GB per GPU holds what the reference spills to host memory."""
    if compute_kernel == EmbeddingComputeKernel.DENSE:
        return dense_cls
    if compute_kernel in _FUSED_KERNELS:
        if compute_kernel != EmbeddingComputeKernel.FUSED:
            _warn_once(f"compute kernel {compute_kernel.value}: no host-memory tier is built; the table stays resident in HBM "
                       "(plan memory accordingly: the planner's UVM storage figures do not apply)")
        return fused_cls
    raise ValueError(f"Compute kernel not supported {compute_kernel}")


_warned: set = set()


def _warn_once(message: str) -> None:
    if message not in _warned:
        _warned.add(message)
        import warnings

        warnings.warn(message, stacklevel=3)


class CommOpGradientScaling(torch.autograd.Function):
    """Identity in forward, scales the gradient in backward (weighted features with gradient division)."""

    @staticmethod
    def forward(ctx: FunctionCtx, input_tensor: torch.Tensor, scale_gradient_factor: int) -> torch.Tensor:
        ctx.scale_gradient_factor = scale_gradient_factor
        return input_tensor

    @staticmethod
    def backward(ctx: FunctionCtx, grad_output: torch.Tensor):
        grad_output.mul_(ctx.scale_gradient_factor)
        return grad_output, None


def fx_wrap_tensor_view2d(x: torch.Tensor, dim0: int, dim1: int) -> torch.Tensor:
    return x.view(dim0, dim1)


def dummy_tensor(sparse_features: KeyedJaggedTensor, dtype: torch.dtype) -> torch.Tensor:
    """What a pooled lookup without tables returns: ``[batch, 0]``."""
    return torch.empty([0], dtype=dtype, device=sparse_features.device()).view(sparse_features.stride(), 0)


def embeddings_cat_empty_rank_handle(embeddings: List[torch.Tensor], dummy_embs_tensor: torch.Tensor, dim: int = 0) -> torch.Tensor:
    """Concatenate the outputs of a rank's kernel groups; a rank without tables returns ``dummy_embs_tensor`` (which keeps autograd and
    the output exchange uniform across ranks), a single group is returned as is."""
    if len(embeddings) == 0:
        return dummy_embs_tensor
    if len(embeddings) == 1:
        return embeddings[0]
    return torch.cat(embeddings, dim=dim)


def embeddings_cat_empty_rank_handle_inference(embeddings: List[torch.Tensor], dim: int = 0, device: Optional[str] = None,
                                               dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """The inference form: an empty tensor of the requested dtype on ``device`` when there is nothing to concatenate."""
    if len(embeddings) == 0:
        return torch.empty([0], dtype=dtype, device=torch.device(device) if device is not None else None)
    if len(embeddings) == 1:
        return embeddings[0]
    return torch.cat(embeddings, dim=dim)


class _GroupedLookupBase(BaseEmbeddingLookup[KeyedJaggedTensor, torch.Tensor]):
    def __init__(self) -> None:
        super().__init__()
        self._emb_modules: nn.ModuleList = nn.ModuleList()
        self._feature_splits: List[int] = []
        self.grouped_configs: List[GroupedEmbeddingConfig] = []

    def _finish_init(self, device: Optional[torch.device]) -> None:
        self.register_buffer("_dummy_embs_tensor", torch.empty([0], dtype=torch.float32, device=device, requires_grad=True), persistent=False)

    @property
    def emb_modules(self) -> nn.ModuleList:
        return self._emb_modules

    def state_dict(self, destination=None, prefix: str = "", keep_vars: bool = False) -> Dict[str, Any]:
        if destination is None:
            destination = {}
        for emb_module in self._emb_modules:
            emb_module.state_dict(destination, prefix, keep_vars)
        return destination

    def load_state_dict(self, state_dict, strict: bool = True):  # type: ignore[override]
        m, u = _load_state_dict(self._emb_modules, state_dict)
        return torch.nn.modules.module._IncompatibleKeys(missing_keys=m, unexpected_keys=u)

    def named_parameters(self, prefix: str = "", recurse: bool = True, remove_duplicate: bool = True) -> Iterator[Tuple[str, nn.Parameter]]:
        for emb_module in self._emb_modules:
            yield from emb_module.named_parameters(prefix, recurse)

    def named_buffers(self, prefix: str = "", recurse: bool = True, remove_duplicate: bool = True) -> Iterator[Tuple[str, torch.Tensor]]:
        for emb_module in self._emb_modules:
            yield from emb_module.named_buffers(prefix, recurse)

    def named_parameters_by_table(self) -> Iterator[Tuple[str, torch.Tensor]]:
        for emb_module in self._emb_modules:
            for cfg, w in zip(emb_module.config.embedding_tables, emb_module.split_embedding_weights()):
                yield cfg.name, w

    def prefetch(self, sparse_features: KeyedJaggedTensor, forward_stream=None) -> None:
        """Every table is resident in HBM, so there are no rows to stage ahead of the lookup; a pipeline that schedules prefetches
        keeps working, and is told once that they are free."""
        _warn_once("embedding prefetch requested: tables are HBM-resident here, prefetch is a no-op")

    def flush(self) -> None:
        for m in self._emb_modules:
            m.flush()

    def purge(self) -> None:
        for m in self._emb_modules:
            m.purge()


class GroupedEmbeddingsLookup(_GroupedLookupBase):
    """Unpooled lookup over the TBE groups of one rank -> ``[sum L, D]``."""

    def __init__(self, grouped_configs: List[GroupedEmbeddingConfig], pg: Optional[dist.ProcessGroup] = None, device: Optional[torch.device] = None) -> None:
        super().__init__()
        self.grouped_configs = grouped_configs
        for config in grouped_configs:
            self._emb_modules.append(self._create_embedding_kernel(config, pg, device))
            self._feature_splits.append(config.num_features())
        self._need_prefetch = False
        self._finish_init(device)

    @staticmethod
    def _create_embedding_kernel(config: GroupedEmbeddingConfig, pg, device) -> BaseEmbedding:
        cls = _kernel_class(config.compute_kernel, BatchedDenseEmbedding, BatchedFusedEmbedding)
        return cls(config=config, pg=pg, device=device)

    def forward(self, sparse_features: KeyedJaggedTensor) -> torch.Tensor:
        kernels = list(self._emb_modules)
        if not kernels:
            return self._dummy_embs_tensor
        width = kernels[0].emb_module.max_D
        if len(kernels) == 1:
            return kernels[0](sparse_features).reshape(-1, width)
        parts = sparse_features.split(self._feature_splits)
        return torch.cat([k(f).reshape(-1) for k, f in zip(kernels, parts)]).view(-1, width)


class GroupedPooledEmbeddingsLookup(_GroupedLookupBase):
    """Pooled lookup over the TBE groups of one rank -> ``[B, sum(D)]``."""

    def __init__(self, grouped_configs: List[GroupedEmbeddingConfig], device: Optional[torch.device] = None, pg: Optional[dist.ProcessGroup] = None,
                 feature_processor: Optional[BaseGroupedFeatureProcessor] = None, scale_weight_gradients: bool = True,
                 sharding_type: Optional[ShardingType] = None) -> None:
        super().__init__()
        self.grouped_configs = grouped_configs
        self._sharding_type = sharding_type
        for config in grouped_configs:
            self._emb_modules.append(self._create_embedding_kernel(config, device, pg, sharding_type))
            self._feature_splits.append(config.num_features())
        self._feature_processor = feature_processor
        self._world_size: int = dist.get_world_size(pg) if pg is not None else 1
        self._scale_gradient_factor: int = self._world_size if scale_weight_gradients else 1
        self._finish_init(device)

    @staticmethod
    def _create_embedding_kernel(config: GroupedEmbeddingConfig, device, pg, sharding_type) -> BaseEmbedding:
        cls = _kernel_class(config.compute_kernel, BatchedDenseEmbeddingBag, BatchedFusedEmbeddingBag)
        return cls(config=config, pg=pg, device=device, sharding_type=sharding_type)

    def forward(self, sparse_features: KeyedJaggedTensor) -> torch.Tensor:
        if len(self._emb_modules) == 0:
            return self._dummy_embs_tensor.view(sparse_features.stride(), 0) if sparse_features.stride() else self._dummy_embs_tensor
        parts = [sparse_features] if len(self._emb_modules) == 1 else sparse_features.split(self._feature_splits)
        pooled = [kernel(self._prepare_group_input(cfg, f)) for cfg, kernel, f in zip(self.grouped_configs, self._emb_modules, parts)]
        return embeddings_cat_empty_rank_handle(pooled, self._dummy_embs_tensor, dim=1)

    def _prepare_group_input(self, config: GroupedEmbeddingConfig, features: KeyedJaggedTensor) -> KeyedJaggedTensor:
        """Feature processors run on the owning rank, after the input dist; learnable per-id weights get their gradient scaled
        back up when the pooled gradient was divided by the world size on its way here."""
        fp = self._feature_processor
        if config.has_feature_processor and isinstance(fp, BaseGroupedFeatureProcessor):
            features = fp(features)
        w = features.weights_or_none()
        if config.is_weighted and self._scale_gradient_factor != 1 and w is not None and w.requires_grad:
            features._weights = CommOpGradientScaling.apply(w, self._scale_gradient_factor)
        return features


def fused_optimizer_of_lookups(lookups: List[nn.Module]) -> KeyedOptimizer:
    """``CombinedOptimizer`` over the fused optimizers of every TBE in ``lookups``."""
    optims: List[KeyedOptimizer] = []
    for lookup in lookups:
        while isinstance(lookup, DistributedDataParallel):
            lookup = lookup.module
        for m in getattr(lookup, "emb_modules", []):
            if isinstance(m, FusedOptimizerModule):
                optims.append(m.fused_optimizer)
    return CombinedOptimizer(optims)


def __getattr__(name: str):
    """The inference lookups live in ``infer_embedding_lookup`` (they pull in the quantized kernels); they are reachable from here
    under the reference's import path."""
    if name in ("MetaInferGroupedEmbeddingsLookup", "MetaInferGroupedPooledEmbeddingsLookup", "InferGroupedEmbeddingsLookup",
                "InferGroupedPooledEmbeddingsLookup", "InferCPUGroupedEmbeddingsLookup"):
        from torchrec_b200.distributed import infer_embedding_lookup

        return getattr(infer_embedding_lookup, name)
    raise AttributeError(name)
