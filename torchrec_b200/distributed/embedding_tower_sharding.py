"""Sharded embedding towers: the tables of a tower and its interaction module live on one rank.

The ids of the tower's features travel to the owning rank (the table-wise input distribution of the embedding module), the
owner looks the rows up for the *global* batch and runs the interaction on them, and only the interaction's output -- usually
much narrower than the concatenated embeddings -- is sent back through the pooled all-to-all.  The interaction's parameters are
therefore trained on the owning rank only and are excluded from the data-parallel wrapper.
Counterpart of ``torchrec/distributed/embedding_tower_sharding.py`` (``ShardedEmbeddingTower`` ``:95``, collection ``:442``); the
reference also spreads a tower over the ranks of one host (table-row-wise), which is not built here.
"""
from __future__ import annotations

from typing import Any, Dict, Iterator, List, Optional, Type

import torch
import torch.distributed as dist
from torch import nn

from torchrec_b200.distributed.comm_ops import alltoall_pooled
from torchrec_b200.distributed.embedding_types import BaseEmbeddingSharder, KJTList, ShardedEmbeddingModule
from torchrec_b200.distributed.embeddingbag import EmbeddingBagCollectionSharder, ShardedEmbeddingBagCollection
from torchrec_b200.distributed.types import Awaitable, LazyAwaitable, NoWait, ParameterSharding, QuantizedCommCodecs, ShardingEnv, ShardingType
from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection
from torchrec_b200.modules.embedding_tower import EmbeddingTower, EmbeddingTowerCollection
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor, KeyedTensor


class _TowerOutput(LazyAwaitable[torch.Tensor]):
    def __init__(self, awaitable: Awaitable[torch.Tensor]) -> None:
        super().__init__()
        self._awaitable = awaitable

    def _wait_impl(self) -> torch.Tensor:
        return self._awaitable.wait()


class ShardedEmbeddingTower(ShardedEmbeddingModule):
    def __init__(self, module: EmbeddingTower, table_name_to_parameter_sharding: Dict[str, ParameterSharding], embedding_sharder: EmbeddingBagCollectionSharder,
                 env: ShardingEnv, device: torch.device, module_fqn: Optional[str] = None) -> None:
        super().__init__()
        assert isinstance(module.embedding, EmbeddingBagCollection), "a sharded tower holds an EmbeddingBagCollection"
        owners = set()
        for name, ps in table_name_to_parameter_sharding.items():
            assert ps.sharding_type == ShardingType.TABLE_WISE.value, f"tower table {name} must be table-wise sharded, got {ps.sharding_type}"
            owners.add(ps.ranks[0])
        assert len(owners) == 1, f"all tables of a tower must live on one rank, got ranks {sorted(owners)}"
        self._owner = owners.pop()
        self._env, self._device = env, device
        self._rank, self._world = env.rank, env.world_size
        self._pg = env.process_group
        self._active = self._rank == self._owner
        self.embedding: ShardedEmbeddingBagCollection = embedding_sharder.shard(module.embedding, table_name_to_parameter_sharding, env=env, device=device,
                                                                              module_fqn=(module_fqn + ".embedding") if module_fqn else None)
        if hasattr(self.embedding, "disable_fused_engine"):
            self.embedding.disable_fused_engine()  # the tower consumes the owner-side lookup before any exchange
        self._lookups = self.embedding._lookups
        self.interaction = module.interaction.to(device) if device.type != "meta" else module.interaction
        self._out_dim: Optional[int] = None

    # ---- stages ------------------------------------------------------------------------------------------------
    def input_dist(self, ctx, features: KeyedJaggedTensor) -> Awaitable[Awaitable[KJTList]]:
        ctx.local_batch = features.stride()
        return self.embedding.input_dist(ctx, features)

    def compute(self, ctx, dist_input: KJTList) -> torch.Tensor:
        embs = self.embedding.compute(ctx, dist_input)
        assert len(embs) == 1
        pooled = embs[0]
        if self._active:
            sharding = self.embedding._embedding_shardings[0]
            kt = KeyedTensor(keys=sharding.embedding_names(), length_per_key=sharding.embedding_dims(), values=pooled)
            out = self.interaction(kt)
            assert out.dim() == 2 and out.shape[0] == pooled.shape[0], "the interaction must return [batch, features]"
            return out
        # ranks that do not own the tower still take part in the exchange with a zero-width slice
        return torch.empty((dist_input[0].stride(), 0), device=self._device, requires_grad=True)

    def _output_dim(self, out: torch.Tensor) -> int:
        if self._out_dim is None:
            t = torch.tensor([out.shape[1] if self._active else 0], device=self._device if self._device.type == "cuda" else torch.device("cpu"))
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self._pg)
            self._out_dim = int(t.item())
        return self._out_dim

    def output_dist(self, ctx, output: torch.Tensor) -> LazyAwaitable[torch.Tensor]:
        O = self._output_dim(output)
        dims = [O if r == self._owner else 0 for r in range(self._world)]
        B = ctx.local_batch
        return _TowerOutput(alltoall_pooled(output.contiguous(), batch_size_per_rank=[B] * self._world, dim_sum_per_rank=dims, group=self._pg))

    def create_context(self):
        ctx = self.embedding.create_context()
        ctx.local_batch = 0
        return ctx

    # ---- parameters: everything here is owned by one rank ------------------------------------------------------------
    def sharded_parameter_names(self, prefix: str = "") -> Iterator[str]:
        p = prefix + "." if prefix else ""
        yield from self.embedding.sharded_parameter_names(p + "embedding")
        for name, _ in self.interaction.named_parameters():
            yield f"{p}interaction.{name}"

    @property
    def owner_rank(self) -> int:
        return self._owner

    @property
    def unsharded_module_type(self) -> Type[EmbeddingTower]:
        return EmbeddingTower


class EmbeddingTowerSharder(BaseEmbeddingSharder[EmbeddingTower]):
    def __init__(self, embedding_sharder: Optional[EmbeddingBagCollectionSharder] = None, qcomm_codecs_registry: Optional[Dict[str, QuantizedCommCodecs]] = None) -> None:
        super().__init__(qcomm_codecs_registry=qcomm_codecs_registry)
        self._embedding_sharder = embedding_sharder or EmbeddingBagCollectionSharder(qcomm_codecs_registry=self.qcomm_codecs_registry)

    def shard(self, module: EmbeddingTower, params: Dict[str, ParameterSharding], env: ShardingEnv, device: Optional[torch.device] = None,
              module_fqn: Optional[str] = None) -> ShardedEmbeddingTower:
        device = device if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")
        return ShardedEmbeddingTower(module, params, self._embedding_sharder, env, device, module_fqn)

    @property
    def fused_params(self) -> Optional[Dict[str, Any]]:
        return self._embedding_sharder.fused_params

    def shardable_parameters(self, module: EmbeddingTower) -> Dict[str, nn.Parameter]:
        return self._embedding_sharder.shardable_parameters(module.embedding)

    @property
    def module_type(self) -> Type[EmbeddingTower]:
        return EmbeddingTower

    def sharding_types(self, compute_device_type: str) -> List[str]:
        return [ShardingType.TABLE_WISE.value]


class ShardedEmbeddingTowerCollection(nn.Module):
    """Every tower sharded on its own; ``forward`` concatenates the tower outputs like the unsharded collection."""

    def __init__(self, module: EmbeddingTowerCollection, tower_to_params: List[Dict[str, ParameterSharding]], tower_sharder: EmbeddingTowerSharder, env: ShardingEnv,
                 device: torch.device) -> None:
        super().__init__()
        self.towers = nn.ModuleList([tower_sharder.shard(t, p, env, device, module_fqn=f"towers.{i}") for i, (t, p) in enumerate(zip(module.towers, tower_to_params))])
        self._input_params = module._input_params

    def forward(self, features: Optional[KeyedJaggedTensor] = None, weighted_features: Optional[KeyedJaggedTensor] = None) -> torch.Tensor:
        pending = []
        for tower, (has_f, has_w) in zip(self.towers, self._input_params):
            pending.append(tower(features if has_f else weighted_features))
        return torch.cat([p.wait() for p in pending], dim=1)
